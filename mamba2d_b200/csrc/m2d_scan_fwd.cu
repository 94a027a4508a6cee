// Forward entry point of the wavefront scan: one fused kernel, y written directly.
#include "launch.cuh"
#include "sweep_rows.cuh"

namespace m2d {

// Several CTAs per image (large maps, few images): the flat step loop with the cross-CTA hand-off.
template <typename io_t, bool VEC>
__global__ void __launch_bounds__(256, 2) m2d_fwd_chained_kernel(const FwdArgs a) {
    constexpr int CB = 1;
    extern __shared__ float4 handoff[];
    const int lane = threadIdx.x & 31;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));

    const int total = (int)(sweep_smem_bytes(blockDim.x >> 5, CB) / sizeof(float4));
    for (int k = threadIdx.x; k < total; k += blockDim.x) handoff[k] = make_float4(0.f, 0.f, 0.f, 0.f);

    const int ch_own = g * kGroup + lane;
    const float D_own = ch_own < a.E ? load1(static_cast<const io_t*>(a.D), ch_own) : 0.f;
    __syncthreads();
    float4* const params = reinterpret_cast<float4*>(reinterpret_cast<char*>(handoff) + sweep_smem_bytes((blockDim.x >> 5), CB));
    if (threadIdx.x < 32) stage_params<io_t>(params, a.AT, a.AL, a.N, ch0, chv, n0, nv, lane, a.a_log);
    __syncthreads();

    // gridDim.x = chains x a.chain: CTA (chain_id, cpos) walks images chain_id, chain_id + chains, ...
    const int chains = (int)gridDim.x / a.chain;
    const int chain_id = (int)blockIdx.x / a.chain, cpos = (int)blockIdx.x % a.chain;
    const int nb = (a.B - chain_id + chains - 1) / chains;
    forward_sweep<io_t, VEC, false, true, CB>(a, handoff, params, D_own, chain_id, chains, nb, cpos, a.chain);
}

// Batch mode (one CTA per image and channel group): the sweep written as nested loops.
template <typename io_t, bool VEC>
__global__ void __launch_bounds__(256, 2) m2d_fwd_kernel(const FwdArgs a) {
    extern __shared__ float4 smem[];
    const int lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));
    const int total = (int)(rows_fwd_smem_bytes(nwarps) / sizeof(float4));
    for (int k = threadIdx.x; k < total; k += blockDim.x) smem[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int ch_own = g * kGroup + lane;
    const float D_own = ch_own < a.E ? load1(static_cast<const io_t*>(a.D), ch_own) : 0.f;
    __syncthreads();
    float4* const params = reinterpret_cast<float4*>(reinterpret_cast<char*>(smem) + rows_fwd_smem_bytes(nwarps));
    if (threadIdx.x < 32) stage_params<io_t>(params, a.AT, a.AL, a.N, ch0, chv, n0, nv, lane, a.a_log);
    __syncthreads();
    const int nb = (a.B - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    forward_rows<io_t, VEC, false>(a, smem, params, D_own, blockIdx.x, gridDim.x, nb);
}

template <typename io_t>
static int launch_fwd(const m2d_scan_desc* d, const Plan& pl, bool vec, cudaStream_t st) {
    FwdArgs a;
    fill_common_args(a, d, pl);
    char* ws = static_cast<char*>(d->workspace);
    a.y = d->y;
    a.status = reinterpret_cast<int*>(ws);
    a.ring = reinterpret_cast<float4*>(ws + kStatusBytes);
    size_t zero_bytes = sizeof(int);
    if (pl.chain > 1) {
        // workspace = [status word][column counters][boundary rows of every band]: one memset clears the
        // status word and the counters
        const size_t nband = (size_t)d->B * pl.groups * pl.nbands;
        a.progress = reinterpret_cast<int*>(ws + kStatusBytes);
        a.bnd = reinterpret_cast<float4*>(ws + kStatusBytes + align256(nband * sizeof(int)));
        zero_bytes = kStatusBytes + nband * sizeof(int);
    }
    if (cudaMemsetAsync(ws, 0, zero_bytes, st) != cudaSuccess) return M2D_ERR_LAUNCH;
    // (the flat kernel with a chain of one CTA is the fallback for maps the nested-loop kernel does not take)
    void (*kern)(const FwdArgs) = pl.rows ? (vec ? m2d_fwd_kernel<io_t, true> : m2d_fwd_kernel<io_t, false>)
                                          : (vec ? m2d_fwd_chained_kernel<io_t, true> : m2d_fwd_chained_kernel<io_t, false>);
    return launch_sweep_kernel(kern, a, pl, d->W, st);
}

}  // namespace m2d

extern "C" uint64_t m2d_scan_fwd_workspace(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, false, false) != M2D_OK) return 0;
    return m2d::plan_fwd(d).scratch;
}

extern "C" int64_t m2d_scan_fwd_status_offset(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, false, false) != M2D_OK) return -1;
    return 0;
}

extern "C" int m2d_scan_fwd_chain(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, false, false) != M2D_OK) return 0;
    return m2d::plan_fwd(d).chain;
}

extern "C" int m2d_scan_chain_bound(int want, int nbands, int steps_per_row, int rows_per_band) {
    if (nbands < 1 || steps_per_row < 1 || rows_per_band < 1) return 0;
    return m2d::bound_chain(want, nbands, steps_per_row, rows_per_band);
}

extern "C" int m2d_scan_fwd(const m2d_scan_desc* d, void* stream) {
    int rc = m2d::check_desc(d, false, true);
    if (rc != M2D_OK) return rc;
    if (!d->y) return M2D_ERR_NULL;
    const m2d::Plan pl = m2d::plan_fwd(d);
    if (!d->workspace || d->workspace_bytes < pl.scratch || (reinterpret_cast<uintptr_t>(d->workspace) & 255))
        return M2D_ERR_WORKSPACE;
    const bool vec = m2d::vector_ok(d, false);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->dtype == M2D_F32) return m2d::launch_fwd<float>(d, pl, vec, st);
    return m2d::launch_fwd<__nv_bfloat16>(d, pl, vec, st);
}
