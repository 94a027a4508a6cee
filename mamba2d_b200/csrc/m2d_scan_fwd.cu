// Forward entry point of the wavefront scan: one fused kernel, y written directly.
#include "plan.cuh"
#include "sweep_fwd.cuh"

namespace m2d {

template <typename io_t, bool VEC, bool CHAINED, int CB>
__global__ void __launch_bounds__(256, 2) m2d_fwd_kernel(const FwdArgs a) {
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
    if (threadIdx.x < 32) stage_params<io_t>(params, a.AT, a.AL, a.N, ch0, chv, n0, nv, lane);
    __syncthreads();

    // gridDim.x = chains x a.chain: CTA (chain_id, cpos) walks images chain_id, chain_id + chains, ...
    const int chains = (int)gridDim.x / a.chain;
    const int chain_id = (int)blockIdx.x / a.chain, cpos = (int)blockIdx.x % a.chain;
    const int nb = (a.B - chain_id + chains - 1) / chains;
    forward_sweep<io_t, VEC, false, CHAINED, CB>(a, handoff, params, D_own, chain_id, chains, nb, cpos, a.chain);
}

template <typename io_t>
static int launch_fwd(const m2d_scan_desc* d, const Plan& pl, bool vec, cudaStream_t st) {
    FwdArgs a;
    a.B = d->B; a.H = d->H; a.W = d->W; a.E = d->E; a.N = d->N;
    a.dir = (d->flags & M2D_SCAN_REVERSE) ? -1 : 1;
    a.x = d->x; a.dT = d->dT; a.dL = d->dL; a.AT = d->AT; a.AL = d->AL;
    a.BT = d->BT; a.BL = d->BL; a.C = d->C; a.D = d->D;
    a.pBT = d->BT_pitch; a.pBL = d->BL_pitch; a.pC = d->C_pitch;
    a.y = d->y;
    a.gy = nullptr;
    a.ring = static_cast<float4*>(d->workspace);
    a.hs = nullptr;
    a.Rb = pl.Rb; a.nbands = pl.nbands;
    a.chain = pl.chain;
    a.bnd = nullptr; a.progress = nullptr; a.status = nullptr;
    if (pl.chain > 1) {
        // workspace = [boundary rows of every band][column counters + status word]
        char* ws = static_cast<char*>(d->workspace);
        const size_t nband = (size_t)d->B * pl.groups * pl.nbands;
        const size_t bnd_bytes = align256(nband * d->W * kSlotF4 * sizeof(float4));
        a.bnd = reinterpret_cast<float4*>(ws);
        a.progress = reinterpret_cast<int*>(ws + bnd_bytes);
        a.status = a.progress + nband;
        if (cudaMemsetAsync(a.progress, 0, (nband + 1) * sizeof(int), st) != cudaSuccess) return M2D_ERR_LAUNCH;
    }
    dim3 block(pl.warps * 32);
    void (*kern)(const FwdArgs);
    if (pl.cb == 2) {
        kern = pl.chain > 1 ? (vec ? m2d_fwd_kernel<io_t, true, true, 2> : m2d_fwd_kernel<io_t, false, true, 2>)
                            : (vec ? m2d_fwd_kernel<io_t, true, false, 2> : m2d_fwd_kernel<io_t, false, false, 2>);
    } else {
        kern = pl.chain > 1 ? (vec ? m2d_fwd_kernel<io_t, true, true, 1> : m2d_fwd_kernel<io_t, false, true, 1>)
                            : (vec ? m2d_fwd_kernel<io_t, true, false, 1> : m2d_fwd_kernel<io_t, false, false, 1>);
    }
    if (pl.smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess)
        return M2D_ERR_LAUNCH;
    if (a.chain > 1) {
        // CTAs of a chain wait on one another, so every CTA of the launch must be resident at the same
        // time.  A cooperative launch guarantees that or fails cleanly; the chain is shortened until
        // the device accepts it (the workspace layout does not depend on the chain length).
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, (int)block.x, pl.smem) != cudaSuccess || per_sm < 1)
            return M2D_ERR_LAUNCH;
        const long long fit = (long long)per_sm * sm_count() / ((long long)pl.grid_x * pl.groups);
        if (fit < a.chain) a.chain = fit < 1 ? 1 : (int)fit;
        for (;;) {
            dim3 grid(pl.grid_x * a.chain, pl.groups);
            void* args[] = {&a};
            const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), grid, block, args, pl.smem, st);
            if (e == cudaSuccess) return M2D_OK;
            cudaGetLastError();
            if (e != cudaErrorCooperativeLaunchTooLarge || a.chain == 1) return M2D_ERR_LAUNCH;
            a.chain = a.chain > 2 ? a.chain - a.chain / 4 - 1 : 1;
        }
    }
    dim3 grid(pl.grid_x, pl.groups);
    kern<<<grid, block, pl.smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? M2D_OK : M2D_ERR_LAUNCH;
}

}  // namespace m2d

extern "C" uint64_t m2d_scan_fwd_workspace(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, false, false) != M2D_OK) return 0;
    return m2d::plan_fwd(d).scratch;
}

extern "C" int64_t m2d_scan_fwd_status_offset(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, false, false) != M2D_OK) return -1;
    const m2d::Plan pl = m2d::plan_fwd(d);
    if (pl.chain <= 1) return -1;
    const size_t nband = (size_t)d->B * pl.groups * pl.nbands;
    return (int64_t)(m2d::align256(nband * d->W * m2d::kSlotF4 * sizeof(float4)) + nband * sizeof(int));
}

extern "C" int m2d_scan_fwd(const m2d_scan_desc* d, void* stream) {
    int rc = m2d::check_desc(d, false, true);
    if (rc != M2D_OK) return rc;
    if (!d->y) return M2D_ERR_NULL;
    const m2d::Plan pl = m2d::plan_fwd(d);
    if (pl.scratch > 0 && (!d->workspace || d->workspace_bytes < pl.scratch || (reinterpret_cast<uintptr_t>(d->workspace) & 255)))
        return M2D_ERR_WORKSPACE;
    const bool vec = m2d::vector_ok(d, false);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->dtype == M2D_F32) return m2d::launch_fwd<float>(d, pl, vec, st);
    return m2d::launch_fwd<__nv_bfloat16>(d, pl, vec, st);
}
