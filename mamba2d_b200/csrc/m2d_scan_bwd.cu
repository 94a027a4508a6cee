// Backward entry point of the wavefront scan: recompute sweep + adjoint sweep in one kernel,
// followed by a small kernel that casts the fp32 accumulators of the reduced gradients.
#include <cstdlib>

#include "launch.cuh"
#include "sweep_bwd.cuh"
#include "sweep_rows.cuh"

// Row-warps per CTA of the backward kernel (two CTAs per SM): the register budget per thread follows
// from it (6 warps: 168 registers).
#ifndef M2D_BWD_MAXW
#define M2D_BWD_MAXW 6
#endif
#ifndef M2D_BWD_MINB
#define M2D_BWD_MINB 2
#endif

namespace m2d {

// Workspace layout of the backward pass (all regions 256-byte aligned):
//   status   one word, nonzero if a wait between CTAs gave up
//   counters chained CTAs only: two column counters per band (recompute sweep, adjoint sweep)
//   ring     per-CTA band-boundary ring, ctas*W*2 KiB (only if nbands > 1); with chained CTAs one
//            boundary row per band instead (h downwards in the recompute sweep, pT upwards in the
//            adjoint sweep)
//   hs       state record written by the recompute sweep     B*groups*H*W*2 KiB (1 KiB with bf16 I/O)
//   acc      bf16 I/O only: fp32 accumulators 3 x [B*H*W][N] | 2 x [E][N] | [E], zeroed before the
//            main kernel and cast by a second kernel.  With fp32 I/O the kernel accumulates straight
//            into the caller's (zeroed) gradient tensors and this region is empty.
struct BwdLayout {
    size_t counters, ring, hs, acc, acc_bytes, total;
};

inline BwdLayout bwd_layout(const m2d_scan_desc* d, const Plan& p) {
    BwdLayout L;
    size_t off = kStatusBytes;
    L.counters = off;
    L.ring = off;
    if (p.chain > 1) {
        const size_t nband = (size_t)d->B * p.groups * p.nbands;
        off += align256(2 * nband * sizeof(int));
        L.ring = off;
        off += align256(nband * d->W * kSlotF4 * sizeof(float4));
    } else if (p.nbands > 1) {
        off += align256((size_t)p.grid_x * p.groups * d->W * kSlotF4 * sizeof(float4));
    }
    L.hs = off;
    off += align256((size_t)d->B * p.groups * d->H * d->W * (d->dtype == M2D_F32 ? 128 : 64) * sizeof(float4));
    L.acc = off;
    L.acc_bytes = 0;
    if (d->dtype != M2D_F32) {
        const size_t npn = (size_t)d->B * d->H * d->W * d->N, en = (size_t)d->E * d->N;
        L.acc_bytes = align256((3 * npn + 2 * en + d->E) * sizeof(float));
    }
    off += L.acc_bytes;
    L.total = off;
    return L;
}

inline Plan plan_bwd(const m2d_scan_desc* d) {
    // tuning knob: M2D_BWD_WARPS=<1..max> overrides the row-warps per CTA of the backward kernel
    int maxw = M2D_BWD_MAXW;
    if (const char* e = getenv("M2D_BWD_WARPS")) { const int v = atoi(e); if (v >= 1 && v <= M2D_BWD_MAXW) maxw = v; }
    Plan p = plan_best(d, maxw, 2 * M2D_BWD_MAXW);
    p.smem = bwd_smem_bytes(p.warps) + kParamF4 * sizeof(float4);
    // few images on a large map: chain CTAs along the bands of an image, as the forward does
    {
        const long long slots = (long long)(2 * M2D_BWD_MAXW / p.warps > 0 ? 2 * M2D_BWD_MAXW / p.warps : 1) * sm_count();
        const long long ctas = (long long)p.grid_x * p.groups;
        if (p.nbands > 1 && ctas * 2 <= slots) p.chain = bound_chain(slots / ctas, p.nbands, d->W, p.Rb);
    }
    if (p.chain == 1 && d->W >= 3) {
        // batch mode: the nested-loop kernel (maps narrower than three columns keep the flat one)
        p = plan_best(d, maxw, 2 * M2D_BWD_MAXW, 1, 2);
        p.rows = true;
        p.smem = rows_bwd_smem_bytes(p.warps) + kParamF4 * sizeof(float4);
    }
    p.scratch = bwd_layout(d, p).total;
    return p;
}

// Several CTAs per image (large maps, few images): the flat step loops with the cross-CTA hand-off.
template <typename io_t, bool VEC>
__global__ void __launch_bounds__(M2D_BWD_MAXW * 32, 2) m2d_bwd_chained_kernel(const ScanArgs a) {
    constexpr bool CHAINED = true;
    extern __shared__ float4 handoff[];
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));

    const int total = (int)(bwd_smem_bytes(nwarps) / sizeof(float4));
    for (int k = threadIdx.x; k < total; k += blockDim.x) handoff[k] = make_float4(0.f, 0.f, 0.f, 0.f);

    const int ch_own = g * kGroup + lane;
    const float D_own = ch_own < a.E ? load1(static_cast<const io_t*>(a.D), ch_own) : 0.f;
    float dAT[4][4], dAL[4][4], dD[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        dD[c] = 0.f;
#pragma unroll
        for (int n = 0; n < 4; ++n) dAT[c][n] = dAL[c][n] = 0.f;
    }
    __syncthreads();
    float4* const params = reinterpret_cast<float4*>(reinterpret_cast<char*>(handoff) + bwd_smem_bytes(nwarps));
    if (threadIdx.x < 32) stage_params<io_t>(params, a.AT, a.AL, a.N, ch0, chv, n0, nv, lane, a.a_log);
    __syncthreads();

    // gridDim.x = chains x a.chain: CTA (chain_id, cpos) walks images chain_id, chain_id + chains, ...
    const int chains = (int)gridDim.x / a.chain;
    const int chain_id = (int)blockIdx.x / a.chain, cpos = (int)blockIdx.x % a.chain;
    for (int b = chain_id; b < a.B; b += chains) {
        forward_sweep<io_t, VEC, true, CHAINED, 1>(a, handoff, params, D_own, b, 0, 1, cpos, a.chain);
        reverse_sweep<io_t, VEC, CHAINED>(a, handoff, params, D_own, dAT, dAL, dD, b, cpos, a.chain);
    }

    // ---- per-(channel,state) sums: fold the CTA's row-warps through shared memory, then one
    //      atomic per value from warp 0 ----------------------------------------------------------
    float* red = reinterpret_cast<float*>(handoff);     // reuse: needs 36 floats per thread
    const int slot = 2 * (nwarps + 1) * kSlotF4 * 4;     // floats available
    const bool fits = (int)blockDim.x * 36 <= slot;
    if (fits && nwarps > 1) {
        float* mine = red + (size_t)threadIdx.x * 36;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int n = 0; n < 4; ++n) { mine[c * 4 + n] = dAT[c][n]; mine[16 + c * 4 + n] = dAL[c][n]; }
            mine[32 + c] = dD[c];
        }
        __syncthreads();
        if (r == 0) {
            for (int w = 1; w < nwarps; ++w) {
                const float* o = red + (size_t)(w * 32 + lane) * 36;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int n = 0; n < 4; ++n) { dAT[c][n] += o[c * 4 + n]; dAL[c][n] += o[16 + c * 4 + n]; }
                    dD[c] += o[32 + c];
                }
            }
        }
    }
    if (r == 0 || !(fits && nwarps > 1)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (c < chv) {
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    if (n < nv) {
                        const long long idx = (long long)(ch0 + c) * a.N + n0 + n;
                        // with A given as A_log the gradient asked for is d_A_log = d_A * A (A = -exp(A_log),
                        // models/kernels/wavefront_cuda.py:72-73); the product is linear, so every CTA
                        // scales its own partial sum
                        const float sT = a.a_log ? load_A<io_t>(a.AT, idx, 1, true) : 1.f;
                        const float sL = a.a_log ? load_A<io_t>(a.AL, idx, 1, true) : 1.f;
                        atomicAdd(a.accAT + idx, dAT[c][n] * sT);
                        atomicAdd(a.accAL + idx, dAL[c][n] * sL);
                    }
                }
                if (nq == 0) atomicAdd(a.accD + ch0 + c, dD[c]);
            }
        }
    }
}

// Batch mode (one CTA per image and channel group): both sweeps written as nested loops.
template <typename io_t, bool VEC>
__global__ void __launch_bounds__(M2D_BWD_MAXW * 32, M2D_BWD_MINB) m2d_bwd_kernel(const ScanArgs a) {
    extern __shared__ float4 smem[];
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));

    const int total = (int)(rows_bwd_smem_bytes(nwarps) / sizeof(float4));
    for (int k = threadIdx.x; k < total; k += blockDim.x) smem[k] = make_float4(0.f, 0.f, 0.f, 0.f);

    const int ch_own = g * kGroup + lane;
    const float D_own = ch_own < a.E ? load1(static_cast<const io_t*>(a.D), ch_own) : 0.f;
    float dAT[4][4], dAL[4][4], dD[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        dD[c] = 0.f;
#pragma unroll
        for (int n = 0; n < 4; ++n) dAT[c][n] = dAL[c][n] = 0.f;
    }
    __syncthreads();
    float4* const params = reinterpret_cast<float4*>(reinterpret_cast<char*>(smem) + rows_bwd_smem_bytes(nwarps));
    if (threadIdx.x < 32) stage_params<io_t>(params, a.AT, a.AL, a.N, ch0, chv, n0, nv, lane, a.a_log);
    __syncthreads();

    for (int b = (int)blockIdx.x; b < a.B; b += (int)gridDim.x) {
        forward_rows<io_t, VEC, true>(a, smem, params, D_own, b, 0, 1);
        reverse_rows<io_t, VEC>(a, smem, params, D_own, dAT, dAL, dD, b);
    }

    // ---- per-(channel,state) sums: fold the CTA's row-warps through shared memory, then one
    //      atomic per value from warp 0 ----------------------------------------------------------
    float* red = reinterpret_cast<float*>(smem);        // reuse: needs 36 floats per thread
    const int slot = (int)rows_handoff_f4(nwarps) * 4;   // floats available
    const bool fits = (int)blockDim.x * 36 <= slot;
    if (fits && nwarps > 1) {
        float* mine = red + (size_t)threadIdx.x * 36;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int n = 0; n < 4; ++n) { mine[c * 4 + n] = dAT[c][n]; mine[16 + c * 4 + n] = dAL[c][n]; }
            mine[32 + c] = dD[c];
        }
        __syncthreads();
        if (r == 0) {
            for (int w = 1; w < nwarps; ++w) {
                const float* o = red + (size_t)(w * 32 + lane) * 36;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int n = 0; n < 4; ++n) { dAT[c][n] += o[c * 4 + n]; dAL[c][n] += o[16 + c * 4 + n]; }
                    dD[c] += o[32 + c];
                }
            }
        }
    }
    if (r == 0 || !(fits && nwarps > 1)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (c < chv) {
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    if (n < nv) {
                        const long long idx = (long long)(ch0 + c) * a.N + n0 + n;
                        // with A given as A_log the gradient asked for is d_A_log = d_A * A (A = -exp(A_log),
                        // models/kernels/wavefront_cuda.py:72-73); the product is linear, so every CTA
                        // scales its own partial sum
                        const float sT = a.a_log ? load_A<io_t>(a.AT, idx, 1, true) : 1.f;
                        const float sL = a.a_log ? load_A<io_t>(a.AL, idx, 1, true) : 1.f;
                        atomicAdd(a.accAT + idx, dAT[c][n] * sT);
                        atomicAdd(a.accAL + idx, dAL[c][n] * sL);
                    }
                }
                if (nq == 0) atomicAdd(a.accD + ch0 + c, dD[c]);
            }
        }
    }
}

// bf16 I/O: cast the fp32 accumulators into the caller's gradient tensors (d_AT / d_AL stay fp32 when
// they are gradients of the fp32 parameter A_log).
template <typename io_t>
__global__ void m2d_bwd_finalize(const float* __restrict__ acc, io_t* d_BT, io_t* d_BL, io_t* d_C, void* d_AT, void* d_AL,
                                 io_t* d_D, long long npn, long long en, int E, int a_log) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    for (long long k = tid; k < npn; k += nthreads) {
        store1(d_BT, k, acc[k]);
        store1(d_BL, k, acc[npn + k]);
        store1(d_C, k, acc[2 * npn + k]);
    }
    const float* accA = acc + 3 * npn;
    for (long long k = tid; k < en; k += nthreads) {
        if (a_log) {
            static_cast<float*>(d_AT)[k] = accA[k];
            static_cast<float*>(d_AL)[k] = accA[en + k];
        } else {
            store1(static_cast<io_t*>(d_AT), k, accA[k]);
            store1(static_cast<io_t*>(d_AL), k, accA[en + k]);
        }
    }
    for (long long k = tid; k < E; k += nthreads) store1(d_D, k, accA[2 * en + k]);
}

template <typename io_t>
static int launch_bwd(const m2d_scan_desc* d, const Plan& pl, bool vec, cudaStream_t st) {
    const BwdLayout L = bwd_layout(d, pl);
    char* ws = static_cast<char*>(d->workspace);
    ScanArgs a;
    fill_common_args(a, d, pl);
    a.status = reinterpret_cast<int*>(ws);
    a.ring = reinterpret_cast<float4*>(ws + L.ring);
    size_t zero_bytes = sizeof(int);
    if (pl.chain > 1) {
        const size_t nband = (size_t)d->B * pl.groups * pl.nbands;
        a.bnd = reinterpret_cast<float4*>(ws + L.ring);
        a.progress = reinterpret_cast<int*>(ws + L.counters);
        zero_bytes = kStatusBytes + 2 * nband * sizeof(int);
    }
    if (cudaMemsetAsync(ws, 0, zero_bytes, st) != cudaSuccess) return M2D_ERR_LAUNCH;
    a.gy = d->gy;
    a.hs = reinterpret_cast<float4*>(ws + L.hs);
    a.d_x = d->d_x; a.d_dT = d->d_dT; a.d_dL = d->d_dL;
    const size_t npn = (size_t)d->B * d->H * d->W * d->N, en = (size_t)d->E * d->N;
    if (d->dtype == M2D_F32) {
        a.accBT = static_cast<float*>(d->d_BT); a.accBL = static_cast<float*>(d->d_BL); a.accC = static_cast<float*>(d->d_C);
        a.accAT = static_cast<float*>(d->d_AT); a.accAL = static_cast<float*>(d->d_AL); a.accD = static_cast<float*>(d->d_D);
        // the six accumulated outputs start from zero; a caller that carved the three per-pixel ones
        // out of one buffer and the three per-channel ones out of another, in this order, gets two
        // memsets instead of six (they are 3 us each against a 200 us kernel at the smallest stage)
        const bool big_adjacent = a.accBL == a.accBT + npn && a.accC == a.accBL + npn;
        const bool small_adjacent = a.accAL == a.accAT + en && a.accD == a.accAL + en;
        bool ok;
        if (big_adjacent && a.accAT == a.accC + npn && small_adjacent) {
            ok = cudaMemsetAsync(a.accBT, 0, (3 * npn + 2 * en + (size_t)d->E) * 4, st) == cudaSuccess;
        } else {
            ok = big_adjacent ? cudaMemsetAsync(a.accBT, 0, 3 * npn * 4, st) == cudaSuccess
                              : (cudaMemsetAsync(a.accBT, 0, npn * 4, st) == cudaSuccess && cudaMemsetAsync(a.accBL, 0, npn * 4, st) == cudaSuccess &&
                                 cudaMemsetAsync(a.accC, 0, npn * 4, st) == cudaSuccess);
            ok = ok && (small_adjacent ? cudaMemsetAsync(a.accAT, 0, (2 * en + (size_t)d->E) * 4, st) == cudaSuccess
                                       : (cudaMemsetAsync(a.accAT, 0, en * 4, st) == cudaSuccess && cudaMemsetAsync(a.accAL, 0, en * 4, st) == cudaSuccess &&
                                          cudaMemsetAsync(a.accD, 0, (size_t)d->E * 4, st) == cudaSuccess));
        }
        if (!ok) return M2D_ERR_LAUNCH;
    } else {
        float* acc = reinterpret_cast<float*>(ws + L.acc);
        a.accBT = acc; a.accBL = acc + npn; a.accC = acc + 2 * npn;
        a.accAT = acc + 3 * npn; a.accAL = a.accAT + en; a.accD = a.accAL + en;
        if (cudaMemsetAsync(acc, 0, L.acc_bytes, st) != cudaSuccess) return M2D_ERR_LAUNCH;
    }
    // (the flat kernel with a chain of one CTA is the fallback for maps the nested-loop kernel does not take)
    void (*kern)(const ScanArgs) = pl.rows ? (vec ? m2d_bwd_kernel<io_t, true> : m2d_bwd_kernel<io_t, false>)
                                           : (vec ? m2d_bwd_chained_kernel<io_t, true> : m2d_bwd_chained_kernel<io_t, false>);
    const int rc = launch_sweep_kernel(kern, a, pl, d->W, st);
    if (rc != M2D_OK) return rc;
    if (d->dtype != M2D_F32) {
        const int fin_blocks = (int)((npn + 255) / 256 < 148 * 8 ? (npn + 255) / 256 : 148 * 8);
        m2d_bwd_finalize<io_t><<<fin_blocks, 256, 0, st>>>(a.accBT, static_cast<io_t*>(d->d_BT), static_cast<io_t*>(d->d_BL),
                                                          static_cast<io_t*>(d->d_C), d->d_AT, d->d_AL, static_cast<io_t*>(d->d_D),
                                                          (long long)npn, (long long)en, d->E, a.a_log);
        if (cudaGetLastError() != cudaSuccess) return M2D_ERR_LAUNCH;
    }
    return M2D_OK;
}

}  // namespace m2d

extern "C" uint64_t m2d_scan_bwd_workspace(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, true, false) != M2D_OK) return 0;
    return m2d::plan_bwd(d).scratch;
}

extern "C" int64_t m2d_scan_bwd_status_offset(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, true, false) != M2D_OK) return -1;
    return 0;
}

extern "C" int m2d_scan_bwd_chain(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, true, false) != M2D_OK) return 0;
    return m2d::plan_bwd(d).chain;
}

extern "C" int m2d_scan_bwd(const m2d_scan_desc* d, void* stream) {
    int rc = m2d::check_desc(d, true, true);
    if (rc != M2D_OK) return rc;
    const m2d::Plan pl = m2d::plan_bwd(d);
    if (!d->workspace || d->workspace_bytes < pl.scratch || (reinterpret_cast<uintptr_t>(d->workspace) & 255))
        return M2D_ERR_WORKSPACE;
    const bool vec = m2d::vector_ok(d, true);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->dtype == M2D_F32) return m2d::launch_bwd<float>(d, pl, vec, st);
    return m2d::launch_bwd<__nv_bfloat16>(d, pl, vec, st);
}
