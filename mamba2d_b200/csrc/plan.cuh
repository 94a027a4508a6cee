// Host-side descriptor validation and launch planning (header-only, used by both entry points).
#pragma once

#include "common.cuh"

namespace m2d {

inline int sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
        cudaGetLastError();   // clear; planning still works on a machine without a device
        n = 148;
    }
    return n;
}

inline int check_desc(const m2d_scan_desc* d, bool bwd, bool need_ptrs) {
    if (!d) return M2D_ERR_NULL;
    if (d->struct_bytes != sizeof(m2d_scan_desc)) return M2D_ERR_ABI;
    if (d->dtype != M2D_F32 && d->dtype != M2D_BF16) return M2D_ERR_DTYPE;
    if (d->B < 1 || d->E < 1 || d->N < 1 || d->H < 2 || d->W < 2) return M2D_ERR_SHAPE;
    if (d->N > kMaxN) return M2D_ERR_UNSUPPORTED_N;
    if (d->BT_pitch < d->N || d->BL_pitch < d->N || d->C_pitch < d->N) return M2D_ERR_PITCH;
    if (need_ptrs) {
        if (!d->x || !d->dT || !d->dL || !d->AT || !d->AL || !d->BT || !d->BL || !d->C || !d->D) return M2D_ERR_NULL;
        if (bwd && (!d->gy || !d->d_x || !d->d_dT || !d->d_dL || !d->d_AT || !d->d_AL || !d->d_BT || !d->d_BL || !d->d_C || !d->d_D))
            return M2D_ERR_NULL;
    }
    return M2D_OK;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// 128-bit (fp32) / 64-bit (bf16) vector loads need channel and state counts that are multiples
// of 4, pitches that are multiples of 4 elements and suitably aligned base pointers.
inline bool vector_ok(const m2d_scan_desc* d, bool bwd) {
    const size_t al = d->dtype == M2D_F32 ? 16 : 8;
    bool ok = (d->E % 4 == 0) && (d->N % 4 == 0) && (d->BT_pitch % 4 == 0) && (d->BL_pitch % 4 == 0) && (d->C_pitch % 4 == 0);
    ok = ok && aligned(d->x, al) && aligned(d->dT, al) && aligned(d->dL, al) && aligned(d->BT, al) && aligned(d->BL, al) && aligned(d->C, al);
    if (bwd) ok = ok && aligned(d->gy, al);
    return ok;
}

inline int pick_warps(int H, int max_warps) {
    if (H <= max_warps) return H;
    int best = max_warps, best_waste = 1 << 30;
    for (int w = max_warps; w >= (max_warps + 1) / 2 + 1; --w) {
        const int waste = (H + w - 1) / w * w - H;
        if (waste < best_waste) { best_waste = waste; best = w; }
    }
    return best;
}

inline Plan plan_common(const m2d_scan_desc* d, int max_warps, int ctas_per_sm) {
    Plan p;
    p.groups = (d->E + kGroup - 1) / kGroup;
    p.warps = pick_warps(d->H, max_warps);
    p.Rb = p.warps;
    p.nbands = (d->H + p.Rb - 1) / p.Rb;
    if (p.nbands > 1 && p.Rb > d->W - 1) {
        // a band boundary must be written at least one step before the next band reads it
        p.Rb = d->W - 1;
        p.warps = p.Rb;
        p.nbands = (d->H + p.Rb - 1) / p.Rb;
    }
    const long long slots = (long long)ctas_per_sm * sm_count();
    const long long units = (long long)d->B * p.groups;
    const long long per = (units + slots - 1) / slots;          // images per CTA
    p.grid_x = (int)((d->B + per - 1) / per);
    p.smem = (size_t)2 * (p.warps + 1) * kSlotF4 * sizeof(float4);
    p.scratch = 0;
    return p;
}

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

inline Plan plan_fwd(const m2d_scan_desc* d) {
    Plan p = plan_common(d, 8, 2);
    if (p.nbands > 1) p.scratch = align256((size_t)p.grid_x * p.groups * d->W * kSlotF4 * sizeof(float4));
    return p;
}

}  // namespace m2d
