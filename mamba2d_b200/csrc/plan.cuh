// Host-side descriptor validation and launch planning (header-only, used by both entry points).
#pragma once

#include <cstdlib>

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

// Test hooks in desc->flags are honoured only when the environment asks for them.
inline bool test_hooks_enabled() {
    const char* e = getenv("M2D_TEST_HOOKS");
    return e && e[0] == '1';
}

inline int check_desc(const m2d_scan_desc* d, bool bwd, bool need_ptrs) {
    if (!d) return M2D_ERR_NULL;
    if (d->struct_bytes != sizeof(m2d_scan_desc)) return M2D_ERR_ABI;
    if (d->dtype != M2D_F32 && d->dtype != M2D_BF16) return M2D_ERR_DTYPE;
    {
        unsigned known = M2D_SCAN_REVERSE | M2D_SCAN_A_LOG;
        if (!bwd) known |= M2D_SCAN_GELU_OUT;      // an output activation exists in the forward only
        if (test_hooks_enabled()) known |= M2D_SCAN_TEST_WITHHOLD;
        if (d->flags & ~known) return M2D_ERR_FLAGS;
    }
    if (d->B < 1 || d->E < 1 || d->N < 1 || d->H < 2 || d->W < 2) return M2D_ERR_SHAPE;
    if (d->N > kMaxN) return M2D_ERR_UNSUPPORTED_N;
    if (d->BT_pitch < d->N || d->BL_pitch < d->N || d->C_pitch < d->N) return M2D_ERR_PITCH;
    {
        // the kernels index every tensor with 31-bit element offsets
        long long widest = d->E > 48 ? d->E : 48;
        if (d->BT_pitch > widest) widest = d->BT_pitch;
        if (d->BL_pitch > widest) widest = d->BL_pitch;
        if (d->C_pitch > widest) widest = d->C_pitch;
        if ((long long)d->B * d->H * d->W * widest >= (1ll << 31)) return M2D_ERR_TOO_LARGE;
    }
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

// Row-warps per CTA: as many as allowed, traded against rows lost to padding in the last band
// (score = warps x fraction of useful rows; ties go to the better fraction).
inline int pick_warps(int H, int max_warps) {
    if (H <= max_warps) return H;
    int best = max_warps;
    double best_score = -1.0, best_eff = 0.0;
    for (int w = max_warps; w >= 2; --w) {
        const int bands = (H + w - 1) / w;
        const double eff = (double)H / ((double)bands * w);
        const double score = w * eff;
        if (score > best_score + 1e-9 || (score > best_score - 1e-9 && eff > best_eff)) {
            best_score = score; best_eff = eff; best = w;
        }
    }
    return best;
}

// `lead`: how many steps before the band below reads a boundary block it must have been written (1 for
// the flat step loops, 2 for the nested-loop sweeps, which request everything two steps ahead).
inline Plan plan_common(const m2d_scan_desc* d, int max_warps, int warps_per_sm, int cb = 1, int lead = 1) {
    Plan p;
    p.cb = cb;
    p.rows = false;
    p.groups = (d->E + kGroup - 1) / kGroup;
    p.warps = pick_warps(d->H, max_warps);
    p.Rb = p.warps;
    p.nbands = (d->H + p.Rb - 1) / p.Rb;
    const int nch = (d->W + cb - 1) / cb;    // steps per row
    if (p.nbands > 1 && p.Rb > nch - lead) {
        // a band boundary must be written at least `lead` steps before the next band reads it
        p.Rb = nch - lead > 1 ? nch - lead : 1;
        p.warps = p.Rb;
        p.nbands = (d->H + p.Rb - 1) / p.Rb;
    }
    const int ctas_per_sm = warps_per_sm / p.warps > 0 ? warps_per_sm / p.warps : 1;
    const long long slots = (long long)ctas_per_sm * sm_count();
    // all CTAs resident at once: CTAs per channel group = floor(slots / groups), images per CTA to match
    long long per_group = slots / p.groups;
    if (per_group < 1) per_group = 1;
    const long long per = (d->B + per_group - 1) / per_group;    // images per CTA
    p.grid_x = (int)((d->B + per - 1) / per);
    p.smem = ((size_t)2 * cb * (p.warps + 1) * kSlotF4 + (size_t)p.warps * 2 * cb * kStageSlots + 256) * sizeof(float4);   // + parameters
    p.scratch = 0;
    p.chain = 1;
    return p;
}

// Try every cap on the row-warps per CTA and keep the plan that keeps the most warps resident,
// discounted by the rows lost to padding; ties go to the larger CTA.
inline Plan plan_best(const m2d_scan_desc* d, int max_warps, int warps_per_sm, int cb = 1, int lead = 1) {
    Plan best = plan_common(d, max_warps, warps_per_sm, cb, lead);
    double best_score = -1.0;
    const double cap = (double)warps_per_sm * sm_count();
    for (int w = max_warps; w >= 2; --w) {
        const Plan p = plan_common(d, w, warps_per_sm, cb, lead);
        double resident = (double)p.grid_x * p.groups * p.warps;
        if (resident > cap) resident = cap;
        const double eff = (double)d->H / ((double)p.nbands * p.Rb);
        const double score = resident * eff;
        if (score > best_score * 1.02) { best_score = score; best = p; }
    }
    return best;
}

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Scratch layout shared by every entry point: [status word, 256 bytes][the rest].
constexpr size_t kStatusBytes = 256;

// CTAs per image that a launch may use.  When a CTA owns more than one band the chain closes into a
// ring: its first warp enters the second band while (through the per-step block barrier) the warps
// behind it are still up to Rb-1 steps back in the first, and so on around the ring.  The ring must
// be shorter than one row of steps, or the head would wait on data that waits on the head.  `want`
// is the chain the resident CTA slots allow; `steps_per_row` the steps a warp needs for one row.
// Every place that picks or shortens a chain goes through this rule.
inline int bound_chain(long long want, int nbands, int steps_per_row, int Rb) {
    if (want > nbands) want = nbands;
    if (want < nbands) {
        const long long lim = steps_per_row / Rb - 1;
        if (want > lim) want = lim;
    }
    return want < 1 ? 1 : (int)want;
}

inline Plan plan_fwd(const m2d_scan_desc* d, bool allow_chain = true) {
    Plan p = plan_best(d, 8, 16, 1);
    // Few images on a large map: give every image a chain of CTAs, each owning every chain-th band,
    // so that the bands of one image run as a pipeline across SMs.  All CTAs must be resident.
    const long long slots = (long long)(16 / p.warps > 0 ? 16 / p.warps : 1) * sm_count();
    const long long ctas = (long long)p.grid_x * p.groups;
    if (allow_chain && p.nbands > 1 && ctas * 2 <= slots)
        p.chain = bound_chain(slots / ctas, p.nbands, (d->W + p.cb - 1) / p.cb, p.Rb);
    if (p.chain == 1 && d->W >= 3) {
        // batch mode: the nested-loop kernel (maps narrower than three columns keep the flat one)
        p = plan_best(d, 8, 16, 1, 2);
        p.rows = true;
        p.smem = rows_fwd_smem_bytes(p.warps) + kParamF4 * sizeof(float4);
    }
    p.scratch = kStatusBytes;
    if (p.chain > 1) {
        const size_t nband = (size_t)d->B * p.groups * p.nbands;
        p.scratch += align256(nband * sizeof(int)) + align256(nband * d->W * kSlotF4 * sizeof(float4));
    } else if (p.nbands > 1) {
        p.scratch += align256((size_t)p.grid_x * p.groups * d->W * kSlotF4 * sizeof(float4));
    }
    return p;
}

}  // namespace m2d
