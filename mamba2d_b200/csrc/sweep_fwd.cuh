// Forward wavefront sweep: discretisation + two-neighbour recurrence + readout, fused.
//
// Math per cell (i,j), per channel e and state n (reference: models/kernels/wf_cuda/wf_cuda.cu:41-69
// for the recurrence, models/kernels/wavefront_cuda.py:156 for the readout):
//     gT = exp(dT*AT)   gL = exp(dL*AL)   uT = dT*BT*x   uL = dL*BL*x
//     h  = wL*(gL*h_left + uL) + wT*(gT*h_top + uT)
//     (wL,wT) = (1,0) on row 0, (0,1) on column 0 below row 0, (1/2,1/2) inside
//     y  = sum_n h*C + x*D
// The weights are folded into the exponent (exp2(dT*AT*log2e + log2 wT)), so a missing neighbour
// costs nothing: its gate is exp2(-inf) = 0.
//
// Work decomposition.  A CTA owns one 32-channel group and walks `nb` images; each image is cut
// into `nbands` bands of `Rb` rows; warp r owns row q*Rb + r of band q and walks its W columns,
// one per step, lagging r steps behind warp 0 so that the row above is always one step ahead (the
// anti-diagonal wavefront).  Warp r hands its fresh state to warp r+1 through a double-buffered
// shared-memory slot; one __syncthreads per step keeps the warps in lock step.  The last row of a
// band reaches the first row of the next band (W - Rb + 1 steps later) through a per-CTA ring in
// global memory; warp 0 pulls its slot back into shared memory with cp.async one step ahead of
// use.  Inputs of the next cell are copied into a per-warp shared-memory stage with cp.async while
// the current cell's arithmetic runs (one copy per distinct 16-byte piece, not per lane), and read
// back from there a step later.  Addresses derive from one running 32-bit pixel index per side
// (load / compute) that is recomputed only at the start of a row.
#pragma once

#include <type_traits>

#include "common.cuh"

namespace m2d {

struct ScanArgs {
    int B, H, W, E, N;
    const void *x, *dT, *dL, *AT, *AL, *BT, *BL, *C, *D;
    long long pBT, pBL, pC;   // pixel pitch (elements) of BT, BL, C
    void* y;
    int dir;                  // +1: scan from the top-left corner; -1: from the bottom-right one (same memory, walked backwards)
    float4* ring;             // per-CTA band-boundary ring: [cta][W][4][32] float4
    int Rb, nbands;
    // ---- several CTAs per image (large maps, few images): CTA c of a chain of `chain` CTAs owns the
    // bands q = c, c + chain, ... of its images; the last row of band q reaches band q+1 (another
    // CTA) through `bnd` and the per-band column counter `progress`
    int chain;                // 1 = one CTA per image
    float4* bnd;              // [image][group][band][W][4][32] float4
    int* progress;            // [image][group][band]: columns of the band's last row published so far
    int* status;              // nonzero if a wait on `progress` gave up (results are then invalid); never null
    int wait_limit;           // polls before such a wait gives up
    int withhold;             // test hook: the first band of image 0 never publishes its column counter
    int act;                  // forward only: 1 = apply GELU (erf form) to y before it is stored
    int a_log;                // AT / AL hold the fp32 parameter A_log (A = -exp(A_log)); d_AT / d_AL are then fp32 d_A_log
    // ---- backward only ----
    const void* gy;
    float4* hs;               // full state record: [b][group][H*W] blocks; a block is [4][32] float4 (fp32 I/O)
                              // or [2][32] uint4 holding 16 bf16 states per lane (bf16 I/O)
    // fp32 accumulators of the reduced gradients, zeroed before the kernel.  For fp32 I/O they are
    // the caller's gradient tensors themselves; for bf16 I/O they live in the workspace.
    float *accBT, *accBL, *accC;   // [B*H*W][N]
    float *accAT, *accAL;          // [E][N]
    float* accD;                   // [E]
    void *d_x, *d_dT, *d_dL;
};
typedef ScanArgs FwdArgs;

// Flat pixel index in memory of scan position (i, j) of image b.  In the reverse direction the
// scan's cell (i, j) is the memory's pixel (H-1-i, W-1-j), i.e. the image's pixels in opposite order.
__device__ __forceinline__ int scan_pixel(const ScanArgs& a, int b, int i, int j) {
    const int p = i * a.W + j;
    return b * a.H * a.W + (a.dir > 0 ? p : a.H * a.W - 1 - p);
}

// Shared-memory hand-off layout: [slot 0..warps][parity 0..1][4][32] float4.  Rank k reads slot k
// and writes slot k+1; slot 0 receives the ring pull.
constexpr int kSlotPair = 2 * kSlotF4;
__host__ __device__ inline size_t handoff_bytes(int warps, int cb = 1) { return (size_t)(warps + 1) * cb * kSlotPair * sizeof(float4); }
// float4 units of one (cell, warp) block of the state record
template <typename io_t> struct HsBlock { static constexpr int f4 = sizeof(io_t) == 2 ? 64 : 128; };

// Dynamic shared memory of a sweep: the hand-off slots followed by one input stage per warp.
__host__ __device__ inline size_t sweep_smem_bytes(int warps, int cb = 1) { return handoff_bytes(warps, cb) + (size_t)warps * 2 * cb * kStageBytes; }
// Element (e, n) of AT / AL as a float.  With `a_log` the tensors hold the fp32 parameter A_log and
// A = -exp(A_log), rounded to the I/O type the way the reference's cast does
// (models/kernels/wavefront_cuda.py:72-73, :89-90); `exact` skips that rounding (used for the
// gradient d_A_log = d_A * A, where the reference multiplies by the fp32 value).
template <typename io_t>
__device__ __forceinline__ float load_A(const void* A, long long idx, int a_log, bool exact = false) {
    if (!a_log) return load1(static_cast<const io_t*>(A), idx);
    const float v = -expf(__ldg(static_cast<const float*>(A) + idx));
    if (sizeof(io_t) == 2 && !exact) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}

template <typename io_t>
__device__ __forceinline__ void stage_params(float4* dst, const void* AT, const void* AL, int N, int ch0, int chv, int n0, int nv, int lane,
                                             int a_log) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        float t[4], l[4];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const bool ok = (c < chv) && (n < nv);
            t[n] = ok ? load_A<io_t>(AT, (long long)(ch0 + c) * N + n0 + n, a_log) * kLog2e : 0.f;
            l[n] = ok ? load_A<io_t>(AL, (long long)(ch0 + c) * N + n0 + n, a_log) * kLog2e : 0.f;
        }
        dst[c * 32 + lane] = make_float4(t[0], t[1], t[2], t[3]);
        dst[128 + c * 32 + lane] = make_float4(l[0], l[1], l[2], l[3]);
    }
}

// Cell inputs held in registers.
struct CellIn {
    float4 x, dT, dL, bT, bL, c;
    float4 gy;   // only loaded by the backward sweeps
};

// Bounded wait of a consumer warp on a producer's column counter (another CTA).  Every lane polls
// with an acquire load (one request per warp), so each lane's later reads of the published data are
// ordered after the counter it saw.  Returns the value seen; after `wait_limit` unsuccessful polls,
// or as soon as any wait of the launch has given up, it records the failure in the status word and
// returns a huge value (the caller then stops waiting for the rest of the row), so a kernel can
// never spin forever.
constexpr int kWaitPolls = 1 << 22;
__device__ __forceinline__ int wait_columns(const int* counter, int need, int* status, int limit) {
    int seen = ld_acquire_gpu(counter);
    int polls = 0;
    while (seen < need) {
        if (++polls > limit || *reinterpret_cast<volatile int*>(status) != 0) {
            atomicExch(status, 1);
            return 0x7fffffff;
        }
        __nanosleep(64);
        seen = ld_acquire_gpu(counter);
    }
    return seen;
}

// Per-warp running state of a forward sweep.  Addresses are rebuilt every step from a running 32-bit
// pixel index (one multiply-add each); the host guarantees that every element index fits 31 bits.
struct FwdRun {
    // ---- load side: the cell whose inputs are fetched next ----
    int pixl;               // flat pixel index in memory of the cell (see scan_pixel)
    int jl, ql, bil;
    bool row_l, pull_l;
    int seen;               // columns of the band above known to be published (chained CTAs)
    const float4* pull;     // boundary row of the band above
    const int* pcount;      // its column counter
    // ---- compute side: the cell whose arithmetic runs now ----
    int pixc;
    float4* phs;            // state record of the current cell (recompute sweep only)
    int jc, qc, bic;
    bool row_c, row0_c, push_c;
    bool silent_c;          // test hook: this band does not publish its column counter
    float4* push;           // where this band's last row goes
    int* ccount;            // its column counter (chained CTAs)
};

// One CTA's forward sweep over images img0, img0 + img_stride, ... (nb of them).  `handoff` is
// shared memory of sweep_smem_bytes(warps, CB), zero-initialised by the caller.  With STORE_HS every
// fresh state block is also written to a.hs and d_C is accumulated (backward's recompute sweep).
// CB = cells per step: each warp advances CB columns of its row between two block barriers (the
// skew between neighbouring rows is CB columns), which amortises the per-step bookkeeping and lets
// the exponentials of one cell overlap the recurrence arithmetic of the other.
template <typename io_t, bool VEC, bool STORE_HS, bool CHAINED = false, int CB = 1>
__device__ __forceinline__ void forward_sweep(const ScanArgs& a, float4* handoff, const float4* params,
                                              float D_own, int img0, int img_stride, int nb, int cpos = 0, int chain_arg = 1) {
    const int chain = CHAINED ? chain_arg : 1;   // compile-time 1 in the batch kernels
    constexpr int SP = 2 * CB * kSlotF4;         // float4 per hand-off slot (two parities x CB cells)
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y, groups = gridDim.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));
    const int W = a.W, H = a.H, E = a.E, Rb = a.Rb, nbands = a.nbands;
    const int nch = (W + CB - 1) / CB;           // chunks of CB columns per row
    const int nq_c = chain > 1 ? (nbands - cpos + chain - 1) / chain : nbands;   // bands of an image this CTA owns
    const int T = nb * nq_c * nch;               // chunks in this warp's sequence
    const int steps = T + Rb - 1;
    const int pBT = (int)a.pBT, pBL = (int)a.pBL, pC = (int)a.pC;
    float4* const ring = a.ring + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * W) * kSlotF4 + lane;
    float4* const my = handoff + r * SP + lane;  // read slot r at my[(par*CB + cc)*128 + k*32], write slot r+1
    char* const stage = reinterpret_cast<char*>(handoff + ((blockDim.x >> 5) + 1) * SP) + r * 2 * CB * kStageBytes;
    const bool y_lane = (g * kGroup + lane) < E;
    const bool ch_copier = (nq == 0) && (chv > 0);   // lanes that copy per-channel / per-state inputs
    const bool st_copier = (cq == 0) && (nv > 0);
    const bool hi16 = (cq & 4) != 0, hi8 = (cq & 2) != 0;
    const int dc_n = n0 + (hi16 ? 2 : 0) + (hi8 ? 1 : 0);
    const bool dc_lane = ((cq & 1) == 0) && dc_n < a.N;
    const float ninf = __int_as_float(0xff800000);

    float h[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int n = 0; n < 4; ++n) h[c][n] = 0.f;

    LaneCopy<io_t> lc;
    lc.init(a.x, a.dT, a.dL, a.gy, a.BT, a.BL, a.C, pBT, pBL, pC, E, a.N, g, lane, STORE_HS);

    // the forward sweep can afford to hold its 32 parameters in registers (the adjoint sweep cannot)
    float aT2r[4][4], aL2r[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float4 pT4 = params[c * 32 + lane], pL4 = params[128 + c * 32 + lane];
        aT2r[c][0] = pT4.x; aT2r[c][1] = pT4.y; aT2r[c][2] = pT4.z; aT2r[c][3] = pT4.w;
        aL2r[c][0] = pL4.x; aL2r[c][1] = pL4.y; aL2r[c][2] = pL4.z; aL2r[c][3] = pL4.w;
    }

    FwdRun st;
    st.jl = st.ql = st.bil = 0;
    st.jc = st.qc = st.bic = 0;
    st.row_l = st.pull_l = st.row_c = st.row0_c = st.push_c = st.silent_c = false;
    st.pixl = st.pixc = 0;
    st.phs = nullptr;
    st.seen = 0; st.pull = ring; st.pcount = nullptr; st.push = ring; st.ccount = nullptr;

    // ---- stage the inputs of the next chunk of this warp's sequence -------------------------------
    auto load_phase = [&](int par) {
        if (st.jl == 0) {   // start of a row
            const int q = cpos + st.ql * chain;
            const int i = q * Rb + r;
            const int b = img0 + st.bil * img_stride;
            st.row_l = (r < Rb) && (i < H);
            st.pull_l = st.row_l && (r == 0) && (q > 0);
            st.pixl = scan_pixel(a, b, i, 0);
            if (chain > 1 && q > 0) {   // the band above belongs to another CTA
                const size_t band = ((size_t)b * groups + g) * nbands + (q - 1);
                st.pull = a.bnd + band * W * kSlotF4 + lane;
                st.pcount = a.progress + band;
                st.seen = 0;
            }
        }
        const int col0 = st.jl * CB;
        if (chain > 1 && st.pull_l) {
            const int need = min(col0 + CB, W);
            if (st.seen < need) st.seen = wait_columns(st.pcount, need, a.status, a.wait_limit);
        }
        if (st.row_l) {
#pragma unroll
            for (int cc = 0; cc < CB; ++cc) {
                const int col = col0 + cc;
                if (CB == 1 || col < W) {
                    char* stg = stage + (par * CB + cc) * kStageBytes;
                    if (VEC) {
                        lc.issue(smem_u32(stg), lane, st.pixl, E);
                    } else {
                        // ragged shapes: one lane per distinct piece, guarded scalar copies (see LaneCopy)
                        const int e0 = st.pixl * E + ch0;
                        stage4<VEC>(ch_copier, stg + cq * 16, static_cast<const io_t*>(a.x), e0, chv);
                        stage4<VEC>(ch_copier, stg + (8 + cq) * 16, static_cast<const io_t*>(a.dT), e0, chv);
                        stage4<VEC>(ch_copier, stg + (16 + cq) * 16, static_cast<const io_t*>(a.dL), e0, chv);
                        if (STORE_HS) stage4<VEC>(ch_copier, stg + (24 + cq) * 16, static_cast<const io_t*>(a.gy), e0, chv);
                        stage4<VEC>(st_copier, stg + (32 + nq) * 16, static_cast<const io_t*>(a.BT), st.pixl * pBT + n0, nv);
                        stage4<VEC>(st_copier, stg + (36 + nq) * 16, static_cast<const io_t*>(a.BL), st.pixl * pBL + n0, nv);
                        stage4<VEC>(st_copier, stg + (40 + nq) * 16, static_cast<const io_t*>(a.C), st.pixl * pC + n0, nv);
                    }
                    // the row above lives in the previous band: pull it from the ring into slot 0
                    cp_async16x4_if(st.pull_l, smem_u32(my + (par * CB + cc) * kSlotF4), st.pull + col * kSlotF4);
                    st.pixl += a.dir;
                }
            }
        }
        if (++st.jl == nch) {
            st.jl = 0;
            if (++st.ql == nq_c) { st.ql = 0; ++st.bil; }
        }
    };

    // ---- arithmetic of the current chunk; reads hand-off parity par^1, writes par -------------------
    auto compute_phase = [&](int par) {
        if (st.jc == 0) {
            const int q = cpos + st.qc * chain;
            const int i = q * Rb + r;
            const int b = img0 + st.bic * img_stride;
            st.row_c = (r < Rb) && (i < H);
            st.row0_c = (i == 0);
            st.push_c = st.row_c && (r == Rb - 1) && (q < nbands - 1);
            if (chain > 1) {
                const size_t band = ((size_t)b * groups + g) * nbands + q;
                st.push = a.bnd + band * W * kSlotF4 + lane;
                st.ccount = a.progress + band;
                st.silent_c = a.withhold != 0 && b == 0 && q == 0;
            }
            st.pixc = scan_pixel(a, b, i, 0);
            // a fresh row starts from no left neighbour: nothing of the previous row, band or image is
            // carried into it (the gate of a missing neighbour is zero, but zero times a diverged
            // state would not be)
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int n = 0; n < 4; ++n) h[c][n] = 0.f;
            if (STORE_HS) st.phs = a.hs + (((size_t)b * groups + g) * H * W + (size_t)i * W) * HsBlock<io_t>::f4 + lane;
        }
        if (st.row_c) {
            const int col0 = st.jc * CB;
            auto cell = [&](auto tag, const int cc, const int col) {
                constexpr bool INTERIOR = decltype(tag)::value;
                    // cells inside the map (row > 0, column > 0) have constant weights; row 0 and
                    // column 0 take the generic path, where a missing neighbour's state is taken as
                    // zero instead of being read
                    float wT, wL, offT, offL;
                    if (INTERIOR) {
                        wT = 0.5f; wL = 0.5f; offT = -1.f; offL = -1.f;
                    } else {
                        const bool first = (col == 0);
                        wT = st.row0_c ? 0.f : (first ? 1.f : 0.5f);
                        wL = first ? (st.row0_c ? 1.f : 0.f) : (st.row0_c ? 1.f : 0.5f);
                        offT = st.row0_c ? ninf : (first ? 0.f : -1.f);
                        offL = first ? ninf : (st.row0_c ? 0.f : -1.f);
                    }

                    float4 top[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        top[k] = my[((par ^ 1) * CB + cc) * kSlotF4 + k * 32];
                        if (!INTERIOR && st.row0_c) top[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    CellIn cur;   // staged during the previous step
                    {
                        const char* stg = stage + ((par ^ 1) * CB + cc) * kStageBytes;
                        cur.x = unstage4<io_t>(stg + cq * 16);
                        cur.dT = unstage4<io_t>(stg + (8 + cq) * 16);
                        cur.dL = unstage4<io_t>(stg + (16 + cq) * 16);
                        if (STORE_HS) cur.gy = unstage4<io_t>(stg + (24 + cq) * 16);
                        else cur.gy = make_float4(0.f, 0.f, 0.f, 0.f);
                        cur.bT = unstage4<io_t>(stg + (32 + nq) * 16);
                        cur.bL = unstage4<io_t>(stg + (36 + nq) * 16);
                        cur.c = unstage4<io_t>(stg + (40 + nq) * 16);
                    }

                    const float xs[4] = {cur.x.x, cur.x.y, cur.x.z, cur.x.w};
                    const float dTs[4] = {cur.dT.x, cur.dT.y, cur.dT.z, cur.dT.w};
                    const float dLs[4] = {cur.dL.x, cur.dL.y, cur.dL.z, cur.dL.w};
                    const float bTs[4] = {cur.bT.x, cur.bT.y, cur.bT.z, cur.bT.w};
                    const float bLs[4] = {cur.bL.x, cur.bL.y, cur.bL.z, cur.bL.w};
                    const float cs[4] = {cur.c.x, cur.c.y, cur.c.z, cur.c.w};
                    const float gys[4] = {cur.gy.x, cur.gy.y, cur.gy.z, cur.gy.w};
                    float yacc[4];
                    float dC[4] = {0.f, 0.f, 0.f, 0.f};   // recompute sweep only: sum over this thread's channels of gy*h
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float tp[4] = {top[c].x, top[c].y, top[c].z, top[c].w};
                        const float dtx = wT * dTs[c] * xs[c];
                        const float dlx = wL * dLs[c] * xs[c];
                        // packed fp32x2 arithmetic (two states per instruction) everywhere except the exponentials
                        float2 acc2 = make_float2(0.f, 0.f);
#pragma unroll
                        for (int n = 0; n < 4; n += 2) {
                            const float2 argT = __ffma2_rn(make_float2(dTs[c], dTs[c]), make_float2(aT2r[c][n], aT2r[c][n + 1]), make_float2(offT, offT));
                            const float2 argL = __ffma2_rn(make_float2(dLs[c], dLs[c]), make_float2(aL2r[c][n], aL2r[c][n + 1]), make_float2(offL, offL));
                            const float2 gT = make_float2(ex2(argT.x), ex2(argT.y));
                            const float2 gL = make_float2(ex2(argL.x), ex2(argL.y));
                            const float2 u = __ffma2_rn(make_float2(dlx, dlx), make_float2(bLs[n], bLs[n + 1]),
                                                        __fmul2_rn(make_float2(dtx, dtx), make_float2(bTs[n], bTs[n + 1])));
                            const float2 hn = __ffma2_rn(gL, make_float2(h[c][n], h[c][n + 1]),
                                                         __ffma2_rn(gT, make_float2(tp[n], tp[n + 1]), u));
                            h[c][n] = hn.x;
                            h[c][n + 1] = hn.y;
                            acc2 = __ffma2_rn(hn, make_float2(cs[n], cs[n + 1]), acc2);
                            if (STORE_HS) {
                                const float2 d2 = __ffma2_rn(make_float2(gys[c], gys[c]), hn, make_float2(dC[n], dC[n + 1]));
                                dC[n] = d2.x;
                                dC[n + 1] = d2.y;
                            }
                        }
                        yacc[c] = acc2.x + acc2.y;
                    }

                    // hand the fresh state to the row below (slot r+1), to the next band, and to the record
                    {
                        const float4 h0 = make_float4(h[0][0], h[0][1], h[0][2], h[0][3]), h1 = make_float4(h[1][0], h[1][1], h[1][2], h[1][3]);
                        const float4 h2 = make_float4(h[2][0], h[2][1], h[2][2], h[2][3]), h3 = make_float4(h[3][0], h[3][1], h[3][2], h[3][3]);
                        float4* dst = my + SP + (par * CB + cc) * kSlotF4;
                        dst[0] = h0; dst[32] = h1; dst[64] = h2; dst[96] = h3;
                        stcg4_if(st.push_c, st.push + col * kSlotF4, h0, h1, h2, h3);
                        if (STORE_HS) {
                            if (sizeof(io_t) == 2) {
                                // bf16 I/O: the record holds bf16 states (the gradients that use it are bf16 anyway)
                                __stcg(st.phs, make_float4(__uint_as_float(pack_bf16x2(h0.x, h0.y)), __uint_as_float(pack_bf16x2(h0.z, h0.w)),
                                                           __uint_as_float(pack_bf16x2(h1.x, h1.y)), __uint_as_float(pack_bf16x2(h1.z, h1.w))));
                                __stcg(st.phs + 32, make_float4(__uint_as_float(pack_bf16x2(h2.x, h2.y)), __uint_as_float(pack_bf16x2(h2.z, h2.w)),
                                                                __uint_as_float(pack_bf16x2(h3.x, h3.y)), __uint_as_float(pack_bf16x2(h3.z, h3.w))));
                            } else {
                                stcg4_if(true, st.phs, h0, h1, h2, h3);
                            }
                        }
                    }

                    if (STORE_HS) {
                        // d_C[pixel][n] = sum over channels of gy*h: finish over the 8 cq lanes, then one
                        // atomic per state from the even-cq lane of each pair
                        float k0 = hi16 ? dC[2] : dC[0], k1 = hi16 ? dC[3] : dC[1];
                        k0 += __shfl_xor_sync(0xffffffffu, hi16 ? dC[0] : dC[2], 16);
                        k1 += __shfl_xor_sync(0xffffffffu, hi16 ? dC[1] : dC[3], 16);
                        float k = hi8 ? k1 : k0;
                        k += __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k1, 8);
                        k += __shfl_xor_sync(0xffffffffu, k, 4);
                        if (dc_lane) atomicAdd(a.accC + ((long long)st.pixc * a.N + dc_n), k);
                        st.phs += HsBlock<io_t>::f4;
                    } else {
                        const float ysum = reduce_states(yacc[0], yacc[1], yacc[2], yacc[3], nq);
                        float yv = fmaf(sel4(cur.x, nq), D_own, ysum);
                        // optional output activation (the block applies GELU right after the scan:
                        // models/mamba2d.py:167-169); one value per lane, so it costs one erf per lane and cell
                        if (a.act) yv = 0.5f * yv * (1.f + erff(yv * 0.70710678118654752f));
                        if (y_lane) store1(static_cast<io_t*>(a.y), st.pixc * E + g * kGroup + lane, yv);
                    }
                    st.pixc += a.dir;
            };
#pragma unroll
            for (int cc = 0; cc < CB; ++cc) {
                const int col = col0 + cc;
                if (CB == 1 || col < W) {
                    if (st.row0_c || col == 0) cell(std::false_type{}, cc, col);
                    else cell(std::true_type{}, cc, col);
                }
            }
            if (chain > 1 && st.push_c) {
                // publish the chunk's columns: data first, then the counter.  __syncwarp orders the other
                // lanes' stores before lane 0's release store, which makes them visible with the counter.
                __syncwarp();
                if (lane == 0 && !st.silent_c) st_release_gpu(st.ccount, min(col0 + CB, W));
            }
        }
        if (++st.jc == nch) {
            st.jc = 0;
            if (++st.qc == nq_c) { st.qc = 0; ++st.bic; }
        }
    };

    // Step s: stage the inputs of chunk (s + 1 - r), compute chunk (s - r).  s runs from -1 so that the
    // first copy has a step of its own.  Two steps per iteration keep the parity a constant.
    int cl = -r;     // index of the chunk staged in the current step
    for (int s = -1; s < steps; s += 2) {
        if ((unsigned)cl < (unsigned)T) load_phase(1);
        if ((unsigned)(cl - 1) < (unsigned)T) compute_phase(1);
        ++cl;
        cp_async_wait_all();
        __syncthreads();
        if (s + 1 < steps) {
            if ((unsigned)cl < (unsigned)T) load_phase(0);
            if ((unsigned)(cl - 1) < (unsigned)T) compute_phase(0);
            ++cl;
            cp_async_wait_all();
            __syncthreads();
        }
    }
}

}  // namespace m2d
