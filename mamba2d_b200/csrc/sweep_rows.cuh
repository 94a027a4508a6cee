// Wavefront sweeps of the batch mode (one CTA per image and channel group), written as nested loops.
//
// Same algorithm and data layout as forward_sweep / reverse_sweep in sweep_fwd.cuh / sweep_bwd.cuh --
// warp r owns row q*Rb + r of band q and lags r steps behind warp 0; one __syncthreads per step -- but
// every warp walks its own sequence "for each (image, band): for each column" instead of decoding a
// flat step counter: all per-row decisions (row 0, pull from the ring, push to the ring, output
// offsets) are taken once per row, and the loop over the columns carries only running indices.  Every
// warp executes the same number of barriers (idle steps where it has no cell).
//
// Everything that arrives asynchronously from global memory (the staged inputs, ring blocks, blocks
// of the state record) is requested TWO steps before the cell that uses it and lands in one of three
// rotating buffers; a step ends with cp.async.wait_group 1, i.e. it waits for the copies issued one
// step earlier, never for its own.  (With one step of lead and two buffers the wait at the end of a
// step was for copies issued at its start, and a step is shorter than a trip to HBM on this part:
// removing the wait altogether gained 9 % in the forward and 10 % in the backward kernel.)  Blocks
// handed from warp to warp inside the CTA keep two parities.  A band boundary must therefore be
// written at least two steps before the band below reads it: the plan keeps Rb <= W - 2.
#pragma once

#include "sweep_bwd.cuh"

namespace m2d {

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_prev() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// With STORE_HS (the backward's recompute sweep) every fresh state block also goes to the state
// record a.hs and d_C is accumulated, and nothing is written to y.
template <typename io_t, bool VEC, bool STORE_HS>
__device__ __forceinline__ void forward_rows(const ScanArgs& a, float4* smem, const float4* params, float D_own,
                                             int img0, int img_stride, int nb) {
    constexpr int HB = HsBlock<io_t>::f4;
    constexpr int PO = kSlotF4;                  // float4 between the two parities of a hand-off slot
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));
    const int W = a.W, H = a.H, E = a.E, Rb = a.Rb, nbands = a.nbands;
    const int pBT = (int)a.pBT, pBL = (int)a.pBL, pC = (int)a.pC;
    float4* const ring = a.ring + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * W) * kSlotF4 + lane;
    float4* const pullbuf = smem + lane;                                  // warp 0: blocks of the row above the band
    float4* const out = smem + 3 * kSlotF4 + r * 2 * kSlotF4 + lane;      // this row's states, for the warp below
    const float4* const in = out - 2 * kSlotF4;                           // the row above (r > 0)
    char* const stage = reinterpret_cast<char*>(smem + rows_handoff_f4(nwarps)) + r * 3 * kStageBytes;
    const bool y_lane = (g * kGroup + lane) < E;
    const bool ch_copier = (nq == 0) && (chv > 0);
    const bool st_copier = (cq == 0) && (nv > 0);
    const float ninf = __int_as_float(0xff800000);
    const int dir = a.dir;
    const bool active = r < Rb;                  // (the plan launches exactly Rb row-warps)
    const bool hi16 = (cq & 4) != 0, hi8 = (cq & 2) != 0;
    const int dc_n = n0 + (hi16 ? 2 : 0) + (hi8 ? 1 : 0);
    const bool dc_lane = ((cq & 1) == 0) && dc_n < a.N;
    const int groups = gridDim.y;

    float h[4][4];
    LaneCopy<io_t> lc;
    lc.init(a.x, a.dT, a.dL, a.gy, a.BT, a.BL, a.C, pBT, pBL, pC, E, a.N, g, lane, STORE_HS);

    float aT2r[4][4], aL2r[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float4 pT4 = params[c * 32 + lane], pL4 = params[128 + c * 32 + lane];
        aT2r[c][0] = pT4.x; aT2r[c][1] = pT4.y; aT2r[c][2] = pT4.z; aT2r[c][3] = pT4.w;
        aL2r[c][0] = pL4.x; aL2r[c][1] = pL4.y; aL2r[c][2] = pL4.z; aL2r[c][3] = pL4.w;
    }

    // Every warp takes part in every step from the first one on (idle steps included), so all warps
    // rotate in lock step.  po: parity of the hand-off slots written in this step (read: po ^ PO).
    // k3: which of the three asynchronous buffers is filled in this step, for the cell two steps on;
    // the cell of this step reads buffer k3 + 1 (mod 3), filled two steps ago.
    int po = PO, k3 = 0;
    auto end_step = [&]() {
        cp_async_commit();
        cp_async_wait_prev();
        __syncthreads();
        po ^= PO;
        k3 = (k3 == 2) ? 0 : k3 + 1;
    };

    struct Row { bool has, row0, pull, push; int pix0; float4* hs0; };
    auto make_row = [&](int bi, int q) {
        Row w;
        const int i = q * Rb + r;
        const int b = img0 + bi * img_stride;
        w.has = active && bi < nb && i < H;
        w.row0 = (i == 0);
        w.pull = (r == 0) && (q > 0);
        w.push = (r == Rb - 1) && (q < nbands - 1);
        w.pix0 = scan_pixel(a, b, i, 0);
        w.hs0 = STORE_HS ? a.hs + (((size_t)b * groups + g) * H * W + (size_t)i * W) * HB + lane : nullptr;
        return w;
    };

    // request the inputs (and the ring block above, for the first row of a band) of cell (w, col)
    auto stage_cell = [&](const Row& w, int col) {
        const int pix = w.pix0 + dir * col;
        char* stg = stage + k3 * kStageBytes;
        if (VEC) {
            lc.issue_plain(smem_u32(stg), lane, pix, E);
        } else {
            const int e0 = pix * E + ch0;
            stage4<VEC>(ch_copier, stg + cq * 16, static_cast<const io_t*>(a.x), e0, chv);
            stage4<VEC>(ch_copier, stg + (8 + cq) * 16, static_cast<const io_t*>(a.dT), e0, chv);
            stage4<VEC>(ch_copier, stg + (16 + cq) * 16, static_cast<const io_t*>(a.dL), e0, chv);
            if (STORE_HS) stage4<VEC>(ch_copier, stg + (24 + cq) * 16, static_cast<const io_t*>(a.gy), e0, chv);
            stage4<VEC>(st_copier, stg + (32 + nq) * 16, static_cast<const io_t*>(a.BT), pix * pBT + n0, nv);
            stage4<VEC>(st_copier, stg + (36 + nq) * 16, static_cast<const io_t*>(a.BL), pix * pBL + n0, nv);
            stage4<VEC>(st_copier, stg + (40 + nq) * 16, static_cast<const io_t*>(a.C), pix * pC + n0, nv);
        }
        if (w.pull) cp_async_block(smem_u32(pullbuf + k3 * kSlotF4), ring + col * kSlotF4, false);
    };

    // one cell: reads what was requested two steps ago and what the warp above wrote in the previous step
    auto cell = [&](auto tag, const Row& w, const int col) {
        constexpr bool INTERIOR = decltype(tag)::value;
        float wT, wL, offT, offL;
        if (INTERIOR) {
            wT = 0.5f; wL = 0.5f; offT = -1.f; offL = -1.f;
        } else {
            const bool first = (col == 0);
            wT = w.row0 ? 0.f : (first ? 1.f : 0.5f);
            wL = first ? (w.row0 ? 1.f : 0.f) : (w.row0 ? 1.f : 0.5f);
            offT = w.row0 ? ninf : (first ? 0.f : -1.f);
            offL = first ? ninf : (w.row0 ? 0.f : -1.f);
        }
        const int rd = (k3 == 2) ? 0 : k3 + 1;
        const float4* const tsrc = (r == 0) ? pullbuf + rd * kSlotF4 : in + (po ^ PO);
        float4 top[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            top[k] = tsrc[k * 32];
            if (!INTERIOR && w.row0) top[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const char* stg = stage + rd * kStageBytes;
        const float4 vx = unstage4<io_t>(stg + cq * 16);
        const float4 vdT = unstage4<io_t>(stg + (8 + cq) * 16);
        const float4 vdL = unstage4<io_t>(stg + (16 + cq) * 16);
        const float4 vgy = STORE_HS ? unstage4<io_t>(stg + (24 + cq) * 16) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 vbT = unstage4<io_t>(stg + (32 + nq) * 16);
        const float4 vbL = unstage4<io_t>(stg + (36 + nq) * 16);
        const float4 vc = unstage4<io_t>(stg + (40 + nq) * 16);
        const float xs[4] = {vx.x, vx.y, vx.z, vx.w};
        const float dTs[4] = {vdT.x, vdT.y, vdT.z, vdT.w};
        const float dLs[4] = {vdL.x, vdL.y, vdL.z, vdL.w};
        const float gys[4] = {vgy.x, vgy.y, vgy.z, vgy.w};
        const float bTs[4] = {vbT.x, vbT.y, vbT.z, vbT.w};
        const float bLs[4] = {vbL.x, vbL.y, vbL.z, vbL.w};
        const float cs[4] = {vc.x, vc.y, vc.z, vc.w};
        float yacc[4];
        float dC[4] = {0.f, 0.f, 0.f, 0.f};   // recompute sweep only: sum over this thread's channels of gy*h
        if (STORE_HS) {
        // recompute sweep of the backward kernel: stage by stage over all 16 states of the thread
        // (exponent arguments, exponentials, input terms, recurrence) rather than channel by channel.
        // Measured: 2 % off the backward kernel, whose register budget this sweep does not use up; in
        // the forward kernel the same order is 3 % slower than the channel-wise one below.
        float2 gT2[4][2], gL2[4][2], u2[4][2];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int n = 0; n < 4; n += 2) {
                gT2[c][n >> 1] = __ffma2_rn(make_float2(dTs[c], dTs[c]), make_float2(aT2r[c][n], aT2r[c][n + 1]), make_float2(offT, offT));
                gL2[c][n >> 1] = __ffma2_rn(make_float2(dLs[c], dLs[c]), make_float2(aL2r[c][n], aL2r[c][n + 1]), make_float2(offL, offL));
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                gT2[c][k] = make_float2(ex2(gT2[c][k].x), ex2(gT2[c][k].y));
                gL2[c][k] = make_float2(ex2(gL2[c][k].x), ex2(gL2[c][k].y));
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float dtx, dlx;
            if (INTERIOR) {
                const float xh = 0.5f * xs[c];
                const float2 dx2 = __fmul2_rn(make_float2(dTs[c], dLs[c]), make_float2(xh, xh));
                dtx = dx2.x;
                dlx = dx2.y;
            } else {
                dtx = wT * dTs[c] * xs[c];
                dlx = wL * dLs[c] * xs[c];
            }
#pragma unroll
            for (int n = 0; n < 4; n += 2)
                u2[c][n >> 1] = __ffma2_rn(make_float2(dlx, dlx), make_float2(bLs[n], bLs[n + 1]),
                                           __fmul2_rn(make_float2(dtx, dtx), make_float2(bTs[n], bTs[n + 1])));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float tp[4] = {top[c].x, top[c].y, top[c].z, top[c].w};
            float2 acc2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int n = 0; n < 4; n += 2) {
                const float2 hn = __ffma2_rn(gL2[c][n >> 1], make_float2(h[c][n], h[c][n + 1]),
                                             __ffma2_rn(gT2[c][n >> 1], make_float2(tp[n], tp[n + 1]), u2[c][n >> 1]));
                h[c][n] = hn.x;
                h[c][n + 1] = hn.y;
                if (STORE_HS) {
                    const float2 d2 = __ffma2_rn(make_float2(gys[c], gys[c]), hn, make_float2(dC[n], dC[n + 1]));
                    dC[n] = d2.x;
                    dC[n + 1] = d2.y;
                } else {
                    acc2 = __ffma2_rn(hn, make_float2(cs[n], cs[n + 1]), acc2);
                }
            }
            yacc[c] = acc2.x + acc2.y;
        }
        } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float tp[4] = {top[c].x, top[c].y, top[c].z, top[c].w};
            float dtx, dlx;
            if (INTERIOR) {
                const float xh = 0.5f * xs[c];
                const float2 dx2 = __fmul2_rn(make_float2(dTs[c], dLs[c]), make_float2(xh, xh));
                dtx = dx2.x;
                dlx = dx2.y;
            } else {
                dtx = wT * dTs[c] * xs[c];
                dlx = wL * dLs[c] * xs[c];
            }
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
            }
            yacc[c] = acc2.x + acc2.y;
        }
        }
        {
            const float4 h0 = make_float4(h[0][0], h[0][1], h[0][2], h[0][3]), h1 = make_float4(h[1][0], h[1][1], h[1][2], h[1][3]);
            const float4 h2 = make_float4(h[2][0], h[2][1], h[2][2], h[2][3]), h3 = make_float4(h[3][0], h[3][1], h[3][2], h[3][3]);
            float4* dst = out + po;
            dst[0] = h0; dst[32] = h1; dst[64] = h2; dst[96] = h3;
            if (w.push) stcg4_if(true, ring + col * kSlotF4, h0, h1, h2, h3);
            if (STORE_HS) {
                float4* phs = w.hs0 + (size_t)col * HB;
                if (sizeof(io_t) == 2) {
                    // bf16 I/O: the record holds bf16 states (the gradients that use it are bf16 anyway)
                    __stcg(phs, make_float4(__uint_as_float(pack_bf16x2(h0.x, h0.y)), __uint_as_float(pack_bf16x2(h0.z, h0.w)),
                                            __uint_as_float(pack_bf16x2(h1.x, h1.y)), __uint_as_float(pack_bf16x2(h1.z, h1.w))));
                    __stcg(phs + 32, make_float4(__uint_as_float(pack_bf16x2(h2.x, h2.y)), __uint_as_float(pack_bf16x2(h2.z, h2.w)),
                                                 __uint_as_float(pack_bf16x2(h3.x, h3.y)), __uint_as_float(pack_bf16x2(h3.z, h3.w))));
                } else {
                    stcg4_if(true, phs, h0, h1, h2, h3);
                }
            }
        }
        if (STORE_HS) {
            // d_C[pixel][n] = sum over channels of gy*h: finish over the 8 cq lanes, then one atomic per
            // state from the even-cq lane of each pair
            float k0 = hi16 ? dC[2] : dC[0], k1 = hi16 ? dC[3] : dC[1];
            k0 += __shfl_xor_sync(0xffffffffu, hi16 ? dC[0] : dC[2], 16);
            k1 += __shfl_xor_sync(0xffffffffu, hi16 ? dC[1] : dC[3], 16);
            float k = hi8 ? k1 : k0;
            k += __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k1, 8);
            k += __shfl_xor_sync(0xffffffffu, k, 4);
            if (dc_lane) atomicAdd(a.accC + ((long long)(w.pix0 + dir * col) * a.N + dc_n), k);
        } else {
            const float ysum = reduce_states(yacc[0], yacc[1], yacc[2], yacc[3], nq);
            float yv = fmaf(sel4(vx, nq), D_own, ysum);
            if (a.act) yv = 0.5f * yv * (1.f + erff(yv * 0.70710678118654752f));
            if (y_lane) store1(static_cast<io_t*>(a.y), (w.pix0 + dir * col) * E + g * kGroup + lane, yv);
        }
    };

    // ---- the warp's sequence ---------------------------------------------------------------------
    // r idle steps, two steps that only request the first two cells, W steps per (image, band) item,
    // Rb-1-r idle steps; in every step with a cell, the cell two columns on is requested first
    for (int k = 0; k < r; ++k) end_step();
    int bi = 0, q = 0;
    Row cur = make_row(0, 0);
    if (cur.has) stage_cell(cur, 0);
    end_step();
    if (cur.has) stage_cell(cur, 1);
    end_step();
    const int items = nb * nbands;
    for (int m = 0; m < items; ++m) {
        if (++q == nbands) { q = 0; ++bi; }
        const Row nxt = make_row(bi, q);                      // (.has is false past the last item)
        if (cur.has) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int n = 0; n < 4; ++n) h[c][n] = 0.f;    // a row starts from no left neighbour
            for (int col = 0; col < W; ++col) {
                if (col + 2 < W) stage_cell(cur, col + 2);
                else if (nxt.has) stage_cell(nxt, col + 2 - W);
                if (cur.row0 || col == 0) cell(std::false_type{}, cur, col);
                else cell(std::true_type{}, cur, col);
                end_step();
            }
        } else {
            for (int col = 0; col + 2 < W; ++col) end_step();
            if (nxt.has) stage_cell(nxt, 0);
            end_step();
            if (nxt.has) stage_cell(nxt, 1);
            end_step();
        }
        cur = nxt;
    }
    for (int k = 0; k < Rb - 1 - r; ++k) end_step();          // until the last warp is done
    cp_async_wait_all();                                      // (only empty groups can be pending here)
}

// Adjoint sweep of one CTA over image b, batch mode, written as nested loops: same algorithm and
// data layout as reverse_sweep in sweep_bwd.cuh.  Bands are visited last to first, the bottom row of
// a band leads (rank rr = Rb-1-r), columns run right to left.  Every warp executes the same number
// of barriers: rr + 2 steps before its first cell (the last three of them request, in this order, the
// right-most state block of its first row for the warp below, cell W-1 and cell W-2), W steps per
// band, and Rb-1-rr idle steps at the end.
template <typename io_t, bool VEC>
__device__ __forceinline__ void reverse_rows(const ScanArgs& a, float4* smem, const float4* params, float D_own,
                                             float (&dAT)[4][4], float (&dAL)[4][4], float (&dD)[4], int b) {
    constexpr int PO = kSlotF4;               // float4 between the two parities of a hand-off slot
    constexpr int HB = HsBlock<io_t>::f4;     // float4 units per state-record block
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y, groups = gridDim.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));
    const int W = a.W, H = a.H, E = a.E, Rb = a.Rb, nbands = a.nbands;
    const int rr = Rb - 1 - r;                 // rank in the reverse sweep
    const int pBT = (int)a.pBT, pBL = (int)a.pBL, pC = (int)a.pC;
    const int dir = a.dir;
    float4* const ring = a.ring + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * W) * kSlotF4 + lane;
    float4* const pullbuf = smem + lane;                                      // rank 0: pT of the row below the band
    float4* const out = smem + 3 * kSlotF4 + rr * 2 * kSlotF4 + lane;         // pT of this row, for the row above
    float4* const in = out - 2 * kSlotF4;                                     // pT of the row below (rr > 0)
    char* const stage = reinterpret_cast<char*>(smem + rows_handoff_f4(nwarps)) + r * 3 * kStageBytes;
    float4* const harea = reinterpret_cast<float4*>(reinterpret_cast<char*>(smem) + rows_fwd_smem_bytes(nwarps)) + lane;
    float4* const h_own = harea + (r + 1) * 3 * kSlotF4;                      // this row's h[i][j-1]
    float4* const h_up = harea + r * 3 * kSlotF4;                             // the row above: h[i-1][j]
    const float4* const hs_img = a.hs + ((size_t)b * groups + g) * H * W * HB + lane;
    const bool y_lane = (g * kGroup + lane) < E;
    const bool ch_copier = (nq == 0) && (chv > 0);
    const bool st_copier = (cq == 0) && (nv > 0);
    const bool feeds_below = (r + 1 < Rb);     // a warp of this CTA owns the row below
    const bool hi16 = (cq & 4) != 0, hi8 = (cq & 2) != 0, hi4 = (cq & 1) != 0;
    const int db_n = n0 + (hi8 ? 2 : 0) + (hi4 ? 1 : 0);
    float* const db_acc = hi16 ? a.accBL : a.accBT;
    const bool db_lane = db_n < a.N;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const float ninf = __int_as_float(0xff800000);

    float pL[4][4];
    LaneCopy<io_t> lc;
    lc.init(a.x, a.dT, a.dL, a.gy, a.BT, a.BL, a.C, pBT, pBL, pC, E, a.N, g, lane, true);

    auto copy_block = [&](unsigned dst, const float4* src) { cp_async_block(dst, src, sizeof(io_t) == 2); };
    auto block_states = [&](const float4* area, int c) -> float4 {
        if (sizeof(io_t) == 2) {
            const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(area + (c >> 1) * 32) + (c & 1) * 8);
            return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                               __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
        }
        return area[c * 32];
    };

    // po: parity of the hand-off slots written in this step (read: po ^ PO); k3: which of the three
    // asynchronous buffers is filled in this step, for the cell two steps on (read: k3 + 1 mod 3)
    int po = PO, k3 = 0;
    auto end_step = [&]() {
        cp_async_commit();
        cp_async_wait_prev();
        __syncthreads();
        po ^= PO;
        k3 = (k3 == 2) ? 0 : k3 + 1;
    };

    // row of band q owned by this warp; pixR = memory pixel of its right-most cell (i, W-1)
    struct Row { bool has, row0, bottom, pull, push, top; int i, pixR; };
    auto make_row = [&](int q) {
        Row w;
        w.i = q * Rb + r;
        w.has = (r < Rb) && q >= 0 && (w.i < H);
        w.row0 = (w.i == 0);
        w.bottom = (w.i + 1 >= H);
        w.pull = (rr == 0) && (w.i + 1 < H);          // pT of the row below comes through the ring
        w.push = (r == 0) && (q > 0);                 // pT of this row goes to the band above through the ring
        w.top = (r == 0) && (w.i > 0);                // h of the row above is not staged by a warp of this band
        w.pixR = scan_pixel(a, b, w.i, W - 1);
        return w;
    };
    // request h[i][W-1] of row w for the warp below (nobody's left neighbour, so no cell's request covers it)
    auto prefetch_row_end = [&](const Row& w) {
        if (feeds_below && w.has) copy_block(smem_u32(h_own + k3 * kSlotF4), hs_img + ((size_t)w.i * W + (W - 1)) * HB);
    };
    // request for cell (w, j): the inputs, h[i][j-1], for the top row of a band h[i-1][j], for the bottom
    // row of a band pT of the band below
    auto stage_cell = [&](const Row& w, int j) {
        const int pix = w.pixR - dir * (W - 1 - j);
        char* stg = stage + k3 * kStageBytes;
        if (VEC) {
            lc.issue_plain(smem_u32(stg), lane, pix, E);
        } else {
            const int e0 = pix * E + ch0;
            stage4<VEC>(ch_copier, stg + cq * 16, static_cast<const io_t*>(a.x), e0, chv);
            stage4<VEC>(ch_copier, stg + (8 + cq) * 16, static_cast<const io_t*>(a.dT), e0, chv);
            stage4<VEC>(ch_copier, stg + (16 + cq) * 16, static_cast<const io_t*>(a.dL), e0, chv);
            stage4<VEC>(ch_copier, stg + (24 + cq) * 16, static_cast<const io_t*>(a.gy), e0, chv);
            stage4<VEC>(st_copier, stg + (32 + nq) * 16, static_cast<const io_t*>(a.BT), pix * pBT + n0, nv);
            stage4<VEC>(st_copier, stg + (36 + nq) * 16, static_cast<const io_t*>(a.BL), pix * pBL + n0, nv);
            stage4<VEC>(st_copier, stg + (40 + nq) * 16, static_cast<const io_t*>(a.C), pix * pC + n0, nv);
        }
        const float4* ph = hs_img + ((size_t)w.i * W + (j - 1)) * HB;            // h[i][j-1]
        if (j > 0) copy_block(smem_u32(h_own + k3 * kSlotF4), ph);
        if (w.top) copy_block(smem_u32(h_up + k3 * kSlotF4), ph + (ptrdiff_t)(1 - W) * HB);   // h[i-1][j]
        if (w.pull) cp_async_block(smem_u32(pullbuf + k3 * kSlotF4), ring + j * kSlotF4, false);
    };

    auto cell = [&](auto tag, const Row& w, const int j) {
          constexpr bool INTERIOR = decltype(tag)::value;
        const int pixc = w.pixR - dir * (W - 1 - j);   // memory pixel of scan cell (i, j)
      // cells inside the map (row > 0, column > 0) have constant weights; row 0 and column 0 take
      // the generic path, where a missing neighbour's state is taken as zero instead of being read
      float cfac, mT, mL, offT, offL;
      if (INTERIOR) {
          cfac = 0.5f; mT = 1.f; mL = 1.f; offT = 0.f; offL = 0.f;
      } else {
          const bool first = (j == 0);   // column 0: no averaging, no left neighbour; the left input term exists only on row 0
          cfac = (w.row0 || first) ? 1.f : 0.5f;
          mT = w.row0 ? 0.f : 1.f;
          mL = (first && !w.row0) ? 0.f : 1.f;
          offT = w.row0 ? ninf : 0.f;
          offL = first ? ninf : 0.f;
      }
      const float2 offT2 = make_float2(offT, offT), offL2 = make_float2(offL, offL);
      const int rd = (k3 == 2) ? 0 : k3 + 1;
      const char* stg = stage + rd * kStageBytes;
      const float4* const hl_src = h_own + rd * kSlotF4;
      const float4* const ht_src = h_up + rd * kSlotF4;
      const float4* const pd_src = (rr == 0) ? pullbuf + rd * kSlotF4 : in + (po ^ PO);
      const float4 vx = unstage4<io_t>(stg + cq * 16);
      const float4 vdT = unstage4<io_t>(stg + (8 + cq) * 16);
      const float4 vdL = unstage4<io_t>(stg + (16 + cq) * 16);
      const float4 vgy = unstage4<io_t>(stg + (24 + cq) * 16);
      const float4 vbT = unstage4<io_t>(stg + (32 + nq) * 16);
      const float4 vbL = unstage4<io_t>(stg + (36 + nq) * 16);
      const float4 vc = unstage4<io_t>(stg + (40 + nq) * 16);
      const float xs[4] = {vx.x, vx.y, vx.z, vx.w};
      const float dTs[4] = {vdT.x, vdT.y, vdT.z, vdT.w};
      const float dLs[4] = {vdL.x, vdL.y, vdL.z, vdL.w};
      const float gys[4] = {vgy.x, vgy.y, vgy.z, vgy.w};
      const float bTs[4] = {vbT.x, vbT.y, vbT.z, vbT.w};
      const float bLs[4] = {vbL.x, vbL.y, vbL.z, vbL.w};
      const float cs[4] = {vc.x, vc.y, vc.z, vc.w};

      float2 dBT2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      float2 dBL2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      float o_dT[4], o_dL[4], o_dx[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
          const float4 hl4 = (INTERIOR || j > 0) ? block_states(hl_src, c) : zero4;
          const float4 ht4 = (INTERIOR || !w.row0) ? block_states(ht_src, c) : zero4;
          const float4 pd4 = pd_src[c * 32];
          const float hls[4] = {hl4.x, hl4.y, hl4.z, hl4.w};
          const float hts[4] = {ht4.x, ht4.y, ht4.z, ht4.w};
          const float pds[4] = {pd4.x, pd4.y, pd4.z, pd4.w};
          const float4 qa = params[c * 32 + lane], qb = params[128 + c * 32 + lane];
          const float aT2c[4] = {qa.x, qa.y, qa.z, qa.w}, aL2c[4] = {qb.x, qb.y, qb.z, qb.w};
          const float wTc = mT * dTs[c] * xs[c];
          const float wLc = mL * dLs[c] * xs[c];
          const float gyc = cfac * gys[c];
          float2 qT2 = make_float2(0.f, 0.f), qL2 = qT2, sT2 = qT2, sL2 = qT2;
          float pt[4];
#pragma unroll
          for (int n = 0; n < 4; n += 2) {
              const float2 aT = make_float2(aT2c[n], aT2c[n + 1]), aL = make_float2(aL2c[n], aL2c[n + 1]);
              const float2 argT = INTERIOR ? __fmul2_rn(make_float2(dTs[c], dTs[c]), aT) : __ffma2_rn(make_float2(dTs[c], dTs[c]), aT, offT2);
              const float2 argL = INTERIOR ? __fmul2_rn(make_float2(dLs[c], dLs[c]), aL) : __ffma2_rn(make_float2(dLs[c], dLs[c]), aL, offL2);
              const float2 gT = make_float2(ex2(argT.x), ex2(argT.y));
              const float2 gL = make_float2(ex2(argL.x), ex2(argL.y));
              const float2 in = __fmul2_rn(make_float2(cfac, cfac),
                                           __fadd2_rn(make_float2(pL[c][n], pL[c][n + 1]), make_float2(pds[n], pds[n + 1])));
              const float2 kap = __ffma2_rn(make_float2(gyc, gyc), make_float2(cs[n], cs[n + 1]), in);
              const float2 pTn = __fmul2_rn(gT, kap), pLn = __fmul2_rn(gL, kap);
              const float2 dzT = __fmul2_rn(pTn, make_float2(hts[n], hts[n + 1]));
              const float2 dzL = __fmul2_rn(pLn, make_float2(hls[n], hls[n + 1]));
              const float2 nAT = __ffma2_rn(dzT, make_float2(dTs[c], dTs[c]), make_float2(dAT[c][n], dAT[c][n + 1]));
              const float2 nAL = __ffma2_rn(dzL, make_float2(dLs[c], dLs[c]), make_float2(dAL[c][n], dAL[c][n + 1]));
              dAT[c][n] = nAT.x; dAT[c][n + 1] = nAT.y;
              dAL[c][n] = nAL.x; dAL[c][n + 1] = nAL.y;
              qT2 = __ffma2_rn(dzT, aT, qT2);
              qL2 = __ffma2_rn(dzL, aL, qL2);
              sT2 = __ffma2_rn(kap, make_float2(bTs[n], bTs[n + 1]), sT2);
              sL2 = __ffma2_rn(kap, make_float2(bLs[n], bLs[n + 1]), sL2);
              dBT2[n >> 1] = __ffma2_rn(kap, make_float2(wTc, wTc), dBT2[n >> 1]);
              dBL2[n >> 1] = __ffma2_rn(kap, make_float2(wLc, wLc), dBL2[n >> 1]);
              pL[c][n] = pLn.x; pL[c][n + 1] = pLn.y;
              pt[n] = pTn.x; pt[n + 1] = pTn.y;
          }
          // pT goes to the row above: next rank's slot, and the ring when that row is in another band
          const float4 pT4 = make_float4(pt[0], pt[1], pt[2], pt[3]);
          out[po + c * 32] = pT4;
          if (w.push) __stcg(ring + j * kSlotF4 + c * 32, pT4);
          const float qT = qT2.x + qT2.y, qL = qL2.x + qL2.y, sT = sT2.x + sT2.y, sL = sL2.x + sL2.y;
          if (INTERIOR) {
              o_dT[c] = fmaf(qT, kLn2, xs[c] * sT);
              o_dL[c] = fmaf(qL, kLn2, xs[c] * sL);
              o_dx[c] = fmaf(dTs[c], sT, dLs[c] * sL);
          } else {
              o_dT[c] = fmaf(qT, kLn2, mT * xs[c] * sT);
              o_dL[c] = fmaf(qL, kLn2, mL * xs[c] * sL);
              o_dx[c] = fmaf(mT * dTs[c], sT, mL * dLs[c] * sL);
          }
          dD[c] = fmaf(gys[c], xs[c], dD[c]);
      }

      // sums over states: 2-step exchange over the nq lanes; lane l ends with channel l of the group
      {
          const float r_dT = reduce_states(o_dT[0], o_dT[1], o_dT[2], o_dT[3], nq);
          const float r_dL = reduce_states(o_dL[0], o_dL[1], o_dL[2], o_dL[3], nq);
          const float r_dx = reduce_states(o_dx[0], o_dx[1], o_dx[2], o_dx[3], nq);
          if (y_lane) {
              const int eo = pixc * E + g * kGroup + lane;
              store1(static_cast<io_t*>(a.d_dT), eo, r_dT);
              store1(static_cast<io_t*>(a.d_dL), eo, r_dL);
              store1(static_cast<io_t*>(a.d_x), eo, fmaf(sel4(vgy, nq), D_own, r_dx));
          }
      }

      // sums over channels: 8 values (d_BT[4], d_BL[4]) over the 8 cq lanes: 4 + 2 + 1 exchanges
      {
          const float dBT[4] = {dBT2[0].x, dBT2[0].y, dBT2[1].x, dBT2[1].y};
          const float dBL[4] = {dBL2[0].x, dBL2[0].y, dBL2[1].x, dBL2[1].y};
          float k0 = hi16 ? dBL[0] : dBT[0], k1 = hi16 ? dBL[1] : dBT[1];
          float k2 = hi16 ? dBL[2] : dBT[2], k3 = hi16 ? dBL[3] : dBT[3];
          k0 += __shfl_xor_sync(0xffffffffu, hi16 ? dBT[0] : dBL[0], 16);
          k1 += __shfl_xor_sync(0xffffffffu, hi16 ? dBT[1] : dBL[1], 16);
          k2 += __shfl_xor_sync(0xffffffffu, hi16 ? dBT[2] : dBL[2], 16);
          k3 += __shfl_xor_sync(0xffffffffu, hi16 ? dBT[3] : dBL[3], 16);
          float m0 = hi8 ? k2 : k0, m1 = hi8 ? k3 : k1;
          m0 += __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k2, 8);
          m1 += __shfl_xor_sync(0xffffffffu, hi8 ? k1 : k3, 8);
          float v = hi4 ? m1 : m0;
          v += __shfl_xor_sync(0xffffffffu, hi4 ? m0 : m1, 4);
          // this lane now owns array (hi16 ? d_BL : d_BT), state n0 + 2*hi8 + hi4
          if (db_lane) atomicAdd(db_acc + ((long long)pixc * a.N + db_n), v);
      }
          };

    // ---- the warp's sequence ---------------------------------------------------------------------
    Row cur = make_row(nbands - 1);
    if (rr >= 1) {
        for (int k = 0; k < rr - 1; ++k) end_step();
        prefetch_row_end(cur);
        end_step();
    }
    if (cur.has) stage_cell(cur, W - 1);
    end_step();
    if (cur.has) stage_cell(cur, W - 2);
    end_step();
    for (int q = nbands - 1; q >= 0; --q) {
        const Row nxt = make_row(q - 1);                      // (.has is false past the last item)
        if (cur.has) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int n = 0; n < 4; ++n) pL[c][n] = 0.f;   // a row starts from no right neighbour
            if (cur.bottom) {
                // the bottom row of the map has no row below: nothing arrives in this rank's incoming
                // buffers during the row, so they are cleared once and the cells read zeros from them
                if (rr == 0) {
#pragma unroll
                    for (int k = 0; k < 12; ++k) pullbuf[k * 32] = zero4;
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) in[k * 32] = zero4;
                }
            }
            for (int j = W - 1; j >= 0; --j) {
                if (j >= 2) {
                    stage_cell(cur, j - 2);
                    // cell (i, 0) has no left block: its buffer is free for the right-most block of the next row
                    if (j == 2 && nxt.has) prefetch_row_end(nxt);
                } else if (nxt.has) {
                    stage_cell(nxt, W - 2 + j);
                }
                if (cur.row0 || j == 0) cell(std::false_type{}, cur, j);
                else cell(std::true_type{}, cur, j);
                end_step();
            }
        } else {
            for (int j = W - 1; j >= 0; --j) {
                if (nxt.has) {
                    if (j == 2) prefetch_row_end(nxt);
                    else if (j < 2) stage_cell(nxt, W - 2 + j);
                }
                end_step();
            }
        }
        cur = nxt;
    }
    for (int k = 0; k < Rb - 1 - rr; ++k) end_step();         // until the last warp is done
    cp_async_wait_all();                                      // (only empty groups can be pending here)
}

}  // namespace m2d
