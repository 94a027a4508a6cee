// Reverse (adjoint) wavefront sweep of the backward pass.
//
// With g = gy*C the direct gradient of a state, c = 1/2 inside the map and 1 on row 0 / column 0,
// lam the total adjoint of h and kap = c*lam (reference: models/kernels/wf_cuda/wf_cuda.cu:108-160;
// the reference's omega buffer equals lam/2 and carries no extra information):
//     lam[i,j] = g[i,j] + gL[i,j+1]*kap[i,j+1] + gT[i+1,j]*kap[i+1,j]
// Each cell computes its own gates once and hands pT = gT*kap to the row above and pL = gL*kap to
// the cell on its left, so the sweep needs two exponentials per state.  All gradient arithmetic
// the reference does afterwards in PyTorch (models/kernels/wavefront_cuda.py:97-139, :176-178,
// :193-194) is fused here:
//     dzT = pT*h[i-1,j]                 dzL = pL*h[i,j-1]
//     d_AT[e,n] += dzT*dT               d_AL[e,n] += dzL*dL
//     d_dT = sum_n dzT*AT + mT*x*sum_n kap*BT      (mT = i>0)
//     d_dL = sum_n dzL*AL + mL*x*sum_n kap*BL      (mL = j>0 or i==0)
//     d_x  = mT*dT*sum_n kap*BT + mL*dL*sum_n kap*BL + gy*D
//     d_BT[n] = sum_e mT*kap*dT*x       d_BL[n] = sum_e mL*kap*dL*x        d_D[e] += gy*x
// (d_C = sum_e gy*h is produced by the recompute sweep, where h is in registers.)
// A missing neighbour is handled as in the forward sweep: its gate gets exponent -inf, so pT / pL
// and with them dzT / dzL vanish on row 0 / column 0 without any masking of h.
//
// The sweep mirrors the forward one: bands are visited last to first, the bottom row of a band
// leads (rank 0), columns run right to left; pT travels through the same shared-memory slots and
// the same global ring.  h comes from the state record the recompute sweep wrote.  Every warp copies
// h[i][j-1] of its own row into shared memory one step ahead (cp.async); the warp of the row below,
// which runs one step ahead, needs exactly that block as its h[i-1][j] in the same step and reads
// it from there, so each block crosses L2 -> SM once.  (The block h[i][W-1] is nobody's left
// neighbour; the row's warp fetches it for the warp below one step before its own row starts.)
#pragma once

#include "sweep_fwd.cuh"

namespace m2d {

// Dynamic shared memory of the backward kernel: [hand-off slots][input stages][h areas], the h
// areas being one per row-warp plus one for the row above the band.
__host__ __device__ inline size_t bwd_smem_bytes(int warps) { return sweep_smem_bytes(warps) + handoff_bytes(warps); }   // + parameters behind

struct RevRun {
    int pixl, jl, ql;       // load side (reversed counters: jl = W-1-j, ql counts this CTA's bands from its last)
    bool row_l, pull_l, top_l;
    int seen;               // columns of the band below known to be published (chained CTAs)
    const float4* pull;     // pT row of the band below
    const int* pcount;      // its column counter
    float4* push;           // where this band's first row puts its pT
    int* ccount;            // its column counter
    const float4* phl;      // state record of h[i][j-1] for the cell being staged
    int pixc, jc, qc;       // compute side
    bool row_c, push_c, bottom_c, row0_c;
};

// One CTA's adjoint sweep over image `b`.  dAT/dAL/dD accumulate across calls.
template <typename io_t, bool VEC, bool CHAINED = false>
__device__ __forceinline__ void reverse_sweep(const ScanArgs& a, float4* handoff, const float4* params,
                                              float D_own, float (&dAT)[4][4],
                                              float (&dAL)[4][4], float (&dD)[4], int b, int cpos = 0, int chain_arg = 1) {
    const int chain = CHAINED ? chain_arg : 1;
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y, groups = gridDim.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));
    const int W = a.W, H = a.H, E = a.E, Rb = a.Rb, nbands = a.nbands;
    const int rr = Rb - 1 - r;                 // rank in the reverse sweep
    const int nq_c = chain > 1 ? (nbands - cpos + chain - 1) / chain : nbands;   // bands this CTA owns
    const int T = nq_c * W;
    const int steps = T + Rb - 1;
    const int pBT = (int)a.pBT, pBL = (int)a.pBL, pC = (int)a.pC;
    float4* const ring = a.ring + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * W) * kSlotF4 + lane;
    float4* const my = handoff + rr * kSlotPair + lane;                       // pT: read slot rr, write slot rr+1
    char* const stage = reinterpret_cast<char*>(handoff + (nwarps + 1) * kSlotPair) + r * 2 * kStageBytes;
    float4* const harea = reinterpret_cast<float4*>(reinterpret_cast<char*>(handoff) + sweep_smem_bytes(nwarps)) + lane;
    float4* const h_own = harea + (r + 1) * kSlotPair;                        // this row's h[i][j-1]
    float4* const h_up = harea + r * kSlotPair;                               // the row above: h[i-1][j]
    constexpr int HB = HsBlock<io_t>::f4;   // float4 units per state-record block
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
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int n = 0; n < 4; ++n) pL[c][n] = 0.f;

    LaneCopy<io_t> lc;
    lc.init(a.x, a.dT, a.dL, a.gy, a.BT, a.BL, a.C, pBT, pBL, pC, E, a.N, g, lane, true);

    RevRun st;
    st.pixl = st.jl = st.ql = 0;
    st.pixc = st.jc = st.qc = 0;
    st.row_l = st.pull_l = st.top_l = st.row_c = st.push_c = st.bottom_c = st.row0_c = false;
    st.phl = nullptr;
    st.seen = 0; st.pull = ring; st.pcount = nullptr; st.push = ring; st.ccount = nullptr;

    // One state-record block, global -> shared (2 KiB of fp32 states or 1 KiB of bf16 states).
    auto copy_block = [&](bool on, unsigned dst, const float4* src) {
        if (sizeof(io_t) == 2) cp_async16x2_if(on, dst, src);
        else cp_async16x4_if(on, dst, src);
    };
    // Four states of channel c of a staged block as floats.
    auto block_states = [&](const float4* area, int c) -> float4 {
        if (sizeof(io_t) == 2) {
            const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(area + (c >> 1) * 32) + (c & 1) * 8);
            return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                               __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
        }
        return area[c * 32];
    };

    // Fetch h[i][W-1] of the row this warp starts next, for the warp of the row below.
    auto prefetch_row_end = [&](int q, int par) {
        const int i = q * Rb + r;
        if (feeds_below && r < Rb && i < H) {
            const float4* src = hs_img + ((size_t)i * W + (W - 1)) * HB;
            copy_block(true, smem_u32(h_own + par * kSlotF4), src);
        }
    };

    // ---- stage the inputs and h[i][j-1] (and h[i-1][j] for the top row of a band) of the next cell
    auto load_phase = [&](int par) {
        if (st.jl == 0) {   // start of a row (its right end)
            const int q = cpos + (nq_c - 1 - st.ql) * chain;
            const int i = q * Rb + r;
            st.row_l = (r < Rb) && (i < H);
            st.pull_l = st.row_l && (rr == 0) && (i + 1 < H);      // pT of the row below comes through the ring
            if (chain > 1 && q + 1 < nbands) {
                // the band below belongs to another CTA: its pT row sits in the boundary slot between
                // band q and band q+1 (the slot the forward sweep used for h in the other direction)
                const size_t band = ((size_t)b * groups + g) * nbands + q;
                st.pull = a.bnd + band * W * kSlotF4 + lane;
                st.pcount = a.progress + (size_t)a.B * groups * nbands + band + 1;
                st.seen = 0;
            }
            st.top_l = st.row_l && (r == 0) && (i > 0);            // h of the row above is not in this band
            st.pixl = scan_pixel(a, b, i, W - 1);
            st.phl = hs_img + ((size_t)i * W + (W - 2)) * HB;
        }
        const int j = W - 1 - st.jl;
        if (chain > 1 && st.pull_l && st.seen < st.jl + 1)
            st.seen = wait_columns(st.pcount, st.jl + 1, a.status, a.wait_limit);
        if (st.row_l) {
            char* stg = stage + par * kStageBytes;
            if (VEC) {
                lc.issue(smem_u32(stg), lane, st.pixl, E);
            } else {
                const int e0 = st.pixl * E + ch0;
                stage4<VEC>(ch_copier, stg + cq * 16, static_cast<const io_t*>(a.x), e0, chv);
                stage4<VEC>(ch_copier, stg + (8 + cq) * 16, static_cast<const io_t*>(a.dT), e0, chv);
                stage4<VEC>(ch_copier, stg + (16 + cq) * 16, static_cast<const io_t*>(a.dL), e0, chv);
                stage4<VEC>(ch_copier, stg + (24 + cq) * 16, static_cast<const io_t*>(a.gy), e0, chv);
                stage4<VEC>(st_copier, stg + (32 + nq) * 16, static_cast<const io_t*>(a.BT), st.pixl * pBT + n0, nv);
                stage4<VEC>(st_copier, stg + (36 + nq) * 16, static_cast<const io_t*>(a.BL), st.pixl * pBL + n0, nv);
                stage4<VEC>(st_copier, stg + (40 + nq) * 16, static_cast<const io_t*>(a.C), st.pixl * pC + n0, nv);
            }
            copy_block(j > 0, smem_u32(h_own + par * kSlotF4), st.phl);
            copy_block(st.top_l, smem_u32(h_up + par * kSlotF4), st.phl + (ptrdiff_t)(1 - W) * HB);
            cp_async16x4_if(st.pull_l, smem_u32(my + par * kSlotF4), st.pull + j * kSlotF4);
            st.pixl -= a.dir;
            st.phl -= HB;
        }
        // last cell of a row: its own h[i][-1] does not exist (that gate is zero), so the slot is
        // free for the right-most block of the row this warp starts next
        if (j == 0 && st.ql + 1 < nq_c) prefetch_row_end(cpos + (nq_c - 2 - st.ql) * chain, par);
        if (++st.jl == W) { st.jl = 0; ++st.ql; }
    };

    // ---- adjoint arithmetic of the current cell ---------------------------------------------------
    auto compute_phase = [&](int par) {
        if (st.jc == 0) {
            const int q = cpos + (nq_c - 1 - st.qc) * chain;
            const int i = q * Rb + r;
            st.row_c = (r < Rb) && (i < H);
            if (chain > 1 && q > 0) {
                const size_t band = ((size_t)b * groups + g) * nbands + q;
                st.push = a.bnd + (band - 1) * W * kSlotF4 + lane;
                st.ccount = a.progress + (size_t)a.B * groups * nbands + band;
            }
            st.row0_c = (i == 0);
            st.bottom_c = (i + 1 >= H);
            st.push_c = st.row_c && (r == 0) && (q > 0);
            st.pixc = scan_pixel(a, b, i, W - 1);
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int n = 0; n < 4; ++n) pL[c][n] = 0.f;
        }
        if (st.row_c) {
            const int j = W - 1 - st.jc;
          auto cell = [&](auto tag) {
            constexpr bool INTERIOR = decltype(tag)::value;
            // cells inside the map (row > 0, column > 0) have constant weights; row 0 and column 0 take
            // the generic path, where a missing neighbour's state is taken as zero instead of being read
            float cfac, mT, mL, offT, offL;
            if (INTERIOR) {
                cfac = 0.5f; mT = 1.f; mL = 1.f; offT = 0.f; offL = 0.f;
            } else {
                const bool first = (j == 0);   // column 0: no averaging, no left neighbour; the left input term exists only on row 0
                cfac = (st.row0_c || first) ? 1.f : 0.5f;
                mT = st.row0_c ? 0.f : 1.f;
                mL = (first && !st.row0_c) ? 0.f : 1.f;
                offT = st.row0_c ? ninf : 0.f;
                offL = first ? ninf : 0.f;
            }
            const float2 offT2 = make_float2(offT, offT), offL2 = make_float2(offL, offL);
            const char* stg = stage + (par ^ 1) * kStageBytes;
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
                const float4 hl4 = (INTERIOR || j > 0) ? block_states(h_own + (par ^ 1) * kSlotF4, c) : zero4;
                const float4 ht4 = (INTERIOR || !st.row0_c) ? block_states(h_up + (par ^ 1) * kSlotF4, c) : zero4;
                const float4 pd4 = st.bottom_c ? zero4 : my[(par ^ 1) * kSlotF4 + c * 32];
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
                my[kSlotPair + par * kSlotF4 + c * 32] = pT4;
                stcg_if(st.push_c, st.push + j * kSlotF4 + c * 32, pT4);
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

            if (chain > 1 && st.push_c) {
                // publish the column (columns are produced right to left): data first, then the counter
                __syncwarp();
                if (lane == 0) st_release_gpu(st.ccount, st.jc + 1);
            }

            // sums over states: 2-step exchange over the nq lanes; lane l ends with channel l of the group
            {
                const float r_dT = reduce_states(o_dT[0], o_dT[1], o_dT[2], o_dT[3], nq);
                const float r_dL = reduce_states(o_dL[0], o_dL[1], o_dL[2], o_dL[3], nq);
                const float r_dx = reduce_states(o_dx[0], o_dx[1], o_dx[2], o_dx[3], nq);
                if (y_lane) {
                    const int eo = st.pixc * E + g * kGroup + lane;
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
                if (db_lane) atomicAdd(db_acc + ((long long)st.pixc * a.N + db_n), v);
            }
          };
            if (st.row0_c || j == 0) cell(std::false_type{});
            else cell(std::true_type{});
            st.pixc -= a.dir;
        }
        if (++st.jc == W) { st.jc = 0; ++st.qc; }
    };

    // Step s: stage cell (s + 1 - rr), compute cell (s - rr); the step before a warp's first copy
    // fetches the right-most block of its first row for the warp below.
    int cl = -rr;
    for (int s = -1; s < steps; s += 2) {
        if ((unsigned)cl < (unsigned)T) load_phase(1);
        else if (cl == -1) prefetch_row_end(cpos + (nq_c - 1) * chain, 1);
        if ((unsigned)(cl - 1) < (unsigned)T) compute_phase(1);
        ++cl;
        cp_async_wait_all();
        __syncthreads();
        if (s + 1 < steps) {
            if ((unsigned)cl < (unsigned)T) load_phase(0);
            else if (cl == -1) prefetch_row_end(cpos + (nq_c - 1) * chain, 0);
            if ((unsigned)(cl - 1) < (unsigned)T) compute_phase(0);
            ++cl;
            cp_async_wait_all();
            __syncthreads();
        }
    }
}

}  // namespace m2d
