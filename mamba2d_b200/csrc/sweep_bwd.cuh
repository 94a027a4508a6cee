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
//
// The sweep mirrors the forward one: bands are visited last to first, the bottom row of a band
// leads, columns run right to left.  h comes from the state record the recompute sweep wrote.
#pragma once

#include "sweep_fwd.cuh"

namespace m2d {

struct RevIn {
    float4 x, dT, dL, gy, bT, bL, c;
    float4 hl[4], ht[4];   // h[i][j-1] and h[i-1][j], one float4 (4 states) per channel
};

template <typename io_t, bool VEC>
__device__ __forceinline__ void load_rev(RevIn& ri, const ScanArgs& a, int b, int g, int i, int j, int lane, int ch0, int chv, int n0, int nv) {
    const long long pix = ((long long)b * a.H + i) * a.W + j;
    if (chv > 0) {   // see load_cell: never read beyond the last channel
        ri.gy = load4<VEC>(static_cast<const io_t*>(a.gy), pix * a.E + ch0, chv);
        ri.x = load4<VEC>(static_cast<const io_t*>(a.x), pix * a.E + ch0, chv);
        ri.dT = load4<VEC>(static_cast<const io_t*>(a.dT), pix * a.E + ch0, chv);
        ri.dL = load4<VEC>(static_cast<const io_t*>(a.dL), pix * a.E + ch0, chv);
    } else {
        ri.gy = ri.x = ri.dT = ri.dL = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (nv > 0) {
        ri.bT = load4<VEC>(static_cast<const io_t*>(a.BT), pix * a.pBT + n0, nv);
        ri.bL = load4<VEC>(static_cast<const io_t*>(a.BL), pix * a.pBL + n0, nv);
        ri.c = load4<VEC>(static_cast<const io_t*>(a.C), pix * a.pC + n0, nv);
    } else {
        ri.bT = ri.bL = ri.c = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const size_t rec = ((size_t)b * gridDim.y + g) * a.H * a.W + (size_t)i * a.W + j;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        ri.hl[k] = (j > 0) ? __ldcg(a.hs + ((rec - 1) * 4 + k) * 32 + lane) : z;
        ri.ht[k] = (i > 0) ? __ldcg(a.hs + ((rec - a.W) * 4 + k) * 32 + lane) : z;
    }
}

// One CTA's adjoint sweep over image `b`.  dAT/dAL/dD accumulate across calls.
template <typename io_t, bool VEC>
__device__ __forceinline__ void reverse_sweep(const ScanArgs& a, float4* handoff, const float (&aT2)[4][4],
                                              const float (&aL2)[4][4], float D_own, float (&dAT)[4][4],
                                              float (&dAL)[4][4], float (&dD)[4], int b) {
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));
    const int W = a.W, H = a.H, Rb = a.Rb, nbands = a.nbands;
    const int rr = Rb - 1 - r;                 // rank in the reverse sweep: the bottom row of a band leads
    const int steps = nbands * W + Rb - 1;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    float4* ring = a.ring + (size_t)cta * W * kSlotF4;
    const int slot_stride = (nwarps + 1) * kSlotF4;

    // destination of this lane's share of the channel sums (see the exchange below)
    const bool hi16 = (cq & 4) != 0, hi8 = (cq & 2) != 0;

    float pL[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int n = 0; n < 4; ++n) pL[c][n] = 0.f;

    // positions are tracked in reversed coordinates (jr = W-1-j, qr = nbands-1-q)
    Pos pn = {0, 0, 0};
    bool vn = (rr == 0) && ((nbands - 1) * Rb + r < H);
    RevIn nxt;
    {
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        nxt.x = nxt.dT = nxt.dL = nxt.gy = nxt.bT = nxt.bL = nxt.c = z;
#pragma unroll
        for (int k = 0; k < 4; ++k) nxt.hl[k] = nxt.ht[k] = z;
    }
    if (vn) load_rev<io_t, VEC>(nxt, a, b, g, (nbands - 1) * Rb + r, W - 1, lane, ch0, chv, n0, nv);

    for (int s = 0; s < steps; ++s) {
        const Pos pc = pn;
        const bool vc = vn;
        const RevIn cur = nxt;
        float4* buf_w = handoff + (s & 1) * slot_stride;
        const float4* buf_r = handoff + ((s & 1) ^ 1) * slot_stride;

        if (s + 1 > rr) pn = advance(pc, W, nbands);
        {
            const int qn = nbands - 1 - pn.q;
            const int in = qn * Rb + r, jn = W - 1 - pn.j;
            vn = (s + 1 >= rr) && (pn.bi < 1) && (in < H);
            if (vn) {
                load_rev<io_t, VEC>(nxt, a, b, g, in, jn, lane, ch0, chv, n0, nv);
                if (rr == 0 && in + 1 < H) {
                    // the row below lives in the band visited before this one: pull its pT from the ring
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        cp_async16(buf_w + k * 32 + lane, ring + ((size_t)jn * 4 + k) * 32 + lane);
                }
            }
        }

        if (vc) {
            const int q = nbands - 1 - pc.q;
            const int i = q * Rb + r, j = W - 1 - pc.j;
            const long long pix = ((long long)b * H + i) * W + j;
            const float cfac = (i > 0 && j > 0) ? 0.5f : 1.f;
            const float mT = (i > 0) ? 1.f : 0.f;
            const float mL = (j > 0 || i == 0) ? 1.f : 0.f;

            float4 pd[4];   // pT of the row below
            if (i + 1 < H) {
#pragma unroll
                for (int k = 0; k < 4; ++k) pd[k] = buf_r[rr * kSlotF4 + k * 32 + lane];
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) pd[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (j == W - 1) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int n = 0; n < 4; ++n) pL[c][n] = 0.f;
            }

            const float xs[4] = {cur.x.x, cur.x.y, cur.x.z, cur.x.w};
            const float dTs[4] = {cur.dT.x, cur.dT.y, cur.dT.z, cur.dT.w};
            const float dLs[4] = {cur.dL.x, cur.dL.y, cur.dL.z, cur.dL.w};
            const float gys[4] = {cur.gy.x, cur.gy.y, cur.gy.z, cur.gy.w};
            const float bTs[4] = {cur.bT.x, cur.bT.y, cur.bT.z, cur.bT.w};
            const float bLs[4] = {cur.bL.x, cur.bL.y, cur.bL.z, cur.bL.w};
            const float cs[4] = {cur.c.x, cur.c.y, cur.c.z, cur.c.w};

            float dBT[4] = {0.f, 0.f, 0.f, 0.f}, dBL[4] = {0.f, 0.f, 0.f, 0.f};
            float o_dT[4], o_dL[4], o_dx[4];
            float4 pTout[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float hls[4] = {cur.hl[c].x, cur.hl[c].y, cur.hl[c].z, cur.hl[c].w};
                const float hts[4] = {cur.ht[c].x, cur.ht[c].y, cur.ht[c].z, cur.ht[c].w};
                const float pds[4] = {pd[c].x, pd[c].y, pd[c].z, pd[c].w};
                const float wTc = mT * dTs[c] * xs[c];
                const float wLc = mL * dLs[c] * xs[c];
                const float gyc = cfac * gys[c];
                float qT = 0.f, qL = 0.f, sT = 0.f, sL = 0.f;
                float pt[4];
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const float kap = fmaf(gyc, cs[n], cfac * (pL[c][n] + pds[n]));
                    const float gT = ex2(dTs[c] * aT2[c][n]);
                    const float gL = ex2(dLs[c] * aL2[c][n]);
                    const float pTn = gT * kap, pLn = gL * kap;
                    const float dzT = pTn * hts[n], dzL = pLn * hls[n];
                    dAT[c][n] = fmaf(dzT, dTs[c], dAT[c][n]);
                    dAL[c][n] = fmaf(dzL, dLs[c], dAL[c][n]);
                    qT = fmaf(dzT, aT2[c][n], qT);
                    qL = fmaf(dzL, aL2[c][n], qL);
                    sT = fmaf(kap, bTs[n], sT);
                    sL = fmaf(kap, bLs[n], sL);
                    dBT[n] = fmaf(kap, wTc, dBT[n]);
                    dBL[n] = fmaf(kap, wLc, dBL[n]);
                    pL[c][n] = pLn;
                    pt[n] = pTn;
                }
                pTout[c] = make_float4(pt[0], pt[1], pt[2], pt[3]);
                o_dT[c] = fmaf(qT, kLn2, mT * xs[c] * sT);
                o_dL[c] = fmaf(qL, kLn2, mL * xs[c] * sL);
                o_dx[c] = fmaf(mT * dTs[c], sT, mL * dLs[c] * sL);
                dD[c] = fmaf(gys[c], xs[c], dD[c]);
            }

            // pT goes to the row above: next rank's slot, and the ring when that row is in another band
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                buf_w[(rr + 1) * kSlotF4 + c * 32 + lane] = pTout[c];
                if (r == 0 && q > 0) __stcg(ring + ((size_t)j * 4 + c) * 32 + lane, pTout[c]);
            }

            // sums over states: 2-step exchange over the nq lanes; lane l ends with channel l of the group
            {
                const float r_dT = reduce_states(o_dT[0], o_dT[1], o_dT[2], o_dT[3], nq);
                const float r_dL = reduce_states(o_dL[0], o_dL[1], o_dL[2], o_dL[3], nq);
                const float r_dx = reduce_states(o_dx[0], o_dx[1], o_dx[2], o_dx[3], nq);
                const int ch = g * kGroup + lane;
                if (ch < a.E) {
                    store1(static_cast<io_t*>(a.d_dT), pix * a.E + ch, r_dT);
                    store1(static_cast<io_t*>(a.d_dL), pix * a.E + ch, r_dL);
                    store1(static_cast<io_t*>(a.d_x), pix * a.E + ch, fmaf(sel4(cur.gy, nq), D_own, r_dx));
                }
            }

            // sums over channels: 8 values (d_BT[4], d_BL[4]) over the 8 cq lanes: 4 + 2 + 1 exchanges
            {
                float k0 = hi16 ? dBL[0] : dBT[0], k1 = hi16 ? dBL[1] : dBT[1];
                float k2 = hi16 ? dBL[2] : dBT[2], k3 = hi16 ? dBL[3] : dBT[3];
                k0 += __shfl_xor_sync(0xffffffffu, hi16 ? dBT[0] : dBL[0], 16);
                k1 += __shfl_xor_sync(0xffffffffu, hi16 ? dBT[1] : dBL[1], 16);
                k2 += __shfl_xor_sync(0xffffffffu, hi16 ? dBT[2] : dBL[2], 16);
                k3 += __shfl_xor_sync(0xffffffffu, hi16 ? dBT[3] : dBL[3], 16);
                float m0 = hi8 ? k2 : k0, m1 = hi8 ? k3 : k1;
                m0 += __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k2, 8);
                m1 += __shfl_xor_sync(0xffffffffu, hi8 ? k1 : k3, 8);
                const bool hi4 = (cq & 1) != 0;
                float v = hi4 ? m1 : m0;
                v += __shfl_xor_sync(0xffffffffu, hi4 ? m0 : m1, 4);
                // this lane now owns array (hi16 ? d_BL : d_BT), state n0 + 2*hi8 + hi4
                const int nn = n0 + (hi8 ? 2 : 0) + (hi4 ? 1 : 0);
                if (nn < a.N) atomicAdd(a.accBC + pix * 48 + (hi16 ? 16 : 0) + nn, v);
            }
        }
        cp_async_wait_all();
        __syncthreads();
    }
}

}  // namespace m2d
