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
// Work decomposition: see Pos in common.cuh.  Warp r hands its fresh state to warp r+1 through a
// double-buffered shared-memory slot; one __syncthreads per step keeps the warps in lock step.
// The last row of a band reaches the first row of the next band (W - Rb + 1 steps later) through a
// per-CTA ring in global memory that stays L2 resident; warp 0 pulls its slot back into shared
// memory with cp.async one step ahead of use.
#pragma once

#include "common.cuh"

namespace m2d {

struct ScanArgs {
    int B, H, W, E, N;
    const void *x, *dT, *dL, *AT, *AL, *BT, *BL, *C, *D;
    long long pBT, pBL, pC;   // pixel pitch (elements) of BT, BL, C
    void* y;
    float4* ring;             // per-CTA band-boundary ring: [cta][W][4][32] float4
    int Rb, nbands;
    // ---- backward only ----
    const void* gy;
    float4* hs;               // full state record: [b][group][H*W][4][32] float4
    float* accBC;             // fp32 accumulators [B*H*W][48]: d_BT | d_BL | d_C
    float* accA;              // fp32 accumulators [2][E][N]:   d_AT | d_AL
    float* accD;              // fp32 accumulators [E]
    void *d_x, *d_dT, *d_dL;
};
typedef ScanArgs FwdArgs;

// Cell inputs held in registers (current step and the prefetched next step).
struct CellIn {
    float4 x, dT, dL, bT, bL, c;
    float4 gy;   // only loaded by the backward sweeps
};

template <typename io_t, bool VEC, bool WITH_GY>
__device__ __forceinline__ void load_cell(CellIn& ci, const FwdArgs& a, long long pix, int ch0, int chv, int n0, int nv) {
    // lanes whose channel block lies beyond E (last group of a width that is not a multiple of 32)
    // must not touch memory: a vector load there would read the next pixel
    if (chv > 0) {
        if (WITH_GY) ci.gy = load4<VEC>(static_cast<const io_t*>(a.gy), pix * a.E + ch0, chv);
        ci.x = load4<VEC>(static_cast<const io_t*>(a.x), pix * a.E + ch0, chv);
        ci.dT = load4<VEC>(static_cast<const io_t*>(a.dT), pix * a.E + ch0, chv);
        ci.dL = load4<VEC>(static_cast<const io_t*>(a.dL), pix * a.E + ch0, chv);
    } else {
        ci.gy = ci.x = ci.dT = ci.dL = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (nv > 0) {
        ci.bT = load4<VEC>(static_cast<const io_t*>(a.BT), pix * a.pBT + n0, nv);
        ci.bL = load4<VEC>(static_cast<const io_t*>(a.BL), pix * a.pBL + n0, nv);
        ci.c = load4<VEC>(static_cast<const io_t*>(a.C), pix * a.pC + n0, nv);
    } else {
        ci.bT = ci.bL = ci.c = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// Load the thread's 4x4 block of a (E,N) parameter, scaled; zero outside the valid range.
template <typename io_t>
__device__ __forceinline__ void load_param_block(float (&dst)[4][4], const void* P, int N, int ch0, int chv, int n0, int nv, float scale) {
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int n = 0; n < 4; ++n)
            dst[c][n] = (c < chv && n < nv) ? load1(static_cast<const io_t*>(P), (long long)(ch0 + c) * N + n0 + n) * scale : 0.f;
}

// One CTA's forward sweep over its work list.  `handoff` is shared memory of
// 2 * (warps + 1) * kSlotF4 float4, zero-initialised by the caller.  With STORE_HS every fresh
// state block is also written to a.hs.
template <typename io_t, bool VEC, bool STORE_HS>
__device__ __forceinline__ void forward_sweep(const FwdArgs& a, float4* handoff, const float (&aT2)[4][4],
                                              const float (&aL2)[4][4], float D_own, int img0, int img_stride, int nb) {
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));
    const int W = a.W, H = a.H, Rb = a.Rb, nbands = a.nbands;
    const int steps = nb * nbands * W + Rb - 1;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    float4* ring = a.ring + (size_t)cta * W * kSlotF4;
    const int slot_stride = (nwarps + 1) * kSlotF4;   // float4 per parity buffer

    float h[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int n = 0; n < 4; ++n) h[c][n] = 0.f;

    Pos pn = {0, 0, 0};
    bool vn = (r == 0) && (r < Rb) && (nb > 0);
    CellIn nxt;
    nxt.x = nxt.dT = nxt.dL = nxt.bT = nxt.bL = nxt.c = nxt.gy = make_float4(0.f, 0.f, 0.f, 0.f);
    if (vn) load_cell<io_t, VEC, STORE_HS>(nxt, a, (long long)img0 * H * W, ch0, chv, n0, nv);

    for (int s = 0; s < steps; ++s) {
        const Pos pc = pn;
        const bool vc = vn;
        const CellIn cur = nxt;
        float4* buf_w = handoff + (s & 1) * slot_stride;          // written this step
        const float4* buf_r = handoff + ((s & 1) ^ 1) * slot_stride;  // written last step

        // ---- where this warp stands next step; prefetch its inputs --------------------------------
        if (s + 1 > r) pn = advance(pc, W, nbands);
        vn = (s + 1 >= r) && (r < Rb) && (pn.bi < nb) && (pn.q * Rb + r < H);
        if (vn) {
            const int bn = img0 + pn.bi * img_stride;
            const long long pix = ((long long)bn * H + (pn.q * Rb + r)) * W + pn.j;
            load_cell<io_t, VEC, STORE_HS>(nxt, a, pix, ch0, chv, n0, nv);
            if (r == 0 && pn.q > 0) {
                // row above lives in the previous band: pull it from the ring into slot 0
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    cp_async16(buf_w + k * 32 + lane, ring + ((size_t)pn.j * 4 + k) * 32 + lane);
            }
        }

        if (vc) {
            const int i = pc.q * Rb + r, j = pc.j;
            const int b = img0 + pc.bi * img_stride;
            const long long pix = ((long long)b * H + i) * W + j;
            const float ninf = __int_as_float(0xff800000);
            const float wT = (i == 0) ? 0.f : (j == 0 ? 1.f : 0.5f);
            const float wL = (j == 0) ? (i == 0 ? 1.f : 0.f) : (i == 0 ? 1.f : 0.5f);
            const float offT = (i == 0) ? ninf : (j == 0 ? 0.f : -1.f);
            const float offL = (j == 0) ? ninf : (i == 0 ? 0.f : -1.f);

            float4 top[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) top[k] = buf_r[r * kSlotF4 + k * 32 + lane];

            const float xs[4] = {cur.x.x, cur.x.y, cur.x.z, cur.x.w};
            const float dTs[4] = {cur.dT.x, cur.dT.y, cur.dT.z, cur.dT.w};
            const float dLs[4] = {cur.dL.x, cur.dL.y, cur.dL.z, cur.dL.w};
            const float bTs[4] = {cur.bT.x, cur.bT.y, cur.bT.z, cur.bT.w};
            const float bLs[4] = {cur.bL.x, cur.bL.y, cur.bL.z, cur.bL.w};
            const float cs[4] = {cur.c.x, cur.c.y, cur.c.z, cur.c.w};
            float yacc[4];
            float dC[4] = {0.f, 0.f, 0.f, 0.f};   // backward only: sum over this thread's channels of gy*h
            const float gys[4] = {cur.gy.x, cur.gy.y, cur.gy.z, cur.gy.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float tp[4] = {top[c].x, top[c].y, top[c].z, top[c].w};
                const float dtx = wT * dTs[c] * xs[c];
                const float dlx = wL * dLs[c] * xs[c];
                float acc = 0.f;
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const float gT = ex2(fmaf(dTs[c], aT2[c][n], offT));
                    const float gL = ex2(fmaf(dLs[c], aL2[c][n], offL));
                    const float u = fmaf(dlx, bLs[n], dtx * bTs[n]);
                    const float hn = fmaf(gL, h[c][n], fmaf(gT, tp[n], u));
                    h[c][n] = hn;
                    acc = fmaf(hn, cs[n], acc);
                    if (STORE_HS) dC[n] = fmaf(gys[c], hn, dC[n]);
                }
                yacc[c] = acc;
            }

            // hand the fresh state to the row below (slot r+1), to the next band, and to hs
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float4 hv = make_float4(h[c][0], h[c][1], h[c][2], h[c][3]);
                buf_w[(r + 1) * kSlotF4 + c * 32 + lane] = hv;
                if (r == Rb - 1 && pc.q < nbands - 1) __stcg(ring + ((size_t)j * 4 + c) * 32 + lane, hv);
                if (STORE_HS) {
                    const size_t rec = ((size_t)b * gridDim.y + g) * H * W + (size_t)i * W + j;
                    __stcg(a.hs + (rec * 4 + c) * 32 + lane, hv);
                }
            }

            if (STORE_HS) {
                // d_C[pixel][n] = sum over channels of gy*h: finish over the 8 cq lanes, then one
                // atomic per state from the even-cq lane of each pair
                const bool hi16 = (cq & 4) != 0, hi8 = (cq & 2) != 0;
                float k0 = hi16 ? dC[2] : dC[0], k1 = hi16 ? dC[3] : dC[1];
                k0 += __shfl_xor_sync(0xffffffffu, hi16 ? dC[0] : dC[2], 16);
                k1 += __shfl_xor_sync(0xffffffffu, hi16 ? dC[1] : dC[3], 16);
                float k = hi8 ? k1 : k0;
                k += __shfl_xor_sync(0xffffffffu, hi8 ? k0 : k1, 8);
                k += __shfl_xor_sync(0xffffffffu, k, 4);
                const int nn = n0 + (hi16 ? 2 : 0) + (hi8 ? 1 : 0);
                if ((cq & 1) == 0 && nn < a.N) atomicAdd(a.accBC + pix * 48 + 32 + nn, k);
            }

            if (a.y != nullptr) {
                const float ysum = reduce_states(yacc[0], yacc[1], yacc[2], yacc[3], nq);
                const int ch = g * kGroup + lane;
                if (ch < a.E) store1(static_cast<io_t*>(a.y), pix * a.E + ch, fmaf(sel4(cur.x, nq), D_own, ysum));
            }
        }
        cp_async_wait_all();
        __syncthreads();
    }
}

}  // namespace m2d
