// Shared device helpers and the launch plan for the sm_100a wavefront-scan kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "m2d_scan.h"

namespace m2d {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kGroup = 32;      // channels owned by one warp (8 lanes x 4 channels)
constexpr int kMaxN = 16;       // states owned by one warp   (4 lanes x 4 states)
constexpr int kSlotF4 = 128;    // float4 per (cell, warp) state record: 4 quads x 32 lanes

// Thread layout inside a warp.  A warp owns 32 channels x 16 states of one pixel; lane = (cq, nq)
// owns the 4x4 block channels [4cq, 4cq+4) x states [4nq, 4nq+4).  Sums over states finish with a
// 2-step exchange across the 4 nq lanes, sums over channels with a 3-step exchange across cq.

__device__ __forceinline__ float ex2(float v) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Release / acquire accesses to a progress counter in global memory shared by CTAs of one launch.
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Predicated forms (no branch, no reconvergence point): the copy / store happens iff `on`.
__device__ __forceinline__ void cp_async16_if(bool on, unsigned smem_addr, const void* gmem) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p cp.async.cg.shared.global [%0], [%1], 16;\n\t}"
                 ::"r"(smem_addr), "l"(gmem), "r"((int)on) : "memory");
}
__device__ __forceinline__ void cp_async8_if(bool on, unsigned smem_addr, const void* gmem) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p cp.async.ca.shared.global [%0], [%1], 8;\n\t}"
                 ::"r"(smem_addr), "l"(gmem), "r"((int)on) : "memory");
}
__device__ __forceinline__ void stcg_if(bool on, float4* p, const float4& v) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t@p st.global.cg.v4.f32 [%0], {%1, %2, %3, %4};\n\t}"
                 ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"((int)on) : "memory");
}
// Unpredicated forms, for call sites that branch on a loop-invariant condition themselves.
__device__ __forceinline__ void cp_async16(unsigned smem_addr, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async8(unsigned smem_addr, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_addr), "l"(gmem) : "memory");
}
// A 2 KiB (four 16-byte pieces per lane, 512 bytes apart) or 1 KiB (two pieces) block.
__device__ __forceinline__ void cp_async_block(unsigned smem_addr, const void* gmem, bool half) {
    if (half) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n\tcp.async.cg.shared.global [%0+512], [%1+512], 16;"
                     ::"r"(smem_addr), "l"(gmem) : "memory");
    } else {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n\tcp.async.cg.shared.global [%0+512], [%1+512], 16;\n\t"
                     "cp.async.cg.shared.global [%0+1024], [%1+1024], 16;\n\tcp.async.cg.shared.global [%0+1536], [%1+1536], 16;"
                     ::"r"(smem_addr), "l"(gmem) : "memory");
    }
}
__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

// Four 16-byte copies under one predicate: a 2 KiB (cell, warp) block, 512 bytes apart on both sides.
__device__ __forceinline__ void cp_async16x4_if(bool on, unsigned smem_addr, const void* gmem) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t"
        "@p cp.async.cg.shared.global [%0], [%1], 16;\n\t"
        "@p cp.async.cg.shared.global [%0+512], [%1+512], 16;\n\t"
        "@p cp.async.cg.shared.global [%0+1024], [%1+1024], 16;\n\t"
        "@p cp.async.cg.shared.global [%0+1536], [%1+1536], 16;\n\t}"
        ::"r"(smem_addr), "l"(gmem), "r"((int)on) : "memory");
}
// Two 16-byte copies under one predicate: a 1 KiB (cell, warp) block of bf16 states.
__device__ __forceinline__ void cp_async16x2_if(bool on, unsigned smem_addr, const void* gmem) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t"
        "@p cp.async.cg.shared.global [%0], [%1], 16;\n\t"
        "@p cp.async.cg.shared.global [%0+512], [%1+512], 16;\n\t}"
        ::"r"(smem_addr), "l"(gmem), "r"((int)on) : "memory");
}
__device__ __forceinline__ unsigned pack_bf16x2(float lo, float hi) {
    unsigned r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// Four 16-byte stores (one 2 KiB block) under one predicate.
__device__ __forceinline__ void stcg4_if(bool on, float4* p, const float4& v0, const float4& v1, const float4& v2, const float4& v3) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %17, 0;\n\t"
        "@p st.global.cg.v4.f32 [%0], {%1, %2, %3, %4};\n\t"
        "@p st.global.cg.v4.f32 [%0+512], {%5, %6, %7, %8};\n\t"
        "@p st.global.cg.v4.f32 [%0+1024], {%9, %10, %11, %12};\n\t"
        "@p st.global.cg.v4.f32 [%0+1536], {%13, %14, %15, %16};\n\t}"
        ::"l"(p), "f"(v0.x), "f"(v0.y), "f"(v0.z), "f"(v0.w), "f"(v1.x), "f"(v1.y), "f"(v1.z), "f"(v1.w),
          "f"(v2.x), "f"(v2.y), "f"(v2.z), "f"(v2.w), "f"(v3.x), "f"(v3.y), "f"(v3.z), "f"(v3.w), "r"((int)on) : "memory");
}

// ---- input staging in shared memory ------------------------------------------------------------
// Per warp and parity: 44 slots of 16 bytes: x[8] dT[8] dL[8] gy[8] (one slot per 4-channel block)
// then BT[4] BL[4] C[4] (one slot per 4-state block).  A slot holds four elements of the I/O type
// (fp32: 16 bytes, bf16: the first 8 bytes).
constexpr int kStageSlots = 44;
constexpr int kStageBytes = kStageSlots * 16;   // per parity

// Asynchronous copy of four consecutive elements into a slot (vector path), or a guarded scalar
// copy with zero fill (ragged path).
template <bool VEC>
__device__ __forceinline__ void stage4(bool on, char* slot, const float* __restrict__ p, int off, int nvalid) {
    if (VEC) { cp_async16_if(on, smem_u32(slot), p + off); return; }
    if (on) {
        float* d = reinterpret_cast<float*>(slot);
#pragma unroll
        for (int k = 0; k < 4; ++k) d[k] = (k < nvalid) ? __ldg(p + off + k) : 0.f;
    }
}
template <bool VEC>
__device__ __forceinline__ void stage4(bool on, char* slot, const __nv_bfloat16* __restrict__ p, int off, int nvalid) {
    if (VEC) { cp_async8_if(on, smem_u32(slot), p + off); return; }
    if (on) {
        unsigned short* d = reinterpret_cast<unsigned short*>(slot);
        const unsigned short* q = reinterpret_cast<const unsigned short*>(p) + off;
#pragma unroll
        for (int k = 0; k < 4; ++k) d[k] = (k < nvalid) ? __ldg(q + k) : (unsigned short)0;
    }
}
// Vector-path staging of one cell: every distinct piece of the seven input tensors is copied by
// exactly one lane, with two instructions per warp.  Lanes 0..31 copy the per-channel tensors
// (tensor = lane >> 3 of x, dT, dL, gy; piece = lane & 7, i.e. four channels); lanes 0..11 copy the
// per-state tensors (tensor = lane >> 2 of BT, BL, C; piece = lane & 3).  The slot order of the
// stage (x[8] dT[8] dL[8] gy[8] BT[4] BL[4] C[4]) makes the destination slot equal to the lane
// (+32 for the second copy).  Pieces beyond E or N are never copied: their slots stay zero.
template <typename io_t>
struct LaneCopy {
    const char* cbase;
    const char* bbase;
    int bpitch;
    bool c_on, b_on;
    __device__ __forceinline__ void init(const void* x, const void* dT, const void* dL, const void* gy, const void* BT,
                                         const void* BL, const void* C, int pBT, int pBL, int pC, int E, int N, int g,
                                         int lane, bool with_gy) {
        const int t = lane >> 3, piece = lane & 7;
        const void* cp = t == 0 ? x : (t == 1 ? dT : (t == 2 ? dL : gy));
        const int ch = g * kGroup + piece * 4;
        c_on = (ch < E) && (t < 3 || with_gy);
        cbase = static_cast<const char*>(cp) + (size_t)ch * sizeof(io_t);
        const int tb = lane >> 2, pb = lane & 3;
        const void* bp = tb == 0 ? BT : (tb == 1 ? BL : C);
        bpitch = tb == 0 ? pBT : (tb == 1 ? pBL : pC);
        b_on = (lane < 12) && (pb * 4 < N);
        bbase = static_cast<const char*>(bp) + (size_t)(pb * 4) * sizeof(io_t);
    }
    // Same as issue() below with ordinary branches on the two lane-invariant conditions (the
    // compiler keeps them as predicates across a loop instead of re-deriving them per copy).
    __device__ __forceinline__ void issue_plain(unsigned stage_addr, int lane, int pix, int E) const {
        const char* src_c = cbase + (size_t)(pix * E) * sizeof(io_t);
        const char* src_b = bbase + (size_t)(pix * bpitch) * sizeof(io_t);
        if (sizeof(io_t) == 4) {
            if (c_on) cp_async16(stage_addr + lane * 16, src_c);
            if (b_on) cp_async16(stage_addr + (32 + lane) * 16, src_b);
        } else {
            if (c_on) cp_async8(stage_addr + lane * 16, src_c);
            if (b_on) cp_async8(stage_addr + (32 + lane) * 16, src_b);
        }
    }
    // stage_addr: shared-space address of the stage (this parity); pix: flat pixel index.
    __device__ __forceinline__ void issue(unsigned stage_addr, int lane, int pix, int E) const {
        const char* src_c = cbase + (size_t)(pix * E) * sizeof(io_t);
        const char* src_b = bbase + (size_t)(pix * bpitch) * sizeof(io_t);
        if (sizeof(io_t) == 4) {
            cp_async16_if(c_on, stage_addr + lane * 16, src_c);
            cp_async16_if(b_on, stage_addr + (32 + lane) * 16, src_b);
        } else {
            cp_async8_if(c_on, stage_addr + lane * 16, src_c);
            cp_async8_if(b_on, stage_addr + (32 + lane) * 16, src_b);
        }
    }
};

// Read a staged slot back as four floats.
template <typename io_t> __device__ __forceinline__ float4 unstage4(const char* slot);
template <> __device__ __forceinline__ float4 unstage4<float>(const char* slot) {
    return *reinterpret_cast<const float4*>(slot);
}
template <> __device__ __forceinline__ float4 unstage4<__nv_bfloat16>(const char* slot) {
    const uint2 u = *reinterpret_cast<const uint2*>(slot);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                       __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}

// ---- scalar element loads / stores --------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(unsigned short b) { return __uint_as_float(static_cast<unsigned>(b) << 16); }
__device__ __forceinline__ float load1(const float* __restrict__ p, long long off) { return __ldg(p + off); }
__device__ __forceinline__ float load1(const __nv_bfloat16* __restrict__ p, long long off) {
    return bf16_bits_to_float(__ldg(reinterpret_cast<const unsigned short*>(p) + off));
}
__device__ __forceinline__ void store1(float* p, long long off, float v) { p[off] = v; }
__device__ __forceinline__ void store1(__nv_bfloat16* p, long long off, float v) { p[off] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float sel4(const float4& v, int k) {
    return k == 0 ? v.x : (k == 1 ? v.y : (k == 2 ? v.z : v.w));
}

// Sum four per-channel partials over the 4 nq lanes.  On return lane nq holds the total of
// channel index nq of its 4-channel block (so lane l of the warp holds channel l of the group).
__device__ __forceinline__ float reduce_states(float v0, float v1, float v2, float v3, int nq) {
    const bool hi2 = (nq & 2) != 0;
    float k0 = hi2 ? v2 : v0, k1 = hi2 ? v3 : v1;
    const float s0 = hi2 ? v0 : v2, s1 = hi2 ? v1 : v3;
    k0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    k1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    const bool hi1 = (nq & 1) != 0;
    const float k = hi1 ? k1 : k0, s = hi1 ? k0 : k1;
    return k + __shfl_xor_sync(0xffffffffu, s, 1);
}

// The per-(channel,state) parameters A*log2(e) of the CTA's 32 channels live in shared memory
// behind everything else: [AT | AL][4 channels][32 lanes] float4 (4 KiB), read block by block.
constexpr int kParamF4 = 2 * 4 * 32;

// Shared memory of the nested-loop sweeps, in this order (the parameters follow):
//   pull    3 x 2 KiB           ring blocks for the warp that leads a band
//   slots   warps x 2 x 2 KiB   hand-off: warp (rank) k writes slot k, the next one reads it
//   stage   warps x 3 x kStageBytes
//   harea   backward only: (warps + 1) x 3 x 2 KiB state blocks for the adjoint sweep
__host__ __device__ inline size_t rows_handoff_f4(int warps) { return (size_t)(3 + 2 * warps) * kSlotF4; }
__host__ __device__ inline size_t rows_fwd_smem_bytes(int warps) {
    return rows_handoff_f4(warps) * sizeof(float4) + (size_t)warps * 3 * kStageBytes;
}
__host__ __device__ inline size_t rows_bwd_smem_bytes(int warps) {
    return rows_fwd_smem_bytes(warps) + (size_t)(warps + 1) * 3 * kSlotF4 * sizeof(float4);
}

// Host-side launch plan shared by the workspace queries and the launches.
struct Plan {
    int groups;        // ceil(E / 32)
    int warps;         // row-warps per CTA
    int Rb;            // rows per band (<= warps)
    int nbands;        // ceil(H / Rb)
    int grid_x;        // image chains per channel group; chain k walks images k, k + grid_x, ...
    int cb;            // cells per step and warp (forward only)
    int chain;         // CTAs per chain (> 1 when there are far fewer images than SMs)
    bool rows;         // batch mode with the nested-loop kernel (its own shared-memory layout)
    size_t smem;       // dynamic shared memory per CTA
    size_t scratch;    // workspace bytes
};

}  // namespace m2d
