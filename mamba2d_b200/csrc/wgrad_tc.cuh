// Weight gradient of the x projection on the 5th-generation tensor cores (bf16 operands, fp32
// accumulation in tensor memory):   d_Wx[k][e] = sum_p d_proj[p][k] * x[p][e].
//
// As a GEMM this is D[M][N] += A[M][Kp] * B[Kp][N] with M = the 2R+3N projection columns (padded to
// 128), N = a tile of up to 256 channels and the reduction dimension Kp = pixels.  Both operands lie
// in memory with the reduction index as the row: they are "MN-major", and a TMA box of 64 pixels x 64
// elements (128 bytes per row, 128-byte swizzle) lands in shared memory in exactly the canonical
// layout tcgen05.mma reads for that case, so nothing is transposed or repacked.  Columns beyond the
// tensors' extents are filled with zeros by the TMA unit.
//
// One CTA per SM and channel tile walks a contiguous range of 64-pixel blocks:
//   warp 0, one lane:  TMA producer (ring of kStages stages, full / empty mbarriers)
//   warp 1, one lane:  issues four tcgen05.mma (K = 16 pixels each) per stage, then tcgen05.commit
//                      onto the stage's empty barrier
//   all four warps:    epilogue, tcgen05.ld of the 128 x N accumulator, rows < K stored as this CTA's
//                      partial result; the existing finalize kernel sums the partials.
// Every wait is bounded; a wait that gives up sets the status word, poisons this CTA's partial result
// with NaN (so nothing wrong is returned silently) and the kernel still frees its tensor memory.
#pragma once

#include <cuda.h>   // CUtensorMap and its enums; the encoder itself is fetched through the runtime
#include <cuda_runtime.h>
#include <stdint.h>

namespace m2d {

constexpr int kTcPix = 64;                    // pixels per stage
constexpr int kTcBlockBytes = kTcPix * 128;   // one 64-pixel x 64-element bf16 block: 8 KiB
constexpr int kTcWaitLimit = 1 << 22;

struct TcArgs {
    int K, E;               // rows (projection columns) and columns (channels) of the result
    int nbk;                // 64-channel blocks per CTA (N = 64 * nbk)
    int stages;
    int total_blocks;       // 64-pixel blocks in all
    int blocks_per_cta;
    float* partials;        // [gridDim.x][K][E]
    int* status;
};

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");   // suspends for at most ~1 us per try
    return ok != 0;
}
// Bounded wait; returns false (and raises *abort) when it gives up or another wait already has.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort) {
    for (int n = 0; n < kTcWaitLimit; ++n) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort) return false;
    }
    *abort = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 32 consecutive fp32 columns of this thread's accumulator row (lane of tensor memory)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of an MN-major bf16 operand in the 128-byte-swizzle layout: rows of
// 128 bytes (64 elements along M or N), eight rows per 1 KiB swizzle atom along the reduction
// dimension ("stride" offset 1 KiB), the next 64 elements along M / N one block (8 KiB) further
// ("leading" offset).  Bit layout: start address >> 4 in [0,14), leading offset >> 4 in [16,30), stride
// offset >> 4 in [32,46), descriptor version 1 in [46,48), swizzle mode 2 (128 bytes) in [61,64).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)(kTcBlockBytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulator (bits [4,6) = 1), bf16 A and B (bits [7,10) and [10,13) = 1),
// A and B MN-major (bits 15, 16), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ inline uint32_t tc_instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}

__global__ void __launch_bounds__(128, 1) xproj_wgrad_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_b, const TcArgs a) {
    extern __shared__ uint8_t tc_smem_raw[];
    __shared__ uint64_t bars[2 * 4 + 1];   // full[stages], empty[stages], done
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem0 = (static_cast<uint32_t>(__cvta_generic_to_shared(tc_smem_raw)) + 1023u) & ~1023u;
    const int stage_bytes = (2 + a.nbk) * kTcBlockBytes;
    const uint32_t bar0 = static_cast<uint32_t>(__cvta_generic_to_shared(bars));
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (4 + s); };
    const uint32_t done_bar = bar0 + 8u * 8;
    const int n_cols = 64 * a.nbk;
    const uint32_t tmem_cols = n_cols <= 64 ? 64u : (n_cols <= 128 ? 128u : 256u);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(done_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(static_cast<uint32_t>(__cvta_generic_to_shared(&tmem_base_slot)), tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = tmem_base_slot;
    volatile int* abort = &abort_flag;

    const int kb0 = blockIdx.x * a.blocks_per_cta;
    const int kb1 = min(a.total_blocks, kb0 + a.blocks_per_cta);
    const int nblocks = kb1 - kb0;           // >= 1 by construction of the grid
    const int e_tile = blockIdx.y * n_cols;  // first channel of this CTA's tile

    if (warp == 0 && lane == 0) {
        // ---- producer ----
        int armed = 0;
        for (int it = 0; it < nblocks; ++it) {
            const int s = it % a.stages;
            const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
            if (!mbar_wait(empty_bar(s), ph ^ 1u, abort)) break;
            const uint32_t dst = smem0 + (uint32_t)s * stage_bytes;
            mbar_expect_tx(full_bar(s), (uint32_t)stage_bytes);
            const int p0 = (kb0 + it) * kTcPix;
            tma_load_2d(dst, &map_a, 0, p0, full_bar(s));
            tma_load_2d(dst + kTcBlockBytes, &map_a, 64, p0, full_bar(s));
            for (int b = 0; b < a.nbk; ++b) tma_load_2d(dst + (2 + b) * kTcBlockBytes, &map_b, e_tile + 64 * b, p0, full_bar(s));
            armed = it + 1;
        }
        if (*abort) {
            // let the copies already requested land before the CTA leaves (bounded)
            for (int it = max(0, armed - a.stages); it < armed; ++it) {
                const int s = it % a.stages;
                const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
                for (int n = 0; n < kTcWaitLimit && !mbar_try_wait(full_bar(s), ph); ++n) {}
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const uint32_t idesc = tc_instr_desc(n_cols);
        bool ok = true;
        for (int it = 0; it < nblocks && ok; ++it) {
            const int s = it % a.stages;
            const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
            ok = mbar_wait(full_bar(s), ph, abort);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem0 + (uint32_t)s * stage_bytes, sb = sa + 2 * kTcBlockBytes;
#pragma unroll
            for (int kk = 0; kk < kTcPix / 16; ++kk) {
                // 16 pixels = 16 rows of 128 bytes further along the reduction dimension
                umma_bf16(tmem_d, tc_smem_desc(sa + kk * 2048), tc_smem_desc(sb + kk * 2048), idesc, (it > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(empty_bar(s));      // arrives when these MMAs have finished reading the stage
        }
        if (ok) umma_commit(done_bar);      // arrives when every MMA above has completed
    }

    // ---- epilogue: thread (warp, lane) owns accumulator row 32*warp + lane ----
    // (the decision is taken CTA-wide: tcgen05.ld below must be executed by whole warps together)
    const bool have = __syncthreads_and(mbar_wait(done_bar, 0u, abort) ? 1 : 0) != 0;
    tc_fence_after();
    const int row = warp * 32 + lane;
    float* out = a.partials + ((size_t)blockIdx.x * a.K + row) * a.E;
    const float poison = __int_as_float(0x7fc00000);
    for (int c0 = 0; c0 < n_cols; c0 += 32) {
        float v[32];
        if (have) {
            tmem_ld32(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = poison;
        }
        if (row < a.K) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const int e = e_tile + c0 + i;
                if (e < a.E) *reinterpret_cast<float4*>(out + e) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            }
        }
    }
    if (!have && threadIdx.x == 0) atomicExch(a.status, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_d, tmem_cols);
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*tc_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline tc_encode_fn tc_encoder() {
    static tc_encode_fn fn = []() -> tc_encode_fn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<tc_encode_fn>(p);
    }();
    return fn;
}

// (rows, cols) bf16 matrix with a row pitch in elements; box = 64 columns x 64 rows, 128-byte swizzle
inline bool tc_make_map(CUtensorMap* map, const void* base, long long rows, int cols, long long pitch) {
    tc_encode_fn enc = tc_encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)kTcPix};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct TcPlan {
    bool ok;
    int nbk, ny, stages, grid_x, blocks_per_cta, total_blocks;
    size_t smem;
};

// Can the tensor-core kernel take this problem, and on which grid?  `max_slabs` partial results fit the workspace.
inline TcPlan tc_plan(long long P, int E, int K, long long pitch, const void* x, const void* d_proj, int max_slabs) {
    TcPlan t{};
    t.ok = false;
    if (const char* e = getenv("M2D_WGRAD_TC")) { if (e[0] == '0') return t; }
    if (K > 128 || E % 8 != 0 || pitch % 8 != 0) return t;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(d_proj) & 15)) return t;
    if (!tc_encoder()) return t;
    const int blocks64 = (E + 63) / 64;
    t.ny = (blocks64 + 3) / 4;
    t.nbk = (blocks64 + t.ny - 1) / t.ny;
    t.stages = t.nbk <= 2 ? 4 : 3;
    t.total_blocks = (int)((P + kTcPix - 1) / kTcPix);
    int gx = sm_count() / t.ny;
    if (gx > max_slabs) gx = max_slabs;
    if (gx > t.total_blocks) gx = t.total_blocks;
    if (gx < 1) return t;
    t.blocks_per_cta = (t.total_blocks + gx - 1) / gx;
    t.grid_x = (t.total_blocks + t.blocks_per_cta - 1) / t.blocks_per_cta;   // no CTA without a block
    t.smem = (size_t)t.stages * (2 + t.nbk) * kTcBlockBytes + 1024;
    t.ok = true;
    return t;
}

}  // namespace m2d
