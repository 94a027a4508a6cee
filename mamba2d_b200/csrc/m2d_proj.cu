// Fused parameter projections around the wavefront scan (C ABI in m2d_proj.h).
//
//   dtproj_fwd   delta = softplus(r @ W^T + b) for both directions, one pass over (P,E)
//   dtproj_bwd   softplus', weight / bias gradients and the gradient of r, one pass over (P,E)
//   xproj_wgrad  d_Wx = d_proj^T @ x, a reduction over all pixels split across the GPU
//
// The reference does this in PyTorch (proj_params, models/kernels/wavefront_cuda.py:63-95, and
// its autograd backward).  All three kernels are HBM-streaming: a thread owns one channel, lanes of
// a warp own consecutive channels of one pixel (coalesced rows), the per-pixel rank-R vectors sit
// in shared memory, and the big reductions over pixels stay in registers until the end of the
// kernel, when each CTA writes one partial result that a small second kernel sums.
#include "m2d_proj.h"

#include "common.cuh"
#include "plan.cuh"
#include "wgrad_tc.cuh"

namespace m2d {

constexpr int kProjIters = 8;          // pixels per thread per tile

struct ProjPlan {
    int EB, PS, threads, TP, RB, gx;
    int ntiles;
    // x-projection weight gradient
    int tilesK, tilesE, slabs, rows_per_slab, K;
    size_t dt_partials, wg_partials;   // bytes
};

struct ProjArgs {
    int P, pitch, ntiles;              // every element index fits 31 bits (checked on the host)
    int E, R, EB, PS, TP;
    int wide16;                        // bf16 backward: rows and pointers allow 16-byte copies
    const void *proj, *WT, *WL, *bT, *bL;
    void *dT, *dL;
    const void *g_dT, *g_dL;
    void* d_proj;
    float* partials;                   // [dir][cta][RB+1][EB]
};

struct WgArgs {
    int P, pitch;
    int E, K, rows_per_slab;
    const void *x, *d_proj;
    float* partials;                   // [slab][K][E]
};

static int check_proj(const m2d_proj_desc* d) {
    if (!d) return M2D_ERR_NULL;
    if (d->struct_bytes != sizeof(m2d_proj_desc)) return M2D_ERR_ABI;
    if (d->dtype != M2D_F32 && d->dtype != M2D_BF16) return M2D_ERR_DTYPE;
    if (d->P < 1 || d->E < 1 || d->R < 1 || d->N < 1) return M2D_ERR_SHAPE;
    if (d->E > M2D_PROJ_MAX_E || d->R > M2D_PROJ_MAX_R) return M2D_ERR_TOO_LARGE;
    if (d->proj_pitch < 2ll * d->R + 3ll * d->N) return M2D_ERR_PITCH;
    {
        // the kernels stage 8 pixels x RB ranks per EB channels with two values per thread at most
        const int EB = (d->E + 31) / 32 * 32;
        const int RB = d->R <= 4 ? 4 : d->R <= 8 ? 8 : d->R <= 16 ? 16 : d->R <= 32 ? 32 : 64;
        if (4 * RB > EB) return M2D_ERR_SHAPE;
    }
    const long long widest = d->proj_pitch > d->E ? d->proj_pitch : d->E;
    // the kernels use 31-bit element indices, as the scan does (with room for the look-ahead of one grid of tiles)
    if (d->P * widest >= (1ll << 31) - (1ll << 26)) return M2D_ERR_TOO_LARGE;
    return M2D_OK;
}

static ProjPlan plan_proj(const m2d_proj_desc* d) {
    ProjPlan p;
    const int sms = sm_count();
    p.EB = (d->E + 31) / 32 * 32;
    p.PS = p.EB >= 256 ? 1 : 256 / p.EB;
    p.threads = p.EB * p.PS;
    p.TP = kProjIters * p.PS;
    p.RB = d->R <= 4 ? 4 : d->R <= 8 ? 8 : d->R <= 16 ? 16 : d->R <= 32 ? 32 : 64;
    p.ntiles = (int)((d->P + p.TP - 1) / p.TP);
    p.gx = p.ntiles < 2 * sms ? p.ntiles : 2 * sms;
    p.dt_partials = (size_t)2 * p.gx * (p.RB + 1) * p.EB * sizeof(float);
    p.K = 2 * d->R + 3 * d->N;
    p.tilesK = (p.K + 63) / 64;
    p.tilesE = (d->E + 63) / 64;
    const int tiles = p.tilesK * p.tilesE;
    long long slabs = (4ll * sms + tiles - 1) / tiles;
    const long long max_slabs = (d->P + 63) / 64;
    if (slabs > max_slabs) slabs = max_slabs;
    if (slabs < 1) slabs = 1;
    p.rows_per_slab = (int)(((d->P + slabs - 1) / slabs + 31) / 32 * 32);
    p.slabs = (int)((d->P + p.rows_per_slab - 1) / p.rows_per_slab);
    p.wg_partials = align256((size_t)p.slabs * p.K * d->E * sizeof(float)) + 256;   // + the status word of the tensor-core kernel
    return p;
}

// softplus with the reference's threshold of 20 (torch.nn.functional.softplus defaults)
// log1p(t) for t in (0, 1] as 2*atanh(t / (2 + t)): the argument stays below 1/3, where seven terms of
// the series are exact to fp32 rounding (next term 2 s^15 / 15 < 1e-8 of the result); half the
// instructions of log1pf, which was a third of the forward kernel.
__device__ __forceinline__ float log1p_unit(float t) {
    const float s = __fdividef(t, 2.f + t), s2 = s * s;
    float p = 1.f / 13.f;
    p = fmaf(p, s2, 1.f / 11.f);
    p = fmaf(p, s2, 1.f / 9.f);
    p = fmaf(p, s2, 1.f / 7.f);
    p = fmaf(p, s2, 1.f / 5.f);
    p = fmaf(p, s2, 1.f / 3.f);
    p = fmaf(p, s2, 1.f);
    return 2.f * s * p;
}
// softplus(z) = max(z, 0) + log1p(exp(-|z|)); past the reference's threshold of 20 the second term is
// below half an ulp of z, so the threshold of torch.nn.functional.softplus needs no branch
__device__ __forceinline__ float softplus_f(float z) {
    // exp(-|z|) = 2^(a + e): a is the rounded product with log2(e); e collects what that rounding and
    // the rounding of the constant lost (without it the error grows with |z|: 3e-6 at |z| = 60)
    const float m = -fabsf(z);
    const float a = m * kLog2e;
    const float e = fmaf(m, kLog2e, -a) + m * 1.92596299e-8f;
    const float t = ex2(a) * fmaf(e, kLn2, 1.f);
    return fmaxf(z, 0.f) + log1p_unit(t);
}

// ------------------------------------------------------------------------------------------------
// delta = softplus(r @ W^T + b).  grid (ctas, 2 directions); block = EB channels x PS pixels.
// ------------------------------------------------------------------------------------------------
template <typename io_t, int RB, int MAXT>
__global__ void __launch_bounds__(MAXT) dtproj_fwd_kernel(const ProjArgs a) {
    extern __shared__ float sm[];                  // rs[TP][RB]: this tile's rank-R rows, zero padded
    const int dir = blockIdx.y;
    const int te = threadIdx.x % a.EB, ps = threadIdx.x / a.EB;
    const bool e_ok = te < a.E;
    const io_t* W = static_cast<const io_t*>(dir ? a.WL : a.WT);
    const io_t* bias = static_cast<const io_t*>(dir ? a.bL : a.bT);
    const io_t* proj = static_cast<const io_t*>(a.proj);
    io_t* out = static_cast<io_t*>(dir ? a.dL : a.dT);
    const int col0 = dir * a.R;

    float w[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) w[r] = (e_ok && r < a.R) ? load1(W, te * a.R + r) : 0.f;
    const float b = e_ok ? load1(bias, te) : 0.f;

    // The rank-R rows of the next tile are fetched into registers while this tile is computed
    // (TP*RB <= 2*blockDim is guaranteed by the host: two values per thread at most).
    const int tile_elems = a.TP * RB;
    auto fetch_rows = [&](int tile, float (&v)[2]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int idx = threadIdx.x + h * blockDim.x;
            const int pp = idx / RB, r = idx % RB;
            const int p = tile * a.TP + pp;
            v[h] = (idx < tile_elems && r < a.R && p < a.P && tile < a.ntiles) ? load1(proj, p * a.pitch + col0 + r) : 0.f;
        }
    };
    float nxt[2];
    fetch_rows(blockIdx.x, nxt);
    for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x) {
        const int p0 = tile * a.TP;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int idx = threadIdx.x + h * blockDim.x;
            if (idx < tile_elems) sm[idx] = nxt[h];
        }
        __syncthreads();
        fetch_rows(tile + gridDim.x, nxt);
        io_t* dst = out + (p0 + ps) * a.E + te;
        const int row_step = a.PS * a.E;
#pragma unroll
        for (int k = 0; k < kProjIters; ++k) {
            const int pp = k * a.PS + ps;
            const float4* rr = reinterpret_cast<const float4*>(sm + pp * RB);
            float z = b;
#pragma unroll
            for (int r4 = 0; r4 < RB / 4; ++r4) {
                const float4 v = rr[r4];
                z = fmaf(v.x, w[4 * r4], z);
                z = fmaf(v.y, w[4 * r4 + 1], z);
                z = fmaf(v.z, w[4 * r4 + 2], z);
                z = fmaf(v.w, w[4 * r4 + 3], z);
            }
            if (e_ok && p0 + pp < a.P) store1(dst, k * row_step, softplus_f(z));
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------------
// Backward of the dt projections.  A thread owns channel te of the pixels k*PS + ps (k = 0..7) of
// each tile: it forms s = g * softplus', keeps d_b and its row of d_W in registers, and parks s in a
// per-warp [8 pixels][32 channels] slab of shared memory.  The warp then re-reads the slab with the
// roles turned round -- a lane owns rank r (and a subset of the 8 pixels), holds W[e][r] of the
// warp's 32 channels in registers and sums over them -- which yields the warp's share of
// d_r = s @ W without any shuffle; the shares of the CTA's warps meet in shared memory.
// Shared memory: rs[TP][RB], drs[TP][RB], slab[warps][8][36] and two buffers of the tile's g and
// delta rows; the end-of-kernel reduction accS[RB+1][EB] reuses the same bytes.
// ------------------------------------------------------------------------------------------------
constexpr int kSlabStride = 36;        // 32 channels + 4: rows of a slab start in different banks
__device__ __forceinline__ float smem_value(const float* p) { return *p; }
__device__ __forceinline__ float smem_value(const __nv_bfloat16* p) { return bf16_bits_to_float(*reinterpret_cast<const unsigned short*>(p)); }

template <typename io_t, int RB, int MAXT>
__global__ void __launch_bounds__(MAXT) dtproj_bwd_kernel(const ProjArgs a) {
    extern __shared__ float sm[];
    float* accS = sm;                              // used after the tile loop only: overlays everything else
    float* rs = sm;
    float* drs = rs + a.TP * RB;
    float* slab = drs + a.TP * RB + (threadIdx.x >> 5) * (kProjIters * kSlabStride);
    io_t* tiles = reinterpret_cast<io_t*>(drs + a.TP * RB + (blockDim.x >> 5) * (kProjIters * kSlabStride));   // [2 buffers][g | delta][TP*E]
    const int dir = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const int te = threadIdx.x % a.EB, ps = threadIdx.x / a.EB;
    const bool e_ok = te < a.E;
    const io_t* W = static_cast<const io_t*>(dir ? a.WL : a.WT);
    const io_t* proj = static_cast<const io_t*>(a.proj);
    const io_t* delta = static_cast<const io_t*>(dir ? a.dL : a.dT);
    const io_t* g = static_cast<const io_t*>(dir ? a.g_dL : a.g_dT);
    io_t* d_proj = static_cast<io_t*>(a.d_proj);
    const int col0 = dir * a.R;

    // roles of the second phase: lane = (pl, rl): ranks rl + 32*h, pixels pl + PL*kk of the warp's 8
    constexpr int RL = RB > 32 ? 32 : RB;          // ranks handled side by side
    constexpr int PL = 32 / RL;                    // pixels handled side by side
    constexpr int KPL = kProjIters / PL;           // pixels per lane
    constexpr int NH = RB / RL;                    // rank halves per lane
    const int rl = lane % RL, pl = lane / RL;
    const int e_slice = te - lane;                 // first channel of this warp
    float wreg[NH][32];
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int e = 0; e < 32; ++e) {
            const int r = h * RL + rl, ch = e_slice + e;
            wreg[h][e] = (ch < a.E && r < a.R) ? load1(W, ch * a.R + r) : 0.f;
        }

    float acc[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) acc[r] = 0.f;
    float accb = 0.f;

    const int tile_elems = a.TP * RB;
    auto fetch_rows = [&](int tile, float (&v)[2]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int idx = threadIdx.x + h * blockDim.x;
            const int pp = idx / RB, r = idx % RB;
            const int p = tile * a.TP + pp;
            v[h] = (idx < tile_elems && r < a.R && p < a.P && tile < a.ntiles) ? load1(proj, p * a.pitch + col0 + r) : 0.f;
        }
    };
    // The tile's g and delta rows (TP consecutive pixels = one contiguous chunk of each tensor) are
    // copied to shared memory with cp.async, one tile ahead, in pieces of 4 elements.
    const int tile_chunk = a.TP * a.E;                       // elements per tensor per tile
    auto issue_inputs = [&](int tile, int buf) {
        io_t* dst_g = tiles + (size_t)(buf * 2) * tile_chunk;
        io_t* dst_d = dst_g + tile_chunk;
        const int base = tile * a.TP * a.E;
        // 16-byte pieces (4 fp32 or 8 bf16 elements, L2-only copies) where rows allow it and both
        // tensors are 16-byte aligned; 8-byte pieces for bf16 rows that are only a multiple of 4
        const bool wide = sizeof(io_t) == 4 || a.wide16;
        const int pe = wide ? 16 / (int)sizeof(io_t) : 4;
        for (int piece = threadIdx.x; piece * pe < tile_chunk; piece += blockDim.x) {
            const int off = piece * pe;
            const bool ok = tile < a.ntiles && tile * a.TP + off / a.E < a.P;
            if (wide) {
                cp_async16_if(ok, smem_u32(dst_g + off), g + base + off);
                cp_async16_if(ok, smem_u32(dst_d + off), delta + base + off);
                if (!ok) {
                    *reinterpret_cast<float4*>(dst_g + off) = make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4*>(dst_d + off) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            } else {
                cp_async8_if(ok, smem_u32(dst_g + off), g + base + off);
                cp_async8_if(ok, smem_u32(dst_d + off), delta + base + off);
                if (!ok) {
                    *reinterpret_cast<uint2*>(dst_g + off) = make_uint2(0u, 0u);
                    *reinterpret_cast<uint2*>(dst_d + off) = make_uint2(0u, 0u);
                }
            }
        }
    };
    float nxt[2];
    fetch_rows(blockIdx.x, nxt);
    issue_inputs(blockIdx.x, 0);
    int buf = 0;
    for (int tile = blockIdx.x; tile < a.ntiles; tile += gridDim.x, buf ^= 1) {
        const int p0 = tile * a.TP;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int idx = threadIdx.x + h * blockDim.x;
            if (idx < tile_elems) {
                rs[idx] = nxt[h];
                drs[idx] = 0.f;
            }
        }
        cp_async_wait_all();
        __syncthreads();
        fetch_rows(tile + gridDim.x, nxt);
        issue_inputs(tile + gridDim.x, buf ^ 1);      // next tile's copies fly while this one is reduced
        const io_t* cur_g = tiles + (size_t)(buf * 2) * tile_chunk + ps * a.E + te;
        const io_t* cur_d = cur_g + tile_chunk;
        float sv[kProjIters];
#pragma unroll
        for (int k = 0; k < kProjIters; ++k) {
            const float gk = e_ok ? smem_value(cur_g + k * a.PS * a.E) : 0.f;
            const float d = e_ok ? smem_value(cur_d + k * a.PS * a.E) : 0.f;
            // softplus'(z) = sigmoid(z) = 1 - exp(-softplus(z)); a short series where 1 - exp cancels
            const float series = d * (1.f - d * (0.5f - d * (1.f / 6.f - d * (1.f / 24.f - d * (1.f / 120.f)))));
            sv[k] = gk * (d < 0.1f ? series : 1.f - __expf(-d));
            slab[k * kSlabStride + lane] = sv[k];
            accb += sv[k];
        }
        __syncwarp();
        // d_W row of this channel: acc[r] += s * r_row[r]
#pragma unroll
        for (int k = 0; k < kProjIters; ++k) {
            const float4* rr = reinterpret_cast<const float4*>(rs + (k * a.PS + ps) * RB);
#pragma unroll
            for (int r4 = 0; r4 < RB / 4; ++r4) {
                const float4 q = rr[r4];
                acc[4 * r4] = fmaf(sv[k], q.x, acc[4 * r4]);
                acc[4 * r4 + 1] = fmaf(sv[k], q.y, acc[4 * r4 + 1]);
                acc[4 * r4 + 2] = fmaf(sv[k], q.z, acc[4 * r4 + 2]);
                acc[4 * r4 + 3] = fmaf(sv[k], q.w, acc[4 * r4 + 3]);
            }
        }
        // d_r of the warp's pixels over the warp's 32 channels
#pragma unroll
        for (int kk = 0; kk < KPL; ++kk) {
            const int k = pl + kk * PL;
            const float4* row = reinterpret_cast<const float4*>(slab + k * kSlabStride);
            float sum[NH];
#pragma unroll
            for (int h = 0; h < NH; ++h) sum[h] = 0.f;
#pragma unroll
            for (int e4 = 0; e4 < 8; ++e4) {
                const float4 q = row[e4];
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    sum[h] = fmaf(q.x, wreg[h][4 * e4], sum[h]);
                    sum[h] = fmaf(q.y, wreg[h][4 * e4 + 1], sum[h]);
                    sum[h] = fmaf(q.z, wreg[h][4 * e4 + 2], sum[h]);
                    sum[h] = fmaf(q.w, wreg[h][4 * e4 + 3], sum[h]);
                }
            }
#pragma unroll
            for (int h = 0; h < NH; ++h) atomicAdd(&drs[(k * a.PS + ps) * RB + h * RL + rl], sum[h]);
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int idx = threadIdx.x + h * blockDim.x;
            const int pp = idx / RB, r = idx % RB;
            if (idx < tile_elems && r < a.R && p0 + pp < a.P) store1(d_proj, (p0 + pp) * a.pitch + col0 + r, drs[idx]);
        }
        __syncthreads();
    }

    // CTA-level sum over the PS pixel rows of the block, then one partial per CTA
    cp_async_wait_all();
    __syncthreads();
    for (int idx = threadIdx.x; idx < (RB + 1) * a.EB; idx += blockDim.x) accS[idx] = 0.f;
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RB; ++r) atomicAdd(&accS[r * a.EB + te], acc[r]);
    atomicAdd(&accS[RB * a.EB + te], accb);
    __syncthreads();
    float* part = a.partials + ((size_t)dir * gridDim.x + blockIdx.x) * (RB + 1) * a.EB;
    for (int idx = threadIdx.x; idx < (RB + 1) * a.EB; idx += blockDim.x) part[idx] = accS[idx];
}

// d_W[e][r] (r < R) and d_b[e] (r == RB) = sum over CTAs of the partials.  Block (32, 8): 32
// neighbouring results, the CTAs dealt round-robin to the 8 rows of the block.
template <typename io_t>
__global__ void dtproj_bwd_finalize(const float* __restrict__ partials, int ctas, int RB, int EB, int E, int R,
                                    io_t* d_WT, io_t* d_WL, io_t* d_bT, io_t* d_bL) {
    __shared__ float red[8][33];
    const int n = 2 * (RB + 1) * EB;
    const int idx = blockIdx.x * 32 + threadIdx.x;
    const size_t step = (size_t)(RB + 1) * EB;
    int dir = 0, r = 0, e = 0;
    float s = 0.f;
    if (idx < n) {
        dir = idx / (int)step;
        const int rem = idx % (int)step;
        r = rem / EB;
        e = rem % EB;
        const float* src = partials + (size_t)dir * ctas * step + rem;
#pragma unroll 4
        for (int c = threadIdx.y; c < ctas; c += 8) s += src[(size_t)c * step];
    }
    red[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && idx < n && e < E && (r < R || r == RB)) {
        float t = 0.f;
#pragma unroll
        for (int y = 0; y < 8; ++y) t += red[y][threadIdx.x];
        if (r == RB) store1(dir ? d_bL : d_bT, e, t);
        else store1(dir ? d_WL : d_WT, (long long)e * R + r, t);
    }
}

// ------------------------------------------------------------------------------------------------
// d_Wx[k][e] = sum_p d_proj[p][k] * x[p][e].  grid (slabs, tilesE, tilesK); a CTA of 256 threads
// computes a 64x64 tile of the result over its slab of pixels, 32 pixels per shared-memory stage,
// each thread a 4x4 block.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float4 load4g(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4g(const __nv_bfloat16* p) {
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                       __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}

template <typename io_t>
__global__ void __launch_bounds__(256) xproj_wgrad_kernel(const WgArgs a) {
    __shared__ float4 As[2][32][16];
    __shared__ float4 Bs[2][32][16];
    const io_t* A = static_cast<const io_t*>(a.d_proj);
    const io_t* B = static_cast<const io_t*>(a.x);
    const int tid = threadIdx.x, te = tid & 15, tk = tid >> 4;
    const int e0 = blockIdx.y * 64, k0 = blockIdx.z * 64;
    const int row0 = blockIdx.x * a.rows_per_slab;
    int row_end = row0 + a.rows_per_slab;
    if (row_end > a.P) row_end = a.P;
    const int chunks = (int)((row_end - row0 + 31) / 32);

    // each thread stages two float4 of A and two of B per chunk: rows lr and lr + 16, column quad lc
    const int lr = tid >> 4, lc = tid & 15;
    auto fetch = [&](int chunk, float4 (&ra)[2], float4 (&rb)[2]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = row0 + chunk * 32 + lr + 16 * h;
            const bool row_ok = p < row_end;
            const int ka = k0 + lc * 4, eb = e0 + lc * 4;
            ra[h] = make_float4(0.f, 0.f, 0.f, 0.f);
            rb[h] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row_ok && ka + 4 <= a.K) {
                ra[h] = load4g(A + p * a.pitch + ka);
            } else if (row_ok && ka < a.K) {       // ragged last quad of the K columns
                float t[4] = {0.f, 0.f, 0.f, 0.f};
                for (int i = 0; i < 4 && ka + i < a.K; ++i) t[i] = load1(A, p * a.pitch + ka + i);
                ra[h] = make_float4(t[0], t[1], t[2], t[3]);
            }
            if (row_ok && eb < a.E) rb[h] = load4g(B + p * a.E + eb);
        }
    };

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    float4 ra[2], rb[2];
    if (chunks > 0) {
        fetch(0, ra, rb);
        As[0][lr][lc] = ra[0]; As[0][lr + 16][lc] = ra[1];
        Bs[0][lr][lc] = rb[0]; Bs[0][lr + 16][lc] = rb[1];
    }
    __syncthreads();
    for (int c = 0; c < chunks; ++c) {
        const int buf = c & 1;
        const bool more = c + 1 < chunks;
        if (more) fetch(c + 1, ra, rb);
#pragma unroll 8
        for (int p = 0; p < 32; ++p) {
            const float4 av = As[buf][p][tk], bv = Bs[buf][p][te];
            const float aa[4] = {av.x, av.y, av.z, av.w}, bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], bb[j], acc[i][j]);
        }
        if (more) {
            As[buf ^ 1][lr][lc] = ra[0]; As[buf ^ 1][lr + 16][lc] = ra[1];
            Bs[buf ^ 1][lr][lc] = rb[0]; Bs[buf ^ 1][lr + 16][lc] = rb[1];
        }
        __syncthreads();
    }
    float* part = a.partials + (size_t)blockIdx.x * a.K * a.E;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k = k0 + tk * 4 + i, e = e0 + te * 4;
        if (k < a.K && e < a.E)
            *reinterpret_cast<float4*>(part + (size_t)k * a.E + e) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
}

template <typename io_t>
__global__ void xproj_wgrad_finalize(const float* __restrict__ partials, int slabs, long long ke, io_t* out) {   // block (32, 8)
    __shared__ float red[8][33];
    const long long idx = (long long)blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (idx < ke) {
#pragma unroll 4
        for (int c = threadIdx.y; c < slabs; c += 8) s += partials[(size_t)c * ke + idx];
    }
    red[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && idx < ke) {
        float t = 0.f;
#pragma unroll
        for (int y = 0; y < 8; ++y) t += red[y][threadIdx.x];
        store1(out, idx, t);
    }
}

// ------------------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------------------
static ProjArgs proj_args(const m2d_proj_desc* d, const ProjPlan& p) {
    ProjArgs a;
    a.P = (int)d->P; a.pitch = (int)d->proj_pitch; a.ntiles = p.ntiles;
    a.E = d->E; a.R = d->R; a.EB = p.EB; a.PS = p.PS; a.TP = p.TP;
    a.proj = d->proj; a.WT = d->WT; a.WL = d->WL; a.bT = d->bT; a.bL = d->bL;
    a.dT = d->dT; a.dL = d->dL; a.g_dT = d->g_dT; a.g_dL = d->g_dL;
    a.d_proj = d->d_proj;
    a.partials = static_cast<float*>(d->workspace);
    a.wide16 = d->E % 8 == 0 && aligned(d->g_dT, 16) && aligned(d->g_dL, 16) && aligned(d->dT, 16) && aligned(d->dL, 16);
    return a;
}

// CTAs per direction: the grid (gx, 2 directions) fills the resident CTA slots of the device exactly
// once, so that every SM gets the same number of CTAs and every CTA the same number of tiles (with the
// planned 2 x SMs per direction some SMs held five CTAs and others three: a quarter of the kernel was
// spent waiting for the fuller ones).  Never more than the plan's gx, which sized the workspace.
template <typename K>
static int balanced_gx(K kern, const ProjPlan& p, size_t smem) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, p.threads, smem) != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        return p.gx;
    }
    const int gx = per_sm * sm_count() / 2;
    return gx < 1 ? 1 : (gx < p.gx ? gx : p.gx);
}

template <typename io_t, int RB>
static int launch_dt_fwd(const ProjArgs& a, const ProjPlan& p, cudaStream_t st) {
    const size_t smem = (size_t)p.TP * RB * sizeof(float);
    auto kern = p.threads <= 256   ? dtproj_fwd_kernel<io_t, RB, 256>
                : p.threads <= 384 ? dtproj_fwd_kernel<io_t, RB, 384>
                : p.threads <= 512 ? dtproj_fwd_kernel<io_t, RB, 512>
                                   : dtproj_fwd_kernel<io_t, RB, M2D_PROJ_MAX_E>;
    kern<<<dim3(balanced_gx(kern, p, smem), 2), p.threads, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? M2D_OK : M2D_ERR_LAUNCH;
}

template <typename io_t, int RB>
static int launch_dt_bwd(const m2d_proj_desc* d, const ProjArgs& a, const ProjPlan& p, cudaStream_t st) {
    const size_t loop_bytes = (2 * (size_t)p.TP * RB + (size_t)(p.threads / 32) * kProjIters * kSlabStride) * sizeof(float) +
                              (size_t)4 * p.TP * d->E * sizeof(io_t);
    const size_t tail_bytes = (size_t)(RB + 1) * p.EB * sizeof(float);
    const size_t smem = loop_bytes > tail_bytes ? loop_bytes : tail_bytes;
    // the launch bound follows the block size, so that small blocks keep their registers
    auto kern = p.threads <= 256   ? dtproj_bwd_kernel<io_t, RB, 256>
                : p.threads <= 384 ? dtproj_bwd_kernel<io_t, RB, 384>
                : p.threads <= 512 ? dtproj_bwd_kernel<io_t, RB, 512>
                                   : dtproj_bwd_kernel<io_t, RB, M2D_PROJ_MAX_E>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return M2D_ERR_LAUNCH;
    const int gx = balanced_gx(kern, p, smem);
    kern<<<dim3(gx, 2), p.threads, smem, st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return M2D_ERR_LAUNCH;
    const int n = 2 * (RB + 1) * p.EB;
    dtproj_bwd_finalize<io_t><<<(n + 31) / 32, dim3(32, 8), 0, st>>>(a.partials, gx, RB, p.EB, d->E, d->R,
                                                             static_cast<io_t*>(d->d_WT), static_cast<io_t*>(d->d_WL),
                                                             static_cast<io_t*>(d->d_bT), static_cast<io_t*>(d->d_bL));
    return cudaGetLastError() == cudaSuccess ? M2D_OK : M2D_ERR_LAUNCH;
}

template <typename io_t>
static int dispatch_dt(const m2d_proj_desc* d, bool bwd, cudaStream_t st) {
    const ProjPlan p = plan_proj(d);
    const ProjArgs a = proj_args(d, p);
    switch (p.RB) {
        case 4: return bwd ? launch_dt_bwd<io_t, 4>(d, a, p, st) : launch_dt_fwd<io_t, 4>(a, p, st);
        case 8: return bwd ? launch_dt_bwd<io_t, 8>(d, a, p, st) : launch_dt_fwd<io_t, 8>(a, p, st);
        case 16: return bwd ? launch_dt_bwd<io_t, 16>(d, a, p, st) : launch_dt_fwd<io_t, 16>(a, p, st);
        case 32: return bwd ? launch_dt_bwd<io_t, 32>(d, a, p, st) : launch_dt_fwd<io_t, 32>(a, p, st);
        default: return bwd ? launch_dt_bwd<io_t, 64>(d, a, p, st) : launch_dt_fwd<io_t, 64>(a, p, st);
    }
}

// bf16 operands: the tensor-core kernel, when the problem meets its alignment rules (otherwise, and for
// fp32, whose 1e-4 bar rules out tf32 operands, the CUDA-core kernel below).  Returns -1 for "not taken".
static int launch_wgrad_tc(const m2d_proj_desc* d, const ProjPlan& p, cudaStream_t st) {
    const TcPlan t = tc_plan(d->P, d->E, p.K, d->proj_pitch, d->x, d->d_proj, p.slabs);
    if (!t.ok) return -1;
    CUtensorMap map_a, map_b;
    if (!tc_make_map(&map_a, d->d_proj, d->P, p.K, d->proj_pitch) || !tc_make_map(&map_b, d->x, d->P, d->E, d->E)) return -1;
    TcArgs a;
    a.K = p.K; a.E = d->E; a.nbk = t.nbk; a.stages = t.stages; a.total_blocks = t.total_blocks; a.blocks_per_cta = t.blocks_per_cta;
    a.partials = static_cast<float*>(d->workspace);
    a.status = reinterpret_cast<int*>(static_cast<char*>(d->workspace) + p.wg_partials - 256);
    if (cudaMemsetAsync(a.status, 0, sizeof(int), st) != cudaSuccess) return M2D_ERR_LAUNCH;
    if (cudaFuncSetAttribute(xproj_wgrad_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem) != cudaSuccess) return M2D_ERR_LAUNCH;
    xproj_wgrad_tc_kernel<<<dim3(t.grid_x, t.ny), 128, t.smem, st>>>(map_a, map_b, a);
    if (cudaGetLastError() != cudaSuccess) return M2D_ERR_LAUNCH;
    const long long ke = (long long)p.K * d->E;
    xproj_wgrad_finalize<__nv_bfloat16><<<(int)((ke + 31) / 32), dim3(32, 8), 0, st>>>(a.partials, t.grid_x, ke, static_cast<__nv_bfloat16*>(d->d_Wx));
    return cudaGetLastError() == cudaSuccess ? M2D_OK : M2D_ERR_LAUNCH;
}

template <typename io_t>
static int launch_wgrad(const m2d_proj_desc* d, cudaStream_t st) {
    const ProjPlan p = plan_proj(d);
    if (sizeof(io_t) == 2) {
        const int rc = launch_wgrad_tc(d, p, st);
        if (rc >= 0) return rc;
    }
    WgArgs a;
    a.P = (int)d->P; a.pitch = (int)d->proj_pitch; a.E = d->E; a.K = p.K; a.rows_per_slab = p.rows_per_slab;
    a.x = d->x; a.d_proj = d->d_proj;
    a.partials = static_cast<float*>(d->workspace);
    xproj_wgrad_kernel<io_t><<<dim3(p.slabs, p.tilesE, p.tilesK), 256, 0, st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return M2D_ERR_LAUNCH;
    const long long ke = (long long)p.K * d->E;
    xproj_wgrad_finalize<io_t><<<(int)((ke + 31) / 32), dim3(32, 8), 0, st>>>(a.partials, p.slabs, ke, static_cast<io_t*>(d->d_Wx));
    return cudaGetLastError() == cudaSuccess ? M2D_OK : M2D_ERR_LAUNCH;
}

static bool workspace_ok(const m2d_proj_desc* d, size_t need) {
    return need == 0 || (d->workspace && d->workspace_bytes >= need && aligned(d->workspace, 256));
}

}  // namespace m2d

using namespace m2d;

extern "C" uint64_t m2d_proj_workspace(const m2d_proj_desc* d) {
    if (check_proj(d) != M2D_OK) return 0;
    const ProjPlan p = plan_proj(d);
    return align256(p.dt_partials > p.wg_partials ? p.dt_partials : p.wg_partials);
}

extern "C" int m2d_dtproj_fwd(const m2d_proj_desc* d, void* stream) {
    const int rc = check_proj(d);
    if (rc != M2D_OK) return rc;
    if (!d->proj || !d->WT || !d->WL || !d->bT || !d->bL || !d->dT || !d->dL) return M2D_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return d->dtype == M2D_F32 ? dispatch_dt<float>(d, false, st) : dispatch_dt<__nv_bfloat16>(d, false, st);
}

extern "C" int m2d_dtproj_bwd(const m2d_proj_desc* d, void* stream) {
    const int rc = check_proj(d);
    if (rc != M2D_OK) return rc;
    if (!d->proj || !d->WT || !d->WL || !d->dT || !d->dL || !d->g_dT || !d->g_dL || !d->d_proj || !d->d_WT || !d->d_WL ||
        !d->d_bT || !d->d_bL)
        return M2D_ERR_NULL;
    {
        // the g / delta rows are copied in 4-element pieces
        const size_t al = d->dtype == M2D_F32 ? 16 : 8;
        if (d->E % 4 != 0 || !aligned(d->g_dT, al) || !aligned(d->g_dL, al) || !aligned(d->dT, al) || !aligned(d->dL, al)) return M2D_ERR_PITCH;
    }
    if (!workspace_ok(d, plan_proj(d).dt_partials)) return M2D_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return d->dtype == M2D_F32 ? dispatch_dt<float>(d, true, st) : dispatch_dt<__nv_bfloat16>(d, true, st);
}

extern "C" int m2d_xproj_wgrad_on_tensor_cores(const m2d_proj_desc* d) {
    if (check_proj(d) != M2D_OK || d->dtype != M2D_BF16 || !d->x || !d->d_proj) return 0;
    const ProjPlan p = plan_proj(d);
    const TcPlan t = tc_plan(d->P, d->E, p.K, d->proj_pitch, d->x, d->d_proj, p.slabs);
    if (!t.ok) return 0;
    CUtensorMap map_a, map_b;
    return tc_make_map(&map_a, d->d_proj, d->P, p.K, d->proj_pitch) && tc_make_map(&map_b, d->x, d->P, d->E, d->E) ? 1 : 0;
}

extern "C" int m2d_xproj_wgrad(const m2d_proj_desc* d, void* stream) {
    const int rc = check_proj(d);
    if (rc != M2D_OK) return rc;
    if (!d->x || !d->d_proj || !d->d_Wx) return M2D_ERR_NULL;
    const size_t al = d->dtype == M2D_F32 ? 16 : 8;
    if (d->E % 4 != 0 || d->proj_pitch % 4 != 0 || !aligned(d->x, al) || !aligned(d->d_proj, al)) return M2D_ERR_PITCH;
    if (!workspace_ok(d, plan_proj(d).wg_partials)) return M2D_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return d->dtype == M2D_F32 ? launch_wgrad<float>(d, st) : launch_wgrad<__nv_bfloat16>(d, st);
}
