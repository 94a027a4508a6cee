// Forward scan for callers that cannot hand the library a workspace buffer.
//
// The regular forward entry point needs a scratch region (the per-CTA ring that carries the last
// row of one band of image rows to the first row of the next band) and expects the caller to
// allocate it.  Some callers have no way to do that: a host runtime that binds this library behind
// a fixed "inputs in, outputs out" plugin signature has no slot for an extra buffer; a service that
// carved up all device memory at start-up has no allocator left to ask; and code running inside a
// latency-critical loop must not call cudaMalloc, which can synchronise the whole device.  For
// them this file keeps the ring in a file-scope __device__ array of fixed size, so the call needs
// nothing but the inputs and the output.
//
// Cost and limits of that choice:
//   - every GPU on which this library is loaded holds M2D_NOALLOC_SCRATCH_BYTES (32 MiB) of
//     device memory from load until the process exits;
//   - problems whose ring would not fit are rejected with M2D_ERR_TOO_LARGE;
//   - all calls on one device share the one array.  Only its first word (the status word the
//     kernels share with the regular entry point's workspace layout) has to start at zero, and the
//     call clears it itself; every other slot is written before it is read within a call, and what
//     an earlier call left behind is never read.  But two calls that overlap in time on the same
//     GPU -- different streams, or different host threads -- would overwrite each other's slots
//     and produce wrong results.  Serialise them (one stream, or events between streams);
//   - the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) and caches it; make that first call before starting any stream
//     capture on that device.
#include <mutex>

#include "launch.cuh"
#include "sweep_rows.cuh"

namespace m2d {

// In host code this name is only a handle for the runtime's symbol table, not a device address:
// it must go through cudaGetSymbolAddress before a kernel can be given a pointer to it.
static __device__ __align__(256) unsigned char g_noalloc_ring[M2D_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_ring_mutex;
static float4* g_ring_ptr[kMaxDevices] = {};   // device address of g_noalloc_ring on each device

// Device address of the ring on the CURRENT device; looked up once per device.
static int ring_address(float4** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return M2D_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_ring_mutex);
    if (g_ring_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_ring) != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return M2D_ERR_LAUNCH;
        }
        g_ring_ptr[dev] = static_cast<float4*>(p);
    }
    *out = g_ring_ptr[dev];
    return M2D_OK;
}

// ROWS: the nested-loop sweep; otherwise the flat step loop (maps narrower than three columns).
template <typename io_t, bool VEC, bool ROWS>
__global__ void __launch_bounds__(256, 2) m2d_fwd_noalloc_kernel(const ScanArgs a) {
    extern __shared__ float4 smem[];
    const int lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int cq = lane >> 2, nq = lane & 3;
    const int g = blockIdx.y;
    const int ch0 = g * kGroup + cq * 4, n0 = nq * 4;
    const int chv = min(4, max(0, a.E - ch0));
    const int nv = min(4, max(0, a.N - n0));
    const size_t bytes = ROWS ? rows_fwd_smem_bytes(nwarps) : sweep_smem_bytes(nwarps);
    const int total = (int)(bytes / sizeof(float4));
    for (int k = threadIdx.x; k < total; k += blockDim.x) smem[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int ch_own = g * kGroup + lane;
    const float D_own = ch_own < a.E ? load1(static_cast<const io_t*>(a.D), ch_own) : 0.f;
    __syncthreads();
    float4* const params = reinterpret_cast<float4*>(reinterpret_cast<char*>(smem) + bytes);
    if (threadIdx.x < 32) stage_params<io_t>(params, a.AT, a.AL, a.N, ch0, chv, n0, nv, lane, a.a_log);
    __syncthreads();
    const int nb = (a.B - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    if (ROWS) forward_rows<io_t, VEC, false>(a, smem, params, D_own, blockIdx.x, gridDim.x, nb);
    else forward_sweep<io_t, VEC, false, false, 1>(a, smem, params, D_own, blockIdx.x, gridDim.x, nb);
}

template <typename io_t>
static int launch_noalloc(const m2d_scan_desc* d, const Plan& pl, bool vec, float4* scratch, cudaStream_t st) {
    ScanArgs a;
    fill_common_args(a, d, pl);
    a.y = d->y;
    // same layout as a caller's workspace: [status word][per-CTA rings]
    char* base = reinterpret_cast<char*>(scratch);
    a.status = reinterpret_cast<int*>(base);
    a.ring = reinterpret_cast<float4*>(base + kStatusBytes);
    a.chain = 1;
    if (cudaMemsetAsync(base, 0, sizeof(int), st) != cudaSuccess) return M2D_ERR_LAUNCH;
    void (*kern)(const ScanArgs) = pl.rows ? (vec ? m2d_fwd_noalloc_kernel<io_t, true, true> : m2d_fwd_noalloc_kernel<io_t, false, true>)
                                           : (vec ? m2d_fwd_noalloc_kernel<io_t, true, false> : m2d_fwd_noalloc_kernel<io_t, false, false>);
    return launch_sweep_kernel(kern, a, pl, d->W, st);
}

}  // namespace m2d

extern "C" uint64_t m2d_scan_fwd_noalloc_need(const m2d_scan_desc* d) {
    if (m2d::check_desc(d, false, false) != M2D_OK) return 0;
    return m2d::plan_fwd(d, false).scratch;
}

extern "C" int m2d_scan_fwd_noalloc(const m2d_scan_desc* d, void* stream) {
    int rc = m2d::check_desc(d, false, true);
    if (rc != M2D_OK) return rc;
    if (!d->y) return M2D_ERR_NULL;
    const m2d::Plan pl = m2d::plan_fwd(d, false);   // one CTA per image: the fixed array holds per-CTA rings only
    if (pl.scratch > M2D_NOALLOC_SCRATCH_BYTES) return M2D_ERR_TOO_LARGE;   // decided before any device work
    float4* ring = nullptr;
    rc = m2d::ring_address(&ring);
    if (rc != M2D_OK) return rc;
    const bool vec = m2d::vector_ok(d, false);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->dtype == M2D_F32) return m2d::launch_noalloc<float>(d, pl, vec, ring, st);
    return m2d::launch_noalloc<__nv_bfloat16>(d, pl, vec, ring, st);
}
