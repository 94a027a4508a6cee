/*
 * m2d_scan.h -- C ABI of the B200 (sm_100a) wavefront 2-D selective scan.
 *
 * This is the drop-in boundary for the native side of the Mamba2D scan.  In the reference project
 * the native boundary is a pybind11 module with two functions taking torch::Tensor by value
 *   wf_fwd(hs, x, deltaT, deltaL, BT, BL, AT, AL)                         models/kernels/wf_cuda/wf_cuda_bind.cpp:24-34
 *   wf_bwd(hs, x, deltaT, deltaL, AT, AL, grad_output, dDAT, dDAL, omega) models/kernels/wf_cuda/wf_cuda_bind.cpp:36-47
 * which each run one anti-diagonal per kernel launch and leave the readout and most of the
 * gradient arithmetic to PyTorch.  The entry points below sit one level higher, at the level of
 * the reference's autograd Function wf_cuda_fn_pr (models/kernels/wavefront_cuda.py:146-196):
 *   forward   (x, dT, dL, AT, AL, BT, BL, C, D)        -> y
 *   backward  (x, dT, dL, AT, AL, BT, BL, C, D, gy)    -> nine gradients
 * so that the forward pass never materialises the 5-D hidden state and autograd never saves it (the
 * backward pass recomputes it into its own workspace, as the reference's partial-recomputation
 * mode does: wavefront_cuda.py:172-173).
 *
 * Conventions
 *   - plain C types only; every pointer is a DEVICE pointer unless stated otherwise;
 *   - the library never allocates or frees device memory: outputs and workspace are the caller's
 *     (as in the reference, where Python allocates every tensor: wavefront_cuda.py:152, :181-183);
 *   - inputs are never modified;
 *   - calls are asynchronous on the given stream; no host synchronisation on the success path;
 *   - every function returns M2D_OK (0) or a negative m2d_status code; m2d_strerror() names it;
 *   - re-entrant, no global mutable state (one exception is documented where it applies).
 */
#ifndef M2D_SCAN_H
#define M2D_SCAN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define M2D_ABI_VERSION 3

typedef enum m2d_dtype {
    M2D_F32 = 0,   /* float in memory, float arithmetic */
    M2D_BF16 = 1   /* bfloat16 in memory, float arithmetic and float state */
} m2d_dtype;

typedef enum m2d_status {
    M2D_OK = 0,
    M2D_ERR_NULL = -1,          /* a required pointer is NULL */
    M2D_ERR_DTYPE = -2,         /* unknown dtype */
    M2D_ERR_SHAPE = -3,         /* B,E,N < 1, or H < 2 or W < 2 (the reference raises ValueError for
                                   the latter: wavefront_cuda.py:322-324) */
    M2D_ERR_UNSUPPORTED_N = -4, /* N > 16 */
    M2D_ERR_PITCH = -5,         /* a BT/BL/C pixel pitch smaller than N */
    M2D_ERR_WORKSPACE = -6,     /* workspace missing, too small or not 256-byte aligned */
    M2D_ERR_LAUNCH = -7,        /* the CUDA runtime rejected a launch or a memset */
    M2D_ERR_ABI = -8,           /* descriptor size does not match this library */
    M2D_ERR_TOO_LARGE = -9,     /* B*H*W*max(E, pitch) >= 2^31 (kernels use 31-bit element indices), or
                                   scratch beyond the capacity of the no-allocation entry point */
    M2D_ERR_FLAGS = -10         /* an unknown bit is set in desc->flags */
} m2d_status;

/*
 * desc->flags bits.
 *
 * M2D_SCAN_REVERSE: scan from the bottom-right corner towards the top-left one.  The result is
 * what the forward-direction call returns on inputs whose H and W axes are both flipped, flipped
 * back -- for y and for every gradient -- but no tensor is copied: the kernels walk the same
 * memory in the opposite order.  The reference gets this direction with torch.flip copies of the
 * activation around the whole block (scan_start == "BR", models/mamba2d.py:162-175, chosen for odd
 * blocks by inter_flip, :350) and around the second scan of double_scans (:190-200); everything
 * between those flips other than the scan acts per pixel, so the flips can be dropped when the
 * scan itself runs in reverse.
 */
#define M2D_SCAN_REVERSE 1u

/*
 * M2D_SCAN_GELU_OUT (m2d_scan_fwd and m2d_scan_fwd_noalloc only; the backward rejects it): store
 * gelu(y) instead of y, GELU in its erf form.  The reference block applies nn.GELU() to the scan's
 * output as a separate elementwise pass (act2, models/mamba2d.py:169); at inference that pass can be
 * folded into the scan's store.  For training the pre-activation y is needed by GELU's backward, so
 * callers that need gradients leave the flag off and apply the activation themselves.
 */
#define M2D_SCAN_GELU_OUT 2u

/*
 * M2D_SCAN_A_LOG: desc->AT and desc->AL point to the FP32 parameters AT_log, AL_log (E,N), whatever
 * `dtype` is, and the kernels use A = -exp(A_log), rounded to `dtype` as the reference's cast does
 * (models/kernels/wavefront_cuda.py:72-73, :89-90).  In the backward desc->d_AT and desc->d_AL then
 * receive the gradient with respect to A_log (= d_A * A) as FP32 (E,N) arrays.  This folds the
 * reference's `-torch.exp(A_log.float())`, its casts and their backward -- a handful of tiny
 * elementwise launches per call -- into the kernels.
 */
#define M2D_SCAN_A_LOG 4u

/*
 * M2D_SCAN_TEST_WITHHOLD: test hook, rejected with M2D_ERR_FLAGS unless the environment variable
 * M2D_TEST_HOOKS is 1.  In a launch that runs several CTAs per image, the CTA that owns the first
 * band of image 0 never publishes that band's column counter and every wait gives up after a few
 * hundred tries instead of a million: the CTA below runs out of patience, the kernel returns
 * normally and the status word is nonzero.  Nothing faults or hangs; the outputs are void.  It
 * exists so that the give-up path of the bounded waits can be exercised by a test.
 */
#define M2D_SCAN_TEST_WITHHOLD 0x100u

/*
 * Problem descriptor.  Tensor layouts are the ones the reference op receives:
 *   x, dT, dL, y, gy, d_x, d_dT, d_dL   (B,H,W,E) contiguous, channels last
 *   AT, AL, d_AT, d_AL                  (E,N) contiguous; A = -exp(A_log) already applied (but see
 *                                       M2D_SCAN_A_LOG)
 *   D, d_D                              (E)
 *   BT, BL, C                           (B,H,W,N) with unit stride over N and a per-tensor pixel
 *                                       pitch in ELEMENTS (row stride W*pitch, batch stride
 *                                       H*W*pitch).  The reference produces these as views into
 *                                       one projection output with pitch 2R+3N
 *                                       (wavefront_cuda.py:78-82); a contiguous tensor has pitch N.
 *   d_BT, d_BL, d_C                     (B,H,W,N) contiguous
 * All tensors share `dtype`.
 */
typedef struct m2d_scan_desc {
    uint32_t struct_bytes;      /* = sizeof(m2d_scan_desc) */
    int32_t dtype;              /* m2d_dtype */
    int32_t B, H, W, E, N;
    uint32_t flags;             /* 0 or M2D_SCAN_* bits */
    const void *x, *dT, *dL;
    const void *AT, *AL;
    const void *BT, *BL, *C;
    int64_t BT_pitch, BL_pitch, C_pitch;
    const void *D;
    void *y;                    /* forward output */
    const void *gy;             /* backward input: upstream gradient of y */
    void *d_x, *d_dT, *d_dL, *d_AT, *d_AL, *d_BT, *d_BL, *d_C, *d_D;   /* backward outputs */
    void *workspace;            /* scratch, 256-byte aligned, see *_workspace() */
    uint64_t workspace_bytes;
} m2d_scan_desc;

/* ABI version of the loaded library (compare with M2D_ABI_VERSION). */
int m2d_abi_version(void);

/* Static string naming a status code. */
const char *m2d_strerror(int status);

/*
 * Bytes of scratch m2d_scan_fwd / m2d_scan_bwd need for this problem on the current device (never
 * 0: the scratch starts with a status word).  Replaces the reference's Python-side allocations of
 * hs / dDAT / dDAL / omega (wavefront_cuda.py:152, :181-183).  Returns 0 for an invalid descriptor.
 */
uint64_t m2d_scan_fwd_workspace(const m2d_scan_desc *desc);
uint64_t m2d_scan_bwd_workspace(const m2d_scan_desc *desc);

/*
 * Forward: y = sum_n h*C + x*D with h the two-neighbour recurrence.
 * Replaces wf_fwd (wf_cuda_bind.cpp:24-34) + the readout (wavefront_cuda.py:156).
 * Reads x,dT,dL,AT,AL,BT,BL,C,D; writes y; uses workspace.  `stream` is a cudaStream_t.
 */
int m2d_scan_fwd(const m2d_scan_desc *desc, void *stream);

/*
 * With few images on a large map several CTAs share an image and wait on one another through
 * global memory (inside a CTA the row-warps meet at block barriers with uniform trip counts).  Every
 * wait between CTAs is bounded.  If one ever gives up (it cannot when the kernel has the GPU
 * to itself), all later waits return at once, the kernel terminates normally and leaves a nonzero
 * int32 status word in the workspace; the outputs are then void.  These return the byte offset of
 * that word inside the workspace (0 today), or -1 for an invalid descriptor.  Read the word after
 * synchronising the stream.  m2d_scan_*_chain return how many CTAs share one image for this problem
 * on the current device (1: none do; 0: invalid descriptor) -- launches with more than one are the
 * ones whose waits cross CTAs.  No counterpart in the reference (its launches are serialised by the
 * host).
 */
int64_t m2d_scan_fwd_status_offset(const m2d_scan_desc *desc);
int64_t m2d_scan_bwd_status_offset(const m2d_scan_desc *desc);   /* same, for m2d_scan_bwd's workspace */
int m2d_scan_fwd_chain(const m2d_scan_desc *desc);
int m2d_scan_bwd_chain(const m2d_scan_desc *desc);

/*
 * The rule every launch applies when it picks, or has to shorten, the number of CTAs per image:
 * at most one CTA per band, and when CTAs own more than one band each (the chain closes into a
 * ring) fewer than one row of steps divided by the rows per band, so that the head of the ring
 * never waits on data that waits on the head.  Host-side arithmetic only; returns 0 for
 * non-positive arguments.  No counterpart in the reference.
 */
int m2d_scan_chain_bound(int want, int nbands, int steps_per_row, int rows_per_band);

/*
 * Backward with recomputation of the hidden state: all nine gradients of the forward.
 * Replaces the body of wf_cuda_fn_pr.backward (wavefront_cuda.py:163-196): the recompute of hs,
 * wf_bwd (wf_cuda_bind.cpp:36-47) and fused_backward_math (wavefront_cuda.py:97-139).
 * Reads the forward inputs and gy; writes d_x..d_D; uses workspace.
 */
int m2d_scan_bwd(const m2d_scan_desc *desc, void *stream);

/*
 * Forward scan that needs no workspace from the caller.  It has no counterpart in the reference
 * project (there, Python allocates every buffer the kernels touch).
 *
 * Same inputs, output and results as m2d_scan_fwd, but desc->workspace is ignored: the scratch the
 * kernel needs lives in a fixed array inside the library.  It exists for callers that cannot
 * provide a scratch buffer -- a host runtime whose plugin signature carries only inputs and
 * outputs, a process that handed out all device memory at start-up, or a loop that must never
 * reach cudaMalloc.  The entry point itself calls no cudaMalloc/cudaFree and no allocating
 * library routine.
 *
 *   - The array is M2D_NOALLOC_SCRATCH_BYTES (32 MiB) and every GPU that loads the library keeps
 *     it until the process exits.
 *   - A problem needing more scratch than that returns M2D_ERR_TOO_LARGE before any device work.
 *     m2d_scan_fwd_noalloc_need() reports the need: a status word plus one ring of W slots of 2 KiB
 *     per CTA when the map has more rows than a CTA has row-warps (8), with at most two CTAs per SM.
 *     This entry always runs one CTA per (image, channel group), so its need can differ from what
 *     m2d_scan_fwd_workspace() reports for the same problem.
 *   - All calls on a device share the array.  The call clears the one word that must start at
 *     zero itself, but calls that overlap in time on one GPU race on the array: keep them on one
 *     stream or order them with events.
 *   - The first call on each device resolves the array's device address and caches it; issue
 *     that first call before any stream capture on that device.
 */
#define M2D_NOALLOC_SCRATCH_BYTES (32u << 20)
int m2d_scan_fwd_noalloc(const m2d_scan_desc *desc, void *stream);
uint64_t m2d_scan_fwd_noalloc_need(const m2d_scan_desc *desc);   /* bytes of the array this problem would use; 0 if invalid */

#ifdef __cplusplus
}
#endif
#endif /* M2D_SCAN_H */
