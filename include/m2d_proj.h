/*
 * m2d_proj.h -- C ABI of the fused parameter projections that feed the wavefront scan.
 *
 * The reference computes the scan's input-dependent parameters in PyTorch
 * (proj_params, models/kernels/wavefront_cuda.py:63-95):
 *     proj           = x @ Wx^T                           (P, 2R+3N)  = [rT | rL | BT | BL | C]
 *     deltaT, deltaL = softplus(rT @ WT^T + bT), softplus(rL @ WL^T + bL)          (P, E)
 * and differentiates them with autograd.  On B200 the x projection is a well-shaped GEMM and
 * stays on the GEMM library; the rest is not:
 *   - the two dt projections have an inner dimension of R = E/16 (4..36) and are followed by an
 *     element-wise softplus: three passes over (P,E) per direction;
 *   - their weight gradients, and the x projection's, are reductions over all P = B*H*W pixels
 *     into a tiny (E,R) or (2R+3N,E) result, the shape GEMM libraries handle worst (measured: a
 *     third of a millisecond each at P = 401 408, 20x the time their operands take to stream).
 * The entry points below do that work in one pass each.  Rows are pixels; every matrix is
 * row-major; conventions (device pointers, caller-owned memory, asynchronous on `stream`, status
 * codes, re-entrancy) are those of m2d_scan.h.
 */
#ifndef M2D_PROJ_H
#define M2D_PROJ_H

#include "m2d_scan.h"

#ifdef __cplusplus
extern "C" {
#endif

#define M2D_PROJ_MAX_E 640   /* channels per call (the shipped models use at most 576) */
#define M2D_PROJ_MAX_R 64    /* dt rank per call (the shipped models use at most 36); also required: the
                                rank, rounded up to 4, 8, 16, 32 or 64, is at most a quarter of E rounded up to
                                a multiple of 32 (M2D_ERR_SHAPE otherwise; the models use R = E/16) */

typedef struct m2d_proj_desc {
    uint32_t struct_bytes;     /* = sizeof(m2d_proj_desc) */
    int32_t dtype;             /* m2d_dtype of every tensor below */
    int64_t P;                 /* pixels = B*H*W; P * max(E, proj_pitch) must stay below 2^31 - 2^26 (M2D_ERR_TOO_LARGE) */
    int32_t E, R, N;           /* channels, dt rank, state size; K = 2R+3N columns are in use */
    int32_t reserved0;
    int64_t proj_pitch;        /* row pitch, in elements, of proj and d_proj (>= K) */
    const void *x;             /* (P,E)      scan input                              [wgrad] */
    const void *proj;          /* (P,pitch)  x-projection output                     [fwd, bwd] */
    const void *WT, *WL;       /* (E,R)      dt projection weights                   [fwd, bwd] */
    const void *bT, *bL;       /* (E)        dt projection biases                    [fwd] */
    void *dT, *dL;             /* (P,E)      softplus outputs: written by fwd, read by bwd */
    const void *g_dT, *g_dL;   /* (P,E)      upstream gradients of dT, dL            [bwd] */
    void *d_proj;              /* (P,pitch)  gradient of proj: bwd writes columns [0,2R); wgrad reads [0,K) */
    void *d_WT, *d_WL;         /* (E,R)                                              [bwd] */
    void *d_bT, *d_bL;         /* (E)                                                [bwd] */
    void *d_Wx;                /* (K,E)      gradient of the x-projection weight     [wgrad] */
    void *workspace;           /* scratch, 256-byte aligned, see m2d_proj_workspace() */
    uint64_t workspace_bytes;
} m2d_proj_desc;

/* Bytes of scratch the three calls below need for this problem (the maximum over the three). */
uint64_t m2d_proj_workspace(const m2d_proj_desc *desc);

/*
 * dT = softplus(proj[:, 0:R] @ WT^T + bT), dL = softplus(proj[:, R:2R] @ WL^T + bL), softplus with
 * the reference's threshold (values above 20 pass through).  Replaces the two F.linear + F.softplus
 * pairs of proj_params (wavefront_cuda.py:84-85).  No workspace.
 */
int m2d_dtproj_fwd(const m2d_proj_desc *desc, void *stream);

/*
 * Backward of the above in one pass over g_dT, g_dL: with s = g * (1 - exp(-delta)) (softplus'
 * expressed through its own output, so the pre-activation need not be kept),
 *     d_W = s^T @ r,   d_b = sum_p s,   d_proj[:, 0:R] = sT @ WT,   d_proj[:, R:2R] = sL @ WL.
 * Replaces what autograd runs for wavefront_cuda.py:84-85 (softplus backward, two bias sums and
 * four GEMMs with a dimension of R).
 */
int m2d_dtproj_bwd(const m2d_proj_desc *desc, void *stream);

/*
 * d_Wx = d_proj[:, 0:K]^T @ x, a reduction over all pixels, split across the GPU and summed in a
 * second small kernel.  Replaces the weight half of the backward of F.linear(x, x_proj_w)
 * (wavefront_cuda.py:75).  Requires E % 4 == 0, proj_pitch % 4 == 0 and 16-byte aligned x and
 * d_proj (M2D_ERR_PITCH otherwise).
 */
int m2d_xproj_wgrad(const m2d_proj_desc *desc, void *stream);

/*
 * 1 if m2d_xproj_wgrad would run this problem on the tensor cores (bf16 operands staged by TMA,
 * tcgen05.mma with an fp32 accumulator in tensor memory), 0 if on the CUDA cores (fp32; bf16 problems
 * with E or proj_pitch not a multiple of 8, pointers not 16-byte aligned, more than 128 projection
 * columns, or M2D_WGRAD_TC=0 in the environment).  Needs x and d_proj set; launches nothing.
 */
int m2d_xproj_wgrad_on_tensor_cores(const m2d_proj_desc *desc);

#ifdef __cplusplus
}
#endif
#endif /* M2D_PROJ_H */
