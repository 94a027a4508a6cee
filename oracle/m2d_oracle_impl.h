/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the Mamba2D wavefront 2-D selective scan.
 *
 * This body is included several times by m2d_oracle.c with different arithmetic:
 *   REAL      storage / arithmetic type (float or double)
 *   RND(v)    rounding hook applied after every arithmetic operation
 *             (identity for f32/f64; round-to-nearest-even bf16 for the bf16 emulation,
 *             which mimics the reference computing in scalar_t = BFloat16)
 *   FN(name)  symbol suffixing
 *
 * Layouts are the ones the reference op receives (all contiguous here):
 *   x, dT, dL, y, gy   (B,H,W,E)      channels last
 *   BT, BL, C          (B,H,W,N)
 *   AT, AL             (E,N)          already A = -exp(A_log)
 *   Dskip              (E)
 *
 * Reference being restated (paths inside the reference project):
 *   forward cell update      models/kernels/wf_cuda/wf_cuda.cu:41-69
 *   readout                  models/kernels/wavefront_cuda.py:156
 *   backward orchestration   models/kernels/wavefront_cuda.py:163-196
 *   adjoint sweep            models/kernels/wf_cuda/wf_cuda.cu:108-160
 *   post-kernel gradients    models/kernels/wavefront_cuda.py:97-139
 *
 * The reference sweeps anti-diagonals with one launch each; cells of one diagonal are
 * independent and every cell's arithmetic is fixed, so a row-major sweep gives the same
 * floating-point value per cell.  The rolling two-slot omega buffer of the reference
 * (wf_cuda.cu:109-112) is held here as a full plane, which stores the same values.
 */

/* One (b,e) plane of the forward recurrence.  hs is [H][W][N] for this plane. */
static void FN(plane_fwd)(int H, int W, int E, int N, int e,
                          const REAL *x, const REAL *dT, const REAL *dL,      /* at batch b: [H][W][E] */
                          const REAL *BT, const REAL *BL,                      /* at batch b: [H][W][N] */
                          const REAL *AT, const REAL *AL,                      /* [E][N] */
                          REAL *hs)
{
    for (int i = 0; i < H; ++i) {
        for (int j = 0; j < W; ++j) {
            const size_t p = (size_t)i * W + j;
            const REAL v_dt = dT[p * E + e];
            const REAL v_dl = dL[p * E + e];
            const REAL v_x  = x[p * E + e];
            for (int n = 0; n < N; ++n) {
                const REAL v_BT = BT[p * N + n];
                const REAL v_BL = BL[p * N + n];
                const REAL v_AT = AT[(size_t)e * N + n];
                const REAL v_AL = AL[(size_t)e * N + n];
                /* wf_cuda.cu:50-53 */
                const REAL gAT = RND(EXPF(RND(v_dt * v_AT)));
                const REAL gAL = RND(EXPF(RND(v_dl * v_AL)));
                const REAL bxT = RND(RND(v_dt * v_BT) * v_x);
                const REAL bxL = RND(RND(v_dl * v_BL) * v_x);
                REAL h;
                /* wf_cuda.cu:58-69 */
                if (i == 0 && j == 0) {
                    h = bxL;
                } else if (i == 0) {
                    h = RND(RND(gAL * hs[(p - 1) * N + n]) + bxL);
                } else if (j == 0) {
                    h = RND(RND(gAT * hs[(p - W) * N + n]) + bxT);
                } else {
                    REAL s = RND(gAL * hs[(p - 1) * N + n]);
                    s = RND(s + bxL);
                    s = RND(s + RND(gAT * hs[(p - W) * N + n]));
                    s = RND(s + bxT);
                    h = RND((REAL)0.5 * s);
                }
                hs[p * N + n] = h;
            }
        }
    }
}

/*
 * Forward: y = sum_n hs*C + x*D.  If hs_out != NULL it receives the full (B,H,W,E,N) state.
 * Returns 0, or -1 on allocation failure / bad shape.
 */
int FN(m2d_oracle_fwd)(int B, int H, int W, int E, int N,
                       const REAL *x, const REAL *dT, const REAL *dL,
                       const REAL *AT, const REAL *AL,
                       const REAL *BT, const REAL *BL, const REAL *C,
                       const REAL *Dskip, REAL *y, REAL *hs_out)
{
    if (B < 1 || H < 1 || W < 1 || E < 1 || N < 1) return -1;
    int fail = 0;
    const long planes = (long)B * E;
#pragma omp parallel
    {
        REAL *hs = (REAL *)malloc(sizeof(REAL) * (size_t)H * W * N);
        if (!hs) {
#pragma omp atomic write
            fail = 1;
        }
#pragma omp barrier
        if (!fail) {
#pragma omp for schedule(static)
            for (long pe = 0; pe < planes; ++pe) {
                const int b = (int)(pe / E), e = (int)(pe % E);
                const size_t ob = (size_t)b * H * W;
                FN(plane_fwd)(H, W, E, N, e, x + ob * E, dT + ob * E, dL + ob * E,
                              BT + ob * N, BL + ob * N, AT, AL, hs);
                for (size_t p = 0; p < (size_t)H * W; ++p) {
                    /* wavefront_cuda.py:156: (hs * C).sum(-1) + x * D */
                    ACC acc = 0;
                    for (int n = 0; n < N; ++n)
                        acc += (ACC)RND(hs[p * N + n] * C[(ob + p) * N + n]);
                    const REAL xe = x[(ob + p) * E + e];
                    y[(ob + p) * E + e] = RND(RND((REAL)acc) + RND(xe * Dskip[e]));
                    if (hs_out)
                        for (int n = 0; n < N; ++n)
                            hs_out[((ob + p) * E + e) * N + n] = hs[p * N + n];
                }
            }
        }
        free(hs);
    }
    return fail ? -1 : 0;
}

/*
 * Backward, following the reference's own algorithm step by step.  All nine gradients:
 *   d_x, d_dT, d_dL (B,H,W,E); d_AT, d_AL (E,N); d_BT, d_BL, d_C (B,H,W,N); d_D (E).
 */
int FN(m2d_oracle_bwd)(int B, int H, int W, int E, int N,
                       const REAL *x, const REAL *dT, const REAL *dL,
                       const REAL *AT, const REAL *AL,
                       const REAL *BT, const REAL *BL, const REAL *C,
                       const REAL *Dskip, const REAL *gy,
                       REAL *d_x, REAL *d_dT, REAL *d_dL,
                       REAL *d_AT, REAL *d_AL,
                       REAL *d_BT, REAL *d_BL, REAL *d_C, REAL *d_D)
{
    if (B < 1 || H < 2 || W < 2 || E < 1 || N < 1) return -1;
    const size_t HW = (size_t)H * W, PN = HW * N;
    int fail = 0;

    /* (E,N) and (E) sums over (b,i,j) accumulate in ACC; every e is owned by one thread at a time. */
    ACC *accAT = (ACC *)calloc((size_t)E * N, sizeof(ACC));
    ACC *accAL = (ACC *)calloc((size_t)E * N, sizeof(ACC));
    ACC *accD  = (ACC *)calloc((size_t)E, sizeof(ACC));
    int nthr = 1;
#ifdef _OPENMP
    nthr = omp_get_max_threads();
#endif
    /* per-thread partial sums over e of d_BT, d_BL, d_C for the current batch element */
    ACC *part = (ACC *)malloc(sizeof(ACC) * (size_t)nthr * 3 * PN);
    if (!accAT || !accAL || !accD || !part) { free(accAT); free(accAL); free(accD); free(part); return -1; }

    for (int b = 0; b < B && !fail; ++b) {
        const size_t ob = (size_t)b * HW;
        memset(part, 0, sizeof(ACC) * (size_t)nthr * 3 * PN);
#pragma omp parallel
        {
            int tid = 0;
#ifdef _OPENMP
            tid = omp_get_thread_num();
#endif
            ACC *pBT = part + (size_t)tid * 3 * PN, *pBL = pBT + PN, *pC = pBL + PN;
            REAL *hs   = (REAL *)malloc(sizeof(REAL) * PN);
            REAL *dbx  = (REAL *)malloc(sizeof(REAL) * PN);   /* grad_output, overwritten in place by dBX */
            REAL *om   = (REAL *)malloc(sizeof(REAL) * PN);   /* omega, full plane */
            REAL *ddat = (REAL *)malloc(sizeof(REAL) * PN);
            REAL *ddal = (REAL *)malloc(sizeof(REAL) * PN);
            if (!hs || !dbx || !om || !ddat || !ddal) {
#pragma omp atomic write
                fail = 1;
            }
#pragma omp barrier
            if (!fail) {
#pragma omp for schedule(static)
                for (int e = 0; e < E; ++e) {
                    /* wavefront_cuda.py:172-173: recompute hs */
                    FN(plane_fwd)(H, W, E, N, e, x + ob * E, dT + ob * E, dL + ob * E,
                                  BT + ob * N, BL + ob * N, AT, AL, hs);
                    /* wavefront_cuda.py:176-178 */
                    for (size_t p = 0; p < HW; ++p) {
                        const REAL g = gy[(ob + p) * E + e];
                        accD[e] += (ACC)RND(g * x[(ob + p) * E + e]);
                        for (int n = 0; n < N; ++n) {
                            pC[p * N + n] += (ACC)RND(g * hs[p * N + n]);
                            dbx[p * N + n] = RND(g * C[(ob + p) * N + n]);
                        }
                    }
                    /* wf_cuda.cu:108-160, cells visited in an order compatible with k = H+W-2 .. 0 */
                    for (int i = H - 1; i >= 0; --i) {
                        for (int j = W - 1; j >= 0; --j) {
                            const size_t p = (size_t)i * W + j;
                            for (int n = 0; n < N; ++n) {
                                const REAL a_T = AT[(size_t)e * N + n], a_L = AL[(size_t)e * N + n];
                                const REAL om_r = (j < W - 1) ? om[(p + 1) * N + n] : (REAL)0;
                                const REAL om_b = (i < H - 1) ? om[(p + W) * N + n] : (REAL)0;
                                const REAL go = dbx[p * N + n];
                                REAL cur_om, cur_dbx;
                                if (i == H - 1 && j == W - 1) {
                                    cur_dbx = go; cur_om = go;
                                } else if (i == H - 1) {
                                    const REAL gL = RND(EXPF(RND(dL[(ob + p + 1) * E + e] * a_L)));
                                    cur_dbx = RND(go + RND(gL * dbx[(p + 1) * N + n]));
                                    cur_om  = RND(go + RND(gL * om_r));
                                } else if (j == W - 1) {
                                    const REAL gT = RND(EXPF(RND(dT[(ob + p + W) * E + e] * a_T)));
                                    cur_dbx = RND(go + RND(gT * dbx[(p + W) * N + n]));
                                    cur_om  = RND(go + RND(gT * om_b));
                                } else {
                                    const REAL gL = RND(EXPF(RND(dL[(ob + p + 1) * E + e] * a_L)));
                                    const REAL gT = RND(EXPF(RND(dT[(ob + p + W) * E + e] * a_T)));
                                    cur_dbx = RND(RND(go + RND(gT * dbx[(p + W) * N + n])) + RND(gL * dbx[(p + 1) * N + n]));
                                    const REAL mT = (j == 0) ? (REAL)2 : (REAL)1;
                                    const REAL mL = (i == 0) ? (REAL)2 : (REAL)1;
                                    cur_om = RND(RND(go + RND(RND(mT * gT) * om_b)) + RND(RND(mL * gL) * om_r));
                                }
                                cur_om = RND(cur_om * (REAL)0.5);
                                if (i > 0 && j > 0) cur_dbx = RND(cur_dbx * (REAL)0.5);
                                dbx[p * N + n] = cur_dbx;
                                om[p * N + n] = cur_om;
                                const REAL mTo = (j == 0) ? (REAL)2 : (REAL)1;
                                const REAL mLo = (i == 0) ? (REAL)2 : (REAL)1;
                                ddat[p * N + n] = (i > 0) ? RND(RND(mTo * cur_om) * hs[(p - W) * N + n]) : (REAL)0;
                                ddal[p * N + n] = (j > 0) ? RND(RND(mLo * cur_om) * hs[(p - 1) * N + n]) : (REAL)0;
                            }
                        }
                    }
                    /* wavefront_cuda.py:97-139 and :193-194 */
                    for (int i = 0; i < H; ++i) {
                        for (int j = 0; j < W; ++j) {
                            const size_t p = (size_t)i * W + j;
                            const REAL v_dt = dT[(ob + p) * E + e], v_dl = dL[(ob + p) * E + e];
                            const REAL v_x = x[(ob + p) * E + e];
                            const REAL maskT = (i > 0) ? (REAL)1 : (REAL)0;
                            const REAL maskL = (j > 0 || i == 0) ? (REAL)1 : (REAL)0;
                            ACC s_ddT = 0, s_ddL = 0, s_ddT2 = 0, s_ddL2 = 0, s_xT = 0, s_xL = 0;
                            for (int n = 0; n < N; ++n) {
                                const REAL a_T = AT[(size_t)e * N + n], a_L = AL[(size_t)e * N + n];
                                const REAL gT = RND(EXPF(RND(v_dt * a_T)));
                                const REAL gL = RND(EXPF(RND(v_dl * a_L)));
                                const REAL dzT = RND(ddat[p * N + n] * gT);
                                const REAL dzL = RND(ddal[p * N + n] * gL);
                                accAT[(size_t)e * N + n] += (ACC)RND(dzT * v_dt);
                                accAL[(size_t)e * N + n] += (ACC)RND(dzL * v_dl);
                                s_ddT += (ACC)RND(dzT * a_T);
                                s_ddL += (ACC)RND(dzL * a_L);
                                const REAL hT = RND(dbx[p * N + n] * maskT);
                                const REAL hL = RND(dbx[p * N + n] * maskL);
                                const REAL bT = BT[(ob + p) * N + n], bL = BL[(ob + p) * N + n];
                                s_ddT2 += (ACC)RND(RND(hT * bT) * v_x);
                                s_ddL2 += (ACC)RND(RND(hL * bL) * v_x);
                                const REAL tT = RND(hT * v_dt), tL = RND(hL * v_dl);
                                pBT[p * N + n] += (ACC)RND(tT * v_x);
                                pBL[p * N + n] += (ACC)RND(tL * v_x);
                                s_xT += (ACC)RND(tT * bT);
                                s_xL += (ACC)RND(tL * bL);
                            }
                            d_dT[(ob + p) * E + e] = RND(RND((REAL)s_ddT) + RND((REAL)s_ddT2));
                            d_dL[(ob + p) * E + e] = RND(RND((REAL)s_ddL) + RND((REAL)s_ddL2));
                            const REAL dxs = RND(RND((REAL)s_xT) + RND((REAL)s_xL));
                            d_x[(ob + p) * E + e] = RND(dxs + RND(gy[(ob + p) * E + e] * Dskip[e]));
                        }
                    }
                }
            }
            free(hs); free(dbx); free(om); free(ddat); free(ddal);
        }
        if (fail) break;
        /* sum the per-thread partials over e */
#pragma omp parallel for schedule(static)
        for (long q = 0; q < (long)PN; ++q) {
            ACC sBT = 0, sBL = 0, sC = 0;
            for (int t = 0; t < nthr; ++t) {
                const ACC *pp = part + (size_t)t * 3 * PN;
                sBT += pp[q]; sBL += pp[PN + q]; sC += pp[2 * PN + q];
            }
            d_BT[ob * N + q] = RND((REAL)sBT);
            d_BL[ob * N + q] = RND((REAL)sBL);
            d_C[ob * N + q]  = RND((REAL)sC);
        }
    }
    if (!fail) {
        for (size_t q = 0; q < (size_t)E * N; ++q) { d_AT[q] = RND((REAL)accAT[q]); d_AL[q] = RND((REAL)accAL[q]); }
        for (int e = 0; e < E; ++e) d_D[e] = RND((REAL)accD[e]);
    }
    free(accAT); free(accAL); free(accD); free(part);
    return fail ? -1 : 0;
}
