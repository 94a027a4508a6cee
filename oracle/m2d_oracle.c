/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the Mamba2D wavefront 2-D selective scan
 * (forward + backward), used as the checker in tests/, in the smoke check and as the timed
 * CPU baseline of bench.py.  The shipped library never links or calls this file.
 *
 * The reference project has no CPU implementation of the recurrence (its launcher
 * models/kernels/wf_cuda/wf_cuda.cu:163-218 has no host branch), so this file restates the
 * kernel bodies and the PyTorch glue around them; see m2d_oracle_impl.h for line citations.
 *
 * Pinning: the reference ships no tests or golden vectors for this path.  The restatement is
 * pinned (a) against the reference's own kernel source executed on the CPU through a
 * thread-index shim (oracle/build_ref.py builds that into oracle/_ref/), (b) against the
 * reference's own PyTorch post-kernel code, and (c) against fp64 autograd through a naive loop.
 * The fixtures produced by (a) and (b) are committed under tests/golden/.
 *
 * Exported variants:
 *   *_f64   double arithmetic (accuracy oracle)
 *   *_f32   float arithmetic, float accumulators (reference-precision; the timed CPU baseline)
 *   *_bf16e float storage holding bf16-representable values, every operation rounded to bf16
 *           (emulates the reference running with scalar_t = BFloat16)
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC m2d_oracle.c -o libm2d_oracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_round(float v)
{
    uint32_t u;
    memcpy(&u, &v, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return v; /* NaN */
    const uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    u &= 0xffff0000u;
    memcpy(&v, &u, 4);
    return v;
}

/* ---- double ---- */
#define REAL double
#define ACC double
#define RND(v) (v)
#define EXPF(v) exp(v)
#define FN(name) name##_f64
#include "m2d_oracle_impl.h"
#undef REAL
#undef ACC
#undef RND
#undef EXPF
#undef FN

/* ---- float ---- */
#define REAL float
#define ACC float
#define RND(v) (v)
#define EXPF(v) expf(v)
#define FN(name) name##_f32
#include "m2d_oracle_impl.h"
#undef REAL
#undef ACC
#undef RND
#undef EXPF
#undef FN

/* ---- bf16 emulation (values stored as float) ---- */
#define REAL float
#define ACC float
#define RND(v) bf16_round((float)(v))
#define EXPF(v) expf(v)
#define FN(name) name##_bf16e
#include "m2d_oracle_impl.h"
#undef REAL
#undef ACC
#undef RND
#undef EXPF
#undef FN

int m2d_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void m2d_oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
