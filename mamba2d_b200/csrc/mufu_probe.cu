// Stand-alone probe (not part of the library): issue rates of ex2.approx, fma.rn.f32, fma.rn.f32x2 and
// integer adds on the current GPU, alone and interleaved.  It answers which instructions overlap with
// the MUFU exponential, which is what bounds the scan at N = 16.  Build and run:
//     python -m mamba2d_b200.build --probe && ./mamba2d_b200/mufu_probe
#include <cstdio>
#include <cuda_runtime.h>
// what overlaps with MUFU.EX2?  all kernels: 8 independent chains per thread.
#define EX2(r) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(r))
#define FMA(r,b,c) asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(r) : "f"(b), "f"(c))
#define FMA2(r,b,c) asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(r) : "l"(b), "l"(c))
#define IADD(r,b) asm volatile("add.s32 %0, %0, %1;" : "+r"(r) : "r"(b))
template<int K, int MODE> __global__ void k_mix(float* out, int iters) {
    float a[8]; float f[8]; unsigned long long p[8]; int q[8];
    for (int i=0;i<8;i++) { a[i] = -0.001f*(threadIdx.x+i); f[i]=0.5f+i; p[i] = 0x3f0000003f000000ull + i; q[i]=i; }
    float b = 0.999f, c = 0.001f; unsigned long long b2 = 0x3f7fbe773f7fbe77ull, c2 = 0x3a83126f3a83126full; int ib = 3;
    for (int it=0; it<iters; ++it) {
#pragma unroll
        for (int i=0;i<8;i++) {
            if (MODE != 3) EX2(a[i]);
#pragma unroll
            for (int k=0;k<K;k++) {
                if (MODE==0 || MODE==3) FMA(f[(i+k)&7], b, c);
                if (MODE==1) FMA2(p[(i+k)&7], b2, c2);
                if (MODE==2) IADD(q[(i+k)&7], ib);
            }
        }
    }
    float s=0; for (int i=0;i<8;i++) s+=a[i]+f[i]+(float)p[i]+q[i]; out[blockIdx.x*blockDim.x+threadIdx.x]=s;
}
// packed half-precision exponentials: two results per instruction
template<int BF> __global__ void k_ex2_packed(float* out, int iters) {
    unsigned a[8]; for (int i=0;i<8;i++) a[i] = (BF ? 0xbf00bf00u : 0xb800b800u) + i;
    for (int it=0; it<iters; ++it) {
#pragma unroll
        for (int i=0;i<8;i++) {
            if (BF) asm volatile("ex2.approx.ftz.bf16x2 %0, %0;" : "+r"(a[i]));
            else asm volatile("ex2.approx.f16x2 %0, %0;" : "+r"(a[i]));
        }
    }
    unsigned s=0; for (int i=0;i<8;i++) s+=a[i]; out[blockIdx.x*blockDim.x+threadIdx.x]=(float)s;
}
template<typename F> float timeit(F f) {
    cudaEvent_t e0,e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    f(); cudaDeviceSynchronize();
    cudaEventRecord(e0); f(); cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms,e0,e1); return ms;
}
int main() {
    int sms; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    const int iters = 4096; float* out; cudaMalloc(&out, sms*8*512*4);
    const double clk = 1.965e9;
    for (int occ = 0; occ < 2; ++occ) {
        const int blocks = sms * (occ ? 1 : 4), threads = 512;   // 16 or 4 warps per scheduler
        const double warps_per_smsp_total = (double)blocks*threads/32/ (sms*4);
        auto rep = [&](const char* name, float ms, int K) {
            // cycles per (ex2 + K others) group per scheduler
            double groups = warps_per_smsp_total * iters * 8;
            printf("%-28s K=%d  %.2f cycles per group per scheduler (warps/sched=%.0f)\n", name, K, ms*1e-3*clk/groups, warps_per_smsp_total);
        };
        rep("ex2 + K ffma", timeit([&]{k_mix<0,0><<<blocks,threads>>>(out,iters);}), 0);
        rep("ex2 + K ffma", timeit([&]{k_mix<4,0><<<blocks,threads>>>(out,iters);}), 4);
        rep("ex2 + K ffma", timeit([&]{k_mix<8,0><<<blocks,threads>>>(out,iters);}), 8);
        rep("ex2 + K ffma2", timeit([&]{k_mix<4,1><<<blocks,threads>>>(out,iters);}), 4);
        rep("ex2 + K ffma2", timeit([&]{k_mix<8,1><<<blocks,threads>>>(out,iters);}), 8);
        rep("ex2 + K iadd", timeit([&]{k_mix<4,2><<<blocks,threads>>>(out,iters);}), 4);
        rep("ex2 + K iadd", timeit([&]{k_mix<8,2><<<blocks,threads>>>(out,iters);}), 8);
        rep("ex2.f16x2 (2 results/instr)", timeit([&]{k_ex2_packed<0><<<blocks,threads>>>(out,iters);}), 0);
        rep("ex2.bf16x2 (2 results/instr)", timeit([&]{k_ex2_packed<1><<<blocks,threads>>>(out,iters);}), 0);
        rep("K ffma only", timeit([&]{k_mix<8,3><<<blocks,threads>>>(out,iters);}), 8);
        rep("K ffma2 only", timeit([&]{k_mix<8,1><<<blocks,threads>>>(out,iters);}), 8);
    }
    return 0;
}
