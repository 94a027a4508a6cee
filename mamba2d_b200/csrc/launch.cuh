// Pieces the scan entry points share: the argument block and the launch.
#pragma once

#include "plan.cuh"
#include "sweep_fwd.cuh"

namespace m2d {

// Everything of the argument block that comes straight from the descriptor and the plan.
inline void fill_common_args(ScanArgs& a, const m2d_scan_desc* d, const Plan& pl) {
    a = ScanArgs{};
    a.B = d->B; a.H = d->H; a.W = d->W; a.E = d->E; a.N = d->N;
    a.dir = (d->flags & M2D_SCAN_REVERSE) ? -1 : 1;
    a.x = d->x; a.dT = d->dT; a.dL = d->dL; a.AT = d->AT; a.AL = d->AL;
    a.BT = d->BT; a.BL = d->BL; a.C = d->C; a.D = d->D;
    a.pBT = d->BT_pitch; a.pBL = d->BL_pitch; a.pC = d->C_pitch;
    a.Rb = pl.Rb; a.nbands = pl.nbands;
    a.chain = pl.chain;
    a.act = (d->flags & M2D_SCAN_GELU_OUT) ? 1 : 0;
    a.a_log = (d->flags & M2D_SCAN_A_LOG) ? 1 : 0;
    const bool hook = (d->flags & M2D_SCAN_TEST_WITHHOLD) != 0;
    a.withhold = hook ? 1 : 0;
    a.wait_limit = hook ? (1 << 9) : kWaitPolls;
}

// Launch a sweep kernel on the plan's grid.  CTAs of a chain wait on one another, so every CTA of a
// chained launch must be resident at the same time: a cooperative launch guarantees that or fails
// cleanly, and the chain is shortened until the device accepts it (the workspace layout depends on
// the planned chain only through "is there one", not on its length).  A shortened chain goes through
// the same bound as a planned one (bound_chain).
inline int launch_sweep_kernel(void (*kern)(const ScanArgs), ScanArgs& a, const Plan& pl, int steps_per_row, cudaStream_t st) {
    dim3 block(pl.warps * 32);
    if (pl.smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess)
        return M2D_ERR_LAUNCH;
    if (a.chain > 1) {
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, (int)block.x, pl.smem) != cudaSuccess || per_sm < 1)
            return M2D_ERR_LAUNCH;
        const long long fit = (long long)per_sm * sm_count() / ((long long)pl.grid_x * pl.groups);
        if (fit < a.chain) a.chain = bound_chain(fit, pl.nbands, steps_per_row, pl.Rb);
        for (;;) {
            dim3 grid(pl.grid_x * a.chain, pl.groups);
            void* args[] = {&a};
            const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), grid, block, args, pl.smem, st);
            if (e == cudaSuccess) return M2D_OK;
            cudaGetLastError();
            if (e != cudaErrorCooperativeLaunchTooLarge || a.chain == 1) return M2D_ERR_LAUNCH;
            a.chain = bound_chain(a.chain > 2 ? a.chain - a.chain / 4 - 1 : 1, pl.nbands, steps_per_row, pl.Rb);
        }
    }
    dim3 grid(pl.grid_x, pl.groups);
    kern<<<grid, block, pl.smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? M2D_OK : M2D_ERR_LAUNCH;
}

}  // namespace m2d
