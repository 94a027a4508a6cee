#include "plan.cuh"
extern "C" uint64_t m2d_scan_bwd_workspace(const m2d_scan_desc* d) { (void)d; return 0; }
extern "C" int m2d_scan_bwd(const m2d_scan_desc* d, void* stream) { (void)d; (void)stream; return M2D_ERR_LAUNCH; }
