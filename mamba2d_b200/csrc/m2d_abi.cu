// C-ABI housekeeping: version and status strings.
#include "m2d_scan.h"

extern "C" int m2d_abi_version(void) { return M2D_ABI_VERSION; }

extern "C" const char* m2d_strerror(int status) {
    switch (status) {
        case M2D_OK: return "ok";
        case M2D_ERR_NULL: return "a required pointer is NULL";
        case M2D_ERR_DTYPE: return "unknown dtype";
        case M2D_ERR_SHAPE: return "bad shape: need B,E,N >= 1 and H,W >= 2";
        case M2D_ERR_UNSUPPORTED_N: return "state size N > 16 is not supported";
        case M2D_ERR_PITCH: return "BT/BL/C pixel pitch smaller than N";
        case M2D_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
        case M2D_ERR_LAUNCH: return "CUDA launch failed";
        case M2D_ERR_ABI: return "descriptor size does not match this library";
        case M2D_ERR_TOO_LARGE: return "problem exceeds the fixed capacity of this entry point";
        case M2D_ERR_FLAGS: return "unknown bit in desc->flags";
        default: return "unknown status";
    }
}
