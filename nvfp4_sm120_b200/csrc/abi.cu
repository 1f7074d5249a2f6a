// Version and status strings of the C ABI.
#include "nvfp4_b200.h"

extern "C" int nvfp4_version(void) { return NVFP4_ABI_VERSION; }

extern "C" const char* nvfp4_status_string(int code) {
  switch (code) {
    case NVFP4_OK: return "ok";
    case NVFP4_E_NULL: return "a required pointer is NULL";
    case NVFP4_E_SHAPE: return "bad shape: a dimension is not positive or not a multiple the operation needs";
    case NVFP4_E_ALIGN: return "bad alignment of a pointer or leading dimension";
    case NVFP4_E_MODE: return "unknown mode or flag value";
    case NVFP4_E_LAUNCH: return "the CUDA runtime refused the launch";
    case NVFP4_E_DRIVER: return "a CUDA driver entry point needed for TMA descriptors is missing";
    case NVFP4_E_WORKSPACE: return "workspace too small";
    case NVFP4_E_LIMIT: return "size beyond the stated maximum of this entry point";
    default: return "unknown status code";
  }
}
