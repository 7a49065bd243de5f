// Version and status strings of the C ABI.
#include "common.cuh"

extern "C" int b200tbe_abi_version(void) { return 3; }

extern "C" const char* b200tbe_status_string(int status) {
  switch (status) {
    case B200TBE_OK: return "ok";
    case B200TBE_ERR_BAD_ARG: return "bad argument";
    case B200TBE_ERR_SCRATCH: return "scratch buffer missing or too small";
    case B200TBE_ERR_LAUNCH: return "CUDA launch failed";
    case B200TBE_ERR_UNSUPPORTED: return "unsupported dtype or shape";
    case B200TBE_ERR_TOO_LARGE: return "size exceeds a fixed capacity";
    default: return "unknown status";
  }
}
