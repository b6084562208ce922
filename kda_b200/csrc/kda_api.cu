// Library-level entry points: ABI version and error text.
#include <cuda_runtime.h>

#include "kda_b200.h"

extern "C" int kda_b200_abi_version(void) { return KDA_B200_ABI_VERSION; }

extern "C" const char* kda_b200_strerror(int code) {
  switch (code) {
    case KDA_OK: return "ok";
    case KDA_E_NULL: return "a required pointer is NULL";
    case KDA_E_SHAPE: return "unsupported or inconsistent sizes";
    case KDA_E_DTYPE: return "unsupported io_dtype for this entry point";
    case KDA_E_ALIGN: return "a pointer is not 16-byte aligned";
    case KDA_E_WORKSPACE: return "workspace too small";
    case KDA_E_DEVICE: return "the current device is not sm_100";
    case KDA_E_LIMIT: return "size beyond a documented fixed maximum";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown kda_b200 error code";
}
