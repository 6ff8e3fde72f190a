// Status strings and the per-thread last-error message of the C ABI.
#include "common.cuh"

namespace b200moe {

static thread_local char g_last_error[512] = "";

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(B200MOE_LAUNCH_FAILED, "%s: %s", what, cudaGetErrorString(e));
  return B200MOE_OK;
}

}  // namespace b200moe

extern "C" {

const char* b200moe_status_string(int status) {
  switch (status) {
    case B200MOE_OK: return "ok";
    case B200MOE_BAD_SHAPE: return "unsupported shape";
    case B200MOE_BAD_ALIGN: return "misaligned pointer or stride";
    case B200MOE_BAD_DTYPE: return "unsupported dtype";
    case B200MOE_BAD_ARG: return "bad argument";
    case B200MOE_WORKSPACE_TOO_SMALL: return "workspace too small";
    case B200MOE_LAUNCH_FAILED: return "CUDA launch failed";
    case B200MOE_DEVICE_TIMEOUT: return "device-side wait timed out";
    case B200MOE_UNSUPPORTED_DEVICE: return "unsupported device or driver";
    default: return "unknown status";
  }
}

const char* b200moe_last_error(void) { return b200moe::g_last_error; }

int b200moe_abi_version(void) { return 2; }

}  // extern "C"
