// Library-level entry points: ABI version and per-thread error messages.
#include "common.cuh"

namespace fmoe {

static thread_local char g_last_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what, cudaGetErrorString(e),
           cudaGetErrorName(e));
  return static_cast<int>(e);
}

}  // namespace fmoe

extern "C" {

int fmoe_abi_version(void) { return 2; }

const char* fmoe_last_error(void) { return fmoe::g_last_error; }

const char* fmoe_status_name(int status) {
  switch (status) {
    case FMOE_OK: return "FMOE_OK";
    case FMOE_ERR_ARG: return "FMOE_ERR_ARG";
    case FMOE_ERR_UNSUPPORTED: return "FMOE_ERR_UNSUPPORTED";
    case FMOE_ERR_WORKSPACE: return "FMOE_ERR_WORKSPACE";
    case FMOE_ERR_DEVICE: return "FMOE_ERR_DEVICE";
    default: return status > 0 ? cudaGetErrorName(static_cast<cudaError_t>(status)) : "FMOE_ERR_?";
  }
}

}  // extern "C"
