// Status strings and the per-thread error detail of the C ABI.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace moa {
namespace {
thread_local char g_detail[512] = "";
}

void set_error_detail(const char* what, cudaError_t err) {
  snprintf(g_detail, sizeof(g_detail), "%s: %s (%s)", what, cudaGetErrorName(err), cudaGetErrorString(err));
}
void set_error_text(const char* what) { snprintf(g_detail, sizeof(g_detail), "%s", what); }
}  // namespace moa

extern "C" {

int moa_abi_version(void) { return MOA_ABI_VERSION; }

const char* moa_strerror(int status) {
  switch (status) {
    case MOA_OK: return "ok";
    case MOA_ERR_INVALID_ARG: return "invalid argument";
    case MOA_ERR_UNSUPPORTED: return "unsupported head_dim or dtype";
    case MOA_ERR_CUDA: return "CUDA call failed";
    case MOA_ERR_WORKSPACE: return "workspace missing or too small";
    case MOA_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel ran out";
    case MOA_ERR_TOO_LARGE: return "size beyond the entry point's fixed limit";
    default: return "unknown status";
  }
}

const char* moa_last_error_detail(void) { return moa::g_detail; }

}  // extern "C"
