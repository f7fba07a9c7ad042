// Status strings, ABI version and the per-thread record of the last CUDA runtime error.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace keepvq {

static thread_local char g_last_cuda_error[256] = "";

int note_cuda_error(cudaError_t err) {
  const char* name = cudaGetErrorName(err);
  const char* text = cudaGetErrorString(err);
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s", name ? name : "?", text ? text : "?");
  return KEEPVQ_ERR_LAUNCH;
}

}  // namespace keepvq

extern "C" {

int keepvq_abi_version(void) { return KEEPVQ_ABI_VERSION; }

const char* keepvq_last_cuda_error(void) { return keepvq::g_last_cuda_error; }

const char* keepvq_status_string(int status) {
  switch (status) {
    case KEEPVQ_OK: return "ok";
    case KEEPVQ_ERR_NULL: return "a required pointer is NULL";
    case KEEPVQ_ERR_SHAPE: return "inconsistent sizes";
    case KEEPVQ_ERR_DTYPE: return "unknown dtype or code width";
    case KEEPVQ_ERR_ALIGN: return "pointer or row pitch is not aligned as the kernel needs";
    case KEEPVQ_ERR_UNSUPPORTED: return "no kernel serves this combination";
    case KEEPVQ_ERR_LAUNCH: return "CUDA launch failed";
    case KEEPVQ_ERR_CAPACITY: return "a fixed-size buffer is too small";
    default: return "unknown status";
  }
}

}  // extern "C"
