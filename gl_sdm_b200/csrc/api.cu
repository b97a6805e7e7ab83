// Status strings, ABI version and the per-thread CUDA error note.
#include <stdio.h>

#include <atomic>

#include "common.cuh"

namespace glsdm {
namespace {
thread_local char g_last_cuda_error[256] = "";
std::atomic<unsigned long long> g_launches{0};
}

void count_launches(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

void note_cuda_error(cudaError_t err, const char* where) {
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s (%s)", where,
           cudaGetErrorName(err), cudaGetErrorString(err));
}
}  // namespace glsdm

extern "C" int glsdm_abi_version(void) { return 1; }

extern "C" const char* glsdm_status_string(int status) {
  switch (status) {
    case GLSDM_OK: return "ok";
    case GLSDM_ERR_ARGUMENT: return "invalid argument (null or misaligned pointer, or inconsistent sizes)";
    case GLSDM_ERR_UNSUPPORTED: return "shape not supported by the sm_100a kernels";
    case GLSDM_ERR_WORKSPACE: return "workspace smaller than the matching *_workspace_bytes()";
    case GLSDM_ERR_CUDA: return "CUDA runtime error (see glsdm_last_cuda_error)";
    case GLSDM_ERR_LIMIT: return "size beyond a built-in capacity";
    default: return "unknown status";
  }
}

extern "C" const char* glsdm_last_cuda_error(void) { return glsdm::g_last_cuda_error; }

extern "C" uint64_t glsdm_kernel_launches(void) { return glsdm::g_launches.load(std::memory_order_relaxed); }
