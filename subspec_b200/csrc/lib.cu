// Library-wide entry points: version string and CUDA error bookkeeping.
#include "common.cuh"

namespace subspec {
namespace {
thread_local cudaError_t g_last_error = cudaSuccess;
}
int cuda_fail(cudaError_t e) {
  g_last_error = e;
  return SUBSPEC_ECUDA;
}
}  // namespace subspec

extern "C" const char* subspec_version(void) { return "subspec_b200 0.1 (sm_100a)"; }

extern "C" const char* subspec_last_cuda_error(void) { return cudaGetErrorString(subspec::g_last_error); }
