// Library-level entry points: version, error strings, last CUDA error.
#include "b200_common.cuh"

#include <atomic>

namespace b200 {
static std::atomic<long long> g_launches{0};
void note_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
static thread_local cudaError_t g_last_cuda_error = cudaSuccess;
const char* set_last_cuda_error(cudaError_t e) {
  g_last_cuda_error = e;
  return cudaGetErrorString(e);
}
}  // namespace b200

extern "C" int b200_abi_version(void) { return B200_ABI_VERSION; }

extern "C" const char* b200_strerror(int code) {
  switch (code) {
    case B200_OK: return "ok";
    case B200_EINVAL: return "invalid argument (null pointer, negative size or rank above B200_MAX_DIMS)";
    case B200_EDTYPE: return "dtype combination not implemented by this kernel";
    case B200_ELAUNCH: return "CUDA launch failed (see b200_last_cuda_error)";
    case B200_ESCRATCH: return "scratch buffer missing, too small, or request beyond the static maximum";
    case B200_EALIGN: return "pointer or stride alignment unusable for this path";
    case B200_EDRIVER: return "driver entry point for tensor-map encoding unavailable";
    default: return "unknown b200 error code";
  }
}

extern "C" const char* b200_last_cuda_error(void) { return cudaGetErrorString(b200::g_last_cuda_error); }

extern "C" long long b200_launch_count(void) { return b200::g_launches.load(std::memory_order_relaxed); }
