// Error reporting and library-level entry points of the natten_b200 C ABI.
#include <mutex>
#include <string>

#include "common.cuh"

namespace b200na {
namespace {
std::mutex g_err_mu;
std::string g_last_cuda_error = "CUDA error (no detail recorded)";
}  // namespace

void set_last_cuda_error(cudaError_t e, const char* where) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  g_last_cuda_error = std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + where;
}
}  // namespace b200na

extern "C" B200NA_API const char* b200na_strerror(int code) {
  switch (code) {
    case B200NA_OK: return "ok";
    case B200NA_ERR_INVALID_ARGUMENT: return "invalid argument (shape, size or flag outside the documented contract)";
    case B200NA_ERR_UNSUPPORTED: return "unsupported configuration for this kernel";
    case B200NA_ERR_ALIGNMENT: return "pointer or row pitch not aligned as required";
    case B200NA_ERR_CUDA: {
      static thread_local std::string copy;
      std::lock_guard<std::mutex> lk(b200na::g_err_mu);
      copy = b200na::g_last_cuda_error;
      return copy.c_str();
    }
    case B200NA_ERR_DEVICE: return "current device is not a compute capability 10.x (B200-class) GPU";
    case B200NA_ERR_WORKSPACE_LIMIT: return "the problem needs more scratch than the 32 MiB built into the library; call b200na_na_forward with your own workspace";
    case B200NA_ERR_KERNEL_TIMEOUT: return "a bounded device-side wait expired; see b200na_device_status";
    default: return "unknown natten_b200 error code";
  }
}

extern "C" B200NA_API int b200na_version(void) { return 100; }
