// Library-wide host helpers: last CUDA error string, version.
#include "common.cuh"
#include <string>
#include <mutex>

static std::string g_last_error;
static std::mutex g_err_mu;

int flb_record_cuda_error(cudaError_t e) {
  std::lock_guard<std::mutex> lock(g_err_mu);
  g_last_error = cudaGetErrorString(e);
  return FLB_ERR_CUDA;
}

FLB_API const char* flb_last_cuda_error() {
  std::lock_guard<std::mutex> lock(g_err_mu);
  static thread_local std::string copy;
  copy = g_last_error;
  return copy.c_str();
}

FLB_API int flb_abi_version() { return 1; }
