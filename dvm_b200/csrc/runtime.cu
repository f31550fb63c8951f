#include "runtime.h"

#include <cuda_runtime.h>

#include <atomic>
#include <string>

#include "../../include/dvm.h"
#include "bounded_wait.cuh"

namespace dvmb {

uint32_t NextLaunchEpoch() {
  static std::atomic<uint32_t> counter{0};
  uint32_t e = counter.fetch_add(1, std::memory_order_relaxed) + 1;
  if (e == 0) e = counter.fetch_add(1, std::memory_order_relaxed) + 1;   // 0 means "no launch has failed yet"
  return e;
}

Runtime &Runtime::Get() {
  static Runtime rt;
  return rt;
}

void Runtime::EnsureInit() {
  if (initialized_) return;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) {
    std::string msg = std::string("no usable CUDA device: ") + cudaGetErrorString(err);
    cudaGetLastError();
    dvm::DvmException(msg.c_str());
  }
  cudaDeviceProp prop;
  err = cudaGetDeviceProperties(&prop, dev);
  if (err != cudaSuccess) {
    std::string msg = std::string("cudaGetDeviceProperties failed: ") + cudaGetErrorString(err);
    dvm::DvmException(msg.c_str());
  }
  if (prop.major < 10) {
    std::string msg = std::string("dvm-b200 needs an sm_100 class GPU, found ") + prop.name;
    dvm::DvmException(msg.c_str());
  }
  device_ = dev;
  sm_count_ = prop.multiProcessorCount;
  initialized_ = true;
}

}  // namespace dvmb
