#include "runtime.h"

#include <cuda_runtime.h>

#include <string>

#include "../../include/dvm.h"

namespace dvmb {

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
