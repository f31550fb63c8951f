// Host-callable entry points of the device interpreters (the counterpart of gpu::InitVM / LaunchVM in the
// reference, src/vm_gpu.h:153-155).
#ifndef DVM_B200_VM_LAUNCH_H_
#define DVM_B200_VM_LAUNCH_H_

#include <cstdint>

#include "isa.h"

namespace dvmb {

constexpr int kVmMaxThreads = 256;
constexpr int kVmMinBlocks = 2;

// Enqueue the vector interpreter. Returns the cudaError_t of the launch (0 = ok).
int LaunchVector(const VmParam &param, uint32_t grid, uint32_t threads, void *stream);

}  // namespace dvmb

#endif  // DVM_B200_VM_LAUNCH_H_
