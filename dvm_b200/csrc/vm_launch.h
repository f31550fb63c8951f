// Host-callable entry points of the device interpreters (the counterpart of gpu::InitVM / LaunchVM in the
// reference, src/vm_gpu.h:153-155).
#ifndef DVM_B200_VM_LAUNCH_H_
#define DVM_B200_VM_LAUNCH_H_

#include <cstdint>

#include "isa.h"

namespace dvmb {

constexpr int kVmMaxThreads = 512;            // consumer threads per CTA (a producer warp is added on top)
constexpr int kVmMinBlocks = 1;
constexpr int kVmFlatThreads = 256;           // consumer threads of a reduce-free launch
constexpr uint32_t kVmMaxSmemBytes = 200 * 1024;
// dynamic shared memory layout: mbarriers, reduce scratch, then ring stages, temporaries, scalar registers
constexpr uint32_t kVmSmemBarriers = 0;       // full[8] at +0, empty[8] at +64
constexpr uint32_t kVmSmemRed = 128;          // float[2][32]
constexpr uint32_t kVmSmemStages = 512;
constexpr uint32_t kVmMaxStages = 8;

// Enqueue the vector interpreter. Returns the cudaError_t of the launch (0 = ok).
int LaunchVector(const VmParam &param, uint32_t grid, uint32_t threads, uint32_t smem_bytes, void *stream);
// Device status word (0 = ok); reading clears it.
unsigned int ReadVectorStatus();

}  // namespace dvmb

#endif  // DVM_B200_VM_LAUNCH_H_
