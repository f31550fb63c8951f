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
constexpr uint32_t kVmMaxSmemBytes = 216 * 1024;
// dynamic shared memory layout: mbarriers, reduce scratch, then ring stages, temporaries, scalar registers
constexpr uint32_t kVmMaxStages = 8;          // streaming ring depth
constexpr uint32_t kVmMaxSlots = 64;          // resident slots (sets x chunks per CTA)
constexpr uint32_t kVmSmemBarriers = 0;       // full[64] at +0, empty[64] at +512
constexpr uint32_t kVmSmemEmpty = 512;
constexpr uint32_t kVmSmemRed = 1024;         // float[2][32]: warp partials of a CTA-wide reduction
constexpr uint32_t kVmSmemXPart = 1280;       // float[2]: this CTA's partial for the cluster-wide combine
constexpr uint32_t kVmSmemXBar = 1296;        // mbarrier of the cluster-wide combine
constexpr uint32_t kVmSmemTensors = 1536;     // copy of the tensor table (shared-memory reads are faster than indexed parameter reads)
constexpr uint32_t kVmSmemCode = kVmSmemTensors + sizeof(dvmb::TensorDesc) * dvmb::kMaxTensors;   // copy of the program words
// the ring stages follow the program at VmParam::stages_off (the program's capacity is fixed at compile time)
// (one word more than the program: the dispatch loops fetch the word after the one they run, also behind the last END)
constexpr uint32_t VmStagesOffset(uint32_t code_words) { return (kVmSmemCode + 8u * (code_words + 1u) + 127u) & ~127u; }

// Enqueue the vector interpreter. Returns the cudaError_t of the launch (0 = ok).
int LaunchVector(const VmParam &param, uint32_t grid, uint32_t threads, uint32_t smem_bytes, void *stream);   // param.cluster > 1 launches clusters
// Device status word (0 = ok); reading clears it.
unsigned int ReadVectorStatus();
// Enqueue a one-thread kernel whose bounded wait must expire after `limit_ms` (at most 1000) with status code 15.
int LaunchWaitSelfTest(unsigned int limit_ms, void *stream);

}  // namespace dvmb

#endif  // DVM_B200_VM_LAUNCH_H_
