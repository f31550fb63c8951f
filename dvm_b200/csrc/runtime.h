// Process-wide device state: lazy CUDA initialisation, SM count, launch helpers and event timing.
// Stands in for the GPU half of the reference's System singleton (src/system.cc:282-359) and its thin
// CUDA wrappers (src/runtime.h:29-86).  There is no CPU execution path: using the runtime without a
// CUDA device raises DvmException.
#ifndef DVM_B200_RUNTIME_H_
#define DVM_B200_RUNTIME_H_

#include <cstddef>
#include <cstdint>

namespace dvmb {

class Runtime {
 public:
  static Runtime &Get();
  // Query the current device once.  Throws dvm::DvmException when no CUDA device is usable.
  void EnsureInit();
  bool initialized() const { return initialized_; }
  int sm_count() const { return sm_count_; }
  int device() const { return device_; }
  // Host-only planning (compile without a device, e.g. disassembly tests) uses the B200 figures.
  int sm_count_or_default() const { return initialized_ ? sm_count_ : 148; }

 private:
  bool initialized_ = false;
  int device_ = 0;
  int sm_count_ = 148;
};

}  // namespace dvmb

#endif  // DVM_B200_RUNTIME_H_
