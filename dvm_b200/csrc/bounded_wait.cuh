// Bounded device-side waits shared by the three interpreters / tensor-core kernels.
//
// Every spin on an mbarrier gives up after a time limit (about two seconds): the thread then records
// (code << 24 | block index) in the kernel family's status record and returns, so the kernel always runs to its
// end (with wrong results) and the host reports the failure instead of the GPU hanging.  Once one wait of a launch
// has expired, the other waits of THAT launch return as soon as they reach their slow path; launches are told
// apart by an epoch number the host hands to each launch, so an expiry neither shortens the waits of later
// launches nor of launches running next to it on another stream.  `first_error` keeps the first expiry until
// the host reads and clears it.
#ifndef DVM_B200_BOUNDED_WAIT_CUH_
#define DVM_B200_BOUNDED_WAIT_CUH_

#include <cstdint>

namespace dvmb {

struct WaitStatus {
  unsigned int first_error;   // 0 = ok; else (code << 24 | block index) of the first wait that expired
  unsigned int abort_epoch;   // epoch of the launch whose wait expired last (0 = none yet)
};

constexpr unsigned long long kWaitLimitNs = 2000000000ull;

// Host side: a fresh non-zero epoch for a launch (runtime.cu).
uint32_t NextLaunchEpoch();

#ifdef __CUDACC__
// Spins on `try_once()` until it succeeds, the launch has been marked as failed, or `limit_ns` have passed.
template <typename TryFn>
__device__ __forceinline__ void bounded_spin(TryFn try_once, uint32_t code, WaitStatus *st, uint32_t epoch,
                                             unsigned long long limit_ns) {
  for (int i = 0; i < 4096; ++i)
    if (try_once()) return;
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    if (*reinterpret_cast<volatile unsigned int *>(&st->abort_epoch) == epoch) return;
    for (int i = 0; i < 1024; ++i)
      if (try_once()) return;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 > limit_ns) {
      atomicCAS(&st->first_error, 0u, (code << 24) | (blockIdx.x & 0xffffffu));
      atomicExch(&st->abort_epoch, epoch);
      return;
    }
  }
}
#endif

}  // namespace dvmb

#endif  // DVM_B200_BOUNDED_WAIT_CUH_
