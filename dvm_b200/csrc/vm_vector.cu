// Persistent bytecode interpreter for fused vector graphs on sm_100a.
//
// One kernel executes every fused elementwise / broadcast / reduce graph the host compiler emits (the role
// of dvm_vm_gpu in the reference, src/vm_gpu.cu:1552-1617).  Differences in kind, not in degree:
//   * a producer warp streams the input chunks of upcoming tiles into a shared-memory ring with bulk async
//     copies (cp.async.bulk, completion on mbarriers), so HBM latency is hidden by the ring depth and not
//     by occupancy; the consumer warps read each operand straight from the ring, converting on the fly;
//   * the running value of the fused chain stays in registers (an 8-lane accumulator); nothing is written
//     back to shared memory between ops except values with several later uses (thread-private temporaries);
//   * results leave the SM once, as 16-byte (fp32) / 8-byte (16-bit) coalesced stores.
// Per-op arithmetic follows the reference's device functors (src/vm_gpu.cu:198-329): IEEE fp32 math,
// fp16/bf16 values rounded to storage precision after every op, float->int by truncation, compares
// yielding 1/0 in the operand representation, max/min as `a > b ? a : b` / `a < b ? a : b`.
// Every wait on an mbarrier is bounded: on expiry the thread records a status code and leaves.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "bounded_wait.cuh"
#include "isa.h"
#include "vm_launch.h"
#include "vm_ops.cuh"
#include "vm_vector_regs.h"

namespace dvmb {

__device__ WaitStatus g_vm_status = {0u, 0u};

namespace {


// ---- mbarrier / bulk copy -------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t addr) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t addr, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(addr), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t addr, uint32_t parity) {
  uint32_t ok;
  asm volatile(
    "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(ok)
    : "r"(addr), "r"(parity)
    : "memory");
  return ok != 0;
}
// Bounded wait (bounded_wait.cuh): gives up after about two seconds and records `code` in the status record.
// (A warp that has to wait sleeps between its polls: polled back to back, the producer warps' waits alone were a fifth of
// the instructions an issue-bound kernel executed.)
constexpr uint32_t kPollSleepNs = 200;
__device__ __noinline__ void mbar_wait_slow(uint32_t addr, uint32_t parity, uint32_t code, uint32_t epoch) {
  bounded_spin(
    [&]() {
      if (mbar_try_wait(addr, parity)) return true;
      __nanosleep(kPollSleepNs);
      return false;
    },
    code, &g_vm_status, epoch, kWaitLimitNs);
}
__device__ __forceinline__ void mbar_wait(uint32_t addr, uint32_t parity, uint32_t code, uint32_t epoch) {
  if (mbar_try_wait(addr, parity)) return;
  mbar_wait_slow(addr, parity, code, epoch);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(mbar)
               : "memory");
}

// ---- cluster-wide combine (distributed shared memory) ------------------------------------------------
__device__ __forceinline__ uint32_t map_shared_rank(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote_release(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t addr, uint32_t parity) {
  uint32_t ok;
  asm volatile(
    "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(ok)
    : "r"(addr), "r"(parity)
    : "memory");
  return ok != 0;
}
// Bounded like every other wait of the kernel (status code 3).
__device__ __noinline__ void mbar_wait_cluster(uint32_t addr, uint32_t parity, uint32_t epoch) {
  bounded_spin([&]() { return mbar_try_wait_cluster(addr, parity); }, 3u, &g_vm_status, epoch, kWaitLimitNs);
}
__device__ __forceinline__ float ld_shared_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

// ---- addressing -----------------------------------------------------------------------------------

constexpr int kGranules = kLanes / 4;

// Per-thread position inside the iteration space.  Granule g of the thread starts `in_chunk0 + g * 4 * tg`
// elements into the chunk.
struct Pos {
  uint32_t k[kMaxKept];   // kept coordinates of this thread's group
  uint32_t e_start;       // first element (inside the group) of the current chunk
  uint32_t in_chunk0;     // element index of granule 0 inside its chunk (the current round's offset included)
  uint32_t gstep;         // 4 * tg
  uint32_t chunk_valid;   // valid elements of the current chunk up to the end of the current round
  bool gvalid;
};

__device__ __forceinline__ void split_enum(const VmParam &P, uint32_t e, uint32_t (&c)[kMaxEnum]) {
#pragma unroll
  for (int j = kMaxEnum - 1; j > 0; --j) {
    uint32_t s = P.enum_size[j];
    uint32_t q = e / s;
    c[j] = e - q * s;
    e = q;
  }
  c[0] = e;
}

__device__ __forceinline__ uint32_t kept_offset(const TensorDesc &td, const uint32_t (&k)[kMaxKept]) {
  uint32_t off = 0;
#pragma unroll
  for (int j = 0; j < kMaxKept; ++j) off += k[j] * td.kstride[j];
  return off;
}

__device__ __forceinline__ uint32_t enum_offset(const TensorDesc &td, const uint32_t (&c)[kMaxEnum]) {
  uint32_t off = 0;
#pragma unroll
  for (int j = 0; j < kMaxEnum; ++j) off += c[j] * td.estride[j];
  return off;
}

// Element offset and inner stride of a granule that starts at element `e0` of the group.
__device__ __forceinline__ uint32_t granule_offset(const VmParam &P, const TensorDesc &td, uint32_t koff, uint32_t e0,
                                                   uint32_t *istride) {
  const uint32_t mode = td.mode;
  *istride = 1;
  if (mode == AM_DENSE) return koff + e0;
  if (mode == AM_GRANULE) {
    uint32_t c[kMaxEnum];
    split_enum(P, e0, c);
    *istride = td.estride[kMaxEnum - 1];
    return koff + enum_offset(td, c);
  }
  *istride = 0;
  return koff;
}

// General fetch of the 16 lanes of tensor `slot` for this thread: from the ring stage when the tensor is
// staged and the granule lies inside the bulk-copied part, else straight from global memory, element by
// element where the layout or a ragged tail needs it.
__device__ __noinline__ void fetch_tensor(const VmParam &P, uint32_t slot, const Pos &pos, uint32_t stage_saddr,
                                          uint32_t (&out)[kLanes]) {
  const TensorDesc &td = P.tensor[slot];
  const uint32_t dtype = td.dtype, mode = td.mode;
  const uint32_t sh = item_shift(dtype);
  const bool staged = td.ring_off != kNoRing;
  // elements of the chunk that the bulk copy delivered (whole 16-byte units)
  const uint32_t bulk_elems = staged ? (((pos.chunk_valid << sh) & ~15u) >> sh) : 0u;
  const uint8_t *base = reinterpret_cast<const uint8_t *>(td.ptr);
  const uint32_t koff = kept_offset(td, pos.k);
#pragma unroll 1
  for (int g = 0; g < kGranules; ++g) {
    uint32_t *o = &out[4 * g];
    const uint32_t ic = pos.in_chunk0 + (uint32_t)g * pos.gstep;
    if (staged && ic + 4 <= bulk_elems) {
      unpack4(dtype, sload4(dtype, stage_saddr + td.ring_off + (ic << sh)), o);
      continue;
    }
    const int32_t left = (int32_t)pos.chunk_valid - (int32_t)ic;
    const int nv = !pos.gvalid ? 0 : (left >= 4 ? 4 : (left > 0 ? left : 0));
    const uint32_t e0 = pos.e_start + ic;
    if (mode == AM_ELEMENT) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        o[i] = 0;
        if (i < nv) {
          uint32_t c[kMaxEnum];
          split_enum(P, e0 + i, c);
          o[i] = load_elem(dtype, base, koff + enum_offset(td, c));
        }
      }
      continue;
    }
    uint32_t istride;
    const uint32_t off = granule_offset(P, td, koff, nv > 0 ? e0 : 0u, &istride);
    if (td.vec_ok && nv == 4) {
      unpack4(dtype, gload4(dtype, base, off), o);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = i < nv ? load_elem(dtype, base, off + i * istride) : 0u;
    }
  }
}

__device__ __noinline__ void store_tensor(const VmParam &P, uint32_t slot, const Pos &pos,
                                          const uint32_t (&val)[kLanes]) {
  const TensorDesc &td = P.tensor[slot];
  uint8_t *base = reinterpret_cast<uint8_t *>(td.ptr);
  const uint32_t dtype = td.dtype, mode = td.mode;
  const uint32_t koff = kept_offset(td, pos.k);
#pragma unroll 1
  for (int g = 0; g < kGranules; ++g) {
    const uint32_t ic = pos.in_chunk0 + (uint32_t)g * pos.gstep;
    const int32_t left = (int32_t)pos.chunk_valid - (int32_t)ic;
    const int nv = !pos.gvalid ? 0 : (left >= 4 ? 4 : (left > 0 ? left : 0));
    const uint32_t e0 = pos.e_start + ic;
    const uint32_t *v = &val[4 * g];
    if (mode == AM_ELEMENT) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (i < nv) {
          uint32_t c[kMaxEnum];
          split_enum(P, e0 + i, c);
          store_elem(dtype, base, koff + enum_offset(td, c), v[i]);
        }
      }
      continue;
    }
    uint32_t istride;
    const uint32_t off = granule_offset(P, td, koff, nv > 0 ? e0 : 0u, &istride);
    if (td.vec_ok && nv == 4) {
      gstore4(dtype, base, off, v);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < nv) store_elem(dtype, base, off + i * istride, v[i]);
    }
  }
}

__device__ __forceinline__ void decompose_group(const VmParam &P, uint32_t gi, uint32_t (&k)[kMaxKept]) {
#pragma unroll
  for (int j = kMaxKept - 1; j > 0; --j) {
    uint32_t sz = P.kept_size[j];
    uint32_t q = gi / sz;
    k[j] = gi - q * sz;
    gi = q;
  }
  k[0] = gi;
}

}  // namespace

namespace {
// kRounds: chunks may hold several rounds (VmParam::rounds > 1).  Only the instantiations with the larger register budget
// carry the round bookkeeping; the others run one round per chunk and the compiler folds the round loop away.
template <bool kResident, bool kCoords, bool kRounds, int kModeOnly = 0>
__device__ __forceinline__ void vm_vector_body(const VmParam &P, const uint32_t epoch) {
  asm volatile(DV_DECLARE);
  asm volatile(DV_LN(DV_SPLATLANE, "va") DV_LN(DV_SPLATLANE, "vb")
               "mov.b32 vp0, %0;\n\tmov.b32 vp1, %0;\n\tmov.b32 vp2, %0;\n\tmov.b32 vp3, %0;" ::"r"(0u));
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t tid = threadIdx.x;
  const uint32_t T = P.tcons;   // consumer threads (a multiple of 32; threads past tg * groups_per_cta idle)
  // (kModeOnly 1: an instantiation for reduce-free launches only, without the group loop and the reduction words; 2: for
  // group launches only)
  constexpr bool kFlatOnly = kModeOnly == 1;
  const bool flat = kFlatOnly || (kModeOnly != 2 && P.mode == VM_FLAT);
  const uint32_t S = P.num_stages;
  const bool ring = P.stage_bytes != 0;
  const uint32_t ngb = flat ? 1u : (P.num_groups + P.groups_per_cta - 1) / P.groups_per_cta;
  // CTAs of a cluster share a group: CTA `rank` of unit `blockIdx.x / cluster` owns chunks [rank * cpc, ...)
  // (only the instantiations with the larger register budget carry the cluster bookkeeping)
  const uint32_t cluster = (kResident || kRounds) ? P.cluster : 1u, rank = cluster > 1 ? blockIdx.x % cluster : 0u;
  const bool resident = kResident;
  const uint32_t gb_begin = flat ? 0u : blockIdx.x / cluster, gb_step = flat ? 1u : gridDim.x / cluster;
  const uint32_t ch_begin = flat ? blockIdx.x : rank * P.cpc, ch_step = flat ? gridDim.x : 1u;
  const uint32_t ch_end = flat ? P.chunks : min(P.chunks, (rank + 1u) * P.cpc);

  // the program and the tensor table are read from shared memory in the loops below
  for (uint32_t i = tid; i < P.n_code; i += blockDim.x) reinterpret_cast<uint64_t *>(smem + kVmSmemCode)[i] = P.code[i];
  for (uint32_t i = tid; i < P.n_tensors * (sizeof(TensorDesc) / 4u); i += blockDim.x)
    reinterpret_cast<uint32_t *>(smem + kVmSmemTensors)[i] = reinterpret_cast<const uint32_t *>(P.tensor)[i];
  if (tid == 0) {
    for (uint32_t s = 0; s < S; ++s) {
      mbar_init(smem_base + kVmSmemBarriers + 8 * s, 1);        // full: one arrival (the producer) + tx bytes
      mbar_init(smem_base + kVmSmemEmpty + 8 * s, T >> 5);      // empty: one arrival per consumer warp
    }
    mbar_init(smem_base + kVmSmemXBar, cluster);                 // one arrival per CTA of the cluster
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (cluster > 1) {
    // every CTA's barriers exist before a peer signals them
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  } else {
    __syncthreads();
  }

  // =============================== producer warp ===============================
  // One warp feeds the ring: it walks the same tile sequence as the consumers, one stage after the other.
  if (tid >= T) {
    const uint32_t plane = tid - T;
    if (resident) {
      // Resident groups: slot set * cpc + ci holds chunk ci of this CTA for the whole group; lane (ci % 32) fills it
      // once, when the previous occupant has been released in its last phase.
      uint32_t mask = 0;
      for (uint32_t ph = 0; ph < P.num_body; ++ph) mask |= P.body_ring_mask[ph];
      uint32_t set = 0, use = 0;
      for (uint32_t gb = gb_begin; gb < ngb; gb += gb_step) {
        uint32_t k[kMaxKept];
        decompose_group(P, gb, k);
        for (uint32_t ch = ch_begin + plane; ch < ch_end; ch += 32u) {
          const uint32_t slot = set * P.cpc + (ch - ch_begin);
          const uint32_t full = smem_base + kVmSmemBarriers + 8 * slot;
          mbar_wait(smem_base + kVmSmemEmpty + 8 * slot, (use & 1u) ^ 1u, 1, epoch);
          const uint32_t e_start = ch * P.chunk_elems;
          const uint32_t valid = min(P.chunk_elems, P.group_elems - e_start);
          // one copy per staged tensor and round of the chunk (a round is one contiguous run of every tensor)
          uint32_t total = 0;
          for (uint32_t r = 0; r * P.round_elems < valid; ++r) {
            const uint32_t rv = min(P.round_elems, valid - r * P.round_elems);
            for (uint32_t m = mask; m; m &= m - 1) total += (rv << item_shift(P.tensor[__ffs(m) - 1].dtype)) & ~15u;
          }
          if (total == 0) {
            mbar_arrive(full);
            continue;
          }
          mbar_arrive_expect_tx(full, total);
          for (uint32_t r = 0; r * P.round_elems < valid; ++r) {
            const uint32_t rv = min(P.round_elems, valid - r * P.round_elems);
            uint32_t c[kMaxEnum] = {0, 0, 0, e_start + r * P.round_elems};
            if (P.need_coords) split_enum(P, c[3], c);
            for (uint32_t m = mask; m; m &= m - 1) {
              const TensorDesc &td = P.tensor[__ffs(m) - 1];
              const uint32_t sh = item_shift(td.dtype);
              const uint32_t bytes = (rv << sh) & ~15u;
              if (bytes == 0) continue;
              const uint32_t off = kept_offset(td, k) + enum_offset(td, c);
              bulk_g2s(smem_base + P.stages_off + slot * P.stage_bytes + td.ring_off + ((r * P.round_elems) << sh),
                       reinterpret_cast<const uint8_t *>(td.ptr) + ((size_t)off << sh), bytes, full);
            }
          }
        }
        if (++set == P.sets) {
          set = 0;
          ++use;
        }
      }
      return;
    }
    // Streaming ring.  The warp walks the consumers' tile sequence in step: every lane waits for the stage to be
    // released, lane 0 posts the byte count, and lane (t * rounds + r) issues the bulk copy of round r of the t-th staged
    // tensor (a round is one contiguous run of the tensor; the rounds of a chunk lie back to back in the stage).  Each
    // lane keeps its tensor's base, strides and element size in registers; its coordinates advance incrementally.
    uint32_t umask = 0;
    for (uint32_t ph = 0; ph < P.num_body; ++ph) umask |= P.body_ring_mask[ph];
    if (umask == 0) return;
    const uint32_t R = P.rounds;
    const uint32_t my_ti = plane / R, my_r = plane - my_ti * R;
    const bool has = my_ti < (uint32_t)__popc(umask);
    const uint32_t my_t = has ? (uint32_t)__fns(umask, 0, my_ti + 1) : (uint32_t)(__ffs(umask) - 1);
    const TensorDesc &td = P.tensor[my_t];
    const uint32_t sh = item_shift(td.dtype);
    const uint32_t my_ring = td.ring_off + ((my_r * P.round_elems) << sh);
    const uint8_t *my_base = reinterpret_cast<const uint8_t *>(td.ptr);
    uint32_t es[kMaxEnum];
#pragma unroll
    for (int j = 0; j < kMaxEnum; ++j) es[j] = td.estride[j];
    const uint32_t step_elems = ch_step * P.chunk_elems;
    uint32_t stage = 0, parity = 1;   // first wait on a fresh "empty" barrier passes at once
    for (uint32_t gb = gb_begin; gb < ngb; gb += gb_step) {
      uint32_t k[kMaxKept];
      decompose_group(P, gb, k);   // groups_per_cta == 1 whenever the ring is on
      const uint32_t koff = kept_offset(td, k);
      for (uint32_t ph = 0; ph < P.num_body; ++ph) {
        const uint32_t mask = P.body_ring_mask[ph];
        if (mask == 0) continue;
        const bool mine = has && ((mask >> my_t) & 1u);
        // this lane's round starts my_r * round_elems into the chunk
        uint32_t r_start = ch_begin * P.chunk_elems + my_r * P.round_elems;
        uint32_t c[kMaxEnum] = {0, 0, 0, r_start};
        if (P.need_coords) split_enum(P, c[3], c);
        for (uint32_t ch = ch_begin; ch < ch_end; ch += ch_step, r_start += step_elems) {
          const uint32_t full = smem_base + kVmSmemBarriers + 8 * stage;
          // everything the copy needs is worked out before the wait, so that the copy leaves right after the release
          const uint32_t valid = r_start < P.group_elems ? min(P.round_elems, P.group_elems - r_start) : 0u;
          const uint32_t bytes = mine ? ((valid << sh) & ~15u) : 0u;
          const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
          const uint32_t off = koff + c[0] * es[0] + c[1] * es[1] + c[2] * es[2] + c[3] * es[3];
          const uint32_t dst = smem_base + P.stages_off + stage * P.stage_bytes + my_ring;
          const uint8_t *const src = my_base + ((size_t)off << sh);
          mbar_wait(smem_base + kVmSmemEmpty + 8 * stage, parity, 1, epoch);
          if (plane == 0) {
            if (total == 0) {
              mbar_arrive(full);
            } else {
              mbar_arrive_expect_tx(full, total);
            }
          }
          __syncwarp();
          if (bytes != 0) bulk_g2s(dst, src, bytes, full);
          // next chunk of this CTA: advance the innermost coordinate and carry
          c[3] += step_elems;
          if (P.need_coords) {
#pragma unroll
            for (int j = kMaxEnum - 1; j > 0; --j)
              while (c[j] >= P.enum_size[j]) {
                c[j] -= P.enum_size[j];
                c[j - 1] += 1u;
              }
          }
          if (++stage == S) {
            stage = 0;
            parity ^= 1u;
          }
        }
      }
    }
    return;
  }

  // =============================== consumer warps ===============================
  // The vector state (accumulator va, operand register vb, reduction partials vp) lives in PTX
  // registers that only inline assembly names.  The compiler therefore carries no vector state across
  // the dispatch loop (nothing to copy at the switch merge), and ptxas keeps each one in a fixed register.
  float *red_buf = reinterpret_cast<float *>(smem + kVmSmemRed);
  const uint32_t temps_saddr = smem_base + P.stages_off + S * P.stage_bytes;
  const uint32_t sregs_saddr = temps_saddr + P.num_temps * T * (4u * kLanes);
  const uint32_t tg = P.tg;
  const uint32_t lane_in_group = flat ? tid : tid % tg;
  const uint32_t group_in_cta = flat ? 0 : tid / tg;

  uint32_t sacc[1] = {0};
  uint32_t sel_mask = 0;   // lanes whose select condition held
  uint32_t red_par = 0;
  uint32_t ring_stage = 0, ring_parity = 0;
  uint32_t xphase = 0, xpar = 0;       // cluster-combine phase and buffer
  uint32_t res_set = 0, res_use = 0;   // resident slot set of the current group and how often it was used
  bool first_group = true;
  Pos pos;
  uint32_t cc[kMaxEnum] = {0, 0, 0, 0};   // coordinates of the chunk's first element (only when some tensor needs them)
  pos.gstep = 4u * tg;
  const uint32_t lane4 = 4u * lane_in_group;   // the thread's first element inside a round
  pos.in_chunk0 = lane4;

  auto temp_addr = [&](uint32_t k, uint32_t g) { return temps_saddr + ((k * kGranules + g) * T + tid) * 16u; };
  auto sreg_addr = [&](uint32_t k) { return sregs_saddr + (k * T + tid) * 4u; };
  const uint32_t code_saddr = smem_base + kVmSmemCode;
  const TensorDesc *const tdesc = reinterpret_cast<const TensorDesc *>(smem + kVmSmemTensors);
  auto lds64 = [](uint32_t a) {
    uint64_t v;
    asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"(a));
    return v;
  };
  auto lds64x2 = [](uint32_t a, uint32_t &lo, uint32_t &hi) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(a));
  };
  auto lds32 = [](uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
  };
  auto get_part = [](uint32_t slot) {
    uint32_t v;
    switch (slot) {
      case 0: asm volatile("mov.b32 %0, vp0;" : "=r"(v)); break;
      case 1: asm volatile("mov.b32 %0, vp1;" : "=r"(v)); break;
      case 2: asm volatile("mov.b32 %0, vp2;" : "=r"(v)); break;
      default: asm volatile("mov.b32 %0, vp3;" : "=r"(v)); break;
    }
    return u2f(v);
  };
  auto set_part = [](uint32_t slot, float f) {
    const uint32_t v = f2u(f);
    switch (slot) {
      case 0: asm volatile("mov.b32 vp0, %0;" ::"r"(v)); break;
      case 1: asm volatile("mov.b32 vp1, %0;" ::"r"(v)); break;
      case 2: asm volatile("mov.b32 vp2, %0;" ::"r"(v)); break;
      default: asm volatile("mov.b32 vp3, %0;" ::"r"(v)); break;
    }
  };

  for (uint32_t gb = gb_begin; gb < ngb; gb += gb_step) {
    if (!first_group && ++res_set == P.sets) {
      res_set = 0;
      ++res_use;
    }
    first_group = false;
    {
      uint32_t gi = gb * P.groups_per_cta + group_in_cta;
      pos.gvalid = gi < P.num_groups && group_in_cta < P.groups_per_cta && (flat || lane_in_group < tg);
      decompose_group(P, pos.gvalid ? gi : 0u, pos.k);
    }
    for (uint32_t ph = 0; ph <= P.num_body; ++ph) {
      // ---------------- scalar side: PRO_ph ----------------
      if (!((P.pro_skip_mask >> ph) & 1u)) {
        uint32_t spc = code_saddr + 8u * P.sec[2 * ph];
        uint32_t wlo, whi, xlo, xhi;   // the current word and the next one, already on its way
        lds64x2(spc, wlo, whi);
        for (;; wlo = xlo, whi = xhi) {
          const uint32_t sop = whi & 0xffu;   // a flat ScalarOp id, or the opcode of a word that takes the general path
          spc += 8u;
          lds64x2(spc, xlo, xhi);
          const uint32_t sub = (whi >> 8) & 0xffu;
          const uint32_t okind = (whi >> 16) & 0xfu, oidx = (whi >> 20) & 0xfu;
          // operand of the flat forms (immediate, scalar register, accumulator), fetched without a branch
          const uint32_t sv = lds32(okind == K_SREG ? sreg_addr(oidx) : code_saddr);
          const uint32_t sb = okind == K_SREG ? sv : (okind == K_ACC ? sacc[0] : wlo);
          switch (sop) {
            case OP_END: goto scalar_done;   // (inside the switch: one indexed jump per word and no test in front of it)
            case SOP_COPY: sacc[0] = sb; break;
            case SOP_MOV: asm volatile("st.shared.u32 [%0], %1;" ::"r"(sreg_addr((whi >> 24) & 0xfu)), "r"(sacc[0]) : "memory"); break;
            case SOP_RINIT: set_part(sub & 3u, red_identity(sub >> 4)); break;
            case SOP_MOV_END:
              asm volatile("st.shared.u32 [%0], %1;" ::"r"(sreg_addr((whi >> 24) & 0xfu)), "r"(sacc[0]) : "memory");
              goto scalar_done;
            case SOP_RINIT_END: set_part(sub & 3u, red_identity(sub >> 4)); goto scalar_done;
            case SOP_RSTD_FAST: {
              // each operation rounded on its own, as in the four separate words
              const float v = __fadd_rn(__fmul_rn(u2f(sacc[0]), u2f(wlo)), u2f(xlo));
              sacc[0] = f2u(fast_div(1.0f, sqrtf(v)));
              spc += 8u;   // the next word only carried the second immediate
              lds64x2(spc, xlo, xhi);
              break;
            }
            case SOP_RFIN: {
              if (kFlatOnly) break;   // (a reduce-free launch has no reductions to finish)
              const uint32_t kind = sub >> 4;
              float v = get_part(sub & 3u);
              set_part(sub & 3u, red_identity(kind));
              if (tg <= 32) {
                // several groups per warp: tg is a power of two; one group per CTA: tg may be any size up to a warp, and
                // the lanes past it hold the identity
                for (uint32_t o = P.groups_per_cta == 1 ? 16u : tg >> 1; o > 0; o >>= 1)
                  v = red_combine(kind, v, __shfl_xor_sync(0xffffffffu, v, o));
              } else {
#pragma unroll
                for (uint32_t o = 16; o > 0; o >>= 1) v = red_combine(kind, v, __shfl_xor_sync(0xffffffffu, v, o));
                if ((tid & 31u) == 0) red_buf[red_par * 32 + (tid >> 5)] = v;
                asm volatile("bar.sync 1, %0;" ::"r"(T) : "memory");   // consumer warps only
                // every warp's partial (at most 16 warps) is read at once and combined as a tree
                const uint32_t nw = T >> 5;
                if (nw == 4u) {
                  // four warps: the same tree without its identity leaves, (p0 + p2) + (p1 + p3)
                  const float4 q = *reinterpret_cast<const float4 *>(&red_buf[red_par * 32]);
                  v = red_combine(kind, red_combine(kind, q.x, q.z), red_combine(kind, q.y, q.w));
                  red_par ^= 1u;
                  if (cluster == 1) {
                    if ((xhi & 0xffu) == SOP_RSTD_FAST) {
                      // the word behind is the fused reciprocal root (its second immediate in the word after it): done
                      // here, and so is a closing move behind that - a normalisation's scalar section in one dispatch
                      // instead of three, with the operations and roundings of the separate words
                      uint32_t dlo, dhi, mlo, mhi;
                      lds64x2(spc + 8u, dlo, dhi);
                      lds64x2(spc + 16u, mlo, mhi);
                      const float t = __fadd_rn(__fmul_rn(v, u2f(xlo)), u2f(dlo));
                      sacc[0] = f2u(fast_div(1.0f, sqrtf(t)));
                      if ((mhi & 0xffu) == SOP_MOV_END) {
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(sreg_addr((mhi >> 24) & 0xfu)), "r"(sacc[0]) : "memory");
                        goto scalar_done;
                      }
                      spc += 16u;
                      xlo = mlo;
                      xhi = mhi;
                      break;
                    }
                    sacc[0] = f2u(v);
                    break;
                  }
                } else {
                float pv[16];
#pragma unroll
                for (uint32_t wi = 0; wi < 16; ++wi) pv[wi] = wi < nw ? red_buf[red_par * 32 + wi] : red_identity(kind);
                if (kind == R_SUM) {
#pragma unroll
                  for (int h = 8; h > 0; h >>= 1)
#pragma unroll
                    for (int i = 0; i < h; ++i) pv[i] += pv[i + h];
                } else {
#pragma unroll
                  for (int h = 8; h > 0; h >>= 1)
#pragma unroll
                    for (int i = 0; i < h; ++i) pv[i] = red_combine(kind, pv[i], pv[i + h]);
                }
                v = pv[0];
                red_par ^= 1u;
                }
              }
              if (cluster > 1) {
                // combine the CTA totals of the cluster in rank order: publish ours, signal every CTA, read all
                float *xpart = reinterpret_cast<float *>(smem + kVmSmemXPart);
                if (tid == 0) {
                  xpart[xpar] = v;
                  for (uint32_t r = 0; r < cluster; ++r) mbar_arrive_remote_release(map_shared_rank(smem_base + kVmSmemXBar, r));
                }
                mbar_wait_cluster(smem_base + kVmSmemXBar, xphase, epoch);
                xphase ^= 1u;
                v = ld_shared_cluster_f32(map_shared_rank(smem_base + kVmSmemXPart + 4u * xpar, 0));
                for (uint32_t r = 1; r < cluster; ++r)
                  v = red_combine(kind, v, ld_shared_cluster_f32(map_shared_rank(smem_base + kVmSmemXPart + 4u * xpar, r)));
                xpar ^= 1u;
              }
              sacc[0] = f2u(v);
              break;
            }
            case SOP_RFIN2: {
              if (kFlatOnly) break;
              // (sums only, more than one warp per group: the lowering sees to both)
              const uint32_t pa = sub & 3u, pb = (sub >> 2) & 3u;
              float v0 = get_part(pa), v1 = get_part(pb);
              set_part(pa, 0.0f);
              set_part(pb, 0.0f);
#pragma unroll
              for (uint32_t o = 16; o > 0; o >>= 1) {
                v0 += __shfl_xor_sync(0xffffffffu, v0, o);
                v1 += __shfl_xor_sync(0xffffffffu, v1, o);
              }
              if ((tid & 31u) == 0) {
                red_buf[red_par * 32 + (tid >> 5)] = v0;
                red_buf[red_par * 32 + 16 + (tid >> 5)] = v1;
              }
              asm volatile("bar.sync 1, %0;" ::"r"(T) : "memory");   // consumer warps only
              const uint32_t nw = T >> 5;
              float pv[16], pw[16];
#pragma unroll
              for (uint32_t wi = 0; wi < 16; ++wi) {
                pv[wi] = wi < nw ? red_buf[red_par * 32 + wi] : 0.0f;
                pw[wi] = wi < nw ? red_buf[red_par * 32 + 16 + wi] : 0.0f;
              }
#pragma unroll
              for (int h = 8; h > 0; h >>= 1)
#pragma unroll
                for (int i = 0; i < h; ++i) {
                  pv[i] += pv[i + h];
                  pw[i] += pw[i + h];
                }
              red_par ^= 1u;
              asm volatile("st.shared.u32 [%0], %1;" ::"r"(sreg_addr((whi >> 24) & 0xfu)), "r"(f2u(pv[0])) : "memory");
              asm volatile("st.shared.u32 [%0], %1;" ::"r"(sreg_addr(oidx)), "r"(f2u(pw[0])) : "memory");
              sacc[0] = f2u(pw[0]);
              break;
            }
#define DV_SUN(K) case SOP_UN_FIRST + K: apply_un<1>(K, sacc); break;
            DV_SUN(U_SQRT) DV_SUN(U_ABS) DV_SUN(U_LOG) DV_SUN(U_EXP) DV_SUN(U_ROUND) DV_SUN(U_FLOOR) DV_SUN(U_CEIL)
            DV_SUN(U_TRUNC) DV_SUN(U_ISFINITE) DV_SUN(U_ABS_I) DV_SUN(U_EXP_FAST) DV_SUN(U_NOP)
#undef DV_SUN
#define DV_SBIN(K) case SOP_BIN_FIRST + K: apply_bin<1>(K, sacc, SplatOperand{sb}); break;
            DV_SBIN(B_ADD) DV_SBIN(B_SUB) DV_SBIN(B_MUL) DV_SBIN(B_DIV) DV_SBIN(B_MAX) DV_SBIN(B_MIN) DV_SBIN(B_POW)
            DV_SBIN(B_RSUB) DV_SBIN(B_RDIV) DV_SBIN(B_ADD_I) DV_SBIN(B_SUB_I) DV_SBIN(B_MUL_I) DV_SBIN(B_MAX_I)
            DV_SBIN(B_MIN_I) DV_SBIN(B_RSUB_I) DV_SBIN(B_DIV_FAST) DV_SBIN(B_RDIV_FAST)
#undef DV_SBIN
#define DV_SCVT(K) case SOP_CVT_FIRST + K: apply_cvt<1>(K, sacc); break;
            DV_SCVT(V_F2I) DV_SCVT(V_I2F) DV_SCVT(V_NEZ_F) DV_SCVT(V_NEZ_I)
#undef DV_SCVT
            default: {
              // general path: the word keeps its opcode (tensor operands, rounding to 16 bit, compares, selects, stores)
              const uint64_t w = ((uint64_t)whi << 32) | wlo;
              uint32_t gb_ = sb;
              if (okind == K_TENSOR && (sop == OP_COPY || sop == OP_BIN || sop == OP_CMP || sop == OP_SEL)) {
                const TensorDesc &td = tdesc[oidx];
                gb_ = load_elem(td.dtype, reinterpret_cast<const uint8_t *>(td.ptr), kept_offset(td, pos.k));
              }
              const SplatOperand bo{gb_};
              switch (sop) {
                case OP_ST: {
                  const TensorDesc &td = tdesc[sub];
                  if (lane_in_group == 0 && pos.gvalid && rank == 0 && (!flat || blockIdx.x == 0))
                    store_elem(td.dtype, reinterpret_cast<uint8_t *>(td.ptr), kept_offset(td, pos.k), sacc[0]);
                  break;
                }
                case OP_COPY: sacc[0] = gb_; break;
                case OP_UN: apply_un<1>(sub, sacc); apply_round<1>(DVMB_RND(w), sacc); break;
                case OP_BIN: apply_bin<1>(sub, sacc, bo); apply_round<1>(DVMB_RND(w), sacc); break;
                case OP_CMP: apply_cmp<1>(sub, DVMB_ISINT(w), sacc, bo); break;
                case OP_SEL: {
                  uint32_t sc[1];
                  sc[0] = lds32(sreg_addr(sub & 15u));
                  apply_sel<1>(DVMB_ISINT(w), DVMB_DST(w) & 1u, sacc, bo, sc);
                  break;
                }
                case OP_CVT: apply_cvt<1>(sub, sacc); apply_round<1>(DVMB_RND(w), sacc); break;
                default: break;
              }
              break;
            }
          }
        }
      }
    scalar_done:
      if (ph == P.num_body) break;
      // ---------------- vector side: BODY_ph over the chunks ----------------
      const uint32_t body_pc = P.sec[2 * ph + 1], body_pc_any = P.sec_any[ph];
      const bool staged_body = ring && (resident || P.body_ring_mask[ph] != 0);
      const bool body_coords = ((P.body_coords_mask >> ph) & 1u) != 0;   // only vector stores to strided tensors read cc
      const bool release_slots = !resident || ph + 1 == P.num_body;
      for (uint32_t ch = ch_begin; ch < ch_end; ch += ch_step) {
        pos.e_start = ch * P.chunk_elems;
        const uint32_t chunk_total = min(P.chunk_elems, P.group_elems - pos.e_start);
        if (kCoords && body_coords) {
          if (ch == ch_begin) {
            split_enum(P, pos.e_start, cc);
          } else if (ch_step > 1u) {
            // the rounds of the previous chunk advanced the coordinates by one chunk; skip the other CTAs' chunks
            cc[3] += (ch_step - 1u) * P.chunk_elems;
#pragma unroll
            for (int j = kMaxEnum - 1; j > 0; --j)
              while (cc[j] >= P.enum_size[j]) {
                cc[j] -= P.enum_size[j];
                cc[j - 1] += 1u;
              }
          }
        }
        uint32_t stage_saddr = 0, empty_bar = 0;
        if (staged_body) {
          if (resident) {
            // the chunk's own slot: filled once per group, waited for in the first phase only
            const uint32_t slot = res_set * P.cpc + (ch - ch_begin);
            stage_saddr = smem_base + P.stages_off + slot * P.stage_bytes;
            empty_bar = smem_base + kVmSmemEmpty + 8 * slot;
            if (ph == 0) mbar_wait(smem_base + kVmSmemBarriers + 8 * slot, res_use & 1u, 2, epoch);
          } else {
            stage_saddr = smem_base + P.stages_off + ring_stage * P.stage_bytes;
            empty_bar = smem_base + kVmSmemEmpty + 8 * ring_stage;
            mbar_wait(smem_base + kVmSmemBarriers + 8 * ring_stage, ring_parity, 2, epoch);
            if (++ring_stage == S) {
              ring_stage = 0;
              ring_parity ^= 1u;
            }
          }
        }
        // A chunk is `rounds` rounds of round_elems elements, back to back in the stage; the body runs once per round on
        // the thread's 16 lanes of it.  Rounds in which every lane of every thread is valid: the first n_full ones.
        const uint32_t n_full = kRounds ? chunk_total / P.round_elems : 1u;
        const uint32_t n_rounds = kRounds ? n_full + (n_full * P.round_elems < chunk_total ? 1u : 0u) : 1u;
        // A thread outside every group of this CTA (the tail of the last warp of a group that does not fill it) has no
        // round to run.  It goes straight to the release, where its warp meets again: walking the rounds to their END
        // word beside the warp's working threads made that warp the last one to release every stage.
        for (uint32_t rnd = (kRounds && !pos.gvalid) ? n_rounds : 0u; rnd < n_rounds; ++rnd) {
        pos.in_chunk0 = kRounds ? lane4 + rnd * P.round_elems : lane4;
        pos.chunk_valid = kRounds ? min(chunk_total, (rnd + 1u) * P.round_elems) : chunk_total;
        // every lane of this thread lies inside the round: the vector fast paths apply
        const bool full_tile = pos.gvalid && pos.in_chunk0 + 3u * pos.gstep + 4u <= pos.chunk_valid;
        // a thread without a single lane inside the round has nothing to fetch, add or store
        const bool lane_active = pos.gvalid && pos.in_chunk0 < pos.chunk_valid;
        // full rounds run the variant without per-lane tests; a thread with nothing to do starts at the final END
        uint32_t pc_saddr = code_saddr + 8u * (full_tile ? body_pc : (lane_active ? body_pc_any : P.n_code - 1u));
        uint32_t ulo, uhi, nlo, nhi;   // the current micro-op and the next one, already on its way
        lds64x2(pc_saddr, ulo, uhi);
        uint32_t rnd_begin = rnd;
        for (;; ulo = nlo, uhi = nhi) {
          const uint32_t uh = ulo & 0xffu;
          const uint32_t aux = (ulo >> 8) & 0xffu;
          const uint32_t arg = ulo >> 16;
          pc_saddr += 8u;
          lds64x2(pc_saddr, nlo, nhi);
          switch (uh) {
            case UH_END: goto body_done;
            // ---------------- operand fetches ----------------
#define DV_LDR_CASE(H, REG, MACRO, SHL)                                                                        \
  case H: {                                                                                                 \
    const uint32_t a0 = stage_saddr + (arg << 4) + (SHL(pos.in_chunk0)), gs = SHL(pos.gstep);               \
    MACRO(REG, a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                      \
    continue;                                                                                               \
  }
#define DV_SHL0(x) (x)
#define DV_SHL1(x) ((x) << 1)
#define DV_SHL2(x) ((x) << 2)
            DV_LDR_CASE(UH_LDR_F32, "vb", DV_LDR32, DV_SHL2)
            DV_LDR_CASE(UH_LDR_F16, "vb", DV_LDR_F16, DV_SHL1)
            DV_LDR_CASE(UH_LDR_BF16, "vb", DV_LDR_BF16, DV_SHL1)
            DV_LDR_CASE(UH_LDR_U8, "vb", DV_LDR_U8, DV_SHL0)
            DV_LDR_CASE(UH_LDRA_F32, "va", DV_LDR32, DV_SHL2)
            DV_LDR_CASE(UH_LDRA_F16, "va", DV_LDR_F16, DV_SHL1)
            DV_LDR_CASE(UH_LDRA_BF16, "va", DV_LDR_BF16, DV_SHL1)
            DV_LDR_CASE(UH_LDRA_U8, "va", DV_LDR_U8, DV_SHL0)
#undef DV_LDR_CASE
            // ---------------- fused forms: ring operand + the operation that follows it ----------------
#define DV_LDX_CASE(H, REG, MACRO, SHL, ...)                                                                   \
  case H: {                                                                                                 \
    const uint32_t a0 = stage_saddr + (arg << 4) + (SHL(pos.in_chunk0)), gs = SHL(pos.gstep);               \
    MACRO(REG, a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                      \
    __VA_ARGS__                                                                                             \
    continue;                                                                                               \
  }
#define DV_LDX_TYPES(FIRST, REG, ...)                                              \
  DV_LDX_CASE(FIRST + FT_F32, REG, DV_LDR32, DV_SHL2, __VA_ARGS__)                 \
  DV_LDX_CASE(FIRST + FT_F16, REG, DV_LDR_F16, DV_SHL1, __VA_ARGS__)               \
  DV_LDX_CASE(FIRST + FT_BF16, REG, DV_LDR_BF16, DV_SHL1, __VA_ARGS__)
            DV_LDX_TYPES(UH_LDOP_FIRST + FO_ADD * 3, "vb", asm volatile(DV_LN(DV_BINVRN_LANE, "add.rn.f32"));)
            DV_LDX_TYPES(UH_LDOP_FIRST + FO_SUB * 3, "vb", asm volatile(DV_LN(DV_BINVRN_LANE, "sub.rn.f32"));)
            DV_LDX_TYPES(UH_LDOP_FIRST + FO_MUL * 3, "vb", asm volatile(DV_LN(DV_BINVRN_LANE, "mul.rn.f32"));)
            // load + reduce forms: as the only micro-op of a body (UA_LOOP) they run every remaining full round of the
            // chunk inside one dispatch; the partial grows round by round exactly as it does with one dispatch per round
#define DV_LDRED_CASE(H, MACRO, SHL, PRE, OPS)                                                                \
  case H: {                                                                                                 \
    uint32_t a0 = stage_saddr + (arg << 4) + (SHL(pos.in_chunk0));                                          \
    const uint32_t gs = SHL(pos.gstep);                                                                     \
    PRE                                                                                                     \
    for (;;) {                                                                                              \
      if (kRounds && (aux & UA_LOOP) && rnd + 1u < n_full) {                                                \
        /* two rounds at a time, one per vector register; the partial takes them in their order */          \
        const uint32_t a1 = a0 + SHL(P.round_elems);                                                        \
        MACRO("va", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                 \
        MACRO("vb", a1, a1 + gs, a1 + 2u * gs, a1 + 3u * gs)                                                 \
        OPS("va")                                                                                           \
        OPS("vb")                                                                                           \
        ++rnd;                                                                                              \
        if (rnd + 1u >= n_full) break;                                                                      \
        ++rnd;                                                                                              \
        a0 = a1 + SHL(P.round_elems);                                                                       \
        continue;                                                                                           \
      }                                                                                                     \
      MACRO("va", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                   \
      OPS("va")                                                                                             \
      if (!kRounds || !(aux & UA_LOOP) || rnd + 1u >= n_full) break;                                        \
      ++rnd;                                                                                                \
      a0 += SHL(P.round_elems);                                                                             \
    }                                                                                                       \
    if (aux & UA_LAST) goto body_done;                                                                      \
    continue;                                                                                               \
  }
#define DV_LDRED_TYPES(FIRST, PRE, OPS)                                            \
  DV_LDRED_CASE(FIRST + FT_F32, DV_LDR32, DV_SHL2, PRE, OPS)                       \
  DV_LDRED_CASE(FIRST + FT_F16, DV_LDR_F16, DV_SHL1, PRE, OPS)                     \
  DV_LDRED_CASE(FIRST + FT_BF16, DV_LDR_BF16, DV_SHL1, PRE, OPS)
#define DV_OPS_SUM0(R) asm volatile(DV_TREE16R(DV_ADDRN2, "0", R));
#define DV_OPS_VAR0(R) asm volatile(DV_LNR(DV_CSQR_LANE_R, R, "")::"r"(sv_)); asm volatile(DV_TREE16R(DV_ADDRN2, "0", R));
#define DV_OPS_VAR1(R) asm volatile(DV_LNR(DV_CSQR_LANE_R, R, "")::"r"(sv_)); asm volatile(DV_TREE16R(DV_ADDRN2, "1", R));
            DV_LDRED_TYPES(UH_LDSUM_FIRST, , DV_OPS_SUM0)
            DV_LDX_TYPES(UH_LDSUBR_FIRST, "va", {
              const uint32_t sv_ = lds32(sreg_addr(uhi));
              asm volatile(DV_LN(DV_BINS_LANE, "sub.rn.f32")::"r"(sv_));
            })
            // two ring operands of one type and their sum / difference / product
#define DV_LD2_CASE(H, MACRO, SHL, OPASM)                                                                      \
  case H: {                                                                                                 \
    const uint32_t o0 = stage_saddr + (SHL(pos.in_chunk0)), gs = SHL(pos.gstep);                            \
    const uint32_t a0 = o0 + (arg << 4), b0 = o0 + (uhi << 4);                                              \
    MACRO("va", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                     \
    MACRO("vb", b0, b0 + gs, b0 + 2u * gs, b0 + 3u * gs)                                                     \
    asm volatile(DV_LN(DV_BINVRN_LANE, OPASM));                                                             \
    continue;                                                                                               \
  }
#define DV_LD2_TYPES(FO, OPASM)                                                   \
  DV_LD2_CASE(UH_LD2OP_FIRST + FO * 3 + FT_F32, DV_LDR32, DV_SHL2, OPASM)         \
  DV_LD2_CASE(UH_LD2OP_FIRST + FO * 3 + FT_F16, DV_LDR_F16, DV_SHL1, OPASM)       \
  DV_LD2_CASE(UH_LD2OP_FIRST + FO * 3 + FT_BF16, DV_LDR_BF16, DV_SHL1, OPASM)
            DV_LD2_TYPES(FO_ADD, "add.rn.f32")
            DV_LD2_TYPES(FO_SUB, "sub.rn.f32")
            DV_LD2_TYPES(FO_MUL, "mul.rn.f32")
#undef DV_LD2_TYPES
#undef DV_LD2_CASE
            case UH_MULR_MULR_ADDR: {
              const uint32_t s1_ = lds32(sreg_addr(arg & 0xfu)), s2_ = lds32(sreg_addr((arg >> 4) & 0xfu)), s3_ = lds32(sreg_addr(arg >> 8));
              asm volatile(DV_LN(DV_BINS3_LANE, "mul.rn.f32", "mul.rn.f32", "add.rn.f32")::"r"(s1_), "r"(s2_), "r"(s3_));
              continue;
            }
            DV_LDRED_TYPES(UH_LDVAR_FIRST, const uint32_t sv_ = lds32(sreg_addr(uhi));, DV_OPS_VAR0)
            DV_LDRED_TYPES(UH_LDVAR_FIRST + 3, const uint32_t sv_ = lds32(sreg_addr(uhi));, DV_OPS_VAR1)
            // deviations from a group scalar, their sum and the sum of their squares in one pass
#define DV_OPS_STATS(R)                                                                                  \
  asm volatile(DV_LNR(DV_SUBS_LANE_R, R, "")::"r"(sv_));                                                   \
  asm volatile(DV_TREE16R(DV_ADDRN2, "0", R));                                                             \
  asm volatile(DV_LNR(DV_SQRRN_LANE_R, R, ""));                                                            \
  asm volatile(DV_TREE16R(DV_ADDRN2, "1", R));
            DV_LDRED_TYPES(UH_LDSTATS_FIRST, const uint32_t sv_ = lds32(sreg_addr(uhi));, DV_OPS_STATS)
#undef DV_OPS_STATS
#undef DV_OPS_SUM0
#undef DV_OPS_VAR0
#undef DV_OPS_VAR1
#undef DV_LDRED_TYPES
#undef DV_LDRED_CASE
            DV_LDX_TYPES(UH_LDNORM_FIRST, "va", {
              const uint32_t s0_ = lds32(sreg_addr(uhi & 0xfu)), s1_ = lds32(sreg_addr((uhi >> 4) & 0xfu));
              const uint32_t s2_ = lds32(sreg_addr((uhi >> 8) & 0xfu)), s3_ = lds32(sreg_addr((uhi >> 12) & 0xfu));
              asm volatile(DV_LN(DV_NORM_LANE, "")::"r"(s0_), "r"(s1_), "r"(s2_), "r"(s3_));
            })
            DV_LDX_TYPES(UH_LDSIGM_FIRST, "va", asm volatile(DV_LN(DV_SIGM_LANE, ""));)
            // a whole normalisation body in one micro-op: ring operand -> ((x - s0) * s1) * s2 + s3 -> vector store in the
            // operand's own type, for every remaining full round of the chunk when it is the body's only micro-op
#define DVMB_ST "st.global"   /* (a cache-streaming form, st.global.cs, measured the same on a three-pass normalisation) */
#define DV_STV32R(R, P0, GS)                                                                                          \
  asm volatile(DVMB_ST ".v4.b32 [%0], {" R "0," R "1," R "2," R "3};\n\t" DVMB_ST ".v4.b32 [%1], {" R "4," R "5," R "6," R "7};\n\t" \
               DVMB_ST ".v4.b32 [%2], {" R "8," R "9," R "10," R "11};\n\t" DVMB_ST ".v4.b32 [%3], {" R "12," R "13," R "14," R "15};" ::"l"(P0), \
               "l"(P0 + GS), "l"(P0 + 2u * GS), "l"(P0 + 3u * GS)                                                      \
               : "memory");
#define DV_STV16R(CVT, R, P0, GS)                                                                             \
  asm volatile("{\n\t.reg .b32 t0, t1;\n\t"                                                                   \
               CVT " t0, " R "1, " R "0;\n\t" CVT " t1, " R "3, " R "2;\n\t" DVMB_ST ".v2.b32 [%0], {t0,t1};\n\t"           \
               CVT " t0, " R "5, " R "4;\n\t" CVT " t1, " R "7, " R "6;\n\t" DVMB_ST ".v2.b32 [%1], {t0,t1};\n\t"           \
               CVT " t0, " R "9, " R "8;\n\t" CVT " t1, " R "11, " R "10;\n\t" DVMB_ST ".v2.b32 [%2], {t0,t1};\n\t"         \
               CVT " t0, " R "13, " R "12;\n\t" CVT " t1, " R "15, " R "14;\n\t" DVMB_ST ".v2.b32 [%3], {t0,t1};\n\t}" ::"l"(P0), \
               "l"(P0 + GS), "l"(P0 + 2u * GS), "l"(P0 + 3u * GS)                                            \
               : "memory");
#define DV_STV32(P0, GS) DV_STV32R("va", P0, GS)
#define DV_STV16(CVT, P0, GS) DV_STV16R(CVT, "va", P0, GS)
#define DV_NORM_SCALARS                                                                                     \
  const uint64_t s0w_ = (static_cast<uint64_t>(s0_) << 32) | s0_, s1w_ = (static_cast<uint64_t>(s1_) << 32) | s1_, \
                 s2w_ = (static_cast<uint64_t>(s2_) << 32) | s2_;
#define DV_NORM_APPLY(R) asm volatile(DV_NORM2_R(R)::"l"(s0w_), "l"(s1w_), "l"(s2w_), "r"(s3_));
#define DV_LDNORMST_CASE(H, MACRO, SHL, ELEM, STORE)                                                          \
  case H: {                                                                                                 \
    const TensorDesc &td = tdesc[(uhi >> 16) & 0xfu];                                                       \
    const uint32_t s0_ = lds32(sreg_addr(uhi & 0xfu)), s1_ = lds32(sreg_addr((uhi >> 4) & 0xfu));           \
    const uint32_t s2_ = lds32(sreg_addr((uhi >> 8) & 0xfu)), s3_ = lds32(sreg_addr((uhi >> 12) & 0xfu));   \
    DV_NORM_SCALARS                                                                                         \
    uint32_t a0 = stage_saddr + (arg << 4) + (SHL(pos.in_chunk0));                                          \
    const uint32_t gs = SHL(pos.gstep), ge = pos.gstep;                                                     \
    const bool by_coords = kCoords && td.mode != AM_DENSE;                                                  \
    ELEM *const base = reinterpret_cast<ELEM *>(td.ptr) + kept_offset(td, pos.k);                           \
    ELEM *p0 = base + (by_coords ? enum_offset(td, cc) + lane4 : pos.e_start + pos.in_chunk0);              \
    /* the result pointer of the round after the one at p0 (the coordinates move on by one round) */       \
    auto next_round = [&](ELEM *p) -> ELEM * {                                                              \
      if (!by_coords) return p + P.round_elems;                                                             \
      rnd_begin += 1u;   /* (the code behind the body adds one round to the coordinates itself) */          \
      cc[3] += P.round_elems;                                                                               \
      _Pragma("unroll") for (int j = kMaxEnum - 1; j > 0; --j) while (cc[j] >= P.enum_size[j]) {            \
        cc[j] -= P.enum_size[j];                                                                            \
        cc[j - 1] += 1u;                                                                                    \
      }                                                                                                     \
      return base + enum_offset(td, cc) + lane4;                                                            \
    };                                                                                                      \
    for (;;) {                                                                                              \
      if (kRounds && (aux & UA_LOOP) && rnd + 1u < n_full) {                                                \
        /* two rounds at a time, one per vector register */                                                 \
        const uint32_t a1 = a0 + SHL(P.round_elems);                                                        \
        ELEM *const p1 = next_round(p0);                                                                    \
        MACRO("va", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                 \
        MACRO("vb", a1, a1 + gs, a1 + 2u * gs, a1 + 3u * gs)                                                 \
        DV_NORM_APPLY("va")                                                                                 \
        DV_NORM_APPLY("vb")                                                                                 \
        STORE("va", p0)                                                                                     \
        STORE("vb", p1)                                                                                     \
        ++rnd;                                                                                              \
        if (rnd + 1u >= n_full) break;                                                                      \
        ++rnd;                                                                                              \
        a0 = a1 + SHL(P.round_elems);                                                                       \
        p0 = next_round(p1);                                                                                \
        continue;                                                                                           \
      }                                                                                                     \
      MACRO("va", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                   \
      DV_NORM_APPLY("va")                                                                                   \
      STORE("va", p0)                                                                                       \
      if (!kRounds || !(aux & UA_LOOP) || rnd + 1u >= n_full) break;                                        \
      ++rnd;                                                                                                \
      a0 += SHL(P.round_elems);                                                                             \
      p0 = next_round(p0);                                                                                  \
    }                                                                                                       \
    if (aux & UA_LAST) goto body_done;                                                                      \
    continue;                                                                                               \
  }
#define DV_ST_NORM32(R, P) DV_STV32R(R, P, ge)
#define DV_ST_NORMF16(R, P) DV_STV16R("cvt.rn.f16x2.f32", R, P, ge)
#define DV_ST_NORMBF16(R, P) DV_STV16R("cvt.rn.bf16x2.f32", R, P, ge)
            DV_LDNORMST_CASE(UH_LDNORMST_FIRST + FT_F32, DV_LDR32, DV_SHL2, uint32_t, DV_ST_NORM32)
            DV_LDNORMST_CASE(UH_LDNORMST_FIRST + FT_F16, DV_LDR_F16, DV_SHL1, unsigned short, DV_ST_NORMF16)
            DV_LDNORMST_CASE(UH_LDNORMST_FIRST + FT_BF16, DV_LDR_BF16, DV_SHL1, unsigned short, DV_ST_NORMBF16)
#undef DV_ST_NORM32
#undef DV_ST_NORMF16
#undef DV_ST_NORMBF16
#undef DV_LDNORMST_CASE
#undef DV_NORM_APPLY
#undef DV_NORM_SCALARS
            // ---- the pieces of a residual RMSNorm + gated activation, one dispatch each (same operations, order and
            // rounding as the micro-ops they replace)
#define DV_RING3(SHL)                                                                                       \
    const uint32_t o0 = stage_saddr + (SHL(pos.in_chunk0)), gs = SHL(pos.gstep);                            \
    const uint32_t a0 = o0 + (arg << 4), b0 = o0 + ((uhi & 0xfffu) << 4), c0 = o0 + (((uhi >> 12) & 0xfffu) << 4);
#define DV_STORE_PTR(ELEM)                                                                                  \
    const TensorDesc &td = tdesc[(uhi >> 24) & 0xfu];                                                       \
    ELEM *const p0 = reinterpret_cast<ELEM *>(td.ptr) + kept_offset(td, pos.k) +                            \
                     ((kCoords && td.mode != AM_DENSE) ? enum_offset(td, cc) + lane4 : pos.e_start + pos.in_chunk0); \
    const uint32_t ge = pos.gstep;
// the arithmetic of the three handlers below in packed f32x2 form (two lanes per instruction)
#define DV_C3_ADDSQR asm volatile(DV_PAIRS8V(DV_P2_ADDSQR, ""));
#define DV_C3_ADDMULS asm volatile(DV_PAIRS8V(DV_P2_ADDMULS, "")::"l"((static_cast<uint64_t>(sv_) << 32) | sv_));
#define DV_C3_MULV asm volatile(DV_PAIRS8V(DV_P2_BINV, "mul.rn.f32x2"));
#define DV_C3_SIGM asm volatile(DV_PAIRS8V(DV_P2_SIGM, "")::"l"(0xbfb8aa3bbfb8aa3bull), "l"(0x3f8000003f800000ull));
#define DV_LD2ADDSQRSUM_CASE(H, MACRO, SHL, SLOT)                                                           \
  case H: {                                                                                                 \
    const uint32_t o0 = stage_saddr + (SHL(pos.in_chunk0)), gs = SHL(pos.gstep);                            \
    const uint32_t a0 = o0 + (arg << 4), b0 = o0 + (uhi << 4);                                              \
    MACRO("va", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                     \
    MACRO("vb", b0, b0 + gs, b0 + 2u * gs, b0 + 3u * gs)                                                     \
    DV_C3_ADDSQR                                                                                            \
    asm volatile(DV_SUMRN_TREE(SLOT));                                                                      \
    if (aux & UA_LAST) goto body_done;                                                                      \
    continue;                                                                                               \
  }
            DV_LD2ADDSQRSUM_CASE(UH_LD2ADDSQRSUM_FIRST + FT_F32, DV_LDR32, DV_SHL2, "0")
            DV_LD2ADDSQRSUM_CASE(UH_LD2ADDSQRSUM_FIRST + FT_F16, DV_LDR_F16, DV_SHL1, "0")
            DV_LD2ADDSQRSUM_CASE(UH_LD2ADDSQRSUM_FIRST + FT_BF16, DV_LDR_BF16, DV_SHL1, "0")
            DV_LD2ADDSQRSUM_CASE(UH_LD2ADDSQRSUM_FIRST + 3 + FT_F32, DV_LDR32, DV_SHL2, "1")
            DV_LD2ADDSQRSUM_CASE(UH_LD2ADDSQRSUM_FIRST + 3 + FT_F16, DV_LDR_F16, DV_SHL1, "1")
            DV_LD2ADDSQRSUM_CASE(UH_LD2ADDSQRSUM_FIRST + 3 + FT_BF16, DV_LDR_BF16, DV_SHL1, "1")
#undef DV_LD2ADDSQRSUM_CASE
#define DV_LD2ADDMULRMULST_CASE(H, MACRO, SHL, ELEM, STORE)                                                   \
  case H: {                                                                                                 \
    DV_RING3(SHL)                                                                                           \
    const uint32_t sv_ = lds32(sreg_addr(uhi >> 28));                                                       \
    DV_STORE_PTR(ELEM)                                                                                      \
    MACRO("va", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                     \
    MACRO("vb", b0, b0 + gs, b0 + 2u * gs, b0 + 3u * gs)                                                     \
    DV_C3_ADDMULS                                                                                           \
    MACRO("vb", c0, c0 + gs, c0 + 2u * gs, c0 + 3u * gs)                                                     \
    DV_C3_MULV                                                                                              \
    STORE                                                                                                   \
    if (aux & UA_LAST) goto body_done;                                                                      \
    continue;                                                                                               \
  }
            DV_LD2ADDMULRMULST_CASE(UH_LD2ADDMULRMULST_FIRST + FT_F32, DV_LDR32, DV_SHL2, uint32_t, DV_STV32(p0, ge))
            DV_LD2ADDMULRMULST_CASE(UH_LD2ADDMULRMULST_FIRST + FT_F16, DV_LDR_F16, DV_SHL1, unsigned short, DV_STV16("cvt.rn.f16x2.f32", p0, ge))
            DV_LD2ADDMULRMULST_CASE(UH_LD2ADDMULRMULST_FIRST + FT_BF16, DV_LDR_BF16, DV_SHL1, unsigned short, DV_STV16("cvt.rn.bf16x2.f32", p0, ge))
#undef DV_LD2ADDMULRMULST_CASE
#define DV_LDSIGMMUL2ST_CASE(H, MACRO, SHL, ELEM, STORE)                                                      \
  case H: {                                                                                                 \
    DV_RING3(SHL)                                                                                           \
    DV_STORE_PTR(ELEM)                                                                                      \
    MACRO("va", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                     \
    DV_C3_SIGM                                                                                              \
    MACRO("vb", b0, b0 + gs, b0 + 2u * gs, b0 + 3u * gs)                                                     \
    DV_C3_MULV                                                                                              \
    MACRO("vb", c0, c0 + gs, c0 + 2u * gs, c0 + 3u * gs)                                                     \
    DV_C3_MULV                                                                                              \
    STORE                                                                                                   \
    if (aux & UA_LAST) goto body_done;                                                                      \
    continue;                                                                                               \
  }
            DV_LDSIGMMUL2ST_CASE(UH_LDSIGMMUL2ST_FIRST + FT_F32, DV_LDR32, DV_SHL2, uint32_t, DV_STV32(p0, ge))
            DV_LDSIGMMUL2ST_CASE(UH_LDSIGMMUL2ST_FIRST + FT_F16, DV_LDR_F16, DV_SHL1, unsigned short, DV_STV16("cvt.rn.f16x2.f32", p0, ge))
            DV_LDSIGMMUL2ST_CASE(UH_LDSIGMMUL2ST_FIRST + FT_BF16, DV_LDR_BF16, DV_SHL1, unsigned short, DV_STV16("cvt.rn.bf16x2.f32", p0, ge))
#undef DV_LDSIGMMUL2ST_CASE
#undef DV_C3_ADDSQR
#undef DV_C3_ADDMULS
#undef DV_C3_MULV
#undef DV_C3_SIGM
#undef DV_STORE_PTR
#undef DV_RING3
#undef DV_STV16
#undef DV_STV32
#undef DV_STV16R
#undef DV_STV32R
#undef DVMB_ST
#define DV_LDMUL2_CASE(H, MACRO, SHL)                                                                          \
  case H: {                                                                                                 \
    const uint32_t o0 = stage_saddr + (SHL(pos.in_chunk0)), gs = SHL(pos.gstep);                            \
    const uint32_t a0 = o0 + (arg << 4), b0 = o0 + (uhi << 4);                                              \
    MACRO("vb", a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)                                                     \
    asm volatile(DV_LN(DV_BINVRN_LANE, "mul.rn.f32"));                                                      \
    MACRO("vb", b0, b0 + gs, b0 + 2u * gs, b0 + 3u * gs)                                                     \
    asm volatile(DV_LN(DV_BINVRN_LANE, "mul.rn.f32"));                                                      \
    continue;                                                                                               \
  }
            DV_LDMUL2_CASE(UH_LDMUL2_FIRST + FT_F32, DV_LDR32, DV_SHL2)
            DV_LDMUL2_CASE(UH_LDMUL2_FIRST + FT_F16, DV_LDR_F16, DV_SHL1)
            DV_LDMUL2_CASE(UH_LDMUL2_FIRST + FT_BF16, DV_LDR_BF16, DV_SHL1)
#undef DV_LDMUL2_CASE
#undef DV_LDX_TYPES
#undef DV_LDX_CASE
            case UH_SQRSUM0:
              asm volatile(DV_LN(DV_SQRRN_LANE, ""));
              asm volatile(DV_SUMRN_TREE("0"));
              if (aux & UA_LAST) goto body_done;
              continue;
            case UH_SQRSUM1:
              asm volatile(DV_LN(DV_SQRRN_LANE, ""));
              asm volatile(DV_SUMRN_TREE("1"));
              if (aux & UA_LAST) goto body_done;
              continue;
#define DV_RR_CASE(H, OP1, OP2)                                                       \
  case H: {                                                                        \
    const uint32_t s1_ = lds32(sreg_addr(arg & 0xffu)), s2_ = lds32(sreg_addr(arg >> 8)); \
    asm volatile(DV_LN(DV_BINS2_LANE, OP1, OP2)::"r"(s1_), "r"(s2_));              \
    continue;                                                                      \
  }
            DV_RR_CASE(UH_SUBR_MULR, "sub.rn.f32", "mul.rn.f32")
            DV_RR_CASE(UH_MULR_ADDR, "mul.rn.f32", "add.rn.f32")
            DV_RR_CASE(UH_MULR_MULR, "mul.rn.f32", "mul.rn.f32")
#undef DV_RR_CASE
            case UH_SIGMOID_FAST: asm volatile(DV_LN(DV_SIGM_LANE, "")); continue;
            case UH_LDG: {
              uint32_t t[kLanes];
              fetch_tensor(P, aux >> 2, pos, stage_saddr, t);
              DV_BY_DEST(aux & 3u, DV_SET, t)
              continue;
            }
            case UH_LDT: {
              const uint32_t a0 = temp_addr(arg, 0), gs = T * 16u;
              DV_BY_DEST(aux & 3u, DV_LDR32, a0, a0 + gs, a0 + 2u * gs, a0 + 3u * gs)
              continue;
            }
            case UH_LDS:
            case UH_LDI: {
              const uint32_t v = uh == UH_LDS ? lds32(sreg_addr(arg)) : uhi;
              DV_BY_DEST(aux & 3u, DV_SPLAT, v)
              continue;
            }
            case UH_MOVA:
              asm volatile(DV_LN(DV_MOV_LANE, "vb", "va"));
              continue;
            case UH_SQR: asm volatile(DV_LN(DV_SQR_LANE, "")); continue;
            case UH_RCP: asm volatile(DV_LN(DV_UN_LANE, "rcp.approx.f32")); continue;
            case UH_STT: {
              const uint32_t a0 = temp_addr(arg, 0), gs = T * 16u;
              asm volatile("st.shared.v4.b32 [%0], {va0,va1,va2,va3};\n\tst.shared.v4.b32 [%1], {va4,va5,va6,va7};\n\t"
                           "st.shared.v4.b32 [%2], {va8,va9,va10,va11};\n\tst.shared.v4.b32 [%3], {va12,va13,va14,va15};" ::"r"(a0),
                           "r"(a0 + gs), "r"(a0 + 2u * gs), "r"(a0 + 3u * gs)
                           : "memory");
              continue;
            }
            // ---------------- arithmetic: acc <- op(acc, vb) / op(acc, scalar) ----------------
            DV_BIN_CASES(B_ADD, DV_BINV_LANE, DV_BINS_LANE, "add.f32")
            DV_BIN_CASES(B_SUB, DV_BINV_LANE, DV_BINS_LANE, "sub.f32")
            DV_BIN_CASES(B_MUL, DV_BINV_LANE, DV_BINS_LANE, "mul.f32")
            DV_BIN_CASES(B_DIV, DV_BINV_LANE, DV_BINS_LANE, "div.rn.f32")
            DV_BIN_CASES(B_RSUB, DV_RBINV_LANE, DV_RBINS_LANE, "sub.f32")
            DV_BIN_CASES(B_RDIV, DV_RBINV_LANE, DV_RBINS_LANE, "div.rn.f32")
            DV_BIN_CASES(B_DIV_FAST, DV_BINV_LANE, DV_BINS_LANE, "div.full.f32")
            DV_BIN_CASES(B_RDIV_FAST, DV_RBINV_LANE, DV_RBINS_LANE, "div.full.f32")
            DV_BIN_CASES(B_ADD_I, DV_BINV_LANE, DV_BINS_LANE, "add.s32")
            DV_BIN_CASES(B_SUB_I, DV_BINV_LANE, DV_BINS_LANE, "sub.s32")
            DV_BIN_CASES(B_MUL_I, DV_BINV_LANE, DV_BINS_LANE, "mul.lo.s32")
            DV_BIN_CASES(B_MAX_I, DV_BINV_LANE, DV_BINS_LANE, "max.s32")
            DV_BIN_CASES(B_MIN_I, DV_BINV_LANE, DV_BINS_LANE, "min.s32")
            DV_BIN_CASES(B_RSUB_I, DV_RBINV_LANE, DV_RBINS_LANE, "sub.s32")
            // float max / min keep the reference's `a > b ? a : b` / `a < b ? a : b`
            case UH_BINV_FIRST + B_MAX: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_PICKV_LANE, "setp.gt.f32") "}"); break;
            case UH_BINV_FIRST + B_MIN: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_PICKV_LANE, "setp.lt.f32") "}"); break;
            case UH_BINS_FIRST + B_MAX:
            case UH_BINR_FIRST + B_MAX: {
              const uint32_t sv = uh == UH_BINR_FIRST + B_MAX ? lds32(sreg_addr(arg)) : uhi;
              asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_PICKS_LANE, "setp.gt.f32") "}" ::"r"(sv));
              break;
            }
            case UH_BINS_FIRST + B_MIN:
            case UH_BINR_FIRST + B_MIN: {
              const uint32_t sv = uh == UH_BINR_FIRST + B_MIN ? lds32(sreg_addr(arg)) : uhi;
              asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_PICKS_LANE, "setp.lt.f32") "}" ::"r"(sv));
              break;
            }
            case UH_BINV_FIRST + B_POW:
            case UH_BINR_FIRST + B_POW:
            case UH_BINS_FIRST + B_POW: {
              uint32_t x[kLanes], y[kLanes];
              DV_GET("va", x)
              if (uh == UH_BINV_FIRST + B_POW) {
                DV_GET("vb", y)
              } else {
                const uint32_t sv = uh == UH_BINR_FIRST + B_POW ? lds32(sreg_addr(arg)) : uhi;
#pragma unroll
                for (int i = 0; i < kLanes; ++i) y[i] = sv;
              }
#pragma unroll
              for (int i = 0; i < kLanes; ++i) x[i] = f2u(powf(u2f(x[i]), u2f(y[i])));
              DV_SET("va", x)
              break;
            }
            // ---------------- unary ----------------
            case UH_UN_FIRST + U_SQRT: asm volatile(DV_LN(DV_UN_LANE, "sqrt.rn.f32")); break;
            case UH_UN_FIRST + U_ABS: asm volatile(DV_LN(DV_UN_LANE, "abs.f32")); break;
            case UH_UN_FIRST + U_ROUND: asm volatile(DV_LN(DV_UN_LANE, "cvt.rni.f32.f32")); break;
            case UH_UN_FIRST + U_FLOOR: asm volatile(DV_LN(DV_UN_LANE, "cvt.rmi.f32.f32")); break;
            case UH_UN_FIRST + U_CEIL: asm volatile(DV_LN(DV_UN_LANE, "cvt.rpi.f32.f32")); break;
            case UH_UN_FIRST + U_TRUNC: asm volatile(DV_LN(DV_UN_LANE, "cvt.rzi.f32.f32")); break;
            case UH_UN_FIRST + U_ABS_I: asm volatile(DV_LN(DV_UN_LANE, "abs.s32")); break;
            case UH_UN_FIRST + U_ISFINITE:
              asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_ISFIN_LANE, "") "}");
              break;
            case UH_UN_FIRST + U_LOG:
            case UH_UN_FIRST + U_EXP: {
              uint32_t x[kLanes];
              DV_GET("va", x)
              if (uh == UH_UN_FIRST + U_EXP) {
#pragma unroll
                for (int i = 0; i < kLanes; ++i) x[i] = f2u(expf(u2f(x[i])));
              } else {
#pragma unroll
                for (int i = 0; i < kLanes; ++i) x[i] = f2u(logf(u2f(x[i])));
              }
              DV_SET("va", x)
              break;
            }
            case UH_UN_FIRST + U_EXP_FAST: asm volatile(DV_LN(DV_EXPF_LANE, "")); break;
            case UH_UN_FIRST + U_NOP: break;
            case UH_RND_F16: asm volatile("{\n\t.reg .b16 h;\n\t" DV_LN(DV_RNDH_LANE, "") "}"); continue;
            case UH_RND_BF16:
              asm volatile("{\n\t.reg .b32 t;\n\t" DV_PAIRS(DV_RNDB_PAIR, "") "}");
              continue;
            // ---------------- compare / select / convert ----------------
            case UH_CMP_F_V:
            case UH_CMP_F_S:
            case UH_CMP_I_V:
            case UH_CMP_I_S: {
              const bool is_int = uh == UH_CMP_I_V || uh == UH_CMP_I_S;
              if (uh == UH_CMP_F_S || uh == UH_CMP_I_S) {
                const uint32_t sv = (aux & UA_CMP_SREG) ? lds32(sreg_addr(arg)) : uhi;
                DV_SPLAT("vb", sv)
              }
              switch ((aux & 7u) | (is_int ? 8u : 0u)) {
                case C_EQ: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPF_LANE, "setp.eq.f32") "}"); break;
                case C_NE: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPF_LANE, "setp.neu.f32") "}"); break;
                case C_GT: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPF_LANE, "setp.gt.f32") "}"); break;
                case C_GE: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPF_LANE, "setp.ge.f32") "}"); break;
                case C_LT: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPF_LANE, "setp.lt.f32") "}"); break;
                case C_LE: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPF_LANE, "setp.le.f32") "}"); break;
                case 8 + C_EQ: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPI_LANE, "setp.eq.s32") "}"); break;
                case 8 + C_NE: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPI_LANE, "setp.ne.s32") "}"); break;
                case 8 + C_GT: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPI_LANE, "setp.gt.s32") "}"); break;
                case 8 + C_GE: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPI_LANE, "setp.ge.s32") "}"); break;
                case 8 + C_LT: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPI_LANE, "setp.lt.s32") "}"); break;
                default: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_CMPI_LANE, "setp.le.s32") "}"); break;
              }
              continue;
            }
            case UH_PRED_F:
              sel_mask = 0;
              asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\t" DV_LN(DV_PRED_LANE, "setp.neu.f32 p, va", ", 0f00000000") "}" : "+r"(sel_mask));
              continue;
            case UH_PRED_I:
              sel_mask = 0;
              asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\t" DV_LN(DV_PRED_LANE, "setp.ne.s32 p, va", ", 0") "}" : "+r"(sel_mask));
              continue;
            case UH_SELM: asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 t;\n\t" DV_LN(DV_SELM_LANE, "") "}" ::"r"(sel_mask)); continue;
            case UH_CVT_F2I: asm volatile(DV_LN(DV_UN_LANE, "cvt.rzi.s32.f32")); break;
            case UH_CVT_I2F: asm volatile(DV_LN(DV_UN_LANE, "cvt.rn.f32.s32")); break;
            case UH_CVT_NEZ_F: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_NEZ_LANE, "setp.neu.f32 p, va", ", 0f00000000") "}"); continue;
            case UH_CVT_NEZ_I: asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(DV_NEZ_LANE, "setp.ne.s32 p, va", ", 0") "}"); continue;
            // ---------------- reductions ----------------
            case UH_RACC_SUM:
            case UH_RACC_MAX:
            case UH_RACC_MIN: {
              // any chunk: lanes past the end of the chunk do not take part
              const uint32_t kind = uh - UH_RACC_SUM;
              uint32_t x[kLanes];
              DV_GET("va", x)
              float v = red_identity(kind);
#pragma unroll
              for (int i = 0; i < kLanes; ++i) {
                const int32_t left = (int32_t)pos.chunk_valid - (int32_t)(pos.in_chunk0 + (uint32_t)(i >> 2) * pos.gstep);
                if (pos.gvalid && (i & 3) < left) v = red_combine(kind, v, u2f(x[i]));
              }
              set_part(arg & 3u, red_combine(kind, get_part(arg & 3u), v));
              continue;
            }
            // full chunks: the 16 lanes are combined as a tree, one handler per partial register
#define DV_RACCF(KIND, SLOT, TREE)         \
  case UH_RACCF_FIRST + KIND * 4 + SLOT:   \
    asm volatile(TREE(#SLOT));             \
    if (aux & UA_LAST) goto body_done;     \
    continue;
#define DV_RACCF4(KIND, TREE) DV_RACCF(KIND, 0, TREE) DV_RACCF(KIND, 1, TREE) DV_RACCF(KIND, 2, TREE) DV_RACCF(KIND, 3, TREE)
            DV_RACCF4(R_SUM, DV_SUM_TREE)
            DV_RACCF4(R_MAX, DV_MAX_TREE)
            DV_RACCF4(R_MIN, DV_MIN_TREE)
#undef DV_RACCF4
#undef DV_RACCF
            // ---------------- stores ----------------
            case UH_ST_F32: {
              const TensorDesc &td = tdesc[arg];
              uint32_t *p0 = reinterpret_cast<uint32_t *>(td.ptr) + kept_offset(td, pos.k) + (!kCoords || td.mode == AM_DENSE ? pos.e_start + pos.in_chunk0 : enum_offset(td, cc) + lane4);
              const uint32_t gs = pos.gstep;
              asm volatile("st.global.v4.b32 [%0], {va0,va1,va2,va3};\n\tst.global.v4.b32 [%1], {va4,va5,va6,va7};\n\t"
                           "st.global.v4.b32 [%2], {va8,va9,va10,va11};\n\tst.global.v4.b32 [%3], {va12,va13,va14,va15};" ::"l"(p0),
                           "l"(p0 + gs), "l"(p0 + 2u * gs), "l"(p0 + 3u * gs)
                           : "memory");
              if (aux & UA_LAST) goto body_done;
              continue;
            }
            case UH_ST_F16:
            case UH_ST_BF16: {
              const TensorDesc &td = tdesc[arg];
              unsigned short *p0 = reinterpret_cast<unsigned short *>(td.ptr) + kept_offset(td, pos.k) + (!kCoords || td.mode == AM_DENSE ? pos.e_start + pos.in_chunk0 : enum_offset(td, cc) + lane4);
              const uint32_t gs = pos.gstep;
#define DV_ST16(CVT)                                                                                          \
  asm volatile("{\n\t.reg .b32 t0, t1;\n\t"                                                                   \
               CVT " t0, va1, va0;\n\t" CVT " t1, va3, va2;\n\tst.global.v2.b32 [%0], {t0,t1};\n\t"           \
               CVT " t0, va5, va4;\n\t" CVT " t1, va7, va6;\n\tst.global.v2.b32 [%1], {t0,t1};\n\t"           \
               CVT " t0, va9, va8;\n\t" CVT " t1, va11, va10;\n\tst.global.v2.b32 [%2], {t0,t1};\n\t"         \
               CVT " t0, va13, va12;\n\t" CVT " t1, va15, va14;\n\tst.global.v2.b32 [%3], {t0,t1};\n\t}" ::"l"(p0), \
               "l"(p0 + gs), "l"(p0 + 2u * gs), "l"(p0 + 3u * gs)                                            \
               : "memory");
              if (uh == UH_ST_BF16) {
                DV_ST16("cvt.rn.bf16x2.f32")
              } else {
                DV_ST16("cvt.rn.f16x2.f32")
              }
#undef DV_ST16
              if (aux & UA_LAST) goto body_done;
              continue;
            }
            case UH_ST_U8:
            case UH_STG: {
              uint32_t x[kLanes];
              DV_GET("va", x)
              store_tensor(P, arg, pos, x);
              continue;
            }
            default: __builtin_unreachable();
          }
        }
      body_done:
        if (kCoords && body_coords) {
          // the coordinates follow the rounds (a looping handler may have run several)
          cc[3] += (rnd - rnd_begin + 1u) * P.round_elems;
#pragma unroll
          for (int j = kMaxEnum - 1; j > 0; --j)
            while (cc[j] >= P.enum_size[j]) {
              cc[j] -= P.enum_size[j];
              cc[j - 1] += 1u;
            }
        }
        }   // rounds
        if (staged_body && release_slots) {
          __syncwarp();
          if ((tid & 31u) == 0) mbar_arrive(empty_bar);
        }
      }
    }
  }
  if (cluster > 1) {
    // no CTA leaves while a peer may still read its partials
    if (tid == 0)
      for (uint32_t r = 0; r < cluster; ++r) mbar_arrive_remote_release(map_shared_rank(smem_base + kVmSmemXBar, r));
    mbar_wait_cluster(smem_base + kVmSmemXBar, xphase, epoch);
  }
}
}  // namespace

// Register budgets of the same interpreter: up to 256 consumer threads per CTA (two CTAs of that size per SM, four
// of the 128-thread ones that reduce graphs with many groups use), and up to 512 (few long groups) with one CTA per SM.
// A third budget of 72 registers (five 128-thread CTAs per SM) was measured 50 % slower: its spills sit in the loop.
#define DVMB_VM_KERNEL(NAME, THREADS, BLOCKS, ...)                                                              \
  __global__ void __launch_bounds__(THREADS, BLOCKS) NAME(const __grid_constant__ VmParam P,                      \
                                                          const uint32_t epoch) {                                 \
    vm_vector_body<__VA_ARGS__>(P, epoch);                                                                        \
  }
// dense layouts (every chunk starts at group offset + element index)
DVMB_VM_KERNEL(dvm_b200_vm_vector, kVmFlatThreads + 32, 2, false, false, false)
DVMB_VM_KERNEL(dvm_b200_vm_vector_wide, kVmMaxThreads + 32, 1, false, false, false)
// ... of reduce-free (flat) launches only
DVMB_VM_KERNEL(dvm_b200_vm_vector_flat, kVmFlatThreads + 32, 2, false, false, false, 1)
// ... of group launches only
DVMB_VM_KERNEL(dvm_b200_vm_vector_group, kVmFlatThreads + 32, 2, false, false, false, 2)
// strided layouts: chunk starts follow from the chunk's coordinates along the iterated axes
DVMB_VM_KERNEL(dvm_b200_vm_vector_nd, kVmFlatThreads + 32, 2, false, true, false)
DVMB_VM_KERNEL(dvm_b200_vm_vector_nd_wide, kVmMaxThreads + 32, 1, false, true, false)
// CTAs of at most 256 threads that run two per SM (groups of up to 224 consumer threads plus the producer warp): the
// bound lets ptxas use up to 128 registers, which keeps the dispatch loop free of spills and pays for the round loop
DVMB_VM_KERNEL(dvm_b200_vm_vector_r128, 256, 2, false, false, true)
DVMB_VM_KERNEL(dvm_b200_vm_vector_nd_r128, 256, 2, false, true, true)
// resident groups (and clusters): every chunk of a group keeps a shared-memory slot for all phases
DVMB_VM_KERNEL(dvm_b200_vm_vector_res, 256, 2, true, true, true)
DVMB_VM_KERNEL(dvm_b200_vm_vector_res_wide, kVmMaxThreads + 32, 1, true, true, true)
#undef DVMB_VM_KERNEL

int LaunchVector(const VmParam &param, uint32_t grid, uint32_t threads, uint32_t smem_bytes, void *stream) {
  static bool attr_set[64] = {false};   // the attribute is per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaSuccess;
    for (auto fn : {dvm_b200_vm_vector, dvm_b200_vm_vector_wide, dvm_b200_vm_vector_nd, dvm_b200_vm_vector_nd_wide,
                    dvm_b200_vm_vector_res, dvm_b200_vm_vector_res_wide, dvm_b200_vm_vector_r128, dvm_b200_vm_vector_nd_r128,
                    dvm_b200_vm_vector_flat, dvm_b200_vm_vector_group})
      if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kVmMaxSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  if (param.cluster > 1) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = param.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  const bool narrow = threads <= kVmFlatThreads + 32;
  static const bool no_flat = getenv("DVM_B200_NO_FLAT_KERNEL") != nullptr;
  static const bool no_group = getenv("DVM_B200_NO_GROUP_KERNEL") != nullptr;
  auto kernel = narrow ? (param.mode == VM_FLAT ? (no_flat ? dvm_b200_vm_vector : dvm_b200_vm_vector_flat)
                                                : (no_group ? dvm_b200_vm_vector : dvm_b200_vm_vector_group))
                       : dvm_b200_vm_vector_wide;
  if (param.resident) {
    kernel = threads <= 256 ? dvm_b200_vm_vector_res : dvm_b200_vm_vector_res_wide;
  } else if (param.need_coords) {
    kernel = narrow ? dvm_b200_vm_vector_nd : dvm_b200_vm_vector_nd_wide;
  }
  // (the 160-thread CTAs run four per SM and need the 96-register build for that)
  static const bool no_r128 = getenv("DVM_B200_NO_R128") != nullptr;
  const bool r128 = !param.resident && threads > 160 && threads <= 256 && !no_r128;
  if (r128) kernel = param.need_coords ? dvm_b200_vm_vector_nd_r128 : dvm_b200_vm_vector_r128;
  if ((param.rounds > 1 || param.cluster > 1) && !r128 && !param.resident) return -4;   // (the compiler only plans rounds and clusters for these kernels)
  if (param.cluster > 1) {
    // A persistent grid of clusters must be resident as a whole: a cluster that has to wait for another one to leave
    // would start its share of the groups only then.  The driver knows how many clusters of this shape fit (fewer than
    // SMs x CTAs per SM / cluster size, since a cluster may not straddle GPCs); the answer is cached per launch shape.
    struct Fit { const void *fn; uint32_t threads, smem, cluster; int dev, clusters; };
    static Fit cache[16];
    static int cached = 0;
    int fit = -1;
    for (int i = 0; i < cached; ++i)
      if (cache[i].fn == reinterpret_cast<const void *>(kernel) && cache[i].threads == threads && cache[i].smem == smem_bytes &&
          cache[i].cluster == param.cluster && cache[i].dev == dev)
        fit = cache[i].clusters;
    if (fit < 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = static_cast<int>(grid / param.cluster);
      }
      fit = n;
      if (cached < 16) cache[cached++] = Fit{reinterpret_cast<const void *>(kernel), threads, smem_bytes, param.cluster, dev, n};
    }
    if (grid / param.cluster > static_cast<uint32_t>(fit)) {
      grid = static_cast<uint32_t>(fit) * param.cluster;
      cfg.gridDim = dim3(grid, 1, 1);
    }
  }
  static const bool debug_launch = getenv("DVM_B200_DEBUG_LAUNCH") != nullptr;
  if (debug_launch) {
    // the launch configuration and what the driver says about its residency (a diagnostic; off by default)
    int per_sm = 0, clusters = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, static_cast<int>(threads), smem_bytes);
    if (param.cluster > 1) cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
    fprintf(stderr, "dvm_b200 launch: grid=%u threads=%u smem=%u cluster=%u resident=%u blocks/SM=%d active clusters=%d\n", grid,
            threads, smem_bytes, param.cluster, param.resident, per_sm, clusters);
  }
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, param, NextLaunchEpoch());
  if (le != cudaSuccess) return static_cast<int>(le);
  return static_cast<int>(cudaGetLastError());
}

// A launch whose only wait can never succeed: one thread spins on an mbarrier that nothing arrives at, through the same
// bounded wait as the interpreter, with a caller-chosen limit.  It exists so that a test can watch the expiry path end
// to end (status recorded, reported by the host, cleared, later launches unaffected) without hanging or faulting the GPU.
__global__ void dvm_b200_wait_selftest(const uint32_t epoch, const unsigned long long limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(&bar));
  mbar_init(addr, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  bounded_spin([&]() { return mbar_try_wait(addr, 0u); }, 15u, &g_vm_status, epoch, limit_ns);
}

int LaunchWaitSelfTest(unsigned int limit_ms, void *stream) {
  if (limit_ms > 1000u) limit_ms = 1000u;
  dvm_b200_wait_selftest<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(NextLaunchEpoch(), 1000000ull * limit_ms);
  return static_cast<int>(cudaGetLastError());
}

// Read (and clear) the first recorded expiry of the vector interpreter; 0 means every bounded wait succeeded.
unsigned int ReadVectorStatus() {
  WaitStatus v = {0u, 0u};
  const unsigned int zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_vm_status, sizeof(v)) != cudaSuccess) return 0xffffffffu;
  if (v.first_error != 0) cudaMemcpyToSymbol(g_vm_status, &zero, sizeof(zero), offsetof(WaitStatus, first_error));
  return v.first_error;
}

}  // namespace dvmb
