// Fused attention  O = softmax(scale * Q K^T) V  on the sm_100a tensor cores.
//
// The reference has no attention operator: its example (examples/03_attention.py:31-52) builds
// MatMul -> scale -> softmax -> MatMul from API ops, which its splitter turns into several kernels with the full
// score matrix in global memory (src/xkernel.cc:1980-2119).  Here the stage planner recognises that pattern and
// runs it as one launch with the scores kept on chip (online softmax over key/value tiles).
//
// One CTA owns 256 query rows of one (batch, head): two tiles of 128 rows that take turns on the tensor core.
//   warp 0      TMA producer: Q once, then K and V tiles of 128 keys through a 3-slot ring
//   warp 1      MMA issuer: S_g = Q_g K^T into TMEM, O_g += P_g V; the two row tiles g = 0, 1 are interleaved so
//               that one tile's softmax overlaps the other tile's MMAs
//   warps 2-5   softmax of tile 0 (one thread per row), warps 6-9 softmax of tile 1: scores TMEM -> registers,
//               running maximum, exp2, row sum, P as bf16/fp16 into shared memory (the A operand of P V)
// The running maximum is only raised when a row's new maximum exceeds it by more than 8 (a factor e^8 of
// head-room in P); only then is the accumulator in TMEM rescaled, which for typical inputs happens once.
// Rounding follows the graph: the score is rounded to the operand type (the MatMul result), scaled (rounded
// again when the scale was applied in the operand type), softmax in fp32, P rounded to the operand type.
// Every mbarrier wait is bounded; on expiry a status word is set and the kernel runs to its end.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "mm_launch.h"
#include "sm100_sync.cuh"
#include "vm_ops.cuh"

namespace dvmb {

__device__ WaitStatus g_attn_status = {0u, 0u};

namespace {

constexpr uint32_t kTileQ = 128, kTileKV = 128;
constexpr uint32_t kQTilesPerCta = 2;
constexpr uint32_t kRingSlots = 3;
constexpr uint32_t kTileBytes = 128 * 128 * 2;      // one [128 x 128] 16-bit tile (two 64-column halves)
constexpr uint32_t kHalfBytes = 128 * 64 * 2;       // [128 rows x 64 elements], 128-byte swizzled rows
constexpr uint32_t kThreads = 64 + 2 * 128;
constexpr uint32_t kHeader = 1024;
// shared memory: header | Q0 Q1 | P0 P1 | ring[3]
constexpr uint32_t kOffQ = kHeader, kOffP = kOffQ + 2 * kTileBytes, kOffRing = kOffP + 2 * kTileBytes;
constexpr uint32_t kSmemBytes = kOffRing + kRingSlots * kTileBytes + 1024;
// tensor memory columns: S0 S1 O0 O1
constexpr uint32_t kTmemS = 0, kTmemO = 256, kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;

struct AttnMaps {
  CUtensorMap q, k, v;
};

// barrier offsets inside the header
constexpr uint32_t kBarQ = 0, kBarKvFull = 8, kBarKvEmpty = 32, kBarSFull = 56, kBarSFree = 72, kBarPReady = 88,
                   kBarPvDone = 104, kTmemSlot = 128;

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
    "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
    "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
    "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
    "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
    "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
    "r"(r[31])
    : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Round two fp32 values to the operand type's precision (hardware packed conversion, then widen again).
template <uint32_t DT>
__device__ __forceinline__ void round_pair(float &a, float &b) {
  if (DT == T_BF16) {
    const uint32_t d = pack_bf16x2(a, b);
    a = __uint_as_float(d << 16);
    b = __uint_as_float(d & 0xffff0000u);
  } else {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 f = __half22float2(h);
    a = f.x;
    b = f.y;
  }
}

// Packed 2 x 16-bit arithmetic in the operand type: the product of two bf16 / fp16 values rounded once to that type
// is exactly "multiply in fp32, round to the type", the graph's scaled score.
template <uint32_t DT>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  uint32_t r;
  if (DT == T_BF16) {
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  } else {
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  }
  return r;
}
template <uint32_t DT>
__device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
  uint32_t r;
  if (DT == T_BF16) {
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  } else {
    asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  }
  return r;
}
template <uint32_t DT>
__device__ __forceinline__ float2 unpack2(uint32_t p) {
  if (DT == T_BF16) return make_float2(__uint_as_float(p << 16), __uint_as_float(p & 0xffff0000u));
  return __half22float2(*reinterpret_cast<const __half2 *>(&p));
}

__device__ __forceinline__ uint32_t pack_pair(uint32_t dtype, float lo, float hi) {
  if (dtype == T_BF16) return pack_bf16x2(lo, hi);
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

}  // namespace

namespace {
template <uint32_t DT, bool SCALE_FIRST>
__device__ __forceinline__ void attention_body(const AttnParam &P, const AttnMaps &maps, const uint32_t epoch) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw_addr);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t dhalves = P.d / 64;                  // 64-element halves of the head dimension (1 or 2)
  const uint32_t qblocks = (P.sq + kTileQ * kQTilesPerCta - 1) / (kTileQ * kQTilesPerCta);
  const uint32_t bz = blockIdx.x / qblocks, qb = blockIdx.x - bz * qblocks;
  const uint32_t q_row0 = qb * kTileQ * kQTilesPerCta;
  const uint32_t nkv = (P.skv + kTileKV - 1) / kTileKV;
  const uint32_t tile_bytes = dhalves * kHalfBytes;   // bytes of one staged Q / K / V tile

  if (threadIdx.x == 0) {
    mbar_init(base + kBarQ, 1);
    for (uint32_t s = 0; s < kRingSlots; ++s) {
      mbar_init(base + kBarKvFull + 8 * s, 1);
      mbar_init(base + kBarKvEmpty + 8 * s, 1);
    }
    for (uint32_t g = 0; g < 2; ++g) {
      mbar_init(base + kBarSFull + 8 * g, 1);
      mbar_init(base + kBarSFree + 8 * g, 4);
      mbar_init(base + kBarPReady + 8 * g, 4);
      mbar_init(base + kBarPvDone + 8 * g, 1);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(base + kTmemSlot, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_before_sync();
  __syncthreads();
  tcgen05_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem + kTmemSlot);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(base + kBarQ, 2 * tile_bytes);
      for (uint32_t g = 0; g < 2; ++g)
        for (uint32_t h = 0; h < dhalves; ++h)
          tma_load_3d(base + kOffQ + g * kTileBytes + h * kHalfBytes, &maps.q, base + kBarQ, (int)(h * 64),
                      (int)(q_row0 + g * kTileQ), (int)bz);
      // ring order = order of need: K0, then per key tile j: K(j+1) (its scores are issued early), V(j)
      uint32_t slot = 0, parity = 1;
      const uint32_t ntiles = 2 * nkv;
      for (uint32_t p = 0; p < ntiles; ++p) {
        // position p holds: K0 at 0; K(j) at 2j - 1; V(j) at 2j + 2, except the last V at 2 nkv - 1
        const bool is_v = p != 0 && ((p & 1u) == 0 || p == ntiles - 1);
        const uint32_t j = p == 0 ? 0u : (is_v ? (p == ntiles - 1 ? nkv - 1 : (p - 2) / 2) : (p + 1) / 2);
        const CUtensorMap *map = is_v ? &maps.v : &maps.k;
        mbar_wait(base + kBarKvEmpty + 8 * slot, parity, 1, &g_attn_status, epoch);
        mbar_expect_tx(base + kBarKvFull + 8 * slot, tile_bytes);
        for (uint32_t h = 0; h < dhalves; ++h)
          tma_load_3d(base + kOffRing + slot * kTileBytes + h * kHalfBytes, map, base + kBarKvFull + 8 * slot, (int)(h * 64),
                      (int)(j * kTileKV), (int)bz);
        if (++slot == kRingSlots) {
          slot = 0;
          parity ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t fmt = DT == T_BF16 ? 1u : 0u;
      // S = Q K^T: both operands have the head dimension innermost; M = 128, N = 128 keys
      const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((kTileKV >> 3) << 17) | ((kTileQ >> 4) << 24);
      // O += P V: V is stored [key][d] (the contraction axis outermost); N = d
      const uint32_t idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((P.d >> 3) << 17) | ((kTileQ >> 4) << 24);
      const uint32_t ksteps_s = P.d / 16;
      auto issue_s = [&](uint32_t g, uint32_t kslot) {
        const uint32_t qa = base + kOffQ + g * kTileBytes, kb = base + kOffRing + kslot * kTileBytes;
        for (uint32_t kk = 0; kk < ksteps_s; ++kk) {
          const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3u) * 32u;
          umma_f16_cta1(tmem_base + kTmemS + g * 128, make_smem_desc(qa + off, 0, 1024), make_smem_desc(kb + off, 0, 1024), idesc_s,
                        kk != 0 ? 1u : 0u);
        }
        umma_commit_cta1(base + kBarSFull + 8 * g);
      };
      auto issue_pv = [&](uint32_t g, uint32_t vslot, bool accumulate) {
        const uint32_t pa = base + kOffP + g * kTileBytes, vb = base + kOffRing + vslot * kTileBytes;
        for (uint32_t kk = 0; kk < kTileKV / 16; ++kk) {
          const uint64_t da = make_smem_desc(pa + (kk >> 2) * kHalfBytes + (kk & 3u) * 32u, 0, 1024);
          const uint64_t db = make_smem_desc(vb + kk * 2048, kHalfBytes, 1024);
          umma_f16_cta1(tmem_base + kTmemO + g * 128, da, db, idesc_o, (accumulate || kk != 0) ? 1u : 0u);
        }
        umma_commit_cta1(base + kBarPvDone + 8 * g);
      };
      // ring position of K(j) / V(j) (see the producer) -> slot and phase parity
      const uint32_t ntiles = 2 * nkv;
      auto k_pos = [&](uint32_t j) { return j == 0 ? 0u : 2 * j - 1; };
      auto v_pos = [&](uint32_t j) { return j + 1 < nkv ? 2 * j + 2 : ntiles - 1; };
      auto full_ready = [&](uint32_t pos) { return mbar_try_wait(base + kBarKvFull + 8 * (pos % kRingSlots), (pos / kRingSlots) & 1u); };
      auto release = [&](uint32_t pos) { umma_commit_cta1(base + kBarKvEmpty + 8 * (pos % kRingSlots)); };
      mbar_wait(base + kBarQ, 0, 2, &g_attn_status, epoch);
      // prologue: scores of key tile 0 for both row tiles
      mbar_wait(base + kBarKvFull, 0, 3, &g_attn_status, epoch);
      tcgen05_after_sync();
      issue_s(0, 0);
      issue_s(1, 0);
      release(0);
      // Event-driven issue: the scores of the next key tile go out as soon as the softmax warps have taken the
      // current ones into registers (so a tile's softmax never waits for its own scores), P V as soon as P is in
      // shared memory.  Bounded: gives up after about two seconds without progress.
      uint32_t s_issued[2] = {1, 1}, pv_issued[2] = {0, 0};
      unsigned long long t_last;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_last));
      uint32_t idle = 0;
      while (pv_issued[0] < nkv || pv_issued[1] < nkv) {
        bool progress = false;
#pragma unroll
        for (uint32_t g = 0; g < 2; ++g) {
          const uint32_t js = s_issued[g];
          if (js < nkv && js <= pv_issued[g] + 1 && mbar_try_wait(base + kBarSFree + 8 * g, (js - 1) & 1u) && full_ready(k_pos(js))) {
            tcgen05_after_sync();
            issue_s(g, k_pos(js) % kRingSlots);
            s_issued[g] = js + 1;
            if (s_issued[g ^ 1u] > js) release(k_pos(js));   // both row tiles have read K(js)
            progress = true;
          }
          const uint32_t jp = pv_issued[g];
          if (jp < nkv && jp < s_issued[g] && mbar_try_wait(base + kBarPReady + 8 * g, jp & 1u) && full_ready(v_pos(jp))) {
            tcgen05_after_sync();
            issue_pv(g, v_pos(jp) % kRingSlots, jp != 0);
            pv_issued[g] = jp + 1;
            if (pv_issued[g ^ 1u] > jp) release(v_pos(jp));
            progress = true;
          }
        }
        if (progress) {
          idle = 0;
        } else if (++idle >= 4096) {
          idle = 0;
          unsigned long long t_now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_now));
          if (*reinterpret_cast<volatile unsigned int *>(&g_attn_status.abort_epoch) == epoch) break;
          if (idle == 0 && t_now - t_last > kWaitLimitNs) {
            atomicCAS(&g_attn_status.first_error, 0u, (11u << 24) | (blockIdx.x & 0xffffffu));
            atomicExch(&g_attn_status.abort_epoch, epoch);
            break;
          }
        }
        if (progress) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_last));
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const uint32_t g = (warp - 2) >> 2;          // row tile of this warp
    const uint32_t quarter = warp & 3u;          // TMEM lane quarter this warp may access
    const uint32_t r = quarter * 32 + lane;      // row inside the tile
    const uint32_t row = q_row0 + g * kTileQ + r;
    const uint32_t lane_base = (quarter * 32u) << 16;
    const uint32_t t_s = tmem_base + lane_base + kTmemS + g * 128, t_o = tmem_base + lane_base + kTmemO + g * 128;
    const float scale = __uint_as_float(P.scale_bits);
    constexpr float kLog2e = 1.4426950408889634f;
    float m_used = -CUDART_INF_F, l = 0.0f;
    const uint32_t p_row = base + kOffP + g * kTileBytes + (r >> 3) * 1024 + (r & 7u) * 128;
    for (uint32_t j = 0; j < nkv; ++j) {
      mbar_wait(base + kBarSFull + 8 * g, j & 1u, 8, &g_attn_status, epoch);
      tcgen05_after_sync();
      uint32_t s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32_nowait(t_s + c * 32, &s[c * 32]);   // four loads in flight, one wait
      tmem_ld_wait();
      tcgen05_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(base + kBarSFree + 8 * g);
      const uint32_t kv_valid = min(kTileKV, P.skv - j * kTileKV);
      float alpha = 1.0f;
      bool rescale = false;
      uint32_t pk[64];
      if (SCALE_FIRST) {
        // The graph's order (score rounded to the operand type, scaled in that type) in packed 16-bit arithmetic:
        // one conversion packs and rounds two scores, one packed multiply scales and rounds them again.
        const uint32_t scale2 = pack_pair(DT, scale, scale);
        const uint32_t ninf2 = DT == T_BF16 ? 0xff80ff80u : 0xfc00fc00u;
#pragma unroll
        for (int i = 0; i < 64; ++i) pk[i] = mul2<DT>(pack_pair(DT, u2f(s[2 * i]), u2f(s[2 * i + 1])), scale2);
        if (kv_valid < kTileKV) {   // the last key tile: mask what lies past the sequence
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            if ((uint32_t)(2 * i + 1) >= kv_valid) pk[i] = (pk[i] & 0x0000ffffu) | (ninf2 & 0xffff0000u);
            if ((uint32_t)(2 * i) >= kv_valid) pk[i] = ninf2;
          }
        }
        uint32_t m8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) m8[c] = pk[c];
#pragma unroll
        for (int i = 8; i < 64; ++i) m8[i & 7] = max2<DT>(m8[i & 7], pk[i]);
        const float2 mm = unpack2<DT>(max2<DT>(max2<DT>(max2<DT>(m8[0], m8[1]), max2<DT>(m8[2], m8[3])),
                                               max2<DT>(max2<DT>(m8[4], m8[5]), max2<DT>(m8[6], m8[7]))));
        const float mx = fmaxf(mm.x, mm.y) * kLog2e;   // running maximum kept in the log2 domain
        if (mx > m_used + kRescaleThreshold * kLog2e || m_used == -CUDART_INF_F) {
          alpha = m_used == -CUDART_INF_F ? 0.0f : fast_exp2(m_used - mx);
          rescale = j != 0;
          m_used = mx;
          l *= alpha;
        }
        float sum8[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        const float mneg = -m_used;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float2 x = unpack2<DT>(pk[i]);
          const float p0 = fast_exp2(fmaf(x.x, kLog2e, mneg));
          const float p1 = fast_exp2(fmaf(x.y, kLog2e, mneg));
          sum8[(2 * i) & 7] += p0;
          sum8[(2 * i + 1) & 7] += p1;
          pk[i] = pack_pair(DT, p0, p1);
        }
        l += ((sum8[0] + sum8[1]) + (sum8[2] + sum8[3])) + ((sum8[4] + sum8[5]) + (sum8[6] + sum8[7]));
      } else {
        // scale applied in fp32 after the cast: round the score once, keep it in the log2 domain
        const float c2 = scale * kLog2e;
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          float x0 = u2f(s[i]), x1 = u2f(s[i + 1]);
          round_pair<DT>(x0, x1);
          s[i] = f2u(x0 * c2);
          s[i + 1] = f2u(x1 * c2);
        }
        if (kv_valid < kTileKV) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if ((uint32_t)i >= kv_valid) s[i] = 0xff800000u;
        }
        float mx8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) mx8[c] = u2f(s[c]);
#pragma unroll
        for (int i = 8; i < 128; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], u2f(s[i]));
        const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
        if (mx > m_used + kRescaleThreshold * kLog2e || m_used == -CUDART_INF_F) {
          alpha = m_used == -CUDART_INF_F ? 0.0f : fast_exp2(m_used - mx);
          rescale = j != 0;
          m_used = mx;
          l *= alpha;
        }
        float sum8[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float p0 = fast_exp2(u2f(s[2 * i]) - m_used);
          const float p1 = fast_exp2(u2f(s[2 * i + 1]) - m_used);
          sum8[(2 * i) & 7] += p0;
          sum8[(2 * i + 1) & 7] += p1;
          pk[i] = pack_pair(DT, p0, p1);
        }
        l += ((sum8[0] + sum8[1]) + (sum8[2] + sum8[3])) + ((sum8[4] + sum8[5]) + (sum8[6] + sum8[7]));
      }
      // P_g and O_g are free once the previous P V of this tile has completed
      if (j != 0) {
        mbar_wait(base + kBarPvDone + 8 * g, (j - 1) & 1u, 9, &g_attn_status, epoch);
        tcgen05_after_sync();
      }
      if (__any_sync(0xffffffffu, rescale)) {
        for (uint32_t c = 0; c < P.d; c += 32) {
          uint32_t t[32];
          tmem_ld_32x32b_x32(t_o + c, t);
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = f2u(u2f(t[i]) * alpha);
          tmem_st_32x32b_x32(t_o + c, t);
        }
        tmem_st_wait();
      }
      // P row -> shared memory in the 128-byte swizzled layout of an MMA A operand
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const uint32_t addr = p_row + (u >> 3) * kHalfBytes + (((uint32_t)(u & 7) ^ (r & 7u)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(pk[4 * u]), "r"(pk[4 * u + 1]), "r"(pk[4 * u + 2]),
                     "r"(pk[4 * u + 3])
                     : "memory");
      }
      fence_async_shared();
      tcgen05_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(base + kBarPReady + 8 * g);
    }
    // ---- result: O / l, rounded to the operand type
    mbar_wait(base + kBarPvDone + 8 * g, (nkv - 1) & 1u, 10, &g_attn_status, epoch);
    tcgen05_after_sync();
    const float inv = 1.0f / l;
    uint8_t *orow = reinterpret_cast<uint8_t *>(P.o_ptr) + ((size_t)bz * P.sq + row) * P.d * 2;
    for (uint32_t c = 0; c < P.d; c += 32) {
      uint32_t t[32];
      tmem_ld_32x32b_x32(t_o + c, t);
      if (row < P.sq) {
        uint32_t o[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = pack_pair(DT, u2f(t[2 * i]) * inv, u2f(t[2 * i + 1]) * inv);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          *reinterpret_cast<uint4 *>(orow + (size_t)c * 2 + u * 16) = make_uint4(o[4 * u], o[4 * u + 1], o[4 * u + 2], o[4 * u + 3]);
      }
    }
  }
  tcgen05_before_sync();
  __syncthreads();
  if (warp == 1) {
    tcgen05_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}
}  // namespace

#define DVMB_ATTN_KERNEL(NAME, DT, SF)                                                                              \
  __global__ void __launch_bounds__(kThreads, 1) NAME(const __grid_constant__ AttnParam P,                          \
                                                      const __grid_constant__ AttnMaps maps, const uint32_t epoch) { \
    attention_body<DT, SF>(P, maps, epoch);                                                                         \
  }
DVMB_ATTN_KERNEL(dvm_b200_attention_bf16, T_BF16, false)
DVMB_ATTN_KERNEL(dvm_b200_attention_bf16_sf, T_BF16, true)
DVMB_ATTN_KERNEL(dvm_b200_attention_f16, T_F16, false)
DVMB_ATTN_KERNEL(dvm_b200_attention_f16_sf, T_F16, true)
#undef DVMB_ATTN_KERNEL

namespace {

PFN_cuTensorMapEncodeTiled GetEncodeFn() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
  }
  return fn;
}

// [batch, rows, d] row-major, box = [1, 128 rows, 64 elements], 128-byte swizzle
int EncodeRows(CUtensorMap *map, uint64_t ptr, uint64_t d, uint64_t rows, uint64_t batch) {
  auto encode = GetEncodeFn();
  if (encode == nullptr) return -10;
  cuuint64_t dims[3] = {d, rows, batch};
  cuuint64_t strides[2] = {d * 2, d * rows * 2};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, reinterpret_cast<void *>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -100 - static_cast<int>(r);
}

}  // namespace

bool AttentionSupported(const AttnParam &p) {
  if (p.d != 64 && p.d != 128) return false;
  if (p.dtype != T_BF16 && p.dtype != T_F16) return false;
  if (p.sq == 0 || p.skv == 0 || p.batch == 0) return false;
  return true;
}

int LaunchAttention(const AttnParam &p, void *stream) {
  if (!AttentionSupported(p)) return -1;
  if ((p.q_ptr | p.k_ptr | p.v_ptr | p.o_ptr) & 15u) return -2;
  int dev = 0;
  cudaGetDevice(&dev);
  using KernelFn = void (*)(const AttnParam, const AttnMaps, const uint32_t);
  static const KernelFn kernels[4] = {dvm_b200_attention_bf16, dvm_b200_attention_bf16_sf, dvm_b200_attention_f16,
                                      dvm_b200_attention_f16_sf};
  static bool attr_set[64] = {false};
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    for (auto fn : kernels) {
      cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    attr_set[dev] = true;
  }
  const KernelFn kernel = kernels[(p.dtype == T_BF16 ? 0 : 2) + (p.scale_first ? 1 : 0)];
  AttnMaps maps;
  int rc = EncodeRows(&maps.q, p.q_ptr, p.d, p.sq, p.batch);
  if (rc == 0) rc = EncodeRows(&maps.k, p.k_ptr, p.d, p.skv, p.batch);
  if (rc == 0) rc = EncodeRows(&maps.v, p.v_ptr, p.d, p.skv, p.batch);
  if (rc != 0) return rc;
  const uint32_t qblocks = (p.sq + kTileQ * kQTilesPerCta - 1) / (kTileQ * kQTilesPerCta);
  kernel<<<p.batch * qblocks, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(p, maps, NextLaunchEpoch());
  return static_cast<int>(cudaGetLastError());
}

unsigned int ReadAttentionStatus() {
  WaitStatus v = {0u, 0u};
  const unsigned int zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(v)) != cudaSuccess) return 0xffffffffu;
  if (v.first_error != 0) cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(zero), offsetof(WaitStatus, first_error));
  return v.first_error;
}

}  // namespace dvmb
