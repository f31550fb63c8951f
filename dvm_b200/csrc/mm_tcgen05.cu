// MatMul (+ bias, + fused post-ops) on the sm_100a tensor cores: tcgen05.mma with the accumulator in tensor
// memory, operands staged by TMA into a shared-memory ring, post-fusion ops applied to the accumulator as it is
// drained from TMEM.
//
// Stands in for the reference's cube path, which exists only for Ascend (CubeOp src/ops_m.cc:271-696, the mix
// kernel that shards post-fusion ops per C tile src/xkernel.cc:157-361); the reference's CUDA backend has no
// MatMul at all (src/system.cc:290-294).  Semantics kept: fp16/bf16 operands, fp32 accumulation, optional bias
// added in fp32, result rounded to the operand dtype, then the fused vector ops.
//
// One CTA = one 128 x 256 tile of C at a time (persistent over tiles, grouped along M for L2 reuse):
//   warp 0     TMA producer: A [128 x 64] and B [256 x 64] per stage (64 x 64 boxes when the operand is stored
//              with the contraction axis outermost)
//   warp 1     MMA issuer: four tcgen05.mma (K = 16) per stage into one of two TMEM accumulators
//   warps 2-5  epilogue: tcgen05.ld 16 columns at a time, bias, rounding, post-fusion program, stores
// Every mbarrier wait is bounded; on expiry a status word is set and the kernel runs to its end.
//
// Problems the copy engine cannot address (row pitch or base not 16-byte aligned) run on a plain SIMT kernel
// with the same epilogue.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "mm_epilogue.cuh"
#include "mm_launch.h"
#include "sm100_sync.cuh"

namespace dvmb {

__device__ WaitStatus g_mm_status = {0u, 0u};

namespace {

// Tile geometry.  One CTA owns 128 rows x 256 columns of C at a time.  In the paired form (CTAS = 2) the two CTAs
// of a cluster share one MMA of 256 x 256: each stages its own 128 rows of A and one half (128 columns) of B, so
// a CTA moves 32 KB per k-block instead of 48 KB.
constexpr uint32_t BM = 128, BN = 256, BK = 64;
constexpr uint32_t kABytes = BM * BK * 2;   // 16 KB
constexpr uint32_t kEpiWarps = 8;
constexpr uint32_t kThreads = 64 + 32 * kEpiWarps;
constexpr uint32_t kTmemCols = 512;   // two 256-column fp32 accumulators
// shared memory: [0, 1024) barriers + tmem pointer, then the stages (1024-byte aligned for the 128B swizzle)
constexpr uint32_t kSmemHeader = 1024;
template <int CTAS>
struct Geo {
  static constexpr uint32_t kBBytes = (BN / CTAS) * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kStages = CTAS == 1 ? 4 : 6;
  static constexpr uint32_t kSmemBytes = kSmemHeader + kStages * kStageBytes + 1024;
};

struct MmMaps {
  CUtensorMap a, b;
};

__device__ __forceinline__ float load_bias(const MmParam &P, uint32_t col) {
  if (P.bias_dtype == T_F32) return __ldg(reinterpret_cast<const float *>(P.bias_ptr) + col);
  const unsigned short raw = __ldg(reinterpret_cast<const unsigned short *>(P.bias_ptr) + col);
  if (P.bias_dtype == T_BF16) return __uint_as_float(static_cast<uint32_t>(raw) << 16);
  return __half2float(__ushort_as_half(raw));
}

__device__ __forceinline__ float round_operand_type(uint32_t dtype, float v) {
  return dtype == T_BF16 ? round_bf16(v) : round_f16(v);
}

// tile index -> (batch, m block, n block), grouped along M so that the A panel of a group stays in L2 while
// the group sweeps over N
__device__ __forceinline__ void tile_coords(uint32_t t, uint32_t mblocks, uint32_t nblocks, uint32_t kGroupM, uint32_t &bz,
                                            uint32_t &mb, uint32_t &nb) {
  const uint32_t per_batch = mblocks * nblocks;
  bz = t / per_batch;
  t -= bz * per_batch;
  const uint32_t group_tiles = kGroupM * nblocks;
  const uint32_t g = t / group_tiles;
  const uint32_t first_m = g * kGroupM;
  const uint32_t gm = min(kGroupM, mblocks - first_m);
  const uint32_t in_group = t - g * group_tiles;
  mb = first_m + in_group % gm;
  nb = in_group / gm;
}

// Bias, rounding to the operand type and the post-fusion program for one 16-column strip of one row.
__device__ __forceinline__ void finish_strip(const MmParam &P, const EpiPos &pos, uint32_t (&r)[16]) {
  const bool whole = pos.valid == 16u;
  if (P.bias_ptr != 0) {
    const uint32_t bsh = P.bias_dtype == T_F32 ? 2u : 1u;
    if (whole && ((P.bias_ptr + ((uint64_t)pos.col << bsh)) & 15u) == 0) {
      // sixteen bias values as 16-byte loads
      if (bsh == 2u) {
        const uint4 *bp = reinterpret_cast<const uint4 *>(P.bias_ptr) + (pos.col >> 2);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4 b = __ldg(bp + g);
          r[4 * g + 0] = __float_as_uint(__uint_as_float(r[4 * g + 0]) + __uint_as_float(b.x));
          r[4 * g + 1] = __float_as_uint(__uint_as_float(r[4 * g + 1]) + __uint_as_float(b.y));
          r[4 * g + 2] = __float_as_uint(__uint_as_float(r[4 * g + 2]) + __uint_as_float(b.z));
          r[4 * g + 3] = __float_as_uint(__uint_as_float(r[4 * g + 3]) + __uint_as_float(b.w));
        }
      } else {
        const uint4 *bp = reinterpret_cast<const uint4 *>(P.bias_ptr) + (pos.col >> 3);
        const uint4 b0 = __ldg(bp), b1 = __ldg(bp + 1);
        const uint32_t w[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float lo, hi;
          if (P.bias_dtype == T_BF16) {
            lo = __uint_as_float(w[i] << 16);
            hi = __uint_as_float(w[i] & 0xffff0000u);
          } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            lo = f.x;
            hi = f.y;
          }
          r[2 * i] = __float_as_uint(__uint_as_float(r[2 * i]) + lo);
          r[2 * i + 1] = __float_as_uint(__uint_as_float(r[2 * i + 1]) + hi);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if ((uint32_t)i < pos.valid) r[i] = __float_as_uint(__uint_as_float(r[i]) + load_bias(P, pos.col + i));
    }
  }
  // The product in the operand type: packed two at a time (hardware round to nearest even, NaN kept).
  uint32_t pk[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (P.in_dtype == T_BF16) {
      pk[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    } else {
      const __half2 h = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      pk[i] = *reinterpret_cast<const uint32_t *>(&h);
    }
  }
  if (P.fast_store_slot != 0xffffffffu && whole) {
    // the whole post-fusion program is one store of the product: write it without interpreting
    const EpiTensor &t = P.tensor[P.fast_store_slot];
    const size_t off = epi_offset(t, pos);
    if (t.dtype == P.in_dtype) {
      uint8_t *dst = reinterpret_cast<uint8_t *>(t.ptr) + (off << 1);
      if ((reinterpret_cast<uint64_t>(dst) & 15u) == 0) {
        *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        return;
      }
    }
  }
  // back to the 32-bit register form of the rounded product
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (P.in_dtype == T_BF16) {
      r[2 * i] = pk[i] << 16;
      r[2 * i + 1] = pk[i] & 0xffff0000u;
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&pk[i]));
      r[2 * i] = __float_as_uint(f.x);
      r[2 * i + 1] = __float_as_uint(f.y);
    }
  }
  if (P.gate_slot != 0xffffffffu && whole) {
    // y = x / (c2 + exp(c1 * (x + c0 * x^3))): each step rounded on its own, as the interpreter's words are
    const EpiTensor &t = P.tensor[P.gate_slot];
    uint8_t *dst = reinterpret_cast<uint8_t *>(t.ptr) + (epi_offset(t, pos) << 1);
    if ((reinterpret_cast<uint64_t>(dst) & 15u) == 0) {
      const float c0 = __uint_as_float(P.gate_c[0]), c1 = __uint_as_float(P.gate_c[1]), c2 = __uint_as_float(P.gate_c[2]);
      float y[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float x = __uint_as_float(r[i]);
        float a = __fmul_rn(x, x);
        a = __fmul_rn(a, x);
        a = __fmul_rn(a, c0);
        a = __fadd_rn(a, x);
        a = __fmul_rn(a, c1);
        a = fast_exp(a);
        a = __fadd_rn(a, c2);
        y[i] = fast_div(x, a);
      }
      uint32_t o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (P.in_dtype == T_BF16) {
          o[i] = pack_bf16x2(y[2 * i], y[2 * i + 1]);
        } else {
          const __half2 h = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
          o[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
      }
      *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(o[4], o[5], o[6], o[7]);
      return;
    }
  }
  if (P.fast_store_slot != 0xffffffffu && whole) {
    const EpiTensor &t = P.tensor[P.fast_store_slot];
    if (t.dtype == T_F32) {
      uint8_t *dst = reinterpret_cast<uint8_t *>(t.ptr) + (epi_offset(t, pos) << 2);
      if ((reinterpret_cast<uint64_t>(dst) & 15u) == 0) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4 *>(dst + 16 * g) = make_uint4(r[4 * g], r[4 * g + 1], r[4 * g + 2], r[4 * g + 3]);
        return;
      }
    }
  }
  run_epilogue(P, pos, r);
}

template <int CTAS>
__device__ __forceinline__ void mm_body(const MmParam &P, const MmMaps &maps, const uint32_t epoch) {
  using G = Geo<CTAS>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte alignment of the stage area (required by the 128-byte swizzle pattern)
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw_addr);
  const uint32_t bar_full = base, bar_empty = base + 64, bar_tfull = base + 128, bar_tempty = base + 160;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + 192);
  const uint32_t stages = base + kSmemHeader;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0u;   // position inside the CTA pair
  const uint32_t unit = blockIdx.x / CTAS, num_units = gridDim.x / CTAS;
  const uint32_t mblocks = (P.M + BM * CTAS - 1) / (BM * CTAS), nblocks = (P.N + BN - 1) / BN;
  const uint32_t batch = P.batch0 * P.batch1;
  const uint32_t num_tiles = mblocks * nblocks * batch;
  const uint32_t kblocks = (P.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < G::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (uint32_t a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, kEpiWarps * CTAS);   // one arrival per epilogue warp of the pair
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    if (CTAS == 2) {
      tmem_alloc_pair(base + 192, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(base + 192, kTmemCols);
      tmem_relinquish();
    }
  }
  tcgen05_before_sync();
  if (CTAS == 2) {
    cluster_sync_all();   // the peer's barriers are initialised before anything signals them
  } else {
    __syncthreads();
  }
  tcgen05_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, parity = 1;
      for (uint32_t t = unit; t < num_tiles; t += num_units) {
        uint32_t bz, mb, nb;
        tile_coords(t, mblocks, nblocks, P.group_m, bz, mb, nb);
        const uint32_t b0 = bz / P.batch1, b1 = bz - b0 * P.batch1;
        const int za = (int)(b0 * P.a_mul0 + b1 * P.a_mul1), zb = (int)(b0 * P.b_mul0 + b1 * P.b_mul1);
        const int row0 = (int)((mb * CTAS + rank) * BM);
        const int col0 = (int)(nb * BN + rank * (BN / CTAS));
        for (uint32_t kb = 0; kb < kblocks; ++kb) {
          mbar_wait(bar_empty + 8 * stage, parity, 1, &g_mm_status, epoch);
          const uint32_t sa = stages + stage * G::kStageBytes, sb = sa + kABytes;
          // the pair's first CTA counts the bytes of both CTAs on its barrier
          uint32_t full = bar_full + 8 * stage;
          if (CTAS == 2) {
            if (rank == 0) mbar_expect_tx(full, 2 * G::kStageBytes);
            full = map_to_cta(full, 0);
          } else {
            mbar_expect_tx(full, G::kStageBytes);
          }
          auto load = [&](uint32_t dst, const CUtensorMap *map, int x, int y, int z) {
            if (CTAS == 2) {
              tma_load_3d_pair(dst, map, full, x, y, z);
            } else {
              tma_load_3d(dst, map, full, x, y, z);
            }
          };
          if (!P.a_mmajor) {
            load(sa, &maps.a, (int)(kb * BK), row0, za);
          } else {
#pragma unroll
            for (uint32_t j = 0; j < BM / 64; ++j) load(sa + j * (64 * BK * 2), &maps.a, row0 + (int)(j * 64), (int)(kb * BK), za);
          }
          if (P.b_kmajor) {
            load(sb, &maps.b, (int)(kb * BK), col0, zb);
          } else {
#pragma unroll
            for (uint32_t j = 0; j < BN / CTAS / 64; ++j)
              load(sb + j * (64 * BK * 2), &maps.b, col0 + (int)(j * 64), (int)(kb * BK), zb);
          }
          if (++stage == G::kStages) {
            stage = 0;
            parity ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (the pair's first CTA only) ------------------------------
    if (lane == 0 && rank == 0) {
      // instruction descriptor: D fp32 (bit 4), A/B format (bits 7, 10: 1 = bf16), A / B stored with the
      // contraction axis outermost (bits 15 / 16), N >> 3 at bit 17, M >> 4 at bit 24
      const uint32_t fmt = P.in_dtype == T_BF16 ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((P.a_mmajor ? 1u : 0u) << 15) |
                             ((P.b_kmajor ? 0u : 1u) << 16) | ((BN >> 3) << 17) | (((BM * CTAS) >> 4) << 24);
      uint32_t stage = 0, parity = 0, acc = 0, acc_parity = 1;
      for (uint32_t t = unit; t < num_tiles; t += num_units) {
        mbar_wait(bar_tempty + 8 * acc, acc_parity, 2, &g_mm_status, epoch);
        tcgen05_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (uint32_t kb = 0; kb < kblocks; ++kb) {
          mbar_wait(bar_full + 8 * stage, parity, 3, &g_mm_status, epoch);
          tcgen05_after_sync();
          const uint32_t sa = stages + stage * G::kStageBytes, sb = sa + kABytes;
#pragma unroll
          for (uint32_t kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = P.a_mmajor ? make_smem_desc(sa + kk * 2048, 64 * BK * 2, 1024) : make_smem_desc(sa + kk * 32, 0, 1024);
            const uint64_t db = P.b_kmajor ? make_smem_desc(sb + kk * 32, 0, 1024) : make_smem_desc(sb + kk * 2048, 64 * BK * 2, 1024);
            if (CTAS == 2) {
              umma_f16_pair(d_tmem, da, db, idesc, (kb | kk) != 0 ? 1u : 0u);
            } else {
              umma_f16_cta1(d_tmem, da, db, idesc, (kb | kk) != 0 ? 1u : 0u);
            }
          }
          // the stage is free (in both CTAs) once these MMAs have read it
          if (CTAS == 2) {
            umma_commit_pair(bar_empty + 8 * stage, 3);
          } else {
            umma_commit_cta1(bar_empty + 8 * stage);
          }
          if (++stage == G::kStages) {
            stage = 0;
            parity ^= 1u;
          }
        }
        // accumulator complete
        if (CTAS == 2) {
          umma_commit_pair(bar_tfull + 8 * acc, 3);
        } else {
          umma_commit_cta1(bar_tfull + 8 * acc);
        }
        if (++acc == 2) {
          acc = 0;
          acc_parity ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const uint32_t ew = warp - 2;
    const uint32_t quarter = warp & 3u;          // TMEM lane quarter this warp may read
    const uint32_t col_half = ew >> 2;           // which 128 columns of the tile
    const uint32_t row_in_tile = quarter * 32 + lane;
    uint32_t acc = 0, acc_parity = 0;
    for (uint32_t t = unit; t < num_tiles; t += num_units) {
      uint32_t bz, mb, nb;
      tile_coords(t, mblocks, nblocks, P.group_m, bz, mb, nb);
      mbar_wait(bar_tfull + 8 * acc, acc_parity, 4, &g_mm_status, epoch);
      tcgen05_after_sync();
      EpiPos pos;
      pos.b0 = bz / P.batch1;
      pos.b1 = bz - pos.b0 * P.batch1;
      pos.row = (mb * CTAS + rank) * BM + row_in_tile;
      const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * BN + col_half * (BN / 2);
      for (uint32_t c0 = 0; c0 < BN / 2; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + c0, r);   // every lane of the warp takes part, valid row or not
        pos.col = nb * BN + col_half * (BN / 2) + c0;
        if (pos.row >= P.M || pos.col >= P.N) continue;
        pos.valid = min(16u, P.N - pos.col);
        finish_strip(P, pos, r);
      }
      tcgen05_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2) {
          mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * acc, 0));
        } else {
          mbar_arrive(bar_tempty + 8 * acc);
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_parity ^= 1u;
      }
    }
  }
  tcgen05_before_sync();
  if (CTAS == 2) {
    cluster_sync_all();   // neither CTA leaves while the other may still read its shared memory or signal it
  } else {
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_after_sync();
    if (CTAS == 2) {
      tmem_dealloc_pair(tmem_base, kTmemCols);
    } else {
      tmem_dealloc(tmem_base, kTmemCols);
    }
  }
}

}  // namespace

__global__ void __launch_bounds__(kThreads, 1) dvm_b200_mm_tcgen05(const __grid_constant__ MmParam P,
                                                                   const __grid_constant__ MmMaps maps,
                                                                   const uint32_t epoch) {
  mm_body<1>(P, maps, epoch);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
  dvm_b200_mm_tcgen05_pair(const __grid_constant__ MmParam P, const __grid_constant__ MmMaps maps, const uint32_t epoch) {
  mm_body<2>(P, maps, epoch);
}

// General SIMT MatMul for problems the copy engine cannot address: one thread per 16-column strip of a row,
// fp32 accumulation in order of k.  Correct for every shape and alignment; not a performance path.
__global__ void __launch_bounds__(128) dvm_b200_mm_simt(const __grid_constant__ MmParam P) {
  const uint32_t strips = (P.N + 15u) / 16u;
  const uint64_t total = (uint64_t)P.batch0 * P.batch1 * P.M * strips;
  for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t strip = (uint32_t)(idx % strips);
    const uint64_t rest = idx / strips;
    EpiPos pos;
    pos.row = (uint32_t)(rest % P.M);
    const uint32_t bz = (uint32_t)(rest / P.M);
    pos.b0 = bz / P.batch1;
    pos.b1 = bz - pos.b0 * P.batch1;
    pos.col = strip * 16u;
    pos.valid = min(16u, P.N - pos.col);
    const size_t za = (size_t)(pos.b0 * P.a_mul0 + pos.b1 * P.a_mul1) * P.M * P.K;
    const size_t zb = (size_t)(pos.b0 * P.b_mul0 + pos.b1 * P.b_mul1) * P.N * P.K;
    const unsigned short *A = reinterpret_cast<const unsigned short *>(P.a_ptr) + za;
    const unsigned short *B = reinterpret_cast<const unsigned short *>(P.b_ptr) + zb;
    float accv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) accv[i] = 0.0f;
    for (uint32_t k = 0; k < P.K; ++k) {
      const unsigned short ar = P.a_mmajor ? A[(size_t)k * P.M + pos.row] : A[(size_t)pos.row * P.K + k];
      const float a = u2f(widen(P.in_dtype, ar));
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if ((uint32_t)i < pos.valid) {
          const uint32_t c = pos.col + i;
          const unsigned short br = P.b_kmajor ? B[(size_t)c * P.K + k] : B[(size_t)k * P.N + c];
          accv[i] = fmaf(a, u2f(widen(P.in_dtype, br)), accv[i]);
        }
      }
    }
    uint32_t r[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = f2u(accv[i]);
    finish_strip(P, pos, r);
  }
}

namespace {

PFN_cuTensorMapEncodeTiled GetEncode() {
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

// 3-d map over a [batches, rows, inner] row-major operand: box = [1, box_rows, 64 elements], 128-byte swizzle
int EncodeOperand(CUtensorMap *map, uint64_t ptr, uint64_t inner, uint64_t rows, uint64_t batches, uint32_t box_rows) {
  auto encode = GetEncode();
  if (encode == nullptr) return -10;
  cuuint64_t dims[3] = {inner, rows, batches ? batches : 1};
  cuuint64_t strides[2] = {inner * 2, inner * rows * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, reinterpret_cast<void *>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -100 - static_cast<int>(r);
}

}  // namespace

bool MatMulUsesTensorCores(const MmParam &p) {
  // the copy engine needs 16-byte aligned bases and row pitches (and slices, for batched operands)
  const uint64_t a_inner = p.a_mmajor ? p.M : p.K, b_inner = p.b_kmajor ? p.K : p.N;
  if ((a_inner & 7u) != 0 || (b_inner & 7u) != 0) return false;
  if ((p.a_ptr & 15u) || (p.b_ptr & 15u)) return false;
  if (p.a_batches > 1 && (((uint64_t)p.M * p.K) & 7u) != 0) return false;
  if (p.b_batches > 1 && (((uint64_t)p.N * p.K) & 7u) != 0) return false;
  if (p.K == 0) return false;
  return true;
}

int LaunchMatMul(const MmParam &p_in, void *stream) {
  MmParam p = p_in;
  static const int group_env = getenv("DVM_B200_MM_GROUP_M") ? atoi(getenv("DVM_B200_MM_GROUP_M")) : 0;
  p.group_m = group_env > 0 ? static_cast<uint32_t>(group_env) : 8u;
  // "copy acc, product; store tensor s; end" with a dense row layout: the kernel stores the product directly
  p.fast_store_slot = 0xffffffffu;
  {
    const uint64_t w0 = p.epilogue[0], w1 = p.epilogue[1], w2 = p.epilogue[2];
    if (DVMB_OPC(w0) == OP_COPY && DVMB_OKIND(w0) == K_TENSOR && DVMB_OIDX(w0) == p.mma_slot && DVMB_OPC(w1) == OP_ST &&
        DVMB_OPC(w2) == OP_END && DVMB_SUB(w1) < p.n_tensors) {
      const EpiTensor &t = p.tensor[DVMB_SUB(w1)];
      if (t.sn == 1 && (t.dtype == p.in_dtype || t.dtype == T_F32)) p.fast_store_slot = DVMB_SUB(w1);
    }
  }
  // the gated form x / (c2 + exp(c1 * (x + c0 * x^3))) of the product, rounded to the operand type and stored
  p.gate_slot = 0xffffffffu;
  {
    static const bool off = getenv("DVM_B200_NO_FUSE") != nullptr;
    const uint64_t *w = p.epilogue;
    auto is = [&](int i, uint32_t opc, uint32_t sub, uint32_t okind) {
      return DVMB_OPC(w[i]) == opc && DVMB_SUB(w[i]) == sub && DVMB_OKIND(w[i]) == okind && DVMB_RND(w[i]) == RN_NONE &&
             (okind != K_TENSOR || DVMB_OIDX(w[i]) == p.mma_slot);
    };
    const uint32_t rnd_out = p.in_dtype == T_BF16 ? RN_BF16 : RN_F16;
    if (!off && DVMB_OPC(w[0]) == OP_COPY && DVMB_OKIND(w[0]) == K_TENSOR && DVMB_OIDX(w[0]) == p.mma_slot &&
        is(1, OP_BIN, B_MUL, K_ACC) && is(2, OP_BIN, B_MUL, K_TENSOR) && is(3, OP_BIN, B_MUL, K_IMM) && is(4, OP_BIN, B_ADD, K_TENSOR) &&
        is(5, OP_BIN, B_MUL, K_IMM) && DVMB_OPC(w[6]) == OP_UN && DVMB_SUB(w[6]) == U_EXP_FAST && DVMB_RND(w[6]) == RN_NONE &&
        is(7, OP_BIN, B_ADD, K_IMM) && is(8, OP_BIN, B_RDIV_FAST, K_TENSOR) && DVMB_OPC(w[9]) == OP_CVT && DVMB_SUB(w[9]) == V_RND &&
        DVMB_RND(w[9]) == rnd_out && DVMB_OPC(w[10]) == OP_ST && DVMB_OPC(w[11]) == OP_END && DVMB_SUB(w[10]) < p.n_tensors) {
      const EpiTensor &t = p.tensor[DVMB_SUB(w[10])];
      if (t.sn == 1 && t.dtype == p.in_dtype) {
        p.gate_slot = DVMB_SUB(w[10]);
        p.gate_c[0] = DVMB_IMM(w[3]);
        p.gate_c[1] = DVMB_IMM(w[5]);
        p.gate_c[2] = DVMB_IMM(w[7]);
      }
    }
  }
  if (p.M == 0 || p.N == 0 || p.batch0 * p.batch1 == 0) return 0;
  if (p.in_dtype != T_BF16 && p.in_dtype != T_F16) return -3;
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (!MatMulUsesTensorCores(p)) {
    const uint64_t total = (uint64_t)p.batch0 * p.batch1 * p.M * ((p.N + 15u) / 16u);
    const uint64_t blocks = (total + 127) / 128;
    const uint32_t grid = static_cast<uint32_t>(blocks < (uint64_t)sms * 16 ? blocks : (uint64_t)sms * 16);
    dvm_b200_mm_simt<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return static_cast<int>(cudaGetLastError());
  }
  if (p.leave_sms != 0 && static_cast<int>(p.leave_sms) + 32 <= sms) sms -= static_cast<int>(p.leave_sms);
  static bool attr_set[64] = {false};
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(dvm_b200_mm_tcgen05, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<1>::kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(dvm_b200_mm_tcgen05_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<2>::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  // CTA pairs pay off once there are at least two row blocks; a single row block runs unpaired
  static const int force = getenv("DVM_B200_MM_CTAS") ? atoi(getenv("DVM_B200_MM_CTAS")) : 0;
  const bool pair = force ? force == 2 : p.M > BM;
  MmMaps maps;
  // fp16 and bf16 are both 2-byte types for the copy engine; the MMA descriptor carries the real format
  int rc = p.a_mmajor ? EncodeOperand(&maps.a, p.a_ptr, p.M, p.K, p.a_batches, 64)
                      : EncodeOperand(&maps.a, p.a_ptr, p.K, p.M, p.a_batches, BM);
  if (rc != 0) return rc;
  rc = p.b_kmajor ? EncodeOperand(&maps.b, p.b_ptr, p.K, p.N, p.b_batches, pair ? BN / 2 : BN)
                  : EncodeOperand(&maps.b, p.b_ptr, p.N, p.K, p.b_batches, 64);
  if (rc != 0) return rc;
  const uint32_t batch = p.batch0 * p.batch1;
  if (pair) {
    const uint32_t tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN) * batch;
    const uint32_t units = tiles < static_cast<uint32_t>(sms / 2) ? tiles : static_cast<uint32_t>(sms / 2);
    dvm_b200_mm_tcgen05_pair<<<units * 2, kThreads, Geo<2>::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(p, maps, NextLaunchEpoch());
  } else {
    const uint32_t tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * batch;
    const uint32_t grid = tiles < static_cast<uint32_t>(sms) ? tiles : static_cast<uint32_t>(sms);
    dvm_b200_mm_tcgen05<<<grid, kThreads, Geo<1>::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(p, maps, NextLaunchEpoch());
  }
  return static_cast<int>(cudaGetLastError());
}

unsigned int ReadMatMulStatus() {
  WaitStatus v = {0u, 0u};
  const unsigned int zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_mm_status, sizeof(v)) != cudaSuccess) return 0xffffffffu;
  if (v.first_error != 0) cudaMemcpyToSymbol(g_mm_status, &zero, sizeof(zero), offsetof(WaitStatus, first_error));
  return v.first_error;
}

}  // namespace dvmb
