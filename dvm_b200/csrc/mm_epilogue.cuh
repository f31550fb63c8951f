// Post-fusion interpreter of the MatMul kernels: runs the fused vector ops (the reference shards them per C
// tile, src/xkernel.cc:309-319) on 16 consecutive columns of one result row while the accumulator is being
// drained, so the product never makes a round trip through global memory.
#ifndef DVM_B200_MM_EPILOGUE_CUH_
#define DVM_B200_MM_EPILOGUE_CUH_

#include "mm_launch.h"
#include "vm_ops.cuh"

namespace dvmb {
namespace {

constexpr int kEpiLanes = 16;

struct EpiPos {
  uint32_t b0, b1, row, col;   // coordinates of lane 0
  uint32_t valid;              // lanes inside the matrix (0..16); lanes past it are neither loaded nor stored
};

__device__ __forceinline__ size_t epi_offset(const EpiTensor &t, const EpiPos &p) {
  return (size_t)((int64_t)p.b0 * t.sb0 + (int64_t)p.b1 * t.sb1 + (int64_t)p.row * t.sm + (int64_t)p.col * t.sn);
}

__device__ __noinline__ void epi_fetch(const EpiTensor &t, const EpiPos &p, uint32_t (&out)[kEpiLanes]) {
  const uint8_t *base = reinterpret_cast<const uint8_t *>(t.ptr);
  const size_t off = epi_offset(t, p);
  const uint32_t sh = item_shift(t.dtype);
  if (t.sn == 0) {
    uint32_t s;
    switch (t.dtype) {
      case T_F32:
      case T_I32: s = __ldg(reinterpret_cast<const uint32_t *>(base) + off); break;
      case T_F16:
      case T_BF16: s = widen(t.dtype, __ldg(reinterpret_cast<const unsigned short *>(base) + off)); break;
      default: s = __ldg(base + off); break;
    }
#pragma unroll
    for (int i = 0; i < kEpiLanes; ++i) out[i] = s;
    return;
  }
  const bool vec = p.valid == kEpiLanes && t.sn == 1 && ((t.ptr + (off << sh)) & 15u) == 0;
  if (vec) {
    if (sh == 2) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(base + ((off + 4 * g) << 2)));
        out[4 * g] = r.x; out[4 * g + 1] = r.y; out[4 * g + 2] = r.z; out[4 * g + 3] = r.w;
      }
    } else if (sh == 1) {
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(base + ((off + 8 * g) << 1)));
        unpack4(t.dtype, make_uint4(r.x, r.y, 0, 0), &out[8 * g]);
        unpack4(t.dtype, make_uint4(r.z, r.w, 0, 0), &out[8 * g + 4]);
      }
    } else {
      const uint4 r = __ldg(reinterpret_cast<const uint4 *>(base + off));
      unpack4(T_BOOL, make_uint4(r.x, 0, 0, 0), &out[0]);
      unpack4(T_BOOL, make_uint4(r.y, 0, 0, 0), &out[4]);
      unpack4(T_BOOL, make_uint4(r.z, 0, 0, 0), &out[8]);
      unpack4(T_BOOL, make_uint4(r.w, 0, 0, 0), &out[12]);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < kEpiLanes; ++i) {
    uint32_t v = 0;
    if ((uint32_t)i < p.valid) {
      const size_t o = off + (size_t)((int64_t)i * t.sn);
      switch (t.dtype) {
        case T_F32:
        case T_I32: v = __ldg(reinterpret_cast<const uint32_t *>(base) + o); break;
        case T_F16:
        case T_BF16: v = widen(t.dtype, __ldg(reinterpret_cast<const unsigned short *>(base) + o)); break;
        default: v = __ldg(base + o); break;
      }
    }
    out[i] = v;
  }
}

__device__ __noinline__ void epi_store(const EpiTensor &t, const EpiPos &p, const uint32_t (&v)[kEpiLanes]) {
  uint8_t *base = reinterpret_cast<uint8_t *>(t.ptr);
  const size_t off = epi_offset(t, p);
  const uint32_t sh = item_shift(t.dtype);
  const bool vec = p.valid == kEpiLanes && t.sn == 1 && ((t.ptr + (off << sh)) & 15u) == 0;
  if (vec) {
    if (sh == 2) {
#pragma unroll
      for (int g = 0; g < 4; ++g)
        *reinterpret_cast<uint4 *>(base + ((off + 4 * g) << 2)) = make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
    } else if (sh == 1) {
      uint32_t pk[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (t.dtype == T_BF16) {
          pk[i] = pack_bf16x2(u2f(v[2 * i]), u2f(v[2 * i + 1]));
        } else {
          const __half2 h = __floats2half2_rn(u2f(v[2 * i]), u2f(v[2 * i + 1]));
          pk[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
      }
      *reinterpret_cast<uint4 *>(base + (off << 1)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      *reinterpret_cast<uint4 *>(base + (off << 1) + 16) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    } else {
      uint32_t pk[4];
#pragma unroll
      for (int g = 0; g < 4; ++g)
        pk[g] = (v[4 * g] & 0xffu) | ((v[4 * g + 1] & 0xffu) << 8) | ((v[4 * g + 2] & 0xffu) << 16) | (v[4 * g + 3] << 24);
      *reinterpret_cast<uint4 *>(base + off) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < kEpiLanes; ++i)
    if ((uint32_t)i < p.valid) {
      const size_t o = off + (size_t)((int64_t)i * t.sn);
      switch (t.dtype) {
        case T_F32:
        case T_I32: reinterpret_cast<uint32_t *>(base)[o] = v[i]; break;
        case T_F16:
        case T_BF16: reinterpret_cast<unsigned short *>(base)[o] = (unsigned short)narrow(t.dtype, v[i]); break;
        default: base[o] = (uint8_t)v[i]; break;
      }
    }
}

// Run the post-fusion program on one 16-column strip.  `frag` is the rounded product in register form.
__device__ __forceinline__ void run_epilogue(const MmParam &P, const EpiPos &pos, const uint32_t (&frag)[kEpiLanes]) {
  uint32_t acc[kEpiLanes];
  uint32_t temps[kNumTemps][kEpiLanes];
#pragma unroll
  for (int i = 0; i < kEpiLanes; ++i) acc[i] = frag[i];
  for (uint32_t pc = 0;; ++pc) {
    const uint64_t w = P.epilogue[pc];
    const uint32_t opc = DVMB_OPC(w);
    if (opc == OP_END) break;
    const uint32_t sub = DVMB_SUB(w);
    uint32_t b[kEpiLanes];
    if (opc == OP_COPY || opc == OP_BIN || opc == OP_CMP || opc == OP_SEL) {
      const uint32_t okind = DVMB_OKIND(w), oidx = DVMB_OIDX(w);
      if (okind == K_TENSOR) {
        if (oidx == P.mma_slot) {
#pragma unroll
          for (int i = 0; i < kEpiLanes; ++i) b[i] = frag[i];
        } else {
          uint32_t tmp[kEpiLanes];
          epi_fetch(P.tensor[oidx], pos, tmp);
#pragma unroll
          for (int i = 0; i < kEpiLanes; ++i) b[i] = tmp[i];
        }
      } else if (okind == K_TEMP) {
#pragma unroll
        for (int i = 0; i < kEpiLanes; ++i) b[i] = temps[oidx][i];
      } else if (okind == K_IMM) {
#pragma unroll
        for (int i = 0; i < kEpiLanes; ++i) b[i] = DVMB_IMM(w);
      } else {
#pragma unroll
        for (int i = 0; i < kEpiLanes; ++i) b[i] = acc[i];
      }
    }
    const VecOperand<kEpiLanes> bo{b};
    switch (opc) {
      case OP_ST: {
        uint32_t tmp[kEpiLanes];
#pragma unroll
        for (int i = 0; i < kEpiLanes; ++i) tmp[i] = acc[i];
        epi_store(P.tensor[sub], pos, tmp);
        break;
      }
      case OP_COPY:
#pragma unroll
        for (int i = 0; i < kEpiLanes; ++i) acc[i] = b[i];
        break;
      case OP_MOV: {
        const uint32_t d = DVMB_DST(w);
#pragma unroll
        for (int i = 0; i < kEpiLanes; ++i) temps[d][i] = acc[i];
        break;
      }
      case OP_UN: apply_un<kEpiLanes>(sub, acc); apply_round<kEpiLanes>(DVMB_RND(w), acc); break;
      case OP_BIN: apply_bin<kEpiLanes>(sub, acc, bo); apply_round<kEpiLanes>(DVMB_RND(w), acc); break;
      case OP_CMP: apply_cmp<kEpiLanes>(sub, DVMB_ISINT(w), acc, bo); break;
      case OP_SEL: {
        uint32_t c[kEpiLanes];
        const uint32_t k2 = sub >> 4, i2 = sub & 15u;
        if (k2 == K_TEMP) {
#pragma unroll
          for (int i = 0; i < kEpiLanes; ++i) c[i] = temps[i2][i];
        } else if (i2 == P.mma_slot) {
#pragma unroll
          for (int i = 0; i < kEpiLanes; ++i) c[i] = frag[i];
        } else {
          uint32_t tmp[kEpiLanes];
          epi_fetch(P.tensor[i2], pos, tmp);
#pragma unroll
          for (int i = 0; i < kEpiLanes; ++i) c[i] = tmp[i];
        }
        apply_sel<kEpiLanes>(DVMB_ISINT(w), DVMB_DST(w) & 1u, acc, bo, c);
        break;
      }
      case OP_CVT: apply_cvt<kEpiLanes>(sub, acc); apply_round<kEpiLanes>(DVMB_RND(w), acc); break;
      default: break;
    }
  }
}

}  // namespace
}  // namespace dvmb

#endif  // DVM_B200_MM_EPILOGUE_CUH_
