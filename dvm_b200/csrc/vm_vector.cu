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

#include <cstdint>

#include "isa.h"
#include "vm_launch.h"

namespace dvmb {

__device__ unsigned int g_vm_status = 0;   // 0 = ok; else (code << 24 | blockIdx)

namespace {

__device__ __forceinline__ float u2f(uint32_t v) { return __uint_as_float(v); }
__device__ __forceinline__ uint32_t f2u(float v) { return __float_as_uint(v); }

__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }
// Round-to-nearest-even to bf16 precision; NaN stays NaN (the host encoder's rule, src/dvm.cc:173-186).
__device__ __forceinline__ float round_bf16(float v) {
  uint32_t u = f2u(v);
  if ((u & 0x7fffffffu) > 0x7f800000u) return u2f(0x7fc00000u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return u2f(u & 0xffff0000u);
}
// Two floats -> packed bf16x2 (lo in bits 0..15), hardware round-to-nearest-even, NaN preserved.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int N>
__device__ __forceinline__ void apply_round(uint32_t rnd, uint32_t (&a)[N]) {
  if (rnd == RN_F16) {
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = f2u(round_f16(u2f(a[i])));
  } else if (rnd == RN_BF16) {
    if constexpr (N % 2 == 0) {
#pragma unroll
      for (int i = 0; i < N; i += 2) {
        uint32_t p = pack_bf16x2(u2f(a[i]), u2f(a[i + 1]));
        a[i] = p << 16;
        a[i + 1] = p & 0xffff0000u;
      }
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = f2u(round_bf16(u2f(a[i])));
    }
  }
}

#define DVMB_UN_LOOP(EXPR)                 \
  _Pragma("unroll") for (int i = 0; i < N; ++i) { \
    float x = u2f(a[i]);                   \
    a[i] = f2u(EXPR);                      \
  }

template <int N>
__device__ __forceinline__ void apply_un(uint32_t kind, uint32_t (&a)[N]) {
  switch (kind) {
    case U_SQRT: DVMB_UN_LOOP(sqrtf(x)) break;
    case U_ABS: DVMB_UN_LOOP(fabsf(x)) break;
    case U_LOG: DVMB_UN_LOOP(logf(x)) break;
    case U_EXP: DVMB_UN_LOOP(expf(x)) break;
    case U_ROUND: DVMB_UN_LOOP(nearbyintf(x)) break;
    case U_FLOOR: DVMB_UN_LOOP(floorf(x)) break;
    case U_CEIL: DVMB_UN_LOOP(ceilf(x)) break;
    case U_TRUNC: DVMB_UN_LOOP(truncf(x)) break;
    case U_ISFINITE: DVMB_UN_LOOP((isfinite(x) ? 1.0f : 0.0f)) break;
    case U_ABS_I:
#pragma unroll
      for (int i = 0; i < N; ++i) {
        int32_t x = (int32_t)a[i];
        a[i] = x < 0 ? (0u - a[i]) : a[i];
      }
      break;
    default: break;
  }
}

// Second operands come either as a per-lane vector or as one value for all lanes.
template <int N>
struct VecOperand {
  const uint32_t (&v)[N];
  __device__ __forceinline__ uint32_t operator()(int i) const { return v[i]; }
};
struct SplatOperand {
  uint32_t v;
  __device__ __forceinline__ uint32_t operator()(int) const { return v; }
};

#define DVMB_BIN_F(EXPR)                   \
  _Pragma("unroll") for (int i = 0; i < N; ++i) { \
    float x = u2f(a[i]), y = u2f(b(i));    \
    a[i] = f2u(EXPR);                      \
  }
#define DVMB_BIN_I(EXPR)                   \
  _Pragma("unroll") for (int i = 0; i < N; ++i) { \
    int32_t x = (int32_t)a[i], y = (int32_t)b(i); \
    a[i] = (uint32_t)(EXPR);               \
  }

template <int N, class B>
__device__ __forceinline__ void apply_bin(uint32_t kind, uint32_t (&a)[N], const B &b) {
  switch (kind) {
    case B_ADD: DVMB_BIN_F(x + y) break;
    case B_SUB: DVMB_BIN_F(x - y) break;
    case B_MUL: DVMB_BIN_F(x * y) break;
    case B_DIV: DVMB_BIN_F(x / y) break;
    case B_MAX: DVMB_BIN_F((x > y ? x : y)) break;
    case B_MIN: DVMB_BIN_F((x < y ? x : y)) break;
    case B_POW: DVMB_BIN_F(powf(x, y)) break;
    case B_RSUB: DVMB_BIN_F(y - x) break;
    case B_RDIV: DVMB_BIN_F(y / x) break;
    case B_ADD_I: DVMB_BIN_I((uint32_t)x + (uint32_t)y) break;
    case B_SUB_I: DVMB_BIN_I((uint32_t)x - (uint32_t)y) break;
    case B_MUL_I: DVMB_BIN_I((uint32_t)x * (uint32_t)y) break;
    case B_MAX_I: DVMB_BIN_I((x > y ? x : y)) break;
    case B_MIN_I: DVMB_BIN_I((x < y ? x : y)) break;
    case B_RSUB_I: DVMB_BIN_I((uint32_t)y - (uint32_t)x) break;
    default: break;
  }
}

template <typename T>
__device__ __forceinline__ bool cmp_value(uint32_t kind, T x, T y) {
  switch (kind) {
    case C_EQ: return x == y;
    case C_NE: return x != y;
    case C_GT: return x > y;
    case C_GE: return x >= y;
    case C_LT: return x < y;
    default: return x <= y;
  }
}

template <int N, class B>
__device__ __forceinline__ void apply_cmp(uint32_t kind, uint32_t isint, uint32_t (&a)[N], const B &b) {
  if (isint) {
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = cmp_value<int32_t>(kind, (int32_t)a[i], (int32_t)b(i)) ? 1u : 0u;
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = cmp_value<float>(kind, u2f(a[i]), u2f(b(i))) ? 0x3f800000u : 0u;
  }
}

// a <- cond(a) ? b : c; `inv` swaps the alternatives (the free-form operand b is then the false value).
template <int N, class B>
__device__ __forceinline__ void apply_sel(uint32_t isint, uint32_t inv, uint32_t (&a)[N], const B &b,
                                          const uint32_t (&c)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) {
    bool t = isint ? (a[i] != 0u) : (u2f(a[i]) != 0.0f);
    if (inv) t = !t;
    a[i] = t ? b(i) : c[i];
  }
}

template <int N>
__device__ __forceinline__ void apply_cvt(uint32_t kind, uint32_t (&a)[N]) {
  switch (kind) {
    case V_F2I:
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = (uint32_t)(int32_t)u2f(a[i]);
      break;
    case V_I2F:
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = f2u((float)(int32_t)a[i]);
      break;
    case V_NEZ_F:
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = u2f(a[i]) != 0.0f ? 1u : 0u;
      break;
    case V_NEZ_I:
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = a[i] != 0u ? 1u : 0u;
      break;
    default: break;
  }
}

__device__ __forceinline__ float red_identity(uint32_t kind) {
  return kind == R_SUM ? 0.0f : (kind == R_MAX ? -CUDART_INF_F : CUDART_INF_F);
}
__device__ __forceinline__ float red_combine(uint32_t kind, float x, float y) {
  return kind == R_SUM ? x + y : (kind == R_MAX ? (x > y ? x : y) : (x < y ? x : y));
}

// ---- element conversion ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t widen(uint32_t dtype, uint32_t raw) {
  switch (dtype) {
    case T_F16: return f2u(__half2float(__ushort_as_half((unsigned short)raw)));
    case T_BF16: return raw << 16;
    default: return raw;
  }
}

__device__ __forceinline__ uint32_t load_elem(uint32_t dtype, const uint8_t *base, uint32_t off) {
  switch (dtype) {
    case T_F32:
    case T_I32: return __ldg(reinterpret_cast<const uint32_t *>(base) + off);
    case T_F16:
    case T_BF16: return widen(dtype, __ldg(reinterpret_cast<const unsigned short *>(base) + off));
    default: return __ldg(base + off);
  }
}

__device__ __forceinline__ uint32_t narrow(uint32_t dtype, uint32_t v) {
  switch (dtype) {
    case T_F16: return __half_as_ushort(__float2half_rn(u2f(v)));
    case T_BF16: return f2u(round_bf16(u2f(v))) >> 16;
    default: return v;
  }
}

__device__ __forceinline__ void store_elem(uint32_t dtype, uint8_t *base, uint32_t off, uint32_t v) {
  switch (dtype) {
    case T_F32:
    case T_I32: reinterpret_cast<uint32_t *>(base)[off] = v; break;
    case T_F16:
    case T_BF16: reinterpret_cast<unsigned short *>(base)[off] = (unsigned short)narrow(dtype, v); break;
    default: base[off] = (uint8_t)v; break;
  }
}

// Unpack one raw 4-element granule (16 / 8 / 4 bytes by dtype) into register form.
__device__ __forceinline__ void unpack4(uint32_t dtype, uint4 raw, uint32_t *out) {
  switch (dtype) {
    case T_F32:
    case T_I32: out[0] = raw.x; out[1] = raw.y; out[2] = raw.z; out[3] = raw.w; break;
    case T_F16: {
      float2 lo = __half22float2(*reinterpret_cast<__half2 *>(&raw.x));
      float2 hi = __half22float2(*reinterpret_cast<__half2 *>(&raw.y));
      out[0] = f2u(lo.x); out[1] = f2u(lo.y); out[2] = f2u(hi.x); out[3] = f2u(hi.y);
      break;
    }
    case T_BF16:
      out[0] = raw.x << 16; out[1] = raw.x & 0xffff0000u; out[2] = raw.y << 16; out[3] = raw.y & 0xffff0000u;
      break;
    default:
      out[0] = raw.x & 0xffu; out[1] = (raw.x >> 8) & 0xffu; out[2] = (raw.x >> 16) & 0xffu; out[3] = raw.x >> 24;
      break;
  }
}

__device__ __forceinline__ uint4 gload4(uint32_t dtype, const uint8_t *base, uint32_t off) {
  uint4 r = make_uint4(0, 0, 0, 0);
  switch (dtype) {
    case T_F32:
    case T_I32: r = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const uint32_t *>(base) + off)); break;
    case T_F16:
    case T_BF16: {
      uint2 v = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const unsigned short *>(base) + off));
      r.x = v.x; r.y = v.y;
      break;
    }
    default: r.x = __ldg(reinterpret_cast<const uint32_t *>(base + off)); break;
  }
  return r;
}

__device__ __forceinline__ uint4 sload4(uint32_t dtype, uint32_t saddr) {
  uint4 r = make_uint4(0, 0, 0, 0);
  switch (dtype) {
    case T_F32:
    case T_I32: asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(saddr)); break;
    case T_F16:
    case T_BF16: asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(saddr)); break;
    default: asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r.x) : "r"(saddr)); break;
  }
  return r;
}

__device__ __forceinline__ void gstore4(uint32_t dtype, uint8_t *base, uint32_t off, const uint32_t *v) {
  switch (dtype) {
    case T_F32:
    case T_I32:
      *reinterpret_cast<uint4 *>(reinterpret_cast<uint32_t *>(base) + off) = make_uint4(v[0], v[1], v[2], v[3]);
      break;
    case T_F16: {
      __half2 lo = __floats2half2_rn(u2f(v[0]), u2f(v[1]));
      __half2 hi = __floats2half2_rn(u2f(v[2]), u2f(v[3]));
      uint2 p;
      p.x = *reinterpret_cast<uint32_t *>(&lo);
      p.y = *reinterpret_cast<uint32_t *>(&hi);
      *reinterpret_cast<uint2 *>(reinterpret_cast<unsigned short *>(base) + off) = p;
      break;
    }
    case T_BF16: {
      uint2 p;
      p.x = pack_bf16x2(u2f(v[0]), u2f(v[1]));
      p.y = pack_bf16x2(u2f(v[2]), u2f(v[3]));
      *reinterpret_cast<uint2 *>(reinterpret_cast<unsigned short *>(base) + off) = p;
      break;
    }
    default:
      *reinterpret_cast<uint32_t *>(base + off) =
        (v[0] & 0xffu) | ((v[1] & 0xffu) << 8) | ((v[2] & 0xffu) << 16) | (v[3] << 24);
      break;
  }
}

__device__ __forceinline__ uint32_t item_shift(uint32_t dtype) {
  return dtype == T_BOOL ? 0u : ((dtype == T_F16 || dtype == T_BF16) ? 1u : 2u);
}

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
// Bounded wait: gives up after about two seconds and records `code` in the status word.  Once any wait
// of the launch has expired every later wait returns at once, so the kernel always runs to its end (with
// wrong results, which the host reports through the status word) instead of hanging.
__device__ __noinline__ void mbar_wait_slow(uint32_t addr, uint32_t parity, uint32_t code) {
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait(addr, parity)) return;
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    if (*reinterpret_cast<volatile unsigned int *>(&g_vm_status) != 0u) return;
    for (int i = 0; i < 1024; ++i)
      if (mbar_try_wait(addr, parity)) return;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 > 2000000000ull) {
      atomicCAS(&g_vm_status, 0u, (code << 24) | (blockIdx.x & 0xffffffu));
      return;
    }
  }
}
__device__ __forceinline__ void mbar_wait(uint32_t addr, uint32_t parity, uint32_t code) {
  if (mbar_try_wait(addr, parity)) return;
  mbar_wait_slow(addr, parity, code);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(mbar)
               : "memory");
}

// ---- addressing -----------------------------------------------------------------------------------

// Per-thread position inside the iteration space.
struct Pos {
  uint32_t k[kMaxKept];      // kept coordinates of this thread's group
  uint32_t e0[2];            // first element (inside the group) of each granule
  int32_t nv[2];             // valid elements of each granule (0..4)
  uint32_t ec[2][kMaxEnum];  // enumerated coordinates of each granule's first element (AM_GRANULE)
  uint32_t in_chunk[2];      // element index of each granule inside its chunk
  uint32_t chunk_valid;      // valid elements of the current chunk
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

// Fetch the 8 lanes of tensor `slot` for this thread: from the ring stage when the tensor is staged and the
// granule lies inside the bulk-copied part, else straight from global memory.
__device__ __forceinline__ void fetch_tensor(const VmParam &P, uint32_t slot, const Pos &pos, uint32_t stage_saddr,
                                             uint32_t (&out)[kLanes]) {
  const TensorDesc &td = P.tensor[slot];
  const uint32_t dtype = td.dtype, mode = td.mode;
  const uint32_t sh = item_shift(dtype);
  const bool staged = td.ring_off != kNoRing;
  // elements of the chunk that the bulk copy delivered (whole 16-byte units)
  const uint32_t bulk_elems = staged ? (((pos.chunk_valid << sh) & ~15u) >> sh) : 0u;
  const uint8_t *base = reinterpret_cast<const uint8_t *>(td.ptr);
  const uint32_t koff = kept_offset(td, pos.k);
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    uint32_t *o = &out[4 * g];
    if (staged && pos.in_chunk[g] + 4 <= bulk_elems) {
      unpack4(dtype, sload4(dtype, stage_saddr + td.ring_off + (pos.in_chunk[g] << sh)), o);
      continue;
    }
    const int nv = pos.gvalid ? pos.nv[g] : 0;
    if (mode == AM_ELEMENT) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        o[i] = 0;
        if (i < nv) {
          uint32_t c[kMaxEnum];
          split_enum(P, pos.e0[g] + i, c);
          o[i] = load_elem(dtype, base, koff + enum_offset(td, c));
        }
      }
      continue;
    }
    uint32_t off = koff;
    uint32_t istride = 1;
    if (mode == AM_GRANULE) {
      off += enum_offset(td, pos.ec[g]);
      istride = td.estride[kMaxEnum - 1];
    } else if (mode == AM_DENSE) {
      off += pos.e0[g];
    } else {
      istride = 0;
    }
    if (td.vec_ok && nv == 4) {
      unpack4(dtype, gload4(dtype, base, off), o);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = i < nv ? load_elem(dtype, base, off + i * istride) : 0u;
    }
  }
}

__device__ __forceinline__ void store_tensor(const VmParam &P, uint32_t slot, const Pos &pos,
                                             const uint32_t (&val)[kLanes]) {
  const TensorDesc &td = P.tensor[slot];
  uint8_t *base = reinterpret_cast<uint8_t *>(td.ptr);
  const uint32_t dtype = td.dtype, mode = td.mode;
  const uint32_t koff = kept_offset(td, pos.k);
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int nv = pos.gvalid ? pos.nv[g] : 0;
    const uint32_t *v = &val[4 * g];
    if (mode == AM_ELEMENT) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (i < nv) {
          uint32_t c[kMaxEnum];
          split_enum(P, pos.e0[g] + i, c);
          store_elem(dtype, base, koff + enum_offset(td, c), v[i]);
        }
      }
      continue;
    }
    uint32_t off = koff;
    uint32_t istride = 1;
    if (mode == AM_GRANULE) {
      off += enum_offset(td, pos.ec[g]);
      istride = td.estride[kMaxEnum - 1];
    } else if (mode == AM_DENSE) {
      off += pos.e0[g];
    } else {
      istride = 0;
    }
    if (td.vec_ok && nv == 4) {
      gstore4(dtype, base, off, v);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < nv) store_elem(dtype, base, off + i * istride, v[i]);
    }
  }
}

#define DVMB_PART_CASES(IDX, STMT) \
  switch (IDX) {                   \
    case 0: { constexpr int J = 0; STMT } break; \
    case 1: { constexpr int J = 1; STMT } break; \
    case 2: { constexpr int J = 2; STMT } break; \
    default: { constexpr int J = 3; STMT } break; \
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
__device__ __forceinline__ void vm_vector_body(const VmParam &P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t tid = threadIdx.x;
  const uint32_t T = P.tg * P.groups_per_cta;   // consumer threads
  const bool flat = P.mode == VM_FLAT;
  const uint32_t S = P.num_stages;
  const bool ring = P.stage_bytes != 0;
  const uint32_t ngb = flat ? 1u : (P.num_groups + P.groups_per_cta - 1) / P.groups_per_cta;
  const uint32_t gb_begin = flat ? 0u : blockIdx.x, gb_step = flat ? 1u : gridDim.x;
  const uint32_t ch_begin = flat ? blockIdx.x : 0u, ch_step = flat ? gridDim.x : 1u;

  if (ring) {
    if (tid == 0) {
      for (uint32_t s = 0; s < S; ++s) {
        mbar_init(smem_base + kVmSmemBarriers + 8 * s, 1);        // full: one arrival (the producer) + tx bytes
        mbar_init(smem_base + kVmSmemBarriers + 64 + 8 * s, T);   // empty: every consumer thread
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
  }

  // =============================== producer warp ===============================
  if (tid >= T) {
    if (tid != T) return;
    uint32_t seq = 0;
    for (uint32_t gb = gb_begin; gb < ngb; gb += gb_step) {
      uint32_t k[kMaxKept];
      decompose_group(P, gb, k);   // groups_per_cta == 1 whenever the ring is on
      for (uint32_t ph = 0; ph < P.num_body; ++ph) {
        const uint32_t mask = P.body_ring_mask[ph];
        if (mask == 0) continue;
        for (uint32_t ch = ch_begin; ch < P.chunks; ch += ch_step, ++seq) {
          const uint32_t stage = seq % S, use = seq / S;
          const uint32_t full = smem_base + kVmSmemBarriers + 8 * stage;
          mbar_wait(full + 64, (use & 1u) ^ 1u, 1);
          const uint32_t e_start = ch * P.chunk_elems;
          const uint32_t valid = min(P.chunk_elems, P.group_elems - e_start);
          uint32_t c[kMaxEnum];
          split_enum(P, e_start, c);
          uint32_t total = 0;
          for (uint32_t m = mask; m; m &= m - 1) {
            const TensorDesc &td = P.tensor[__ffs(m) - 1];
            total += (valid << item_shift(td.dtype)) & ~15u;
          }
          if (total == 0) {
            mbar_arrive(full);
            continue;
          }
          mbar_arrive_expect_tx(full, total);
          const uint32_t stage_saddr = smem_base + kVmSmemStages + stage * P.stage_bytes;
          for (uint32_t m = mask; m; m &= m - 1) {
            const TensorDesc &td = P.tensor[__ffs(m) - 1];
            const uint32_t sh = item_shift(td.dtype);
            const uint32_t bytes = (valid << sh) & ~15u;
            if (bytes == 0) continue;
            const uint32_t off = kept_offset(td, k) + enum_offset(td, c);
            bulk_g2s(stage_saddr + td.ring_off, reinterpret_cast<const uint8_t *>(td.ptr) + ((size_t)off << sh), bytes, full);
          }
        }
      }
    }
    return;
  }

  // =============================== consumer warps ===============================
  float *red_buf = reinterpret_cast<float *>(smem + kVmSmemRed);
  const uint32_t temps_saddr = smem_base + kVmSmemStages + S * P.stage_bytes;
  const uint32_t sregs_saddr = temps_saddr + P.num_temps * T * 32u;
  const uint32_t tg = P.tg;
  const uint32_t lane_in_group = flat ? tid : tid % tg;
  const uint32_t group_in_cta = flat ? 0 : tid / tg;

  uint32_t acc[kLanes], b[kLanes], c[kLanes];
  uint32_t sacc[1] = {0};
  float part[kNumRSlots];
#pragma unroll
  for (int i = 0; i < kLanes; ++i) acc[i] = b[i] = c[i] = 0;
#pragma unroll
  for (int j = 0; j < kNumRSlots; ++j) part[j] = 0.0f;
  uint32_t red_par = 0;
  uint32_t seq = 0;
  Pos pos;

  auto temp_addr = [&](uint32_t k, uint32_t g) { return temps_saddr + ((k * 2 + g) * T + tid) * 16u; };
  auto sreg_addr = [&](uint32_t k) { return sregs_saddr + (k * T + tid) * 4u; };
  auto lds32 = [](uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
  };

  for (uint32_t gb = gb_begin; gb < ngb; gb += gb_step) {
    {
      uint32_t gi = gb * P.groups_per_cta + group_in_cta;
      pos.gvalid = gi < P.num_groups;
      decompose_group(P, pos.gvalid ? gi : 0u, pos.k);
    }
    for (uint32_t ph = 0; ph <= P.num_body; ++ph) {
      // ---------------- scalar side: PRO_ph ----------------
      for (uint32_t pc = P.sec[2 * ph];;) {
        const uint64_t w = P.code[pc++];
        const uint32_t opc = DVMB_OPC(w);
        if (opc == OP_END) break;
        const uint32_t sub = DVMB_SUB(w);
        uint32_t sb = 0;
        if (opc == OP_COPY || opc == OP_BIN || opc == OP_CMP || opc == OP_SEL) {
          const uint32_t okind = DVMB_OKIND(w), oidx = DVMB_OIDX(w);
          if (okind == K_SREG) {
            sb = lds32(sreg_addr(oidx));
          } else if (okind == K_IMM) {
            sb = DVMB_IMM(w);
          } else if (okind == K_TENSOR) {
            const TensorDesc &td = P.tensor[oidx];
            sb = load_elem(td.dtype, reinterpret_cast<const uint8_t *>(td.ptr), kept_offset(td, pos.k));
          } else {
            sb = sacc[0];
          }
        }
        const SplatOperand bo{sb};
        switch (opc) {
          case OP_ST: {
            const TensorDesc &td = P.tensor[sub];
            if (lane_in_group == 0 && pos.gvalid && (!flat || blockIdx.x == 0))
              store_elem(td.dtype, reinterpret_cast<uint8_t *>(td.ptr), kept_offset(td, pos.k), sacc[0]);
            break;
          }
          case OP_COPY: sacc[0] = sb; break;
          case OP_MOV: asm volatile("st.shared.u32 [%0], %1;" ::"r"(sreg_addr(DVMB_DST(w))), "r"(sacc[0]) : "memory"); break;
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
          case OP_RINIT: {
            const float id = red_identity(sub >> 4);
            DVMB_PART_CASES(sub & 3u, part[J] = id;)
            break;
          }
          case OP_RFIN: {
            const uint32_t kind = sub >> 4;
            float v = 0.0f;
            DVMB_PART_CASES(sub & 3u, v = part[J]; part[J] = red_identity(kind);)
            if (tg <= 32) {
              for (uint32_t o = tg >> 1; o > 0; o >>= 1) v = red_combine(kind, v, __shfl_xor_sync(0xffffffffu, v, o));
            } else {
#pragma unroll
              for (uint32_t o = 16; o > 0; o >>= 1) v = red_combine(kind, v, __shfl_xor_sync(0xffffffffu, v, o));
              if ((tid & 31u) == 0) red_buf[red_par * 32 + (tid >> 5)] = v;
              asm volatile("bar.sync 1, %0;" ::"r"(T) : "memory");   // consumer warps only
              const uint32_t nw = T >> 5;
              v = red_buf[red_par * 32];
              for (uint32_t wi = 1; wi < nw; ++wi) v = red_combine(kind, v, red_buf[red_par * 32 + wi]);
              red_par ^= 1u;
            }
            sacc[0] = f2u(v);
            break;
          }
          default: break;
        }
      }
      if (ph == P.num_body) break;
      // ---------------- vector side: BODY_ph over the chunks ----------------
      const uint32_t body_pc = P.sec[2 * ph + 1];
      const bool staged_body = ring && P.body_ring_mask[ph] != 0;
      for (uint32_t ch = ch_begin; ch < P.chunks; ch += ch_step) {
        const uint32_t e_start = ch * P.chunk_elems;
        pos.chunk_valid = min(P.chunk_elems, P.group_elems - e_start);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const uint32_t ic = (uint32_t)g * 4u * tg + 4u * lane_in_group;
          const int32_t left = (int32_t)pos.chunk_valid - (int32_t)ic;
          pos.in_chunk[g] = ic;
          pos.nv[g] = left >= 4 ? 4 : (left > 0 ? left : 0);
          pos.e0[g] = e_start + ic;
          if (P.need_coords) split_enum(P, pos.nv[g] > 0 ? pos.e0[g] : 0u, pos.ec[g]);
        }
        uint32_t stage_saddr = 0, empty_bar = 0;
        if (staged_body) {
          const uint32_t stage = seq % S, use = seq / S;
          ++seq;
          stage_saddr = smem_base + kVmSmemStages + stage * P.stage_bytes;
          empty_bar = smem_base + kVmSmemBarriers + 64 + 8 * stage;
          mbar_wait(smem_base + kVmSmemBarriers + 8 * stage, use & 1u, 2);
        }
        const bool full_tile = pos.chunk_valid == P.chunk_elems && pos.gvalid;
        const uint32_t ring_lane = stage_saddr;   // + offset + (in_chunk << shift) per fetch
        for (uint32_t pc = body_pc;; ++pc) {
          const uint64_t u = P.code[pc];
          const uint32_t uh = DVMB_UH(u);
          const uint32_t aux = DVMB_UAUX(u);
          const uint32_t arg = DVMB_UARG(u);
          if (uh == UH_END) break;
          uint32_t slot;
#define DVMB_TO_DEST(FN)                       \
  {                                            \
    const uint32_t d_ = aux & 3u;              \
    if (d_ == UD_ACC) { FN(acc) } else if (d_ == UD_B) { FN(b) } else { FN(c) } \
  }
#define DVMB_BINV(K, TYPE, CONV_IN, CONV_OUT, EXPR)              \
  case UH_BINV_FIRST + K: {                                      \
    _Pragma("unroll") for (int i = 0; i < kLanes; ++i) {         \
      TYPE x = CONV_IN(acc[i]), y = CONV_IN(b[i]);               \
      acc[i] = CONV_OUT(EXPR);                                   \
    }                                                            \
    continue;                                                    \
  }                                                              \
  case UH_BINS_FIRST + K: {                                      \
    const uint32_t sv_ = (aux & 1u) ? lds32(sreg_addr(arg)) : DVMB_UIMM(u); \
    const TYPE y = CONV_IN(sv_);                                 \
    _Pragma("unroll") for (int i = 0; i < kLanes; ++i) {         \
      TYPE x = CONV_IN(acc[i]);                                  \
      acc[i] = CONV_OUT(EXPR);                                   \
    }                                                            \
    continue;                                                    \
  }
#define DVMB_UNOP(K, EXPR)                                       \
  case UH_UN_FIRST + K: {                                        \
    _Pragma("unroll") for (int i = 0; i < kLanes; ++i) {         \
      float x = u2f(acc[i]);                                     \
      acc[i] = f2u(EXPR);                                        \
    }                                                            \
    continue;                                                    \
  }
#define DVMB_AS_INT(v) ((int32_t)(v))
#define DVMB_AS_U32(v) ((uint32_t)(v))
          switch (uh) {
            // ---------------- operand fetches ----------------
            case UH_LDR_F32: {
              slot = aux >> 2;
              if (!full_tile) goto fetch_generic;
              const uint32_t a0 = ring_lane + (arg << 4) + (pos.in_chunk[0] << 2);
              const uint32_t a1 = a0 + ((4u * tg) << 2);
#define DVMB_FN(V)                                                                                                  \
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(V[0]), "=r"(V[1]), "=r"(V[2]), "=r"(V[3]) : "r"(a0)); \
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(V[4]), "=r"(V[5]), "=r"(V[6]), "=r"(V[7]) : "r"(a1));
              DVMB_TO_DEST(DVMB_FN)
#undef DVMB_FN
              continue;
            }
            case UH_LDR_F16:
            case UH_LDR_BF16: {
              slot = aux >> 2;
              if (!full_tile) goto fetch_generic;
              const uint32_t a0 = ring_lane + (arg << 4) + (pos.in_chunk[0] << 1);
              const uint32_t a1 = a0 + ((4u * tg) << 1);
              uint2 r0, r1;
              asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r0.x), "=r"(r0.y) : "r"(a0));
              asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r1.x), "=r"(r1.y) : "r"(a1));
              if (uh == UH_LDR_BF16) {
#define DVMB_FN(V)                                                                                      \
  V[0] = r0.x << 16; V[1] = r0.x & 0xffff0000u; V[2] = r0.y << 16; V[3] = r0.y & 0xffff0000u;           \
  V[4] = r1.x << 16; V[5] = r1.x & 0xffff0000u; V[6] = r1.y << 16; V[7] = r1.y & 0xffff0000u;
                DVMB_TO_DEST(DVMB_FN)
#undef DVMB_FN
              } else {
#define DVMB_FN(V)                                                           \
  {                                                                          \
    float2 f0 = __half22float2(*reinterpret_cast<__half2 *>(&r0.x));         \
    float2 f1 = __half22float2(*reinterpret_cast<__half2 *>(&r0.y));         \
    float2 f2 = __half22float2(*reinterpret_cast<__half2 *>(&r1.x));         \
    float2 f3 = __half22float2(*reinterpret_cast<__half2 *>(&r1.y));         \
    V[0] = f2u(f0.x); V[1] = f2u(f0.y); V[2] = f2u(f1.x); V[3] = f2u(f1.y);  \
    V[4] = f2u(f2.x); V[5] = f2u(f2.y); V[6] = f2u(f3.x); V[7] = f2u(f3.y);  \
  }
                DVMB_TO_DEST(DVMB_FN)
#undef DVMB_FN
              }
              continue;
            }
            case UH_LDR_U8: {
              slot = aux >> 2;
              if (!full_tile) goto fetch_generic;
              const uint32_t a0 = ring_lane + (arg << 4) + pos.in_chunk[0];
              const uint32_t r0 = lds32(a0), r1 = lds32(a0 + 4u * tg);
#define DVMB_FN(V)                                                                                \
  V[0] = r0 & 0xffu; V[1] = (r0 >> 8) & 0xffu; V[2] = (r0 >> 16) & 0xffu; V[3] = r0 >> 24;        \
  V[4] = r1 & 0xffu; V[5] = (r1 >> 8) & 0xffu; V[6] = (r1 >> 16) & 0xffu; V[7] = r1 >> 24;
              DVMB_TO_DEST(DVMB_FN)
#undef DVMB_FN
              continue;
            }
            case UH_LDG: {
              slot = aux >> 2;
            fetch_generic:
#define DVMB_FN(V) fetch_tensor(P, slot, pos, stage_saddr, V);
              DVMB_TO_DEST(DVMB_FN)
#undef DVMB_FN
              continue;
            }
            case UH_LDT: {
#define DVMB_FN(V)                                                                                              \
  _Pragma("unroll") for (int g = 0; g < 2; ++g)                                                                  \
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"                                                         \
                 : "=r"(V[4 * g]), "=r"(V[4 * g + 1]), "=r"(V[4 * g + 2]), "=r"(V[4 * g + 3])                    \
                 : "r"(temp_addr(arg, g)));
              DVMB_TO_DEST(DVMB_FN)
#undef DVMB_FN
              continue;
            }
            case UH_LDS:
            case UH_LDI: {
              const uint32_t v = uh == UH_LDS ? lds32(sreg_addr(arg)) : DVMB_UIMM(u);
#define DVMB_FN(V) _Pragma("unroll") for (int i = 0; i < kLanes; ++i) V[i] = v;
              DVMB_TO_DEST(DVMB_FN)
#undef DVMB_FN
              continue;
            }
            case UH_MOVA: {
              if ((aux & 3u) == UD_B) {
#pragma unroll
                for (int i = 0; i < kLanes; ++i) b[i] = acc[i];
              } else {
#pragma unroll
                for (int i = 0; i < kLanes; ++i) c[i] = acc[i];
              }
              continue;
            }
            case UH_STT: {
#pragma unroll
              for (int g = 0; g < 2; ++g)
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(temp_addr(arg, g)), "r"(acc[4 * g]),
                             "r"(acc[4 * g + 1]), "r"(acc[4 * g + 2]), "r"(acc[4 * g + 3])
                             : "memory");
              continue;
            }
            // ---------------- arithmetic ----------------
            DVMB_BINV(B_ADD, float, u2f, f2u, x + y)
            DVMB_BINV(B_SUB, float, u2f, f2u, x - y)
            DVMB_BINV(B_MUL, float, u2f, f2u, x * y)
            DVMB_BINV(B_DIV, float, u2f, f2u, x / y)
            DVMB_BINV(B_MAX, float, u2f, f2u, (x > y ? x : y))
            DVMB_BINV(B_MIN, float, u2f, f2u, (x < y ? x : y))
            DVMB_BINV(B_POW, float, u2f, f2u, powf(x, y))
            DVMB_BINV(B_RSUB, float, u2f, f2u, y - x)
            DVMB_BINV(B_RDIV, float, u2f, f2u, y / x)
            DVMB_BINV(B_ADD_I, uint32_t, DVMB_AS_U32, DVMB_AS_U32, x + y)
            DVMB_BINV(B_SUB_I, uint32_t, DVMB_AS_U32, DVMB_AS_U32, x - y)
            DVMB_BINV(B_MUL_I, uint32_t, DVMB_AS_U32, DVMB_AS_U32, x * y)
            DVMB_BINV(B_MAX_I, int32_t, DVMB_AS_INT, DVMB_AS_U32, (x > y ? x : y))
            DVMB_BINV(B_MIN_I, int32_t, DVMB_AS_INT, DVMB_AS_U32, (x < y ? x : y))
            DVMB_BINV(B_RSUB_I, uint32_t, DVMB_AS_U32, DVMB_AS_U32, y - x)
            DVMB_UNOP(U_SQRT, sqrtf(x))
            DVMB_UNOP(U_ABS, fabsf(x))
            DVMB_UNOP(U_LOG, logf(x))
            DVMB_UNOP(U_EXP, expf(x))
            DVMB_UNOP(U_ROUND, nearbyintf(x))
            DVMB_UNOP(U_FLOOR, floorf(x))
            DVMB_UNOP(U_CEIL, ceilf(x))
            DVMB_UNOP(U_TRUNC, truncf(x))
            DVMB_UNOP(U_ISFINITE, (isfinite(x) ? 1.0f : 0.0f))
            case UH_UN_FIRST + U_ABS_I: {
#pragma unroll
              for (int i = 0; i < kLanes; ++i) acc[i] = (int32_t)acc[i] < 0 ? (0u - acc[i]) : acc[i];
              continue;
            }
            case UH_UN_FIRST + U_NOP: continue;
            case UH_RND_F16: apply_round<kLanes>(RN_F16, acc); continue;
            case UH_RND_BF16: apply_round<kLanes>(RN_BF16, acc); continue;
            case UH_CMP_F_V: apply_cmp<kLanes>(aux & 7u, 0, acc, VecOperand<kLanes>{b}); continue;
            case UH_CMP_I_V: apply_cmp<kLanes>(aux & 7u, 1, acc, VecOperand<kLanes>{b}); continue;
            case UH_CMP_F_S:
            case UH_CMP_I_S: {
              const SplatOperand so{(aux & 0x80u) ? lds32(sreg_addr(arg)) : DVMB_UIMM(u)};
              apply_cmp<kLanes>(aux & 7u, uh == UH_CMP_I_S ? 1u : 0u, acc, so);
              continue;
            }
            case UH_SEL_F: apply_sel<kLanes>(0, 0, acc, VecOperand<kLanes>{b}, c); continue;
            case UH_SEL_I: apply_sel<kLanes>(1, 0, acc, VecOperand<kLanes>{b}, c); continue;
            case UH_CVT_F2I: apply_cvt<kLanes>(V_F2I, acc); continue;
            case UH_CVT_I2F: apply_cvt<kLanes>(V_I2F, acc); continue;
            case UH_CVT_NEZ_F: apply_cvt<kLanes>(V_NEZ_F, acc); continue;
            case UH_CVT_NEZ_I: apply_cvt<kLanes>(V_NEZ_I, acc); continue;
            case UH_RACC_SUM:
            case UH_RACC_MAX:
            case UH_RACC_MIN: {
              const uint32_t kind = uh - UH_RACC_SUM;
              float v = red_identity(kind);
              if (full_tile) {
#pragma unroll
                for (int i = 0; i < kLanes; ++i) v = red_combine(kind, v, u2f(acc[i]));
              } else {
#pragma unroll
                for (int i = 0; i < kLanes; ++i)
                  if (pos.gvalid && (i & 3) < pos.nv[i >> 2]) v = red_combine(kind, v, u2f(acc[i]));
              }
              DVMB_PART_CASES(arg & 3u, part[J] = red_combine(kind, part[J], v);)
              continue;
            }
            // ---------------- stores ----------------
            case UH_ST_F32:
            case UH_ST_F16:
            case UH_ST_BF16:
            case UH_ST_U8: {
              if (!full_tile) goto store_generic;
              const TensorDesc &td = P.tensor[arg];
              uint8_t *base = reinterpret_cast<uint8_t *>(td.ptr);
              const uint32_t off0 = kept_offset(td, pos.k) + pos.e0[0];
              const uint32_t off1 = off0 + 4u * tg;
              gstore4(uh == UH_ST_F32 ? T_F32 : (uh == UH_ST_F16 ? T_F16 : (uh == UH_ST_BF16 ? T_BF16 : T_BOOL)), base, off0, &acc[0]);
              gstore4(uh == UH_ST_F32 ? T_F32 : (uh == UH_ST_F16 ? T_F16 : (uh == UH_ST_BF16 ? T_BF16 : T_BOOL)), base, off1, &acc[4]);
              continue;
            }
            case UH_STG: {
            store_generic:
              store_tensor(P, arg, pos, acc);
              continue;
            }
            default: continue;
          }
        }
        if (staged_body) mbar_arrive(empty_bar);
      }
    }
  }
}
}  // namespace

// Two register budgets of the same interpreter: up to 256 consumer threads with three CTAs per SM (the
// streaming shapes), and up to 512 consumer threads (long reduction rows) with one.
__global__ void __launch_bounds__(kVmFlatThreads + 32, 3) dvm_b200_vm_vector(const __grid_constant__ VmParam P) {
  vm_vector_body(P);
}
__global__ void __launch_bounds__(kVmMaxThreads + 32, 1) dvm_b200_vm_vector_wide(const __grid_constant__ VmParam P) {
  vm_vector_body(P);
}

int LaunchVector(const VmParam &param, uint32_t grid, uint32_t threads, uint32_t smem_bytes, void *stream) {
  static bool attr_set[64] = {false};   // the attribute is per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(dvm_b200_vm_vector, cudaFuncAttributeMaxDynamicSharedMemorySize, kVmMaxSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(dvm_b200_vm_vector_wide, cudaFuncAttributeMaxDynamicSharedMemorySize, kVmMaxSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  if (threads <= kVmFlatThreads + 32) {
    dvm_b200_vm_vector<<<grid, threads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(param);
  } else {
    dvm_b200_vm_vector_wide<<<grid, threads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(param);
  }
  return static_cast<int>(cudaGetLastError());
}

// Read (and clear) the device status word of the vector interpreter; 0 means every bounded wait succeeded.
unsigned int ReadVectorStatus() {
  unsigned int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_vm_status, sizeof(v)) != cudaSuccess) return 0xffffffffu;
  if (v != 0) cudaMemcpyToSymbol(g_vm_status, &zero, sizeof(zero));
  return v;
}

}  // namespace dvmb
