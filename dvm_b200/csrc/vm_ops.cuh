// Per-op device arithmetic shared by the sm_100a interpreters (vector VM, MatMul and attention epilogues).
//
// Follows the reference's device functors (src/vm_gpu.cu:198-329): IEEE fp32 math, fp16/bf16 values rounded
// to storage precision after every op, float->int by truncation, compares yielding 1/0 in the operand
// representation, max/min as `a > b ? a : b` / `a < b ? a : b`.
#ifndef DVM_B200_VM_OPS_CUH_
#define DVM_B200_VM_OPS_CUH_

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstdint>

#include "isa.h"

namespace dvmb {
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

// exp through the hardware exp2 approximation: relative error about 1e-6 for |x| below 10, 5e-6 at the range ends.
__device__ __forceinline__ float fast_exp(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x * 1.4426950408889634f));
  return r;
}

// Full-range division with a 2-ulp bound (div.full.f32).
__device__ __forceinline__ float fast_div(float a, float b) {
  float r;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
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
    case U_EXP_FAST: DVMB_UN_LOOP(fast_exp(x)) break;
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
    case B_DIV_FAST: DVMB_BIN_F(fast_div(x, y)) break;
    case B_RDIV_FAST: DVMB_BIN_F(fast_div(y, x)) break;
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

}  // namespace
}  // namespace dvmb

#endif  // DVM_B200_VM_OPS_CUH_
