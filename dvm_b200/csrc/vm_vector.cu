// Persistent register-resident bytecode interpreter for fused vector graphs on sm_100a.
//
// One kernel executes every fused elementwise / broadcast / reduce graph the host compiler emits
// (the role of dvm_vm_gpu in the reference, src/vm_gpu.cu:1552-1617, whose operands live in shared
// memory; here every intermediate stays in registers and a fused graph touches HBM once per tensor).
// Per-op arithmetic follows the reference's device functors (src/vm_gpu.cu:198-329): IEEE fp32 math,
// fp16/bf16 values rounded to storage precision after every op, float->int by truncation, compares
// yielding 1/0 in the operand representation, max/min as `a > b ? a : b` / `a < b ? a : b`.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstdint>

#include "isa.h"
#include "vm_launch.h"

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

template <int N>
__device__ __forceinline__ void apply_round(uint32_t rnd, uint32_t (&a)[N]) {
  if (rnd == RN_F16) {
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = f2u(round_f16(u2f(a[i])));
  } else if (rnd == RN_BF16) {
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = f2u(round_bf16(u2f(a[i])));
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

#define DVMB_BIN_F(EXPR)                   \
  _Pragma("unroll") for (int i = 0; i < N; ++i) { \
    float x = u2f(a[i]), y = u2f(b[i]);    \
    a[i] = f2u(EXPR);                      \
  }
#define DVMB_BIN_I(EXPR)                   \
  _Pragma("unroll") for (int i = 0; i < N; ++i) { \
    int32_t x = (int32_t)a[i], y = (int32_t)b[i]; \
    a[i] = (uint32_t)(EXPR);               \
  }

template <int N>
__device__ __forceinline__ void apply_bin(uint32_t kind, uint32_t (&a)[N], const uint32_t (&b)[N]) {
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

template <int N>
__device__ __forceinline__ void apply_cmp(uint32_t kind, uint32_t isint, uint32_t (&a)[N], const uint32_t (&b)[N]) {
  if (isint) {
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = cmp_value<int32_t>(kind, (int32_t)a[i], (int32_t)b[i]) ? 1u : 0u;
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = cmp_value<float>(kind, u2f(a[i]), u2f(b[i])) ? 0x3f800000u : 0u;
  }
}

// a <- cond(a) ? b : c; `inv` swaps the alternatives (the free-form operand b is then the false value).
template <int N>
__device__ __forceinline__ void apply_sel(uint32_t isint, uint32_t inv, uint32_t (&a)[N], const uint32_t (&b)[N],
                                          const uint32_t (&c)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) {
    bool t = isint ? (a[i] != 0u) : (u2f(a[i]) != 0.0f);
    if (inv) t = !t;
    a[i] = t ? b[i] : c[i];
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

// ---- global memory access -------------------------------------------------------------------------

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

__device__ __forceinline__ void load_vec4(uint32_t dtype, const uint8_t *base, uint32_t off, uint32_t *out) {
  switch (dtype) {
    case T_F32:
    case T_I32: {
      uint4 v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const uint32_t *>(base) + off));
      out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
      break;
    }
    case T_F16: {
      uint2 v = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const unsigned short *>(base) + off));
      float2 lo = __half22float2(*reinterpret_cast<__half2 *>(&v.x));
      float2 hi = __half22float2(*reinterpret_cast<__half2 *>(&v.y));
      out[0] = f2u(lo.x); out[1] = f2u(lo.y); out[2] = f2u(hi.x); out[3] = f2u(hi.y);
      break;
    }
    case T_BF16: {
      uint2 v = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const unsigned short *>(base) + off));
      out[0] = v.x << 16; out[1] = v.x & 0xffff0000u; out[2] = v.y << 16; out[3] = v.y & 0xffff0000u;
      break;
    }
    default: {
      uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(base + off));
      out[0] = v & 0xffu; out[1] = (v >> 8) & 0xffu; out[2] = (v >> 16) & 0xffu; out[3] = v >> 24;
      break;
    }
  }
}

__device__ __forceinline__ void store_vec4(uint32_t dtype, uint8_t *base, uint32_t off, const uint32_t *v) {
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
      p.x = (f2u(round_bf16(u2f(v[0]))) >> 16) | (f2u(round_bf16(u2f(v[1]))) & 0xffff0000u);
      p.y = (f2u(round_bf16(u2f(v[2]))) >> 16) | (f2u(round_bf16(u2f(v[3]))) & 0xffff0000u);
      *reinterpret_cast<uint2 *>(reinterpret_cast<unsigned short *>(base) + off) = p;
      break;
    }
    default:
      *reinterpret_cast<uint32_t *>(base + off) =
        (v[0] & 0xffu) | ((v[1] & 0xffu) << 8) | ((v[2] & 0xffu) << 16) | (v[3] << 24);
      break;
  }
}

// Per-thread position inside the iteration space.
struct Pos {
  uint32_t k[kMaxKept];   // kept coordinates of this thread's group
  uint32_t e0[2];         // first element (inside the group) of each granule
  int32_t nv[2];          // valid elements of each granule (0..4)
  uint32_t ec[2][kMaxEnum];  // enumerated coordinates of each granule's first element (AM_GRANULE)
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

__device__ __forceinline__ uint32_t kept_offset(const TensorDesc &td, const Pos &pos) {
  uint32_t off = 0;
#pragma unroll
  for (int j = 0; j < kMaxKept; ++j) off += pos.k[j] * td.kstride[j];
  return off;
}

__device__ __forceinline__ uint32_t enum_offset(const TensorDesc &td, const uint32_t (&c)[kMaxEnum]) {
  uint32_t off = 0;
#pragma unroll
  for (int j = 0; j < kMaxEnum; ++j) off += c[j] * td.estride[j];
  return off;
}

__device__ __forceinline__ void load_tile(const VmParam &P, uint32_t slot, const Pos &pos, uint32_t (&out)[kLanes]) {
  const TensorDesc &td = P.tensor[slot];
  const uint8_t *base = reinterpret_cast<const uint8_t *>(td.ptr);
  const uint32_t dtype = td.dtype, mode = td.mode;
  const uint32_t koff = kept_offset(td, pos);
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int nv = pos.gvalid ? pos.nv[g] : 0;
    uint32_t *o = &out[4 * g];
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
      load_vec4(dtype, base, off, o);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = i < nv ? load_elem(dtype, base, off + i * istride) : 0u;
    }
  }
}

__device__ __forceinline__ void store_tile(const VmParam &P, uint32_t slot, const Pos &pos,
                                           const uint32_t (&val)[kLanes]) {
  const TensorDesc &td = P.tensor[slot];
  uint8_t *base = reinterpret_cast<uint8_t *>(td.ptr);
  const uint32_t dtype = td.dtype, mode = td.mode;
  const uint32_t koff = kept_offset(td, pos);
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
      store_vec4(dtype, base, off, v);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < nv) store_elem(dtype, base, off + i * istride, v[i]);
    }
  }
}

#define DVMB_VREG_CASES(IDX, STMT) \
  switch (IDX) {                   \
    case 0: { constexpr int J = 0; STMT } break; \
    case 1: { constexpr int J = 1; STMT } break; \
    case 2: { constexpr int J = 2; STMT } break; \
    case 3: { constexpr int J = 3; STMT } break; \
    case 4: { constexpr int J = 4; STMT } break; \
    default: { constexpr int J = 5; STMT } break; \
  }

#define DVMB_SREG_CASES(IDX, STMT) \
  switch (IDX) {                   \
    case 0: { constexpr int J = 0; STMT } break; \
    case 1: { constexpr int J = 1; STMT } break; \
    case 2: { constexpr int J = 2; STMT } break; \
    case 3: { constexpr int J = 3; STMT } break; \
    case 4: { constexpr int J = 4; STMT } break; \
    case 5: { constexpr int J = 5; STMT } break; \
    case 6: { constexpr int J = 6; STMT } break; \
    case 7: { constexpr int J = 7; STMT } break; \
    case 8: { constexpr int J = 8; STMT } break; \
    case 9: { constexpr int J = 9; STMT } break; \
    case 10: { constexpr int J = 10; STMT } break; \
    default: { constexpr int J = 11; STMT } break; \
  }

#define DVMB_PART_CASES(IDX, STMT) \
  switch (IDX) {                   \
    case 0: { constexpr int J = 0; STMT } break; \
    case 1: { constexpr int J = 1; STMT } break; \
    case 2: { constexpr int J = 2; STMT } break; \
    default: { constexpr int J = 3; STMT } break; \
  }

}  // namespace

__global__ void __launch_bounds__(kVmMaxThreads, kVmMinBlocks) dvm_b200_vm_vector(const __grid_constant__ VmParam P) {
  __shared__ float red_buf[2][32];

  uint32_t acc[kLanes];
  uint32_t r[kNumVRegs][kLanes];
  uint32_t s[kNumSRegs];
  uint32_t sacc[1] = {0};
  float part[kNumRSlots];
#pragma unroll
  for (int i = 0; i < kLanes; ++i) acc[i] = 0;
#pragma unroll
  for (int j = 0; j < kNumVRegs; ++j)
#pragma unroll
    for (int i = 0; i < kLanes; ++i) r[j][i] = 0;
#pragma unroll
  for (int j = 0; j < kNumSRegs; ++j) s[j] = 0;
#pragma unroll
  for (int j = 0; j < kNumRSlots; ++j) part[j] = 0.0f;

  const uint32_t tid = threadIdx.x;
  const uint32_t tg = P.tg;
  const bool flat = P.mode == VM_FLAT;
  const uint32_t lane_in_group = flat ? tid : tid % tg;
  const uint32_t group_in_cta = flat ? 0 : tid / tg;
  const uint32_t ngb = flat ? 1u : (P.num_groups + P.groups_per_cta - 1) / P.groups_per_cta;
  const uint32_t gb_begin = flat ? 0u : blockIdx.x, gb_step = flat ? 1u : gridDim.x;
  const uint32_t ch_begin = flat ? blockIdx.x : 0u, ch_step = flat ? gridDim.x : 1u;
  uint32_t red_par = 0;

  Pos pos;

  for (uint32_t gb = gb_begin; gb < ngb; gb += gb_step) {
    {
      uint32_t gi = gb * P.groups_per_cta + group_in_cta;
      pos.gvalid = gi < P.num_groups;
      if (!pos.gvalid) gi = 0;
#pragma unroll
      for (int j = kMaxKept - 1; j > 0; --j) {
        uint32_t sz = P.kept_size[j];
        uint32_t q = gi / sz;
        pos.k[j] = gi - q * sz;
        gi = q;
      }
      pos.k[0] = gi;
    }
    for (uint32_t ph = 0; ph <= P.num_body; ++ph) {
      // ---------------- scalar side: PRO_ph ----------------
      for (uint32_t pc = P.sec[2 * ph];;) {
        const uint64_t w = P.code[pc++];
        const uint32_t opc = DVMB_OPC(w);
        if (opc == OP_END) break;
        const uint32_t sub = DVMB_SUB(w);
        uint32_t b[1] = {0};
        if (opc == OP_COPY || opc == OP_BIN || opc == OP_CMP || opc == OP_SEL) {
          const uint32_t okind = DVMB_OKIND(w), oidx = DVMB_OIDX(w);
          if (okind == K_SREG) {
            DVMB_SREG_CASES(oidx, b[0] = s[J];)
          } else if (okind == K_IMM) {
            b[0] = DVMB_IMM(w);
          } else {
            b[0] = sacc[0];
          }
        }
        switch (opc) {
          case OP_LD: {
            const TensorDesc &td = P.tensor[sub];
            uint32_t v = load_elem(td.dtype, reinterpret_cast<const uint8_t *>(td.ptr), kept_offset(td, pos));
            const uint32_t dst = DVMB_DST(w);
            if (dst == kAccIdx) {
              sacc[0] = v;
            } else {
              DVMB_SREG_CASES(dst, s[J] = v;)
            }
            break;
          }
          case OP_ST: {
            const TensorDesc &td = P.tensor[sub];
            if (lane_in_group == 0 && pos.gvalid && (!flat || blockIdx.x == 0))
              store_elem(td.dtype, reinterpret_cast<uint8_t *>(td.ptr), kept_offset(td, pos), sacc[0]);
            break;
          }
          case OP_COPY: sacc[0] = b[0]; break;
          case OP_MOV: {
            const uint32_t dst = DVMB_DST(w);
            DVMB_SREG_CASES(dst, s[J] = sacc[0];)
            break;
          }
          case OP_UN: apply_un<1>(sub, sacc); apply_round<1>(DVMB_RND(w), sacc); break;
          case OP_BIN: apply_bin<1>(sub, sacc, b); apply_round<1>(DVMB_RND(w), sacc); break;
          case OP_CMP: apply_cmp<1>(sub, DVMB_ISINT(w), sacc, b); break;
          case OP_SEL: {
            uint32_t c[1] = {0};
            const uint32_t k2 = sub >> 4, i2 = sub & 15u;
            if (k2 == K_SREG) {
              DVMB_SREG_CASES(i2, c[0] = s[J];)
            } else {
              c[0] = sacc[0];
            }
            apply_sel<1>(DVMB_ISINT(w), DVMB_DST(w) & 1u, sacc, b, c);
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
              if ((tid & 31u) == 0) red_buf[red_par][tid >> 5] = v;
              __syncthreads();
              const uint32_t nw = blockDim.x >> 5;
              v = red_buf[red_par][0];
              for (uint32_t wi = 1; wi < nw; ++wi) v = red_combine(kind, v, red_buf[red_par][wi]);
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
      for (uint32_t ch = ch_begin; ch < P.chunks; ch += ch_step) {
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          // 64-bit so that a chunk past the end of a 2^31-element group cannot wrap
          const uint64_t e = (uint64_t)ch * (8ull * tg) + (uint64_t)g * 4ull * tg + 4ull * lane_in_group;
          const int64_t left = (int64_t)P.group_elems - (int64_t)e;
          pos.nv[g] = left >= 4 ? 4 : (left > 0 ? (int32_t)left : 0);
          pos.e0[g] = (uint32_t)e;
          if (P.need_coords) split_enum(P, pos.nv[g] > 0 ? pos.e0[g] : 0u, pos.ec[g]);
        }
        for (uint32_t pc = body_pc;;) {
          const uint64_t w = P.code[pc++];
          const uint32_t opc = DVMB_OPC(w);
          if (opc == OP_END) break;
          const uint32_t sub = DVMB_SUB(w);
          uint32_t b[kLanes];
          if (opc == OP_COPY || opc == OP_BIN || opc == OP_CMP || opc == OP_SEL) {
            const uint32_t okind = DVMB_OKIND(w), oidx = DVMB_OIDX(w);
            if (okind == K_VREG) {
              DVMB_VREG_CASES(oidx, _Pragma("unroll") for (int i = 0; i < kLanes; ++i) b[i] = r[J][i];)
            } else if (okind == K_ACC) {
#pragma unroll
              for (int i = 0; i < kLanes; ++i) b[i] = acc[i];
            } else {
              uint32_t v = DVMB_IMM(w);
              if (okind == K_SREG) {
                DVMB_SREG_CASES(oidx, v = s[J];)
              }
#pragma unroll
              for (int i = 0; i < kLanes; ++i) b[i] = v;
            }
          }
          switch (opc) {
            case OP_LD: {
              const uint32_t dst = DVMB_DST(w);
              if (dst == kAccIdx) {
                load_tile(P, sub, pos, acc);
              } else {
                uint32_t t[kLanes];
                load_tile(P, sub, pos, t);
                DVMB_VREG_CASES(dst, _Pragma("unroll") for (int i = 0; i < kLanes; ++i) r[J][i] = t[i];)
              }
              break;
            }
            case OP_ST: store_tile(P, sub, pos, acc); break;
            case OP_COPY:
#pragma unroll
              for (int i = 0; i < kLanes; ++i) acc[i] = b[i];
              break;
            case OP_MOV: {
              const uint32_t dst = DVMB_DST(w);
              DVMB_VREG_CASES(dst, _Pragma("unroll") for (int i = 0; i < kLanes; ++i) r[J][i] = acc[i];)
              break;
            }
            case OP_UN: apply_un<kLanes>(sub, acc); apply_round<kLanes>(DVMB_RND(w), acc); break;
            case OP_BIN: apply_bin<kLanes>(sub, acc, b); apply_round<kLanes>(DVMB_RND(w), acc); break;
            case OP_CMP: apply_cmp<kLanes>(sub, DVMB_ISINT(w), acc, b); break;
            case OP_SEL: {
              uint32_t c[kLanes];
              const uint32_t k2 = sub >> 4, i2 = sub & 15u;
              if (k2 == K_VREG) {
                DVMB_VREG_CASES(i2, _Pragma("unroll") for (int i = 0; i < kLanes; ++i) c[i] = r[J][i];)
              } else if (k2 == K_SREG) {
                uint32_t v = 0;
                DVMB_SREG_CASES(i2, v = s[J];)
#pragma unroll
                for (int i = 0; i < kLanes; ++i) c[i] = v;
              } else {
#pragma unroll
                for (int i = 0; i < kLanes; ++i) c[i] = acc[i];
              }
              apply_sel<kLanes>(DVMB_ISINT(w), DVMB_DST(w) & 1u, acc, b, c);
              break;
            }
            case OP_CVT: apply_cvt<kLanes>(sub, acc); apply_round<kLanes>(DVMB_RND(w), acc); break;
            case OP_RACC: {
              const uint32_t kind = sub >> 4;
              float v = red_identity(kind);
#pragma unroll
              for (int i = 0; i < kLanes; ++i)
                if (pos.gvalid && (i & 3) < pos.nv[i >> 2]) v = red_combine(kind, v, u2f(acc[i]));
              DVMB_PART_CASES(sub & 3u, part[J] = red_combine(kind, part[J], v);)
              break;
            }
            default: break;
          }
        }
      }
    }
  }
}

int LaunchVector(const VmParam &param, uint32_t grid, uint32_t threads, void *stream) {
  dvm_b200_vm_vector<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(param);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dvmb
