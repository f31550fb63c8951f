// dvm::Kernel builder methods and the dtype-lowering rules that define each API op's numerical contract.
//
// The lowering follows the reference's src/dvm.cc on its GPU architecture branch (every
// `!= kAiCore_C310` branch taken, no `== kAiCore_C220` branch): which ops are promoted to fp32 or fp16,
// how scalars are encoded, which casts chain through which intermediate type.  The code is organised
// differently (one run-time operand variant instead of 13 template instantiations per op).
#include <cmath>
#include <cstring>
#include <stdexcept>
#include <string>

#include "comm.h"
#include "graph.h"
#include "numeric.h"
#include "runtime.h"

namespace dvm {

[[noreturn]] void DvmException(const char *error_str) {
  throw std::runtime_error(std::string("DVM EXCEPTION. reason: ") + error_str);
}

// ---- Float16 / BFloat16 ---------------------------------------------------------------------------
Float16::Float16(float v) : value_(F32ToF16Bits(v)) {}
Float16::Float16(int32_t v) : value_(F32ToF16Bits(static_cast<float>(v))) {}
Float16::operator float() const { return F16BitsToF32(value_); }
Float16::operator int32_t() const { return static_cast<int32_t>(F16BitsToF32(value_)); }
BFloat16::BFloat16(float v) : value_(F32ToBF16Bits(v)) {}
BFloat16::BFloat16(int32_t v) : value_(F32ToBF16Bits(static_cast<float>(v))) {}
BFloat16::operator float() const { return BF16BitsToF32(value_); }
BFloat16::operator int32_t() const { return static_cast<int32_t>(BF16BitsToF32(value_)); }

// ---- Config (Comm lives in comm.cc) --------------------------------------------------------------
namespace {
class ConfigImpl : public Config {
 public:
  Config &SetDeterm() override { return *this; }
  Config &UnsetDeterm() override { return *this; }
  Config &SetOnlineTuner() override { return *this; }
  Config &UnsetOnlineTuner() override { return *this; }
  Config &SetLazyTuner() override { return *this; }
  Config &UnsetLazyTuner() override { return *this; }
  Config &SetVfFusion(int) override { return *this; }
  Config &UnsetVfFusion() override { return *this; }
};
}  // namespace
Config &Config::Instance() {
  static ConfigImpl impl;
  return impl;
}
bool Config::IsInitialized() const { return dvmb::Runtime::Get().initialized(); }

// ---- scalar operands ------------------------------------------------------------------------------
namespace {

// A scalar operand as passed by the caller, before encoding into a tensor dtype.
struct Scalar {
  enum Tag { kF32, kI32, kI64, kF16, kBF16, kRef } tag;
  double v = 0;            // numeric value (fp16/bf16 operands widened exactly)
  ScalarRef *ref = nullptr;
  bool is_ref() const { return tag == kRef; }
  bool is_integer_valued() const {   // the reference's isInteger(): integral types, or float with no fraction
    if (tag == kI32 || tag == kI64) return true;
    if (tag == kF32) return std::floor(v) == v;
    return false;
  }
};

Scalar MakeScalar(float v) { return {Scalar::kF32, v, nullptr}; }
Scalar MakeScalar(int32_t v) { return {Scalar::kI32, static_cast<double>(v), nullptr}; }
Scalar MakeScalar(int64_t v) { return {Scalar::kI64, static_cast<double>(v), nullptr}; }
Scalar MakeScalar(Float16 v) { return {Scalar::kF16, static_cast<float>(v), nullptr}; }
Scalar MakeScalar(BFloat16 v) { return {Scalar::kBF16, static_cast<float>(v), nullptr}; }
Scalar MakeScalar(ScalarRef *r) { return {Scalar::kRef, 0, r}; }

// Encode a numeric scalar in `dtype`, widened to the interpreter's 32-bit register form
// (fp16/bf16/fp32 -> float bits of the rounded value, int32/bool -> integer bits).
// ref: EncodeScalar, src/dvm.cc:188-223.
uint32_t EncodeNumeric(double v, bool from_float, DataType dtype) {
  const float f = from_float ? static_cast<float>(v) : static_cast<float>(static_cast<int64_t>(v));
  switch (dtype) {
    case kFloat16: return FloatBits(F16BitsToF32(F32ToF16Bits(f)));
    case kBFloat16: return FloatBits(BF16BitsToF32(F32ToBF16Bits(f)));
    case kFloat32: return FloatBits(f);
    case kInt32: return static_cast<uint32_t>(from_float ? static_cast<int32_t>(static_cast<float>(v))
                                                          : static_cast<int32_t>(static_cast<int64_t>(v)));
    case kBool: return v != 0 ? 1u : 0u;
    default: DvmException("scalar operand for an unsupported tensor dtype");
  }
}

uint32_t EncodeScalar(const Scalar &s, DataType dtype) {
  return EncodeNumeric(s.v, s.tag == Scalar::kF32 || s.tag == Scalar::kF16 || s.tag == Scalar::kBF16, dtype);
}

}  // namespace

// Encode the current value of a ScalarRef (called at code generation).  ref: src/dvm.cc:281-310
uint32_t EncodeScalarRefNow(const ScalarRef *ref, DataType dtype) {
  switch (ref->type) {
    case kFloat16: return EncodeNumeric(F16BitsToF32(ref->f16), true, dtype);
    case kBFloat16: return EncodeNumeric(BF16BitsToF32(ref->f16), true, dtype);
    case kFloat32: return EncodeNumeric(ref->f32, true, dtype);
    case kInt32: return EncodeNumeric(ref->i32, false, dtype);
    case kInt64: return EncodeNumeric(static_cast<double>(ref->i64), false, dtype);
    default: DvmException("ScalarRef has no value type; call update() first");
  }
}

// ---- lowering helpers -----------------------------------------------------------------------------
namespace {

[[noreturn]] void Unsupported(const char *what) {
  std::string msg = std::string(what) + ": unsupported on this backend";
  DvmException(msg.c_str());
}

// Next hop of the cast chain from `cur` towards `target` (ref: g_cast_staff_type, src/dvm.cc:416-423).
DataType CastHop(DataType cur, DataType target) {
  if (cur == target) return target;
  if (cur == kBool) return kFloat16;
  if (target == kBool) {
    if (cur == kFloat16 || cur == kInt64) return kBool;
    return cur == kBFloat16 ? kFloat32 : kFloat16;
  }
  switch (cur) {
    case kFloat16: return target == kInt32 ? kInt32 : kFloat32;
    case kBFloat16: return target == kInt32 ? kInt32 : kFloat32;
    case kFloat32: return target;
    case kInt32: return target == kFloat16 ? kFloat16 : (target == kInt64 ? kInt64 : kFloat32);
    default: return target == kInt32 ? kInt32 : kFloat32;  // from int64
  }
}

struct Lower {
  Kernel *k;
  VKernel *vk;

  NDObject *CastStep(NDObject *in, DataType to, bool noloss) {
    auto n = vk->NewNode(N_CAST, to);
    n->in[0] = in;
    n->noloss_cast = noloss;
    return n;
  }

  // ref: NoLossCast, src/dvm.cc:425-443 - a promotion cast that undoes a previous promotion instead of
  // stacking on it, so compare -> select of one dtype emits no cast at all.
  NDObject *NoLossCast(NDObject *in, DataType type) {
    DataType cur = in->dtype;
    while (cur != type) {
      DataType hop = CastHop(cur, type);
      if (in->kind == N_CAST && in->noloss_cast && in->in[0]->dtype == hop) {
        in = in->in[0];
      } else {
        in = CastStep(in, hop, true);
      }
      cur = hop;
    }
    return in;
  }

  NDObject *ScalarArith(ScalarBin op, NDObject *x, const Scalar &s) {
    auto n = vk->NewNode(N_BINARY_S, x->dtype);
    n->sub = op;
    n->in[0] = x;
    if (s.is_ref()) {
      n->scalar_ref = s.ref;
    } else {
      n->scalar_bits = EncodeScalar(s, x->dtype);
    }
    return n;
  }

  // x ^ n for an integral n as a multiply chain.  ref: PowS, src/dvm.cc:255-279
  NDObject *PowInteger(NDObject *x, const Scalar &s) {
    int32_t n = std::abs(static_cast<int32_t>(s.v));
    if (n == 0) {
      return BroadcastScalar(Scalar{s.tag, 1.0, nullptr}, nullptr, x->dtype, x);
    }
    NDObject *res = nullptr;
    if (n == 1) {
      res = k->Copy(x);
    } else {
      while (n) {
        if (n & 1) res = res == nullptr ? x : k->Binary<kMul>(res, x);
        if (n != 1) x = k->Binary<kMul>(x, x);
        n >>= 1;
      }
    }
    if (s.v < 0) res = k->Unary<kReciprocal>(res);
    return res;
  }

  NDObject *BroadcastScalar(const Scalar &s, IntArrayRef *shape, DataType type, NDObject *like) {
    if (type == kBool) return k->Cast(BroadcastScalar(s, shape, kFloat16, like), kBool);
    if (type == kInt64) Unsupported("int64 broadcast");
    auto n = vk->NewNode(N_BROADCAST_S, type);
    n->shape_ref = shape;
    n->in[0] = like;   // when set, the result takes this node's shape (shape_ref is null)
    if (s.is_ref()) {
      n->scalar_ref = s.ref;
    } else {
      n->scalar_bits = EncodeScalar(s, type);
    }
    return n;
  }

  // tensor (op) scalar with the scalar on the right (`scalar_rhs`) or left.  Returns null when the rule
  // table has no scalar form; the caller then broadcasts the scalar.  ref: GetBinaryS, src/dvm.cc:586-676
  NDObject *BinaryScalar(BinaryType op, const Scalar &s, NDObject *x, bool scalar_rhs) {
    if (x->dtype == kInt64) Unsupported("int64 arithmetic");
    switch (op) {
      case kAdd: return ScalarArith(SB_ADD, x, s);
      case kMul: return ScalarArith(SB_MUL, x, s);
      case kMinimum: return ScalarArith(SB_MIN, x, s);
      case kMaximum: return ScalarArith(SB_MAX, x, s);
      case kDiv: {
        if (x->dtype == kBFloat16) {
          auto r = BinaryScalar(op, s, k->Cast(x, kFloat32), scalar_rhs);
          return k->Cast(r, kBFloat16);
        }
        return ScalarArith(scalar_rhs ? SB_DIV : SB_SDIV, x, s);
      }
      case kEqual: case kNotEqual: case kGreater: case kGreaterEqual: case kLess: case kLessEqual: {
        if (x->dtype == kInt32) return nullptr;
        static const BinaryType mirrored[] = {kEqual, kNotEqual, kLess, kLessEqual, kGreater, kGreaterEqual};
        auto n = vk->NewNode(N_COMPARE_S, x->dtype);
        n->sub = scalar_rhs ? op : mirrored[op];
        n->in[0] = x;
        if (s.is_ref()) {
          n->scalar_ref = s.ref;
        } else {
          n->scalar_bits = EncodeScalar(s, x->dtype);
        }
        return NoLossCast(n, kBool);
      }
      case kPow: {
        if (s.is_ref()) return nullptr;
        if (scalar_rhs) return s.is_integer_valued() ? PowInteger(x, s) : nullptr;
        if (s.v > 0) {
          if (x->dtype != kFloat32) {
            auto r = BinaryScalar(kPow, MakeScalar(static_cast<float>(s.v)), k->Cast(x, kFloat32), false);
            return k->Cast(r, x->dtype);
          }
          auto t = ScalarArith(SB_MUL, x, MakeScalar(std::log(static_cast<float>(s.v))));
          return k->Unary<kExp>(t);
        }
        return nullptr;
      }
      case kSub: {
        if (s.is_ref()) return nullptr;
        Scalar neg = s;
        neg.v = -s.v;
        if (scalar_rhs) return ScalarArith(SB_ADD, x, neg);
        Scalar minus_one = s;
        minus_one.v = -1;
        return ScalarArith(SB_ADD, ScalarArith(SB_MUL, x, minus_one), s);
      }
      default: return nullptr;
    }
  }

  NDObject *TensorBinary(BinaryType op, NDObject *a, NDObject *b) {
    switch (a->dtype) {
      case kBool: {
        auto r = TensorBinary(op, NoLossCast(a, kFloat16), NoLossCast(b, kFloat16));
        return NoLossCast(r, kBool);
      }
      case kBFloat16:
        if (op == kPow || op == kDiv) return Promoted(op, a, b, kFloat32);
        break;
      case kFloat16:
        if (op == kPow) return Promoted(op, a, b, kFloat32);
        break;
      case kInt64: Unsupported("int64 arithmetic");
      default: break;
    }
    if (op < kAdd) {
      auto n = vk->NewNode(N_COMPARE, a->dtype);
      n->sub = op;
      n->in[0] = a;
      n->in[1] = b;
      return NoLossCast(n, kBool);
    }
    auto n = vk->NewNode(N_BINARY, a->dtype);
    n->sub = op;
    n->in[0] = a;
    n->in[1] = b;
    return n;
  }

  NDObject *Promoted(BinaryType op, NDObject *a, NDObject *b, DataType via) {
    DataType orig = a->dtype;
    auto r = TensorBinary(op, k->Cast(a, via), k->Cast(b, via));
    return k->Cast(r, orig);
  }

  NDObject *ScalarTensor(BinaryType op, const Scalar &s, NDObject *x, bool scalar_rhs) {
    if (x->dtype == kBool) {
      auto r = ScalarTensor(op, s, NoLossCast(x, kFloat16), scalar_rhs);
      return NoLossCast(r, kBool);
    }
    if (auto r = BinaryScalar(op, s, x, scalar_rhs)) return r;
    auto full = BroadcastScalar(s, nullptr, x->dtype, x);
    return scalar_rhs ? TensorBinary(op, x, full) : TensorBinary(op, full, x);
  }
};

}  // namespace

// ---- Kernel ---------------------------------------------------------------------------------------
Kernel::Kernel() : kernel_(nullptr) {}
Kernel::~Kernel() { delete kernel_; }
Kernel &Kernel::operator=(Kernel &other) {
  if (this != &other) {
    delete kernel_;
    kernel_ = other.kernel_;
    other.kernel_ = nullptr;
  }
  return *this;
}
Kernel::Kernel(Kernel &other) : kernel_(other.kernel_) { other.kernel_ = nullptr; }

void Kernel::Reset(KernelType type, uint32_t flags) {
  if (type < 0 || type >= kKernelTypeEnd) DvmException("invalid kernel type");
  delete kernel_;
  kernel_ = new VKernel(type, flags);
}

void Kernel::Clear() {
  if (kernel_ == nullptr) return;
  auto type = kernel_->type_;
  auto flags = kernel_->flags_;
  delete kernel_;
  kernel_ = new VKernel(type, flags);
}

// ref: include/dvm.h:255-259, src/dvm.cc:1183-1191 - this kernel becomes a copy of `base`'s graph: same type and flags, every
// op copied in order with its operands mapped through the helper, every borrowed IntArrayRef / ScalarRef replaced by what the
// helper maps it to (itself when the helper has nothing for it).  Addresses are not copied: the clone is bound by relocation.
void Kernel::Clone(const Kernel &base, CloneHelper &helper) {
  const VKernel *src = base.GetImpl();
  if (src == nullptr) DvmException("Clone of a kernel that was never reset");
  delete kernel_;
  kernel_ = new VKernel(src->type_, src->flags_);
  kernel_->name_ = src->name_;
  for (const NDObject *n : src->nodes_) {
    NDObject *c = kernel_->NewNode(n->kind, n->dtype);
    const int id = c->id;
    *c = *n;
    c->id = id;
    c->cidx = -1;
    c->addr = nullptr;
    c->origin = nullptr;
    for (int k = 0; k < 3; ++k)
      if (n->in[k]) {
        c->in[k] = helper.GetClone(n->in[k]);
        if (c->in[k] == nullptr) DvmException("Clone: an operand was not cloned before its user");
      }
    auto ints = [&](IntArrayRef *r) { return r ? helper.GetClone(r) : nullptr; };
    auto scal = [&](ScalarRef *r) { return r ? helper.GetClone(r) : nullptr; };
    c->shape_ref = n->reduce_all ? nullptr : ints(n->shape_ref);   // (a reduce over every dim finds its dims at Normalize)
    c->stride_ref = ints(n->stride_ref);
    c->aux_ref = ints(n->aux_ref);
    c->slice_a = ints(n->slice_a);
    c->slice_b = ints(n->slice_b);
    c->slice_c = ints(n->slice_c);
    c->scalar_ref = scal(n->scalar_ref);
    c->scalar_ref2 = scal(n->scalar_ref2);
    helper.SetClone(const_cast<NDObject *>(n), c);
  }
  kernel_->cur_sub_ = src->cur_sub_;
}
void Kernel::SetNameHint(const char *name, const char *) {
  if (kernel_ && name) kernel_->name_ = name;
}

static VKernel *Impl(Kernel *k) {
  if (k->GetImpl() == nullptr) DvmException("Kernel::Reset must be called before building");
  return k->GetImpl();
}

NDObject *Kernel::Load(void *addr, IntArrayRef *shape, DataType type) {
  auto n = Impl(this)->NewNode(N_LOAD, type);
  n->addr = addr;
  n->shape_ref = shape;
  return n;
}
// ref: include/dvm.h:286-294 - a tensor that is not contiguous in memory: `stride` gives the element stride of every dim
// of `shape` (re-read at every Normalize, like the shape)
NDObject *Kernel::Load(void *addr, IntArrayRef *shape, IntArrayRef *stride, DataType type) {
  NDObject *n = Load(addr, shape, type);
  n->stride_ref = stride;
  return n;
}
NDObject *Kernel::GlobalAccess(void *, IntArrayRef *, DataType) { Unsupported("GlobalAccess"); }
NDObject *Kernel::GatherLoad(void *, IntArrayRef *, NDObject *, int, DataType, GatherMode) { Unsupported("GatherLoad"); }
// ref: include/dvm.h:305-317 - a window of a tensor in memory, given by start + size or by start / end / step per dim: a
// strided load (the window is never copied)
NDObject *Kernel::SliceLoad(void *addr, IntArrayRef *shape, IntArrayRef *start, IntArrayRef *size, DataType type) {
  NDObject *n = Load(addr, shape, type);
  n->slice_mode = 1;
  n->slice_a = start;
  n->slice_b = size;
  return n;
}
NDObject *Kernel::StridedSliceLoad(void *addr, IntArrayRef *shape, IntArrayRef *start, IntArrayRef *end, IntArrayRef *step,
                                   DataType type) {
  NDObject *n = Load(addr, shape, type);
  n->slice_mode = 2;
  n->slice_a = start;
  n->slice_b = end;
  n->slice_c = step;
  return n;
}
NDObject *Kernel::MultiLoad(void *, IntArrayRef *, DataType, const Comm *) { Unsupported("MultiLoad"); }

NDObject *Kernel::Store(void *addr, NDObject *input) {
  if (input->kind == N_LOAD) input = Copy(input);   // ref: src/dvm.cc:1547-1549
  auto n = Impl(this)->NewNode(N_STORE, input->dtype);
  n->in[0] = input;
  n->addr = addr;
  return n;
}
// ref: include/dvm.h:332-339 - the result written with the element strides `stride` (what lies between is left as it is)
NDObject *Kernel::Store(void *addr, NDObject *input, IntArrayRef *stride) {
  NDObject *n = Store(addr, input);
  n->stride_ref = stride;
  return n;
}
// ref: src/dvm.cc:1572-1576, NDPadStore::Normalize src/ops.cc:1399-1412 - the result in a buffer whose rows are `pad_size`
// elements longer than the tensor's (dense strides of that longer shape; the padding is left as it is).  GetShape of the
// store reports the padded shape, which is the buffer the caller provides.
NDObject *Kernel::PadStore(void *addr, NDObject *input, int64_t pad_size) {
  if (pad_size < 0) DvmException("PadStore: negative pad size");
  NDObject *n = Store(addr, input);
  n->pad_size = pad_size;
  return n;
}
// ref: src/dvm.cc:1578-1580, src/xkernel.h:322.  The reference's flag keeps its workspace pool from handing the store's
// buffer to another temporary.  Workspace temporaries here are bump-allocated once per compile and never reused, and a
// user's buffer is never used as workspace, so the mark needs no action beyond being recorded (listed by DumpR).
void Kernel::SetStoreInplace(NDObject *store) {
  if (store == nullptr || store->kind != N_STORE) DvmException("SetStoreInplace expects a Store operation");
  store->store_inplace = true;
}
void Kernel::SetStoreTemp(NDObject *store) { store->store_temp = true; }
void Kernel::SetLoadBind(NDObject *, NDObject *) { Unsupported("SetLoadBind"); }

// ref: Kernel::Unary, src/dvm.cc:1245-1283
template <UnaryType op_type>
NDObject *Kernel::Unary(NDObject *input) {
  Lower lw{this, Impl(this)};
  switch (input->dtype) {
    case kBool: {
      auto r = Unary<op_type>(lw.NoLossCast(input, kFloat16));
      return lw.NoLossCast(r, kBool);
    }
    case kBFloat16: return Cast(Unary<op_type>(Cast(input, kFloat32)), kBFloat16);
    case kFloat16:
      if (op_type >= kRound && op_type <= kTrunc) return Cast(Unary<op_type>(Cast(input, kFloat32)), kFloat16);
      break;
    case kInt64: Unsupported("int64 arithmetic");
    default: break;
  }
  if (op_type == kLogicalNot) return Binary<kSub>(static_cast<int32_t>(1), input);
  if (op_type == kReciprocal) return Binary<kDiv>(static_cast<int32_t>(1), input);
  if (input->dtype == kInt32 && op_type != kAbs) Unsupported("int32 unary op other than Abs");
  auto n = kernel_->NewNode(N_UNARY, input->dtype);
  n->sub = op_type;
  n->in[0] = input;
  return n;
}

#define DVM_DEF_UNARY(op) template DVM_API NDObject *Kernel::Unary<op>(NDObject *);
DVM_DEF_UNARY(kSqrt) DVM_DEF_UNARY(kAbs) DVM_DEF_UNARY(kLog) DVM_DEF_UNARY(kExp) DVM_DEF_UNARY(kReciprocal)
DVM_DEF_UNARY(kIsFinite) DVM_DEF_UNARY(kLogicalNot) DVM_DEF_UNARY(kRound) DVM_DEF_UNARY(kFloor)
DVM_DEF_UNARY(kCeil) DVM_DEF_UNARY(kTrunc)
#undef DVM_DEF_UNARY

NDObject *Kernel::Unary(int op_type, NDObject *input) {
  switch (op_type) {
    case kSqrt: return Unary<kSqrt>(input);
    case kAbs: return Unary<kAbs>(input);
    case kLog: return Unary<kLog>(input);
    case kExp: return Unary<kExp>(input);
    case kReciprocal: return Unary<kReciprocal>(input);
    case kIsFinite: return Unary<kIsFinite>(input);
    case kLogicalNot: return Unary<kLogicalNot>(input);
    case kRound: return Unary<kRound>(input);
    case kFloor: return Unary<kFloor>(input);
    case kCeil: return Unary<kCeil>(input);
    case kTrunc: return Unary<kTrunc>(input);
    default: return nullptr;
  }
}

// ref: Kernel::Binary, src/dvm.cc:1298-1382
template <BinaryType op_type, typename L, typename R>
NDObject *Kernel::Binary(L lhs, R rhs) {
  Lower lw{this, Impl(this)};
  if constexpr (!std::is_same<L, NDObject *>::value) {
    return lw.ScalarTensor(op_type, MakeScalar(lhs), rhs, false);
  } else if constexpr (!std::is_same<R, NDObject *>::value) {
    return lw.ScalarTensor(op_type, MakeScalar(rhs), lhs, true);
  } else {
    return lw.TensorBinary(op_type, lhs, rhs);
  }
}

#define DVM_DEF_BINARY(op)                                                     \
  template DVM_API NDObject *Kernel::Binary<op>(NDObject *, NDObject *);       \
  template DVM_API NDObject *Kernel::Binary<op>(NDObject *, float);            \
  template DVM_API NDObject *Kernel::Binary<op>(NDObject *, int32_t);          \
  template DVM_API NDObject *Kernel::Binary<op>(NDObject *, int64_t);          \
  template DVM_API NDObject *Kernel::Binary<op>(NDObject *, Float16);          \
  template DVM_API NDObject *Kernel::Binary<op>(NDObject *, BFloat16);         \
  template DVM_API NDObject *Kernel::Binary<op>(NDObject *, ScalarRef *);      \
  template DVM_API NDObject *Kernel::Binary<op>(float, NDObject *);            \
  template DVM_API NDObject *Kernel::Binary<op>(int32_t, NDObject *);          \
  template DVM_API NDObject *Kernel::Binary<op>(int64_t, NDObject *);          \
  template DVM_API NDObject *Kernel::Binary<op>(Float16, NDObject *);          \
  template DVM_API NDObject *Kernel::Binary<op>(BFloat16, NDObject *);         \
  template DVM_API NDObject *Kernel::Binary<op>(ScalarRef *, NDObject *);
DVM_DEF_BINARY(kEqual) DVM_DEF_BINARY(kNotEqual) DVM_DEF_BINARY(kGreater) DVM_DEF_BINARY(kGreaterEqual)
DVM_DEF_BINARY(kLess) DVM_DEF_BINARY(kLessEqual) DVM_DEF_BINARY(kAdd) DVM_DEF_BINARY(kSub) DVM_DEF_BINARY(kMul)
DVM_DEF_BINARY(kDiv) DVM_DEF_BINARY(kPow) DVM_DEF_BINARY(kMaximum) DVM_DEF_BINARY(kMinimum)
DVM_DEF_BINARY(kLogicalAnd) DVM_DEF_BINARY(kLogicalOr)
#undef DVM_DEF_BINARY

// ref: src/dvm.cc:1415-1427
NDObject *Kernel::Select(NDObject *cond, NDObject *lhs, NDObject *rhs) {
  Lower lw{this, Impl(this)};
  if (lhs->dtype == kInt64) Unsupported("int64 select");
  if (cond->dtype != lhs->dtype) cond = lw.NoLossCast(cond, lhs->dtype);
  auto n = kernel_->NewNode(N_SELECT, lhs->dtype);
  n->in[0] = cond;
  n->in[1] = lhs;
  n->in[2] = rhs;
  return n;
}

// ref: src/dvm.cc:1429-1447
NDObject *Kernel::Cast(NDObject *input, DataType type) {
  Lower lw{this, Impl(this)};
  if (input->dtype == type) return input;
  if (type == kInt64 || input->dtype == kInt64) Unsupported("int64 cast");
  if (type == kBool) input = Binary<kNotEqual>(input, static_cast<int32_t>(0));
  DataType cur = input->dtype;
  while (cur != type) {
    DataType hop = CastHop(cur, type);
    input = lw.CastStep(input, hop, false);
    cur = hop;
  }
  return input;
}

NDObject *Kernel::Copy(NDObject *input) {
  auto n = Impl(this)->NewNode(N_COPY, input->dtype);
  n->in[0] = input;
  return n;
}

// ref: src/dvm.cc:1461-1493
template <typename T>
NDObject *Kernel::Broadcast(T val, IntArrayRef *shape, DataType type) {
  Lower lw{this, Impl(this)};
  return lw.BroadcastScalar(MakeScalar(val), shape, type, nullptr);
}
template DVM_API NDObject *Kernel::Broadcast<float>(float, IntArrayRef *, DataType);
template DVM_API NDObject *Kernel::Broadcast<int32_t>(int32_t, IntArrayRef *, DataType);
template DVM_API NDObject *Kernel::Broadcast<int64_t>(int64_t, IntArrayRef *, DataType);
template DVM_API NDObject *Kernel::Broadcast<Float16>(Float16, IntArrayRef *, DataType);
template DVM_API NDObject *Kernel::Broadcast<BFloat16>(BFloat16, IntArrayRef *, DataType);
template DVM_API NDObject *Kernel::Broadcast<ScalarRef *>(ScalarRef *, IntArrayRef *, DataType);

// ref: src/dvm.cc:1495-1507
NDObject *Kernel::Broadcast(NDObject *input, IntArrayRef *shape) {
  Lower lw{this, Impl(this)};
  if (input->dtype == kBool) return lw.NoLossCast(Broadcast(lw.NoLossCast(input, kFloat16), shape), kBool);
  if (input->dtype == kInt64) Unsupported("int64 broadcast");
  auto n = kernel_->NewNode(N_BROADCAST, input->dtype);
  n->in[0] = input;
  n->shape_ref = shape;
  return n;
}

NDObject *Kernel::Reshape(NDObject *input, IntArrayRef *shape) {
  auto n = Impl(this)->NewNode(N_RESHAPE, input->dtype);
  n->in[0] = input;
  n->shape_ref = shape;
  return n;
}

// Views (ref: include/dvm.h:428-453, 470-479; the reference's view schedules src/schedule.h:23-167): the input's memory
// seen through another shape, strides and offset.  No data moves where the input is a tensor in memory (a Load, another
// view); a computed input is written to the workspace first and viewed there.
static NDObject *View(VKernel *vk, uint8_t kind, NDObject *input) {
  auto n = vk->NewNode(N_VIEW, input->dtype);
  n->sub = kind;
  n->in[0] = input;
  return n;
}
NDObject *Kernel::Permute(NDObject *input, IntArrayRef *dims) {
  auto n = View(Impl(this), VIEW_PERMUTE, input);
  n->shape_ref = dims;
  return n;
}
NDObject *Kernel::Slice(NDObject *input, IntArrayRef *start, IntArrayRef *size) {
  auto n = View(Impl(this), VIEW_SLICE, input);
  n->shape_ref = start;
  n->aux_ref = size;
  return n;
}
NDObject *Kernel::Slice(NDObject *input, int dim, ScalarRef *begin, ScalarRef *end) {
  auto n = View(Impl(this), VIEW_SLICE_DIM, input);
  n->view_dim = dim;
  n->scalar_ref = begin;
  n->scalar_ref2 = end;
  return n;
}
// ref: include/dvm.h:455-469 - the inputs one after the other along `dim` (same type, same extents elsewhere)
NDObject *Kernel::Concat(NDObject **inputs, size_t input_num, int dim) {
  if (inputs == nullptr || input_num == 0) DvmException("Concat needs at least one input");
  auto vk = Impl(this);
  NDObject *acc = inputs[0];
  if (input_num == 1) return Copy(acc);
  for (size_t i = 1; i < input_num; ++i) {
    if (inputs[i]->dtype != acc->dtype) DvmException("Concat inputs must have one type");
    auto n = vk->NewNode(N_CONCAT, acc->dtype);
    n->in[0] = acc;
    n->in[1] = inputs[i];
    n->view_dim = dim;
    acc = n;
  }
  return acc;
}
// ref: include/dvm.h:470-479 - equal chunks along `dim` (the last may be smaller); the returned array is owned by the kernel
NDObject **Kernel::Split(NDObject *input, int dim, int64_t split_size, size_t split_num) {
  auto vk = Impl(this);
  vk->split_outs_.emplace_back(split_num);
  auto &outs = vk->split_outs_.back();
  for (size_t i = 0; i < split_num; ++i) {
    auto n = View(vk, VIEW_SPLIT, input);
    n->view_dim = dim;
    n->view_arg = split_size;
    n->view_index = static_cast<int64_t>(i);
    outs[i] = n;
  }
  return outs.data();
}
template <typename T>
NDObject *Kernel::OneHot(NDObject *, IntArrayRef *, int, T, T) {
  Unsupported("OneHot");
}
template DVM_API NDObject *Kernel::OneHot<float>(NDObject *, IntArrayRef *, int, float, float);
template DVM_API NDObject *Kernel::OneHot<int32_t>(NDObject *, IntArrayRef *, int, int32_t, int32_t);
template DVM_API NDObject *Kernel::OneHot<Float16>(NDObject *, IntArrayRef *, int, Float16, Float16);
template DVM_API NDObject *Kernel::OneHot<BFloat16>(NDObject *, IntArrayRef *, int, BFloat16, BFloat16);
// ref: include/dvm.h:493-496 (private in the reference; python element_any, tests/ut/test_element_any.py): one element
// that is 1 when any element of the input differs from 0, else 0 - the maximum over every dim of (x != 0), in fp32
NDObject *Kernel::ElemAny(NDObject *input) {
  auto vk = Impl(this);
  NDObject *x = input->dtype == kFloat32 ? input : Cast(input, kFloat32);
  auto ne = vk->NewNode(N_COMPARE_S, kFloat32);
  ne->sub = kNotEqual;
  ne->in[0] = x;
  ne->scalar_bits = 0;   // 0.0f
  auto r = vk->NewNode(N_REDUCE, kFloat32);
  r->sub = kMax;
  r->in[0] = ne;
  r->keepdims = false;
  r->reduce_all = true;
  static const int64_t kOne[1] = {1};
  static IntArrayRef one_ref;
  one_ref.data = kOne;
  one_ref.size = 1;
  return Reshape(r, &one_ref);
}

// ref: src/dvm.cc:1537-1544 - a sum of anything but fp32 is refused with a null result.
NDObject *Kernel::_Reduce(int op_type, NDObject *input, IntArrayRef *dims, bool keepdims) {
  if (op_type < 0 || op_type >= kReduceTypeEnd) return nullptr;
  if (input->dtype != kFloat32 && op_type == kSum) return nullptr;
  if (input->dtype == kInt32 || input->dtype == kInt64 || input->dtype == kBool) return nullptr;
  auto n = Impl(this)->NewNode(N_REDUCE, input->dtype);
  n->sub = static_cast<uint8_t>(op_type);
  n->in[0] = input;
  n->shape_ref = dims;
  n->keepdims = keepdims;
  return n;
}

// ref: src/dvm.cc:1679-1686; operand rules ops_m.h:29-141 (fp16/bf16 inputs, result in the input dtype)
NDObject *Kernel::MatMul(NDObject *lhs, NDObject *rhs, bool trans_a, bool trans_b, NDObject *bias) {
  if (lhs->dtype != rhs->dtype || (lhs->dtype != kFloat16 && lhs->dtype != kBFloat16))
    DvmException("MatMul operands must both be float16 or both bfloat16");
  auto n = Impl(this)->NewNode(N_MATMUL, lhs->dtype);
  n->in[0] = lhs;
  n->in[1] = rhs;
  n->in[2] = bias;
  n->trans_a = trans_a;
  n->trans_b = trans_b;
  return n;
}
NDObject *Kernel::GroupedMatMul(NDObject *, NDObject *, bool, bool, NDObject *, NDObject *, GmmSplitType, GmmListType) {
  Unsupported("GroupedMatMul");
}
// ref: Kernel::_AllReduce, src/dvm.cc:1646-1655 (AllReduceOp, src/ops_c.h:124-132): the value of `input` combined over
// the ranks of `comm`.  Sum and max / min on fp32, fp16, bf16 and int32 tensors.
NDObject *Kernel::_AllReduce(int op_type, NDObject *input, const Comm *comm) {
  if (op_type < 0 || op_type >= kReduceTypeEnd) DvmException("invalid all-reduce type");
  if (comm == nullptr || comm->GetImpl() == nullptr) DvmException("AllReduce needs an initialised Comm");
  if (input->dtype == kBool || input->dtype == kInt64) DvmException("AllReduce of bool / int64 tensors is not supported");
  auto n = Impl(this)->NewNode(N_ALLREDUCE, input->dtype);
  n->sub = static_cast<uint8_t>(op_type);
  n->in[0] = input;
  n->comm = comm->GetImpl();
  return n;
}
// ref: Kernel::AllGather / ReduceScatter, src/dvm.cc:1657-1677 (AllGatherOp, ReduceScatterOp: src/ops_c.cc:951-962, 90-111)
static NDObject *Collective(VKernel *vk, uint8_t coll, NDObject *input, const Comm *comm) {
  if (comm == nullptr || comm->GetImpl() == nullptr) DvmException("a collective needs an initialised Comm");
  if (input->dtype == kBool || input->dtype == kInt64) DvmException("collectives on bool / int64 tensors are not supported");
  auto n = vk->NewNode(N_ALLREDUCE, input->dtype);
  n->sub = kSum;
  n->coll = coll;
  n->in[0] = input;
  n->comm = comm->GetImpl();
  return n;
}
NDObject *Kernel::AllGather(NDObject *input, const Comm *comm) { return Collective(Impl(this), 2, input, comm); }
NDObject *Kernel::AllGatherV2(NDObject *, const Comm *) { Unsupported("AllGatherV2"); }
NDObject *Kernel::ReduceScatter(NDObject *input, const Comm *comm) { return Collective(Impl(this), 1, input, comm); }
NDObject *Kernel::ExtOut(NDObject *, int) { Unsupported("ExtOut"); }
// ref: src/dvm.cc:1721-1725 (kernel.h:405).  In the reference the call moves a speculative vector kernel to its next
// fallback stage: a hint where to cut if the graph cannot stay one kernel.  It never changes what the graph computes.
// The stage planner here finds its cuts from the graph alone, so the hint is accepted and not needed; on any other
// kernel type the call is an error, as it is undefined in the reference.
void Kernel::SpecNext() {
  auto vk = Impl(this);
  if (vk->type_ != kVector || !(vk->flags_ & kSpeculate)) DvmException("SpecNext needs a kVector kernel with the kSpeculate flag");
}
// ref: src/dvm.cc:1704-1707, ParallelKernel::AddKernel src/xkernel.cc:1009-1151.  Sub-kernels are independent graphs;
// each becomes launches of its own on the caller's stream (the reference packs them into one launch through a per-core
// program table, src/vm_gpu.cu:1567-1583 - same results, one launch more per sub-kernel here).
void Kernel::ParallelAdd(KernelType type, uint32_t, size_t) {
  auto vk = Impl(this);
  if (vk->type_ != kParallel) DvmException("ParallelAdd needs a kParallel kernel");
  if (type >= kParallel) DvmException("invalid parallel add kernel type");   // (kVector, kCube or kMix graphs)
  vk->cur_sub_ += 1;
}
// ref: src/dvm.cc:1709-1719, SequenceKernel::AddStage src/xkernel.cc:1226-1468.  Ops appended from here on form the
// next stage: it is launched after the previous ones and reads their results through the workspace.
void Kernel::SequenceAdd(KernelType type, uint32_t) {
  auto vk = Impl(this);
  if (vk->type_ != kSequence) DvmException("SequenceAdd needs a kSequence kernel");
  if (type >= kSequence) DvmException("invalid sequence add kernel type");
  vk->cur_sub_ += 1;
}

void Kernel::Normalize() { Impl(this)->Normalize(); }

size_t Kernel::PreCodeGen() {
  auto vk = Impl(this);
  vk->Normalize();
  return vk->Compile();
}

void Kernel::CodeGen(const RelocEntry *relocs, size_t reloc_size, WsAllocator *ws_alloc) {
  auto vk = Impl(this);
  if (!vk->normalized_) vk->Normalize();
  size_t ws = vk->Compile();
  void *workspace = nullptr;
  if (ws > 0) {
    if (ws_alloc == nullptr) DvmException("this kernel needs a workspace but no WsAllocator was given");
    workspace = ws_alloc->Alloc(ws);
  }
  vk->Bind(relocs, reloc_size, workspace);
}

int Kernel::Launch(void *stream) { return Impl(this)->Launch(stream); }

int Kernel::Launch(const RelocEntry *relocs, size_t reloc_size, void *workspace, void *stream) {
  auto vk = Impl(this);
  if (!vk->compiled_) DvmException("Launch(relocs, ...) requires PreCodeGen() first");
  vk->Bind(relocs, reloc_size, workspace);
  return vk->Launch(stream);
}

IntArrayRef *Kernel::GetShape(NDObject *op) {
  op->out_ref.data = op->shape.d;
  op->out_ref.size = static_cast<size_t>(op->shape.rank);
  if (op->kind == N_STORE && op->pad_size > 0 && op->shape.rank > 0) {   // the buffer's shape: rows longer by the pad
    for (int i = 0; i < op->shape.rank; ++i) op->out_dims[i] = op->shape.d[i];
    op->out_dims[op->shape.rank - 1] += op->pad_size;
    op->out_ref.data = op->out_dims;
  }
  return &op->out_ref;
}
DataType Kernel::GetDType(NDObject *op) { return op->dtype; }

const char *Kernel::Dump() const { return kernel_ ? kernel_->Dump() : ""; }
const char *Kernel::DumpR() const { return kernel_ ? kernel_->DumpR() : ""; }
const char *Kernel::Das() const { return kernel_ ? kernel_->Das() : ""; }
const char *Kernel::Inspect() const { return kernel_ ? kernel_->Inspect() : ""; }

}  // namespace dvm
