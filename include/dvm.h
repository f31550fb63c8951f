// dvm-b200: C++ builder API of the B200-native device virtual machine.
//
// Source-compatible with the builder API of mindspore-ai/dvm (its include/dvm.h): the same namespace,
// enumerators (same numeric values), class names, method names, argument order and ownership rules, so
// code written against that header recompiles against this one.  Each declaration cites the
// reference declaration it stands in for as `ref: include/dvm.h:<line>`.
//
// Ownership (ref: include/dvm.h:149-217, docs/tutorial.md:59-117):
//   * a Kernel owns every NDObject* it hands out; callers never free them;
//   * IntArrayRef* / ScalarRef* arguments are borrowed and re-read at every Normalize()/CodeGen(),
//     which is how runtime shapes and scalars enter; the caller keeps them alive;
//   * tensor addresses are borrowed device pointers, may be null while building and are supplied or
//     replaced through RelocEntry at CodeGen()/Launch();
//   * strings returned by Dump/DumpR/Das/Inspect stay valid until the next such call on the same Kernel.
// A Kernel is not re-entrant; different phases may run on different threads one after another.
#ifndef DVM_B200_DVM_H_
#define DVM_B200_DVM_H_

#include <cstddef>
#include <cstdint>
#include <vector>

#define DVM_API __attribute__((visibility("default")))

namespace dvm {

// ref: include/dvm.h:27-35
enum DataType { kBool = 0, kFloat16, kBFloat16, kFloat32, kInt32, kInt64, kDataTypeEnd };
// ref: include/dvm.h:37-40
enum GatherMode { kElementGather = 0, kSliceGather = 1 };
// ref: include/dvm.h:42-55
enum UnaryType {
  kSqrt = 0, kAbs, kLog, kExp, kReciprocal, kIsFinite, kLogicalNot, kRound, kFloor, kCeil, kTrunc, kUnaryTypeEnd
};
// ref: include/dvm.h:57-74
enum BinaryType {
  kEqual = 0, kNotEqual, kGreater, kGreaterEqual, kLess, kLessEqual,
  kAdd, kSub, kMul, kDiv, kPow, kMaximum, kMinimum, kLogicalAnd, kLogicalOr, kBinaryTypeEnd
};
// ref: include/dvm.h:76-81
enum ReduceType { kSum = 0, kMax, kMin, kReduceTypeEnd };
// ref: include/dvm.h:83-94
enum GmmSplitType { kSplit_M = 0, kSplit_N, kSplit_K, kGroupTypeEnd };
enum GmmListType { kListBound = 0, kListSize, kEnd };

// ref: include/dvm.h:97-106.  On this backend every type lowers to launches of the sm_100a interpreters:
// kVector/kEager/kSplit/kSequence build fused vector stages (cut only where on-chip fusion is impossible),
// kCube/kMix put one MatMul on the tcgen05 path with the vector ops that follow it in its epilogue.
enum KernelType { kVector = 0, kCube, kMix, kParallel, kSequence, kSplit, kEager, kKernelTypeEnd };

// ref: include/dvm.h:109-117
enum KernelFlag {
  kDynamic = 0x1,
  kUnifyWS = 0x2,
  kSpeculate = 0x4,
  kLazyCodeGen = 0x8,
  kOptFractalTrans = 1u << 29,
  kPrivate1 = 1u << 30,
  kPrivate2 = 1u << 31,
};

class NDObject;
class VKernel;
class Communicator;

// IEEE binary16 value holder; conversions round to nearest even.  ref: include/dvm.h:123-134
class DVM_API Float16 {
 public:
  explicit Float16(uint16_t bits) : value_(bits) {}
  explicit Float16(float v);
  explicit Float16(int32_t v);
  explicit operator float() const;
  explicit operator int32_t() const;
  uint16_t int_value() const { return value_; }

 private:
  uint16_t value_;
};

// bfloat16 value holder; conversions round to nearest even, NaN maps to 0x7fc0.  ref: include/dvm.h:136-147
class DVM_API BFloat16 {
 public:
  explicit BFloat16(uint16_t bits) : value_(bits) {}
  explicit BFloat16(float v);
  explicit BFloat16(int32_t v);
  explicit operator float() const;
  explicit operator int32_t() const;
  uint16_t int_value() const { return value_; }

 private:
  uint16_t value_;
};

// Borrowed view of an int64 array (shape, dims, strides).  ref: include/dvm.h:149-159
struct DVM_API IntArrayRef {
  IntArrayRef() {}
  explicit IntArrayRef(const std::vector<int64_t> &v) : data(v.data()), size(v.size()) {}
  IntArrayRef &operator=(const std::vector<int64_t> &v) {
    data = v.data();
    size = v.size();
    return *this;
  }
  const int64_t *data;
  size_t size;
};

// Borrowed runtime scalar, re-read at every code generation.  ref: include/dvm.h:161-199
struct DVM_API ScalarRef {
  ScalarRef() = default;
  template <typename T>
  ScalarRef(T v) {
    *this = v;
  }
  ScalarRef &operator=(float v) { type = kFloat32; f32 = v; return *this; }
  ScalarRef &operator=(int32_t v) { type = kInt32; i32 = v; return *this; }
  ScalarRef &operator=(Float16 v) { type = kFloat16; f16 = v.int_value(); return *this; }
  ScalarRef &operator=(BFloat16 v) { type = kBFloat16; f16 = v.int_value(); return *this; }
  ScalarRef &operator=(int64_t v) { type = kInt64; i64 = v; return *this; }
  DataType type;
  union {
    float f32;
    int32_t i32;
    uint16_t f16;
    int64_t i64;
  };
};

// (load/store object, device address) pair used to bind or re-bind tensors.  ref: include/dvm.h:201-206
struct DVM_API RelocEntry {
  RelocEntry() {}
  RelocEntry(NDObject *p, void *a) : io(p), addr(a) {}
  NDObject *io;
  void *addr;
};

// Workspace callback used by CodeGen(); the library never frees what it returns.  ref: include/dvm.h:208-210
struct DVM_API WsAllocator {
  virtual void *Alloc(size_t size) = 0;
};

// ref: include/dvm.h:212-217
struct DVM_API CloneHelper {
  virtual IntArrayRef *GetClone(IntArrayRef *shape) = 0;
  virtual ScalarRef *GetClone(ScalarRef *scalar) = 0;
  virtual NDObject *GetClone(NDObject *op) = 0;
  virtual void SetClone(NDObject *op, NDObject *clone) = 0;
};

// Rank information for collectives.  On this backend the data path is NCCL: Init records rank/size and
// the process binds an NCCL communicator separately (see dvm_c.h).  ref: include/dvm.h:219-231
class DVM_API Comm {
 public:
  enum { kMemory, kHccl, kDummy };
  Comm() = default;
  ~Comm();
  bool Init(int rank_id, int rank_size, int comm_type, const uint32_t *group_ranks = nullptr);
  bool Init(int rank_id, int rank_size) { return Init(rank_id, rank_size, kMemory); }
  void Init(void *nccl_comm);
  inline const Communicator *GetImpl() const { return comm_; }

 protected:
  Communicator *comm_{nullptr};
};

// Graph builder + JIT + launcher.  ref: include/dvm.h:236-722
class DVM_API Kernel {
 public:
  Kernel();
  ~Kernel();
  // Copying transfers the implementation: afterwards only the destination is usable.  ref: :241-245
  Kernel &operator=(Kernel &other);
  explicit Kernel(Kernel &other);

  void Reset(KernelType type, uint32_t flags);              // ref: :252
  void Clone(const Kernel &base, CloneHelper &helper);      // ref: :259
  void SetNameHint(const char *name, const char *fullname);  // ref: :266

  NDObject *Load(void *addr, IntArrayRef *shape, DataType type);                       // ref: :276
  NDObject *GlobalAccess(void *addr, IntArrayRef *shape, DataType type);               // ref: :285
  NDObject *Load(void *addr, IntArrayRef *shape, IntArrayRef *stride, DataType type);  // ref: :294
  NDObject *GatherLoad(void *addr, IntArrayRef *shape, NDObject *index, int axis, DataType type,
                       GatherMode gather_mode = kElementGather);                      // ref: :306
  NDObject *SliceLoad(void *addr, IntArrayRef *shape, IntArrayRef *start, IntArrayRef *size, DataType type);
  NDObject *StridedSliceLoad(void *addr, IntArrayRef *shape, IntArrayRef *start, IntArrayRef *end,
                             IntArrayRef *step, DataType type);
  NDObject *MultiLoad(void *addr, IntArrayRef *shape, DataType type, const Comm *comm);
  NDObject *Store(void *addr, NDObject *input);                       // ref: :331
  NDObject *Store(void *addr, NDObject *input, IntArrayRef *stride);  // ref: :339
  NDObject *PadStore(void *addr, NDObject *input, int64_t pad_size);
  void SetStoreInplace(NDObject *store);
  void SetStoreTemp(NDObject *store);
  void SetLoadBind(NDObject *load, NDObject *access);

  template <UnaryType op_type>
  NDObject *Unary(NDObject *input);  // ref: :372
  template <BinaryType op_type, typename L, typename R>
  NDObject *Binary(L lhs, R rhs);  // ref: :381; L/R: NDObject*, float, int32_t, int64_t, Float16, BFloat16, ScalarRef*
  template <ReduceType op_type>
  NDObject *Reduce(NDObject *input, IntArrayRef *dims, bool keepdims) {  // ref: :391
    return _Reduce(op_type, input, dims, keepdims);
  }
  NDObject *Select(NDObject *cond, NDObject *lhs, NDObject *rhs);  // ref: :401
  NDObject *Cast(NDObject *input, DataType type);                  // ref: :409
  NDObject *Broadcast(NDObject *input, IntArrayRef *shape);        // ref: :417
  template <typename T>
  NDObject *Broadcast(T val, IntArrayRef *shape, DataType type);   // ref: :426
  NDObject *Reshape(NDObject *input, IntArrayRef *shape);          // ref: :434
  NDObject *Permute(NDObject *input, IntArrayRef *dims);
  NDObject *Slice(NDObject *input, IntArrayRef *start, IntArrayRef *size);
  NDObject *Slice(NDObject *input, int dim, ScalarRef *begin, ScalarRef *end);
  NDObject *Copy(NDObject *input);  // ref: :466
  NDObject *Concat(NDObject **inputs, size_t input_num, int dim);
  NDObject **Split(NDObject *input, int dim, int64_t split_size, size_t split_num);
  template <typename T>
  NDObject *OneHot(NDObject *indices, IntArrayRef *depth, int axis, T on_value, T off_value);
  NDObject *ElemAny(NDObject *input);
  // C[..., M, N] = op(A) * op(B) (+ bias); fp16/bf16 operands, fp32 accumulation.  ref: :509
  NDObject *MatMul(NDObject *lhs, NDObject *rhs, bool trans_a, bool trans_b, NDObject *bias);
  NDObject *GroupedMatMul(NDObject *lhs, NDObject *rhs, bool trans_a, bool trans_b, NDObject *bias,
                          NDObject *group_list, GmmSplitType group_type, GmmListType group_list_type);
  template <ReduceType op_type>
  NDObject *AllReduce(NDObject *input, const Comm *comm) {  // ref: :531
    return _AllReduce(op_type, input, comm);
  }
  NDObject *AllGather(NDObject *input, const Comm *comm);
  NDObject *AllGatherV2(NDObject *input, const Comm *comm);
  NDObject *ReduceScatter(NDObject *input, const Comm *comm);
  NDObject *ExtOut(NDObject *op, int index);
  void SpecNext();
  void ParallelAdd(KernelType type, uint32_t flags, size_t thread_limit = 0);
  void SequenceAdd(KernelType type, uint32_t flags);

  void Normalize();                                                                  // ref: :566 shape inference
  void CodeGen(const RelocEntry *relocs, size_t reloc_size, WsAllocator *ws_alloc);  // ref: :572
  int Launch(void *stream);                                                          // ref: :578 (0 = ok)
  void Clear();
  size_t PreCodeGen();  // ref: :590 static-shape compile; returns workspace bytes
  int Launch(const RelocEntry *relocs, size_t reloc_size, void *workspace, void *stream);  // ref: :599

  static IntArrayRef *GetShape(NDObject *op);  // ref: :606
  static DataType GetDType(NDObject *op);      // ref: :612
  const char *Dump() const;                    // ref: :619 graph after scheduling
  const char *DumpR() const;                   // ref: :625 graph as built
  const char *Das() const;                     // ref: :631 bytecode disassembly
  const char *Inspect() const;                 // ref: :637
  VKernel *GetImpl() const { return kernel_; }

 protected:
  NDObject *_Reduce(int op_type, NDObject *input, IntArrayRef *dims, bool keepdims);
  NDObject *_AllReduce(int op_type, NDObject *input, const Comm *comm);
  VKernel *kernel_;

 public:
  // Run-time dispatched spellings kept for callers that pass the op as an int.  ref: :652-721
  NDObject *Unary(int op_type, NDObject *input);
  template <typename L, typename R>
  NDObject *Binary(int op_type, L lhs, R rhs);
  NDObject *Reduce(int op_type, NDObject *input, IntArrayRef *dims, bool keepdims) {
    return _Reduce(op_type, input, dims, keepdims);
  }
  NDObject *AllReduce(int op_type, NDObject *input, const Comm *comm) { return _AllReduce(op_type, input, comm); }
  void ParallelNext() { return ParallelAdd(KernelType::kVector, 0); }
  void Infer() { Normalize(); }
  size_t CodeGen() { return PreCodeGen(); }
};

template <typename L, typename R>
NDObject *Kernel::Binary(int op_type, L lhs, R rhs) {
#define DVM_BINARY_CASE(T) \
  case BinaryType::T: return Binary<BinaryType::T>(lhs, rhs);
  switch (op_type) {
    DVM_BINARY_CASE(kEqual) DVM_BINARY_CASE(kNotEqual) DVM_BINARY_CASE(kGreater) DVM_BINARY_CASE(kGreaterEqual)
    DVM_BINARY_CASE(kLess) DVM_BINARY_CASE(kLessEqual) DVM_BINARY_CASE(kAdd) DVM_BINARY_CASE(kSub)
    DVM_BINARY_CASE(kMul) DVM_BINARY_CASE(kDiv) DVM_BINARY_CASE(kPow) DVM_BINARY_CASE(kMaximum)
    DVM_BINARY_CASE(kMinimum) DVM_BINARY_CASE(kLogicalAnd) DVM_BINARY_CASE(kLogicalOr)
    default: return nullptr;
  }
#undef DVM_BINARY_CASE
}

// Process-wide switches.  ref: include/dvm.h:727-741.  Determinism is always on here (reductions use a
// fixed tree); the tuner and VF-fusion switches are accepted and ignored.
class DVM_API Config {
 public:
  Config() = default;
  ~Config() = default;
  static Config &Instance();
  bool IsInitialized() const;
  virtual Config &SetDeterm() = 0;
  virtual Config &UnsetDeterm() = 0;
  virtual Config &SetOnlineTuner() = 0;
  virtual Config &UnsetOnlineTuner() = 0;
  virtual Config &SetLazyTuner() = 0;
  virtual Config &UnsetLazyTuner() = 0;
  virtual Config &SetVfFusion(int mode = 1) = 0;
  virtual Config &UnsetVfFusion() = 0;
};

// Older spellings.  ref: include/dvm.h:743-750
using DType = DataType;
using UnaryOpType = UnaryType;
using BinaryOpType = BinaryType;
using ReduceOpType = ReduceType;
using GroupType = GmmSplitType;
using GroupListType = GmmListType;
using ShapeRef = IntArrayRef;

// Throws std::runtime_error("DVM EXCEPTION. reason: ...").  ref: include/dvm.h:752, src/system.cc:276-280
[[noreturn]] DVM_API void DvmException(const char *error_str);

}  // namespace dvm

#endif  // DVM_B200_DVM_H_
