// Operator graph of one dvm::Kernel: node type, shape inference, stage plans and launch.
//
// Replaces the reference's NDObject class family (src/ops.h:30-77, 444-554) and its kernel models
// (src/kernel.h:52-104, src/xkernel.h) with one node struct and one compile pipeline aimed at the
// sm_100a interpreters.
#ifndef DVM_B200_GRAPH_H_
#define DVM_B200_GRAPH_H_

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../../include/dvm.h"
#include "isa.h"
#include "mm_launch.h"

namespace dvm {

constexpr int kMaxRank = 10;   // the reference's DimArray limit (src/ops.h:165)

struct Shape {
  int64_t d[kMaxRank];
  int rank = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= d[i];
    return n;
  }
  bool operator==(const Shape &o) const {
    if (rank != o.rank) return false;
    for (int i = 0; i < rank; ++i)
      if (d[i] != o.d[i]) return false;
    return true;
  }
};

enum NodeKind : uint8_t {
  N_LOAD = 0,
  N_STORE,
  N_UNARY,      // sub = UnaryType
  N_BINARY,     // sub = BinaryType (arithmetic / logical / pow), two tensor operands
  N_BINARY_S,   // sub = ScalarBin, tensor (in[0]) op scalar
  N_COMPARE,    // sub = BinaryType (< kAdd), two tensor operands; result is 1/0 in the operand dtype
  N_COMPARE_S,  // tensor (in[0]) cmp scalar
  N_SELECT,     // in[0] cond (same dtype as data), in[1], in[2]
  N_CAST,       // one direct conversion step
  N_BROADCAST,  // tensor -> shape
  N_BROADCAST_S,  // scalar -> shape
  N_RESHAPE,
  N_COPY,
  N_REDUCE,     // sub = ReduceType
  N_MATMUL,
  N_VIEW,       // Permute / Slice / Split: the input's memory seen through another shape, strides and offset
  N_CONCAT,     // in[0] followed by in[1] along dim `view_dim`; Kernel::Concat of n inputs is a chain of n - 1 of these, which
                // the stage planner writes as n slabs of one workspace tensor
  N_ALLREDUCE,  // a collective over the ranks of `comm`: `coll` 0 all-reduce (sub = ReduceType), 1 reduce-scatter (sum),
                // 2 all-gather along the leading dim
};

// Scalar-operand arithmetic kinds (the reference's BinaryScalarOp opcodes ADDS/MULS/DIVS/SDIV/MAXS/MINS,
// src/vm_gpu.cu:1178-1297).
enum ViewKind : uint8_t { VIEW_PERMUTE = 0, VIEW_SLICE, VIEW_SLICE_DIM, VIEW_SPLIT };

enum ScalarBin : uint8_t { SB_ADD = 0, SB_MUL, SB_DIV, SB_SDIV, SB_MAX, SB_MIN };

class NDObject {
 public:
  NodeKind kind;
  DataType dtype;
  uint8_t sub = 0;
  bool noloss_cast = false;   // cast inserted by the dtype-promotion rules (may be peeled again)
  bool keepdims = false;
  bool trans_a = false, trans_b = false;
  bool store_temp = false;
  bool store_inplace = false;   // Kernel::SetStoreInplace: the caller's buffer also feeds this kernel (see dvm_api.cc)
  int sub_kernel = 0;           // sub-kernel of a kSequence / kParallel kernel this op was appended to (0 before the first add)
  int id = 0;
  mutable int cidx = -1;   // position in the op list of the vector compiler that is looking at this node (scratch)
  NDObject *in[3] = {nullptr, nullptr, nullptr};
  // scalar operand: fixed code (already encoded in `dtype`, widened to the 32-bit register form) or a
  // borrowed ScalarRef re-read at code generation
  uint32_t scalar_bits = 0;
  ScalarRef *scalar_ref = nullptr;
  IntArrayRef *shape_ref = nullptr;   // Load/Broadcast/Reshape target shape, Reduce dims (borrowed)
  IntArrayRef *stride_ref = nullptr;  // strided (view) Load / Store: element strides of the tensor in memory (borrowed)
  bool strided = false;               // results of Normalize() for a view: `stride` holds one element stride per dim
  int64_t stride[kMaxRank] = {0};
  // SliceLoad / StridedSliceLoad: a window of the tensor at `addr` whose full shape is shape_ref.  slice_mode 1: start +
  // size (slice_a, slice_b); 2: start, end, step (slice_a, slice_b, slice_c; indices as in Python slicing).  Normalize()
  // turns it into a strided load: shape = the window, stride = the tensor's strides times the steps, addr_off = the start
  // a reduction over every dim of its input, whatever the rank turns out to be (ElemAny): Normalize() fills the dims
  bool reduce_all = false;
  int64_t all_dims[kMaxRank] = {0};
  IntArrayRef all_ref;
  int64_t pad_size = 0;               // PadStore: elements added behind every row of the result in memory (never written)
  uint8_t slice_mode = 0;
  IntArrayRef *slice_a = nullptr, *slice_b = nullptr, *slice_c = nullptr;
  void *addr = nullptr;               // Load/Store device address
  // nodes the stage planner makes: a clone of a user's Load/Store (`origin` supplies the address) or a
  // temporary in the kernel's workspace (`ws_off` >= 0, bytes from the workspace base)
  NDObject *origin = nullptr;
  int64_t ws_off = -1;
  int64_t addr_off = 0;               // bytes added to the address above (a rank's row block of a tensor)
  const Communicator *comm = nullptr; // N_ALLREDUCE: the communicator (borrowed from the caller's Comm)
  uint8_t coll = 0;                   // N_ALLREDUCE: which collective (see NodeKind)
  // N_VIEW: sub = ViewKind.  Permute: shape_ref = dims.  Slice: shape_ref = start, aux_ref = size.  Slice along one dim:
  // view_dim, scalar_ref = begin, scalar_ref2 = end.  Split: view_dim, view_arg = chunk size, view_index = which chunk.
  IntArrayRef *aux_ref = nullptr;
  ScalarRef *scalar_ref2 = nullptr;
  int view_dim = 0;
  int64_t view_arg = 0, view_index = 0;
  // results of Normalize() for a view: per result dim the input dim it walks and the element offset into the input
  int view_from[kMaxRank] = {0};
  int64_t view_start[kMaxRank] = {0};   // per INPUT dim: first index taken
  // results of Normalize()
  Shape shape;
  IntArrayRef out_ref;                // view of `shape` handed out by Kernel::GetShape
  int64_t out_dims[kMaxRank] = {0};   // ... of the padded shape for a PadStore
};

// One launch of the vector interpreter.
struct VectorStage {
  dvmb::VmParam param;
  uint32_t grid = 0, threads = 0, smem_bytes = 0;
  uint32_t body_tensor_mask[dvmb::kMaxPhases] = {0, 0, 0, 0};   // tensor slots each BODY reads
  bool idle = false;                       // zero-size domain: nothing to launch
  uint64_t lowered_for = ~0ull;            // per-tensor (vector access, ring slot) flags the micro-ops in `param` were lowered for
  uint32_t sregs_used = 0;                 // scalar registers the program names; the rest up to param.num_sregs hold
                                           // reciprocals of group scalars that the lowering turns fast divisions into
  uint32_t fused_away = 0;                 // micro-ops the last lowering's peephole pass merged into fused handlers (a
                                           // rebind that drops a ring slot can lengthen the program by up to this much)
  std::vector<uint64_t> bytecode;          // instruction words of every section (what Das() prints)
  uint16_t bsec[2 * dvmb::kMaxPhases + 2] = {0};   // section offsets inside `bytecode`
  std::vector<NDObject *> slot_obj;        // tensor slot -> load/store node (relocation sites)
  std::vector<int64_t> slot_ws_off;        // >= 0: slot is a workspace temporary at this byte offset
  // byte offset inside a ring stage that the compiler planned for each bulk-staged tensor (kNoRing otherwise).  Bind()
  // writes it into the descriptor when the bound address is 16-byte aligned and kNoRing when it is not, so a later
  // rebind to an aligned address gets the planned offset back
  uint32_t ring_plan_off[dvmb::kMaxTensors] = {0};
  uint64_t algo_bytes = 0;
};

// One launch of the tensor-core MatMul with its fused post-ops.
struct MatMulStage {
  dvmb::MmParam param;
  NDObject *a = nullptr, *b = nullptr, *bias = nullptr;   // nodes whose addresses feed the operands
  std::vector<NDObject *> slot_obj;     // post-fusion tensor slot -> node (nullptr for the product itself)
  std::vector<uint64_t> bytecode;       // the post-fusion program (what Das() prints)
  bool idle = false;
  uint64_t algo_bytes = 0, flops = 0;
};

// One launch of the fused attention kernel.
struct AttnStage {
  dvmb::AttnParam param;
  NDObject *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr;
  bool idle = false;
  uint64_t algo_bytes = 0, flops = 0;
};

// One collective on the launch stream (comm.h): all-reduce, or the reduce-scatter / all-gather halves it is split
// into when the ops behind it can run on a rank's own row block.
struct CollStage {
  uint32_t kind = 0;                       // dvmb::CollKind
  int reduce_type = 0, dtype = 0;
  const Communicator *comm = nullptr;
  NDObject *send = nullptr, *recv = nullptr;   // nodes whose addresses feed the call
  int64_t send_off = 0, recv_off = 0;      // bytes added to them
  uint64_t count = 0;                      // elements per NCCL's definition of the call
  uint64_t send_ptr = 0, recv_ptr = 0;     // bound addresses
  uint64_t wire_bytes = 0;                 // bytes this rank sends over the links
};

enum StageKind : uint8_t { STAGE_VECTOR = 0, STAGE_MATMUL, STAGE_ATTENTION, STAGE_COLLECTIVE };

struct Stage {
  StageKind kind = STAGE_VECTOR;
  // A pipelined plan (the row chunks of a K-split MatMul whose exchange overlaps the next chunk's product): stages are
  // enqueued in list order, lane 0 on the launch stream, lane 1 (the collectives) on a second stream of the kernel's own;
  // a stage first waits for the stage `after` (an index into the plan, -1: none) where that one ran on the other lane.
  int lane = 0;
  int after = -1;
  VectorStage vec;
  MatMulStage mm;
  AttnStage attn;
  CollStage coll;
};

class VKernel {
 public:
  VKernel(KernelType type, uint32_t flags) : type_(type), flags_(flags) {}
  void ClearStages();
  // stat_fusion.cc: the op list with sums of squared deviations folded into the pass that makes their mean
  std::vector<NDObject *> FuseDeviationSums(const std::vector<NDObject *> &ops);
  void PlanStages(const std::vector<NDObject *> &ops);   // partition.cc: general multi-stage planner
  ~VKernel();

  NDObject *NewNode(NodeKind kind, DataType dtype);
  void Normalize();
  size_t Compile();   // build stages for the current shapes; returns workspace bytes
  void Bind(const RelocEntry *relocs, size_t n, void *workspace);
  int Launch(void *stream);
  int LaunchStage(size_t index, void *stream);   // one launch (or collective) of the plan, for per-stage timing
  int LaunchPipelined(void *stream);             // a plan with two lanes (see Stage::lane)
  void *side_stream_ = nullptr;                  // lane 1; created at the first pipelined launch
  std::vector<void *> stage_events_;             // one event per stage that another lane waits for
  void *join_event_ = nullptr;

  const char *Dump();
  const char *DumpR();
  const char *Das();
  const char *Inspect();

  KernelType type_;
  uint32_t flags_;
  std::vector<NDObject *> nodes_;          // append (= topological) order
  std::vector<std::unique_ptr<Stage>> stages_;
  std::vector<NDObject *> synth_;          // planner-made nodes (clones, workspace temporaries), owned
  std::vector<std::vector<NDObject *>> split_outs_;   // arrays handed out by Kernel::Split (valid for the kernel's life)
  size_t ws_bytes_ = 0;
  int cur_sub_ = 0;                        // sub-kernel that NewNode() tags ops with (SequenceAdd / ParallelAdd advance it)
  void *workspace_ = nullptr;
  bool normalized_ = false;
  bool compiled_ = false;
  std::string text_;
  std::string name_;
  double last_jit_us_ = 0.0;               // host time of the last Normalize+Compile+Bind
};

// vcompile.cc
bool CompileVectorStage(const std::vector<NDObject *> &ops, VectorStage *out, std::string *why);
// Compile `ops` (a pseudo-load `mma_src` standing for the MatMul product, the fused elementwise ops, stores) into
// the post-fusion program of a MatMul stage.
bool CompileEpilogue(const std::vector<NDObject *> &ops, const NDObject *mma_src, MatMulStage *out, std::string *why);
std::string DisassembleEpilogue(const MatMulStage &st);
std::string DisassembleStage(const VectorStage &st);
// Turn the stage's instruction words into the launch program (scalar sections + micro-ops) for the tensor
// addresses now in the descriptors; called whenever addresses are (re)bound.
void LowerStage(VectorStage *st);
// The per-tensor properties the lowering depends on, packed: a rebind that leaves them unchanged keeps the micro-ops.
inline uint64_t LoweringKey(const VectorStage &st) {
  uint64_t key = 0;
  for (uint32_t s = 0; s < st.param.n_tensors; ++s)
    key |= (static_cast<uint64_t>(st.param.tensor[s].vec_ok ? 1 : 0) | (st.param.tensor[s].ring_off != dvmb::kNoRing ? 2ull : 0ull)) << (2 * s);
  return key;
}

// normalize.cc
void InferShape(NDObject *n);
int ItemSize(DataType t);
const char *DTypeName(DataType t);

}  // namespace dvm

#endif  // DVM_B200_GRAPH_H_
