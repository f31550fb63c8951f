// VKernel: owns the graph of one dvm::Kernel, runs shape inference, plans the launches and runs them.
// Counterpart of the reference's VKernel / VKernelS lifecycle (Normalize/CodeGen/CodeGenR/Launch,
// src/kernel.cc:104-156, 2113-2209) for the sm_100a interpreters.
#include <chrono>
#include <cstring>
#include <string>

#include <cuda_runtime.h>

#include "comm.h"
#include "graph.h"
#include "runtime.h"
#include "vm_launch.h"
#include "mm_launch.h"

namespace dvm {

VKernel::~VKernel() {
  ClearStages();
  for (auto n : nodes_) delete n;
  for (void *e : stage_events_)
    if (e) cudaEventDestroy(static_cast<cudaEvent_t>(e));
  if (join_event_) cudaEventDestroy(static_cast<cudaEvent_t>(join_event_));
  if (side_stream_) cudaStreamDestroy(static_cast<cudaStream_t>(side_stream_));
}

void VKernel::ClearStages() {
  stages_.clear();
  for (auto n : synth_) delete n;
  synth_.clear();
}

// Device address of a load/store node: a workspace temporary, a clone of a user's node, or the node itself.
static void *AddrOf(const NDObject *n, void *workspace) {
  void *base = n->addr;
  if (n->ws_off >= 0) {
    base = workspace ? static_cast<char *>(workspace) + n->ws_off : nullptr;
  } else if (n->origin) {
    base = n->origin->addr;
  }
  return base ? static_cast<char *>(base) + n->addr_off : nullptr;
}

NDObject *VKernel::NewNode(NodeKind kind, DataType dtype) {
  auto n = new NDObject();
  n->kind = kind;
  n->dtype = dtype;
  n->id = static_cast<int>(nodes_.size());
  n->sub_kernel = cur_sub_;
  nodes_.push_back(n);
  normalized_ = false;
  compiled_ = false;
  return n;
}

void VKernel::Normalize() {
  // a Store handed to a later op as an operand stands for the value it stores (the reference's sequence kernels read a
  // stage's stored result back in a later stage, tests/ut/test_sequence_fusion.py:170-205)
  for (auto n : nodes_)
    for (int k = 0; k < 3; ++k)
      while (n->in[k] && n->in[k]->kind == N_STORE && n->in[k]->in[0]) n->in[k] = n->in[k]->in[0];
  for (auto n : nodes_) InferShape(n);
  normalized_ = true;
  compiled_ = false;
}

// Drop ops that no store depends on (the reference's dead-code pass, src/pass.cc:838-849).
static std::vector<NDObject *> LiveOps(const std::vector<NDObject *> &nodes) {
  std::vector<char> live(nodes.size(), 0);
  for (size_t i = nodes.size(); i-- > 0;) {
    NDObject *n = nodes[i];
    if (n->kind == N_STORE) live[i] = 1;
    if (!live[i]) continue;
    for (int k = 0; k < 3; ++k)
      if (n->in[k]) live[n->in[k]->id] = 1;
  }
  std::vector<NDObject *> out;
  for (size_t i = 0; i < nodes.size(); ++i)
    if (live[i]) out.push_back(nodes[i]);
  return out;
}

size_t VKernel::Compile() {
  if (!normalized_) Normalize();
  ClearStages();
  ws_bytes_ = 0;
  std::vector<NDObject *> ops = LiveOps(nodes_);
  if (ops.empty()) {
    compiled_ = true;
    return 0;
  }
  bool has_matmul = false, has_empty = false, stacked = false;
  for (auto n : ops) {
    has_matmul |= n->kind == N_MATMUL || n->kind == N_ALLREDUCE || n->kind == N_VIEW || n->kind == N_CONCAT;   // (anything that needs the stage planner)
    has_empty |= n->shape.numel() == 0;   // the planner drops empty tensors and keeps what still has elements
    stacked |= n->sub_kernel != ops.front()->sub_kernel;   // kSequence / kParallel: every sub-kernel gets launches of its own
  }
  if (!has_matmul && !has_empty && !stacked) {
    // the common case: the whole graph is one launch of the vector interpreter
    std::string why;
    const std::vector<NDObject *> folded = FuseDeviationSums(ops);
    if (folded != ops) {
      auto st = std::make_unique<Stage>();
      if (CompileVectorStage(folded, &st->vec, &why)) {
        stages_.push_back(std::move(st));
        compiled_ = true;
        return 0;
      }
    }
    auto st = std::make_unique<Stage>();
    if (CompileVectorStage(ops, &st->vec, &why)) {
      stages_.push_back(std::move(st));
      compiled_ = true;
      return 0;
    }
  }
  PlanStages(ops);
  compiled_ = true;
  return ws_bytes_;
}

void VKernel::Bind(const RelocEntry *relocs, size_t n, void *workspace) {
  workspace_ = workspace;
  for (size_t i = 0; i < n; ++i) relocs[i].io->addr = relocs[i].addr;
  for (auto &stp : stages_) {
    if (stp->kind == STAGE_MATMUL) {
      MatMulStage &mm = stp->mm;
      mm.param.a_ptr = reinterpret_cast<uint64_t>(AddrOf(mm.a, workspace));
      mm.param.b_ptr = reinterpret_cast<uint64_t>(AddrOf(mm.b, workspace));
      mm.param.bias_ptr = mm.bias ? reinterpret_cast<uint64_t>(AddrOf(mm.bias, workspace)) : 0;
      for (size_t s = 0; s < mm.slot_obj.size(); ++s)
        if (mm.slot_obj[s]) mm.param.tensor[s].ptr = reinterpret_cast<uint64_t>(AddrOf(mm.slot_obj[s], workspace));
      continue;
    }
    if (stp->kind == STAGE_COLLECTIVE) {
      CollStage &co = stp->coll;
      void *sp = AddrOf(co.send, workspace), *rp = AddrOf(co.recv, workspace);
      co.send_ptr = sp ? reinterpret_cast<uint64_t>(sp) + co.send_off : 0;
      co.recv_ptr = rp ? reinterpret_cast<uint64_t>(rp) + co.recv_off : 0;
      continue;
    }
    if (stp->kind == STAGE_ATTENTION) {
      AttnStage &at = stp->attn;
      at.param.q_ptr = reinterpret_cast<uint64_t>(AddrOf(at.q, workspace));
      at.param.k_ptr = reinterpret_cast<uint64_t>(AddrOf(at.k, workspace));
      at.param.v_ptr = reinterpret_cast<uint64_t>(AddrOf(at.v, workspace));
      at.param.o_ptr = reinterpret_cast<uint64_t>(AddrOf(at.o, workspace));
      continue;
    }
    VectorStage &st = stp->vec;
    dvmb::VmParam &P = st.param;
    uint32_t staged = 0;
    for (size_t s = 0; s < st.slot_obj.size(); ++s) {
      dvmb::TensorDesc &td = P.tensor[s];
      td.ptr = reinterpret_cast<uint64_t>(AddrOf(st.slot_obj[s], workspace));
      const uint64_t align = 4ull * ItemSize(static_cast<DataType>(td.dtype));
      td.vec_ok = (td.layout_vec && td.ptr != 0 && td.ptr % align == 0) ? 1 : 0;
      // a tensor planned for bulk staging keeps its ring slot only if its address is 16-byte aligned
      const bool on_ring = td.ring_layout && st.ring_plan_off[s] != dvmb::kNoRing && td.ptr % 16 == 0;
      td.ring_off = on_ring ? st.ring_plan_off[s] : dvmb::kNoRing;
      if (on_ring) staged |= 1u << s;
    }
    for (uint32_t q = 0; q < P.num_body; ++q) P.body_ring_mask[q] = st.body_tensor_mask[q] & staged;
    if (LoweringKey(st) != st.lowered_for) {   // (an unaligned address took a tensor off its fast path)
      LowerStage(&st);
      st.lowered_for = LoweringKey(st);
    }
  }
}

// A plan with two lanes: every stage goes to its lane's stream in list order; a stage whose `after` ran on the other lane
// waits for that stage's event first.  The launch stream finally waits for the second stream, so that the caller sees
// the usual contract (everything enqueued on `stream` is ordered behind the kernel).
int VKernel::LaunchPipelined(void *stream) {
  cudaStream_t main_s = static_cast<cudaStream_t>(stream);
  if (side_stream_ == nullptr) {
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) DvmException("cannot create the second launch stream");
    side_stream_ = s;
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) DvmException("cannot create an event");
    join_event_ = e;
  }
  cudaStream_t side_s = static_cast<cudaStream_t>(side_stream_);
  if (stage_events_.size() < stages_.size()) stage_events_.resize(stages_.size(), nullptr);
  std::vector<char> signals(stages_.size(), 0);
  for (auto &st : stages_)
    if (st->after >= 0 && stages_[st->after]->lane != st->lane) signals[st->after] = 1;
  bool side_used = false;
  for (size_t i = 0; i < stages_.size(); ++i) {
    Stage &st = *stages_[i];
    cudaStream_t s = st.lane ? side_s : main_s;
    if (st.after >= 0 && stages_[st.after]->lane != st.lane) {
      if (cudaStreamWaitEvent(s, static_cast<cudaEvent_t>(stage_events_[st.after]), 0) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    } else if (st.lane && !side_used) {
      // the first stage of the second stream is ordered behind whatever the launch stream holds
      if (cudaEventRecord(static_cast<cudaEvent_t>(join_event_), main_s) != cudaSuccess ||
          cudaStreamWaitEvent(side_s, static_cast<cudaEvent_t>(join_event_), 0) != cudaSuccess)
        return static_cast<int>(cudaGetLastError());
    }
    side_used |= st.lane != 0;
    int err = LaunchStage(i, s);
    if (err != 0) return err;
    if (signals[i]) {
      if (stage_events_[i] == nullptr) {
        cudaEvent_t e = nullptr;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) DvmException("cannot create an event");
        stage_events_[i] = e;
      }
      if (cudaEventRecord(static_cast<cudaEvent_t>(stage_events_[i]), s) != cudaSuccess) return static_cast<int>(cudaGetLastError());
    }
  }
  if (side_used) {
    if (cudaEventRecord(static_cast<cudaEvent_t>(join_event_), side_s) != cudaSuccess ||
        cudaStreamWaitEvent(main_s, static_cast<cudaEvent_t>(join_event_), 0) != cudaSuccess)
      return static_cast<int>(cudaGetLastError());
  }
  return 0;
}

int VKernel::Launch(void *stream) {
  if (!compiled_) DvmException("Launch before CodeGen");
  dvmb::Runtime::Get().EnsureInit();
  for (auto &st : stages_)
    if (st->lane != 0) return LaunchPipelined(stream);
  for (size_t i = 0; i < stages_.size(); ++i) {
    int err = LaunchStage(i, stream);
    if (err != 0) return err;
  }
  return 0;
}

int VKernel::LaunchStage(size_t index, void *stream) {
  if (!compiled_ || index >= stages_.size()) DvmException("LaunchStage: no such stage");
  dvmb::Runtime::Get().EnsureInit();
  {
    auto &stp = stages_[index];
    if (stp->kind == STAGE_MATMUL) {
      MatMulStage &mm = stp->mm;
      if (mm.idle) return 0;
      if (mm.param.a_ptr == 0 || mm.param.b_ptr == 0) DvmException("Launch with an unbound tensor address");
      for (size_t s = 0; s < mm.slot_obj.size(); ++s)
        if (mm.slot_obj[s] && mm.param.tensor[s].ptr == 0) DvmException("Launch with an unbound tensor address");
      return dvmb::LaunchMatMul(mm.param, stream);
    }
    if (stp->kind == STAGE_COLLECTIVE) {
      CollStage &co = stp->coll;
      if (co.count == 0) return 0;
      if (co.send_ptr == 0 || co.recv_ptr == 0) DvmException("Launch with an unbound tensor address");
      std::string err;
      int rc = dvmb::RunCollective(co.comm, static_cast<dvmb::CollKind>(co.kind), co.reduce_type, co.dtype,
                                   reinterpret_cast<const void *>(co.send_ptr), reinterpret_cast<void *>(co.recv_ptr), co.count,
                                   stream, &err);
      if (rc != 0) DvmException(("collective failed: " + err).c_str());
      return 0;
    }
    if (stp->kind == STAGE_ATTENTION) {
      AttnStage &at = stp->attn;
      if (at.idle) return 0;
      if (!at.param.q_ptr || !at.param.k_ptr || !at.param.v_ptr || !at.param.o_ptr)
        DvmException("Launch with an unbound tensor address");
      return dvmb::LaunchAttention(at.param, stream);
    }
    VectorStage &st = stp->vec;
    if (st.idle) return 0;
    for (size_t s = 0; s < st.slot_obj.size(); ++s)
      if (st.param.tensor[s].ptr == 0) DvmException("Launch with an unbound tensor address");
    return dvmb::LaunchVector(st.param, st.grid, st.threads, st.smem_bytes, stream);
  }
}

// ---- text dumps -------------------------------------------------------------------------------------
static const char *KindName(const NDObject *n) {
  static const char *un[] = {"Sqrt", "Abs", "Log", "Exp", "Reciprocal", "IsFinite", "LogicalNot", "Round", "Floor", "Ceil", "Trunc"};
  static const char *bin[] = {"Equal", "NotEqual", "Greater", "GreaterEqual", "Less", "LessEqual", "Add", "Sub", "Mul",
                              "Div", "Pow", "Maximum", "Minimum", "LogicalAnd", "LogicalOr"};
  static const char *sb[] = {"Adds", "Muls", "Divs", "SDiv", "Maxs", "Mins"};
  static const char *red[] = {"ReduceSum", "ReduceMax", "ReduceMin"};
  switch (n->kind) {
    case N_LOAD: return "Load";
    case N_STORE: return "Store";
    case N_UNARY: return un[n->sub];
    case N_BINARY: return bin[n->sub];
    case N_BINARY_S: return sb[n->sub];
    case N_COMPARE: return bin[n->sub];
    case N_COMPARE_S: return bin[n->sub];
    case N_SELECT: return "Select";
    case N_CAST: return "Cast";
    case N_BROADCAST: return "Broadcast";
    case N_BROADCAST_S: return "BroadcastS";
    case N_RESHAPE: return "Reshape";
    case N_COPY: return "Copy";
    case N_REDUCE: return red[n->sub];
    case N_VIEW: {
      static const char *views[] = {"Permute", "Slice", "Slice", "Split"};
      return views[n->sub & 3];
    }
    case N_CONCAT: return "Concat";
    case N_ALLREDUCE:
      if (n->coll == 1) return "ReduceScatter";
      if (n->coll == 2) return "AllGather";
      return n->sub == kSum ? "AllReduceSum" : (n->sub == kMax ? "AllReduceMax" : "AllReduceMin");
    default: return "MatMul";
  }
}

static std::string GraphText(const std::vector<NDObject *> &nodes, bool with_shapes) {
  std::string o;
  char buf[160];
  for (auto n : nodes) {
    snprintf(buf, sizeof(buf), "%%%d = %s.%s(", n->id, KindName(n), DTypeName(n->dtype));
    o += buf;
    bool first = true;
    for (int k = 0; k < 3; ++k)
      if (n->in[k]) {
        snprintf(buf, sizeof(buf), "%s%%%d", first ? "" : ", ", n->in[k]->id);
        o += buf;
        first = false;
      }
    if (n->kind == N_BINARY_S || n->kind == N_COMPARE_S || n->kind == N_BROADCAST_S) {
      snprintf(buf, sizeof(buf), "%s%s", first ? "" : ", ", n->scalar_ref ? "<scalar ref>" : "");
      o += buf;
      if (!n->scalar_ref) {
        snprintf(buf, sizeof(buf), "#0x%08x", n->scalar_bits);
        o += buf;
      }
    }
    o += ")";
    if (with_shapes) {
      o += " [";
      for (int i = 0; i < n->shape.rank; ++i) {
        snprintf(buf, sizeof(buf), "%s%lld", i ? "," : "", static_cast<long long>(n->shape.d[i]));
        o += buf;
      }
      o += "]";
    }
    o += "\n";
  }
  return o;
}

const char *VKernel::DumpR() {
  text_ = GraphText(nodes_, normalized_);
  return text_.c_str();
}

const char *VKernel::Dump() {
  if (!normalized_) Normalize();
  text_ = GraphText(LiveOps(nodes_), true);
  return text_.c_str();
}

const char *VKernel::Das() {
  if (!compiled_) Compile();
  text_.clear();
  for (auto &st : stages_) {
    if (st->kind == STAGE_MATMUL) {
      text_ += DisassembleEpilogue(st->mm);
    } else if (st->kind == STAGE_COLLECTIVE) {
      const CollStage &c = st->coll;
      static const char *names[] = {"all_reduce", "reduce_scatter", "all_gather"};
      static const char *ops[] = {"sum", "max", "min"};
      char buf[320];
      snprintf(buf, sizeof(buf), "cmain.nccl(%s%s%s, %s, count=%llu, rank=%d of %d, wire_bytes=%llu) {\n  %s 0x%llx, load(0x%llx)\n}\n",
               names[c.kind], c.kind == dvmb::COLL_ALL_GATHER ? "" : ".", c.kind == dvmb::COLL_ALL_GATHER ? "" : ops[c.reduce_type],
               DTypeName(static_cast<DataType>(c.dtype)), static_cast<unsigned long long>(c.count), c.comm ? c.comm->rank : 0,
               c.comm ? c.comm->size : 1, static_cast<unsigned long long>(c.wire_bytes), names[c.kind],
               static_cast<unsigned long long>(c.recv_ptr), static_cast<unsigned long long>(c.send_ptr));
      text_ += buf;
    } else if (st->kind == STAGE_ATTENTION) {
      const dvmb::AttnParam &a = st->attn.param;
      char buf[256];
      snprintf(buf, sizeof(buf), "amain.sm100(batch=%u, sq=%u, skv=%u, d=%u, %s) {\n  attention 0x%llx, load(0x%llx), load(0x%llx), load(0x%llx)\n}\n",
               a.batch, a.sq, a.skv, a.d, DTypeName(static_cast<DataType>(a.dtype)), static_cast<unsigned long long>(a.o_ptr),
               static_cast<unsigned long long>(a.q_ptr), static_cast<unsigned long long>(a.k_ptr),
               static_cast<unsigned long long>(a.v_ptr));
      text_ += buf;
    } else {
      text_ += DisassembleStage(st->vec);
    }
  }
  return text_.c_str();
}

const char *VKernel::Inspect() {
  if (!compiled_) Compile();
  char buf[256];
  text_.clear();
  int i = 0;
  for (auto &stp : stages_) {
    if (stp->kind == STAGE_MATMUL) {
      snprintf(buf, sizeof(buf), "stage %d: matmul flops=%llu algorithmic_bytes=%llu%s\n", i++,
               static_cast<unsigned long long>(stp->mm.flops), static_cast<unsigned long long>(stp->mm.algo_bytes),
               stp->mm.idle ? " (idle: zero-size result)" : "");
    } else if (stp->kind == STAGE_COLLECTIVE) {
      snprintf(buf, sizeof(buf), "stage %d: collective kind=%u count=%llu wire_bytes=%llu\n", i++, stp->coll.kind,
               static_cast<unsigned long long>(stp->coll.count), static_cast<unsigned long long>(stp->coll.wire_bytes));
    } else if (stp->kind == STAGE_ATTENTION) {
      snprintf(buf, sizeof(buf), "stage %d: attention flops=%llu algorithmic_bytes=%llu\n", i++,
               static_cast<unsigned long long>(stp->attn.flops), static_cast<unsigned long long>(stp->attn.algo_bytes));
    } else {
      VectorStage &st = stp->vec;
      snprintf(buf, sizeof(buf), "stage %d: grid=%u threads=%u code_words=%u tensors=%u algorithmic_bytes=%llu%s\n", i++,
               st.grid, st.threads, st.param.n_code, st.param.n_tensors, static_cast<unsigned long long>(st.algo_bytes),
               st.idle ? " (idle: zero-size domain)" : "");
    }
    text_ += buf;
  }
  snprintf(buf, sizeof(buf), "workspace_bytes=%zu last_jit_us=%.2f\n", ws_bytes_, last_jit_us_);
  text_ += buf;
  return text_.c_str();
}

}  // namespace dvm
