// Host JIT for one fused vector stage: operator list -> VmParam (geometry, tensor table, bytecode).
//
// This is the new-backend counterpart of the reference's vector scheduling and emission path
// (VectorKernel::BuildDomain/ShapeTiling/ApplyTiling src/kernel.cc:765-1194, GPU CodeGenHelper::Generate
// src/kernel.cc:206-257, op emitters src/ops.cc:769-3171).  The strategy is different: instead of tiling
// into shared-memory slots, every op of the stage is evaluated over one iteration domain by an
// accumulator machine held in registers; reductions split the program into phases and values needed
// after a reduction are recomputed from the (cache-resident) inputs instead of being parked on chip.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>
#include <unordered_map>

#include "graph.h"
#include "runtime.h"
#include "vm_launch.h"

namespace dvm {

void LowerStage(VectorStage *st);

uint32_t EncodeScalarRefNow(const ScalarRef *ref, DataType dtype);

namespace {

using namespace dvmb;

struct Fail {
  std::string why;
};

bool IsIntRepr(DataType t) { return t == kInt32 || t == kBool; }

struct Info {
  int axis[kMaxRank];        // domain axis of each API dim
  int64_t asz[kMaxRank];     // size per domain axis (1 where absent or broadcast)
  bool scalar_space = false;
  int level = 0;
  NDObject *canon = nullptr;  // value this node aliases (itself for real ops)
  int slot = -1;              // tensor slot (loads / stores)
  int rslot = -1;             // reduce partial slot
  int sreg = -1;              // scalar register while live
  int last_section = -1;      // last section index reading this scalar-space value
};

enum LocKind { L_NONE, L_ACC, L_REG, L_IMM };

struct Compiler {
  const std::vector<NDObject *> &ops;
  VectorStage *out;
  std::vector<Info> info;
  int R = 0;                       // domain rank
  int64_t dom[kMaxRank];
  bool reduced[kMaxRank];
  bool has_reduce = false;
  // A reduce-free graph over more iterated axes than a tile walks (kMaxEnum after coalescing, e.g. a 5-d window of a
  // larger tensor) is run like a reduction's: its outer axes become group axes (forced_outer) and the tile walks the
  // rest.  There is no reduction, so the groups only serve as the outer loop.
  bool forced_outer[kMaxRank] = {false};
  int num_forced_outer = 0;
  std::vector<int> kept_axes, enum_axes;   // domain axes, outer -> inner
  // coalesced geometry
  struct CoAxis {
    int64_t size;
    std::vector<int> members;   // domain axes merged into this one (outer -> inner)
  };
  std::vector<CoAxis> ckept, cenum;
  int num_body = 0;
  std::vector<uint64_t> code;
  std::vector<NDObject *> slot_nodes;
  int max_temp = 0, max_sreg = 0;
  uint32_t body_tensor_mask[kMaxPhases] = {0, 0, 0, 0};   // tensor slots each BODY reads as operands
  // nodes whose value can reach an op of the exact class (compare, select condition, cast to int / bool, rounding,
  // IsFinite): those keep IEEE division and the accurate exp; every other float value may use the fast forms,
  // whose error (2 ulp / about 1e-6 relative) is far inside the fp32 tolerance of the path
  std::vector<char> exact;
  bool epilogue = false;           // compiling the post-fusion program of a MatMul stage
  const NDObject *mma_src = nullptr;

  void NoteTensorUse(int section, int slot) {
    if (section & 1) body_tensor_mask[section / 2] |= 1u << slot;
  }

  Compiler(const std::vector<NDObject *> &o, VectorStage *st) : ops(o), out(st) {}

  int IndexOf(const NDObject *n) const {
    if (n->cidx < 0 || static_cast<size_t>(n->cidx) >= ops.size() || ops[n->cidx] != n) throw Fail{"internal: node outside the stage"};
    return n->cidx;
  }
  Info &I(const NDObject *n) { return info[IndexOf(n)]; }

  // ---- step 1: align every node's dims to domain axes -------------------------------------------
  void AlignAxes() {
    R = 0;
    for (auto n : ops) R = std::max(R, n->shape.rank);
    if (R > kMaxRank) throw Fail{"domain rank above 10"};
    for (auto n : ops) {
      Info &fi = I(n);
      const int r = n->shape.rank;
      auto right_align = [&]() {
        for (int i = 0; i < r; ++i) fi.axis[i] = R - r + i;
      };
      switch (n->kind) {
        case N_LOAD:
        case N_BROADCAST_S: right_align(); break;
        case N_REDUCE: {
          const NDObject *src = n->in[0];
          const Info &si = I(src);
          bool red[kMaxRank] = {false};
          for (size_t i = 0; i < n->shape_ref->size; ++i) {
            int64_t d = n->shape_ref->data[i];
            if (d < 0) d += src->shape.rank;
            red[d] = true;
          }
          int o = 0;
          for (int i = 0; i < src->shape.rank; ++i) {
            if (red[i] && !n->keepdims) continue;
            fi.axis[o++] = si.axis[i];
          }
          break;
        }
        case N_RESHAPE: {
          // Supported in-stage only when it inserts or removes unit dims: non-unit dims keep their axes.
          const NDObject *src = n->in[0];
          const Info &si = I(src);
          std::vector<int> src_axes;
          std::vector<int64_t> src_sizes;
          for (int i = 0; i < src->shape.rank; ++i)
            if (src->shape.d[i] != 1) {
              src_axes.push_back(si.axis[i]);
              src_sizes.push_back(src->shape.d[i]);
            }
          size_t j = 0;
          right_align();
          // unit dims of the result sit on their right-aligned axis only if that axis is not claimed
          for (int i = 0; i < r; ++i) {
            if (n->shape.d[i] == 1) continue;
            if (j >= src_axes.size() || src_sizes[j] != n->shape.d[i]) throw Fail{"general reshape inside a stage"};
            fi.axis[i] = src_axes[j++];
          }
          if (j != src_axes.size()) throw Fail{"general reshape inside a stage"};
          // give unit dims any axis that keeps the list strictly increasing; fall back to -1 (ignored)
          for (int i = 0; i < r; ++i)
            if (n->shape.d[i] == 1) fi.axis[i] = -1;
          break;
        }
        case N_BROADCAST: {
          const NDObject *src = n->in[0];
          const Info &si = I(src);
          right_align();
          for (int i = 0; i < src->shape.rank; ++i) {
            int oi = i + (r - src->shape.rank);
            if (si.axis[i] >= 0) fi.axis[oi] = si.axis[i];
          }
          break;
        }
        case N_BINARY:
        case N_COMPARE:
        case N_SELECT: {
          right_align();
          bool fixed[kMaxRank] = {false};
          int nin = n->kind == N_SELECT ? 3 : 2;
          for (int k = 0; k < nin; ++k) {
            NDObject *src = n->in[k];
            Info &si = I(src);
            const int sr = src->shape.rank;
            for (int i = 0; i < sr; ++i) {
              int oi = i + (r - sr);
              if (src->shape.d[i] == 1 || si.axis[i] < 0) continue;
              if (!fixed[oi]) {
                fi.axis[oi] = si.axis[i];
                fixed[oi] = true;
              } else if (fi.axis[oi] != si.axis[i]) {
                // a plain input can simply be re-anchored onto the axes its partner uses
                if (src->kind == N_LOAD || src->kind == N_BROADCAST_S) {
                  si.axis[i] = fi.axis[oi];
                } else {
                  throw Fail{"operands iterate different axes"};
                }
              }
            }
          }
          break;
        }
        default: {
          const Info &si = I(n->in[0]);
          for (int i = 0; i < r; ++i) fi.axis[i] = si.axis[i];
          break;
        }
      }
      // two dims of one value on the same axis: a reshape moved a dim across its partner's position, which only a
      // view of memory can express (the planner then gives the reshape a stage boundary)
      for (int i = 0; i < r; ++i)
        for (int j = i + 1; j < r; ++j)
          if (fi.axis[i] >= 0 && fi.axis[i] == fi.axis[j] && n->shape.d[i] != 1 && n->shape.d[j] != 1)
            throw Fail{"general reshape inside a stage"};
    }
    // domain sizes
    for (int a = 0; a < R; ++a) dom[a] = 1;
    for (auto n : ops) {
      Info &fi = I(n);
      for (int a = 0; a < R; ++a) fi.asz[a] = 1;
      for (int i = 0; i < n->shape.rank; ++i) {
        int a = fi.axis[i];
        if (a < 0) continue;
        if (a >= R) throw Fail{"axis out of range"};
        if (n->shape.d[i] != 1) {
          fi.asz[a] = n->shape.d[i];
          if (dom[a] != 1 && dom[a] != n->shape.d[i]) throw Fail{"ops disagree on a domain extent"};
          dom[a] = n->shape.d[i];
        }
      }
    }
  }

  // ---- step 2: reductions, spaces, levels ---------------------------------------------------------
  void Classify() {
    for (int a = 0; a < R; ++a) reduced[a] = false;
    bool first = true;
    for (auto n : ops) {
      if (n->kind != N_REDUCE) continue;
      if (epilogue) throw Fail{"reduction inside a MatMul epilogue"};
      const NDObject *src = n->in[0];
      const Info &si = I(src);
      bool mine[kMaxRank] = {false};
      for (size_t i = 0; i < n->shape_ref->size; ++i) {
        int64_t d = n->shape_ref->data[i];
        if (d < 0) d += src->shape.rank;
        int a = si.axis[d];
        if (a >= 0 && dom[a] != 1) mine[a] = true;
      }
      if (first) {
        for (int a = 0; a < R; ++a) reduced[a] = mine[a];
        first = false;
      } else {
        for (int a = 0; a < R; ++a)
          if (reduced[a] != mine[a]) throw Fail{"reductions over different axes in one stage"};
      }
      has_reduce = true;
    }
    if (!has_reduce && num_forced_outer > 0) {
      has_reduce = true;
      for (int a = 0; a < R; ++a) reduced[a] = !forced_outer[a];
    }
    int nred = 0;
    for (int a = 0; a < R; ++a) nred += reduced[a] ? 1 : 0;
    if (has_reduce && nred == 0) has_reduce = false;   // every reduced axis has extent 1: plain copies
    for (auto n : ops) {
      Info &fi = I(n);
      bool varies = false;
      for (int a = 0; a < R; ++a) {
        if (fi.asz[a] == 1) continue;
        if (!has_reduce || reduced[a]) varies = true;
      }
      fi.scalar_space = epilogue ? false : !varies;
      // canonical value
      fi.canon = n;
      switch (n->kind) {
        case N_BROADCAST:
        case N_RESHAPE:
        case N_COPY: fi.canon = I(n->in[0]).canon; break;
        case N_CAST:
          if ((n->in[0]->dtype == kFloat16 || n->in[0]->dtype == kBFloat16) && n->dtype == kFloat32)
            fi.canon = I(n->in[0]).canon;
          break;
        case N_REDUCE:
          if (!has_reduce) fi.canon = I(n->in[0]).canon;
          break;
        default: break;
      }
      int lvl = 0;
      for (int k = 0; k < 3; ++k)
        if (n->in[k]) lvl = std::max(lvl, I(n->in[k]).level);
      if (n->kind == N_REDUCE && has_reduce) {
        if (I(n->in[0]).scalar_space) throw Fail{"reduction of a value that does not vary along the reduced axes"};
        lvl += 1;
      }
      fi.level = lvl;
      if (n->kind == N_REDUCE && has_reduce && !fi.scalar_space) throw Fail{"partial reduction result is not group-constant"};
    }
  }

  void MarkExact() {
    exact.assign(ops.size(), 0);
    static const bool off = getenv("DVM_B200_EXACT_MATH") != nullptr;
    if (off) {
      exact.assign(ops.size(), 1);
      return;
    }
    for (size_t i = ops.size(); i-- > 0;) {
      const NDObject *n = ops[i];
      bool sink = false;   // this op needs exact inputs
      switch (n->kind) {
        case N_COMPARE:
        case N_COMPARE_S: sink = true; break;
        case N_CAST: sink = IsIntRepr(n->dtype); break;
        case N_UNARY: sink = n->sub == kIsFinite || n->sub >= kRound; break;
        default: break;
      }
      for (int k = 0; k < 3; ++k) {
        if (!n->in[k]) continue;
        const bool cond = n->kind == N_SELECT && k == 0;
        if (sink || cond || exact[i]) exact[IndexOf(n->in[k])] = 1;
      }
    }
  }

  // ---- step 3: geometry ---------------------------------------------------------------------------
  // Element stride of tensor node `n` (contiguous in its own API shape) along domain axis `a`.
  int64_t StrideOn(const NDObject *n, int a) {
    const Info &fi = I(n);
    if (n->strided) {   // a view: the strides the caller gave
      for (int i = n->shape.rank - 1; i >= 0; --i)
        if (fi.axis[i] == a && n->shape.d[i] != 1) return n->stride[i];
      return 0;
    }
    int64_t st = 1;
    for (int i = n->shape.rank - 1; i >= 0; --i) {
      if (fi.axis[i] == a && n->shape.d[i] != 1) return st;
      st *= n->shape.d[i];
    }
    return 0;
  }

  void Coalesce(const std::vector<int> &axes, std::vector<CoAxis> *outv, bool vector_only) {
    outv->clear();
    for (int a : axes) {
      if (dom[a] == 1) continue;
      if (!outv->empty()) {
        CoAxis &prev = outv->back();
        int pa = prev.members.back();   // innermost member of the previous (outer) group
        bool ok = true;
        for (auto n : slot_nodes) {
          if (vector_only && I(n).scalar_space) continue;
          // merging requires stride(outer) == stride(inner) * size(inner) for every tensor
          int64_t so = StrideOn(n, pa), si = StrideOn(n, a);
          if (so != si * dom[a]) {
            ok = false;
            break;
          }
        }
        if (ok) {
          prev.size *= dom[a];
          prev.members.push_back(a);
          continue;
        }
      }
      outv->push_back(CoAxis{dom[a], {a}});
    }
  }

  void Geometry() {
    for (auto n : ops)
      if (n->kind == N_LOAD || n->kind == N_STORE) {
        I(n).slot = static_cast<int>(slot_nodes.size());
        slot_nodes.push_back(n);
      }
    if (slot_nodes.size() > static_cast<size_t>(kMaxTensors)) throw Fail{"more than 16 tensors in one stage"};
    if (epilogue) return;
    kept_axes.clear();
    enum_axes.clear();
    for (int a = 0; a < R; ++a) {
      if (has_reduce && !reduced[a]) {
        kept_axes.push_back(a);
      } else {
        enum_axes.push_back(a);
      }
    }
    Coalesce(kept_axes, &ckept, false);
    Coalesce(enum_axes, &cenum, true);
    if (ckept.size() > static_cast<size_t>(kMaxKept)) throw Fail{"more than 3 kept axes after coalescing"};
    if (cenum.size() > static_cast<size_t>(kMaxEnum)) throw Fail{"more than 4 iterated axes after coalescing"};
  }

  // ---- step 4: code emission ----------------------------------------------------------------------
  uint32_t RoundOf(const NDObject *n) {
    return n->dtype == kFloat16 ? RN_F16 : (n->dtype == kBFloat16 ? RN_BF16 : RN_NONE);
  }

  uint32_t ScalarBits(const NDObject *n) {
    return n->scalar_ref ? EncodeScalarRefNow(n->scalar_ref, n->dtype) : n->scalar_bits;
  }

  struct Operand {
    uint32_t kind, idx, imm;
  };

  // One section's accumulator-machine emitter.  Vector side: values live in acc / vregs for the section
  // only.  Scalar side: values live in sacc / sregs and persist across sections (Info::sreg).
  struct Side {
    Compiler *c;
    bool scalar;
    int section;
    const NDObject *acc_val = nullptr;
    std::vector<const NDObject *> reg_val;
    std::vector<int> uses_;      // by node position: remaining uses inside this section
    std::vector<int> vreg_of_;   // by node position: register holding the value, or -1 (vector side only)
    int &uses(const NDObject *v) {
      if (uses_.empty()) uses_.assign(c->ops.size(), 0);
      return uses_[c->IndexOf(v)];
    }
    int &vreg_of(const NDObject *v) {
      if (vreg_of_.empty()) vreg_of_.assign(c->ops.size(), -1);
      return vreg_of_[c->IndexOf(v)];
    }

    void Push(uint32_t opc, uint32_t sub, Operand o, uint32_t dst, uint32_t rnd, uint32_t isint) {
      c->code.push_back(Insn::make(opc, sub, o.kind, o.idx, dst, rnd, isint, scalar ? 1 : 0, o.imm));
    }
    void Push0(uint32_t opc, uint32_t sub, uint32_t dst = 0, uint32_t rnd = 0, uint32_t isint = 0) {
      Push(opc, sub, Operand{0, 0, 0}, dst, rnd, isint);
    }

    int RegOf(const NDObject *v) {
      if (scalar) return c->I(v).sreg;
      return vreg_of(v);
    }

    bool NeededLater(const NDObject *v) {
      if (uses(v) > 0) return true;
      if (scalar && c->I(v).last_section > section) return true;
      return false;
    }

    int AllocReg(const NDObject *v) {
      const int n = scalar ? kNumSRegs : kNumTemps;
      if (static_cast<int>(reg_val.size()) < n) reg_val.resize(n, nullptr);
      for (int i = 0; i < n; ++i) {
        if (reg_val[i] == nullptr) {
          reg_val[i] = v;
          if (scalar) {
            c->I(v).sreg = i;
            c->max_sreg = std::max(c->max_sreg, i + 1);
          } else {
            vreg_of(v) = i;
            c->max_temp = std::max(c->max_temp, i + 1);
          }
          return i;
        }
      }
      throw Fail{scalar ? "out of scalar registers" : "out of vector registers"};
    }

    void FreeIfDead(const NDObject *v) {
      if (NeededLater(v)) return;
      int r = RegOf(v);
      if (r >= 0) {
        reg_val[r] = nullptr;
        if (scalar) {
          c->I(v).sreg = -1;
        } else {
          vreg_of(v) = -1;
        }
      }
    }

    // Keep the accumulator's value alive in a register if something still needs it.
    void SaveAcc() {
      if (acc_val == nullptr) return;
      if (RegOf(acc_val) >= 0) return;
      if (!scalar && acc_val->kind == N_LOAD) return;   // an input is simply read again where it lives
      if (!NeededLater(acc_val)) return;
      int r = AllocReg(acc_val);
      Push0(OP_MOV, 0, r);
    }

    // The accumulator is about to be overwritten by an op that reads it: park its value if later ops
    // still need it (call after Consume()).
    void ParkAccIfNeeded() { SaveAcc(); }

    int AllocTemp() {
      const int n = scalar ? kNumSRegs : kNumTemps;
      if (static_cast<int>(reg_val.size()) < n) reg_val.resize(n, nullptr);
      static const NDObject kTempMarker{};
      for (int i = 0; i < n; ++i)
        if (reg_val[i] == nullptr) {
          reg_val[i] = &kTempMarker;
          if (scalar) c->max_sreg = std::max(c->max_sreg, i + 1); else c->max_temp = std::max(c->max_temp, i + 1);
          return i;
        }
      throw Fail{scalar ? "out of scalar registers" : "out of vector registers"};
    }
    void FreeTemp(int r) { reg_val[r] = nullptr; }

    // Location of a value as a non-accumulator operand.  Inputs are read in place: a tensor operand names
    // the tensor slot (the interpreter takes it from the shared-memory ring or from global memory).
    Operand OperandOf(const NDObject *v) {
      if (v->kind == N_BROADCAST_S) return Operand{K_IMM, 0, c->ScalarBits(v)};
      const Info &vi = c->I(v);
      if (!scalar && vi.scalar_space) {
        if (vi.sreg < 0) throw Fail{"internal: group-constant value has no scalar register"};
        return Operand{K_SREG, static_cast<uint32_t>(vi.sreg), 0};
      }
      int r = RegOf(v);
      if (r >= 0) return Operand{scalar ? K_SREG : K_TEMP, static_cast<uint32_t>(r), 0};
      if (acc_val == v) return Operand{K_ACC, 0, 0};
      if (v->kind == N_LOAD) {
        c->NoteTensorUse(section, vi.slot);
        return Operand{K_TENSOR, static_cast<uint32_t>(vi.slot), 0};
      }
      throw Fail{"internal: operand value is not available"};
    }

    // Bring `v` into the accumulator.
    void ToAcc(const NDObject *v) {
      if (acc_val == v) return;
      SaveAcc();
      Operand o = OperandOf(v);
      Push(OP_COPY, 0, o, 0, 0, 0);
      acc_val = v;
    }

    void Consume(const NDObject *v) {
      if (uses(v) > 0) --uses(v);
    }

    void Release(const NDObject *v) {
      if (v->kind == N_BROADCAST_S) return;
      if (!scalar && c->I(v).scalar_space) return;
      FreeIfDead(v);
    }
  };

  const NDObject *Canon(const NDObject *n) { return I(n).canon; }

  // Emit the computation of canonical node `n` on `s`; the value ends in the accumulator.
  // Protocol: operands are located (loading inputs on demand) while their use counts still include
  // this op, so anything the accumulator must give up is parked in a register first; then the uses are
  // consumed, the accumulator operand is parked if later ops still read it, and the op is pushed.
  void EmitNode(Side &s, const NDObject *n) {
    const uint32_t rnd = RoundOf(n);
    const bool isint = IsIntRepr(n->dtype);
    auto finish_unary_like = [&](const NDObject *x) {
      s.Consume(x);
      s.ParkAccIfNeeded();
    };
    switch (n->kind) {
      case N_LOAD:
      case N_BROADCAST_S: return;   // fetched on demand / immediate
      case N_UNARY: {
        const NDObject *x = Canon(n->in[0]);
        s.ToAcc(x);
        finish_unary_like(x);
        static const uint32_t map[] = {U_SQRT, U_ABS, U_LOG, U_EXP, U_NOP, U_ISFINITE, U_NOP, U_ROUND, U_FLOOR, U_CEIL, U_TRUNC};
        uint32_t kind = map[n->sub];
        if (n->sub == kAbs && isint) kind = U_ABS_I;
        if (kind == U_EXP && !exact[IndexOf(n)]) kind = U_EXP_FAST;
        const bool noround = n->sub == kAbs || n->sub == kIsFinite || n->sub >= kRound;
        s.Push0(OP_UN, kind, 0, noround ? RN_NONE : rnd);
        s.acc_val = n;
        s.Release(x);
        return;
      }
      case N_CAST: {
        const NDObject *x = Canon(n->in[0]);
        s.ToAcc(x);
        finish_unary_like(x);
        const DataType from = n->in[0]->dtype, to = n->dtype;
        const bool from_int = IsIntRepr(from), to_int = IsIntRepr(to);
        uint32_t kind = V_RND, r = RN_NONE;
        if (to == kBool) {
          kind = from_int ? V_NEZ_I : V_NEZ_F;
        } else if (from_int && !to_int) {
          kind = V_I2F;
          r = rnd;
        } else if (!from_int && to_int) {
          kind = V_F2I;
        } else if (!from_int) {
          r = rnd;   // float narrowing; bool -> int32 keeps its bits
        }
        s.Push0(OP_CVT, kind, 0, r);
        s.acc_val = n;
        s.Release(x);
        return;
      }
      case N_BINARY_S:
      case N_COMPARE_S: {
        const NDObject *x = Canon(n->in[0]);
        s.ToAcc(x);
        finish_unary_like(x);
        Operand o{K_IMM, 0, ScalarBits(n)};
        if (n->kind == N_COMPARE_S) {
          s.Push(OP_CMP, n->sub, o, 0, 0, isint);
        } else {
          static const uint32_t fmap[] = {B_ADD, B_MUL, B_DIV, B_RDIV, B_MAX, B_MIN};
          static const uint32_t imap[] = {B_ADD_I, B_MUL_I, B_COUNT, B_COUNT, B_MAX_I, B_MIN_I};
          uint32_t kind = isint ? imap[n->sub] : fmap[n->sub];
          if (kind == B_COUNT) throw Fail{"integer division is not supported"};
          if (!exact[IndexOf(n)]) kind = kind == B_DIV ? B_DIV_FAST : (kind == B_RDIV ? B_RDIV_FAST : kind);
          const bool noround = n->sub == SB_MAX || n->sub == SB_MIN;
          s.Push(OP_BIN, kind, o, 0, noround ? RN_NONE : rnd, 0);
        }
        s.acc_val = n;
        s.Release(x);
        return;
      }
      case N_BINARY:
      case N_COMPARE: {
        const NDObject *x = Canon(n->in[0]);
        const NDObject *y = Canon(n->in[1]);
        uint32_t kind = 0, rkind = B_COUNT;   // rkind: the same op with its operands swapped
        bool noround = false;
        if (n->kind == N_BINARY) {
          switch (n->sub) {
            case kAdd: kind = rkind = isint ? B_ADD_I : B_ADD; break;
            case kMul: kind = rkind = isint ? B_MUL_I : B_MUL; break;
            case kSub: kind = isint ? B_SUB_I : B_SUB; rkind = isint ? B_RSUB_I : B_RSUB; break;
            case kDiv:
              if (isint) throw Fail{"integer division is not supported"};
              kind = B_DIV; rkind = B_RDIV;
              if (!exact[IndexOf(n)]) { kind = B_DIV_FAST; rkind = B_RDIV_FAST; }
              break;
            case kPow:
              if (isint) throw Fail{"integer pow is not supported"};
              kind = B_POW; break;
            // float max/min are `a > b ? a : b`: not symmetric for NaN and signed zero, so never mirrored
            case kMaximum: case kLogicalOr: kind = isint ? B_MAX_I : B_MAX; noround = true; if (isint) rkind = kind; break;
            case kMinimum: case kLogicalAnd: kind = isint ? B_MIN_I : B_MIN; noround = true; if (isint) rkind = kind; break;
            default: throw Fail{"unknown binary op"};
          }
        } else {
          static const uint32_t mirrored[] = {C_EQ, C_NE, C_LT, C_LE, C_GT, C_GE};
          kind = n->sub;
          rkind = mirrored[n->sub];
        }
        Operand o;
        bool swapped = false;
        if (x == y) {
          s.ToAcc(x);
          o = Operand{K_ACC, 0, 0};
        } else if (s.acc_val == y && rkind != B_COUNT) {
          swapped = true;
          o = s.OperandOf(x);
        } else {
          s.ToAcc(x);          // parks y first if y sat in the accumulator
          o = s.OperandOf(y);
        }
        s.Consume(x);
        s.Consume(y);
        s.ParkAccIfNeeded();
        if (n->kind == N_COMPARE) {
          s.Push(OP_CMP, swapped ? rkind : kind, o, 0, 0, IsIntRepr(n->in[0]->dtype));
        } else {
          s.Push(OP_BIN, swapped ? rkind : kind, o, 0, noround ? RN_NONE : rnd, 0);
        }
        s.acc_val = n;
        s.Release(x);
        if (y != x) s.Release(y);
        return;
      }
      case N_SELECT: {
        const NDObject *cnd = Canon(n->in[0]);
        const NDObject *a = Canon(n->in[1]);
        const NDObject *b = Canon(n->in[2]);
        // The instruction takes one free-form operand (register / scalar / immediate / accumulator) and
        // one register-or-scalar operand; `inv` makes the free-form one the "false" alternative.
        auto reg_like = [&](const NDObject *v) {
          if (v->kind == N_BROADCAST_S) return false;
          if (!s.scalar && I(v).scalar_space) return true;
          if (s.scalar && v->kind == N_LOAD) return false;   // the scalar side reads tensors only as the free operand
          return v != cnd;   // anything else sits in (or can be given) a register, or is an input read in place
        };
        bool inv = false;
        const NDObject *free_v = a, *reg_v = b;
        if (!reg_like(b)) {
          if (!reg_like(a)) {
            // both alternatives are immediates (or the condition itself): materialise b in a register
            s.SaveAcc();
            s.Push(OP_COPY, 0, s.OperandOf(b), 0, 0, 0);
            int r = s.AllocTemp();
            s.Push0(OP_MOV, 0, r);
            s.acc_val = nullptr;
            s.ToAcc(cnd);
            Operand oa = a == cnd ? Operand{K_ACC, 0, 0} : s.OperandOf(a);
            s.Consume(cnd); s.Consume(a); s.Consume(b);
            s.ParkAccIfNeeded();
            s.Push(OP_SEL, ((s.scalar ? K_SREG : K_TEMP) << 4) | r, oa, 0, 0, IsIntRepr(n->in[0]->dtype));
            s.FreeTemp(r);
            s.acc_val = n;
            s.Release(cnd); s.Release(a); s.Release(b);
            return;
          }
          inv = true;
          free_v = b;
          reg_v = a;
        }
        // reg_v needs a register (or scalar register) location before the condition takes the accumulator
        if (s.acc_val == reg_v && s.RegOf(reg_v) < 0 && !(!s.scalar && I(reg_v).scalar_space)) {
          int r = s.AllocReg(reg_v);
          s.Push0(OP_MOV, 0, r);
        }
        Operand orr = s.OperandOf(reg_v);
        s.ToAcc(cnd);
        if (orr.kind == K_ACC) throw Fail{"internal: select alternative lost its register"};
        Operand of = free_v == cnd ? Operand{K_ACC, 0, 0} : s.OperandOf(free_v);
        s.Consume(cnd); s.Consume(a); s.Consume(b);
        s.ParkAccIfNeeded();
        s.Push(OP_SEL, (orr.kind << 4) | orr.idx, of, inv ? 1 : 0, 0, IsIntRepr(n->in[0]->dtype));
        s.acc_val = n;
        s.Release(cnd); s.Release(a); s.Release(b);
        return;
      }
      default: throw Fail{"op kind cannot run inside a vector stage"};
    }
  }

  // Nodes (canonical, in program order) the vector body of level `q` must evaluate.
  std::vector<const NDObject *> BodyNeeds(int q, std::vector<const NDObject *> *roots) {
    std::vector<char> need(ops.size(), 0);
    roots->clear();
    for (auto n : ops) {
      if (n->kind == N_STORE && !I(n).scalar_space && I(n).level == q) roots->push_back(n);
      if (n->kind == N_REDUCE && has_reduce && I(n->in[0]).level == q) roots->push_back(n);
    }
    std::vector<const NDObject *> stack;
    for (auto r : *roots) stack.push_back(Canon(r->in[0]));
    while (!stack.empty()) {
      const NDObject *v = stack.back();
      stack.pop_back();
      if (I(v).scalar_space || v->kind == N_BROADCAST_S) continue;
      int idx = IndexOf(v);
      if (need[idx]) continue;
      need[idx] = 1;
      for (int k = 0; k < 3; ++k)
        if (v->in[k]) stack.push_back(Canon(v->in[k]));
    }
    std::vector<const NDObject *> order;
    for (size_t i = 0; i < ops.size(); ++i)
      if (need[i]) order.push_back(ops[i]);
    return order;
  }

  void CountUses(Side &s, const std::vector<const NDObject *> &order, const std::vector<const NDObject *> &roots) {
    for (auto v : order)
      for (int k = 0; k < 3; ++k)
        if (v->in[k]) s.uses(Canon(v->in[k]))++;
    for (auto r : roots) s.uses(Canon(r->in[0]))++;
  }

  void Emit() {
    // levels present
    int max_vec_level = -1, max_level = 0;
    for (auto n : ops) {
      const Info &fi = I(n);
      max_level = std::max(max_level, fi.level);
      if (n->kind == N_STORE && !fi.scalar_space) max_vec_level = std::max(max_vec_level, fi.level);
      if (n->kind == N_REDUCE && has_reduce) max_vec_level = std::max(max_vec_level, I(n->in[0]).level);
    }
    num_body = max_vec_level + 1;
    if (num_body > kMaxPhases) throw Fail{"more than 4 dependent reduction phases"};
    // reduce slots
    int nslots = 0;
    for (auto n : ops)
      if (n->kind == N_REDUCE && has_reduce) {
        if (nslots >= kNumRSlots) throw Fail{"more than 4 reductions in one stage"};
        I(n).rslot = nslots++;
      }
    // body plans first: they define how long group-constant values must stay in scalar registers
    std::vector<std::vector<const NDObject *>> body_order(num_body), body_roots(num_body);
    for (int q = 0; q < num_body; ++q) body_order[q] = BodyNeeds(q, &body_roots[q]);
    auto touch = [&](const NDObject *v, int section) {
      Info &vi = I(v);
      if (vi.scalar_space) vi.last_section = std::max(vi.last_section, section);
    };
    for (int q = 0; q < num_body; ++q) {
      for (auto v : body_order[q])
        for (int k = 0; k < 3; ++k)
          if (v->in[k]) touch(Canon(v->in[k]), 2 * q + 1);
      for (auto r : body_roots[q]) touch(Canon(r->in[0]), 2 * q + 1);
    }
    // scalar-side plans
    if (max_level > num_body) throw Fail{"internal: scalar work beyond the last phase"};
    const int num_pro = num_body + 1;
    std::vector<std::vector<const NDObject *>> pro_order(num_pro);
    int deferred_stores = 0;
    for (auto n : ops) {
      const Info &fi = I(n);
      if (!fi.scalar_space) continue;
      if (n->kind == N_STORE) {
        // A group scalar that is only stored (a mean, a variance) leaves for memory in the last scalar section instead
        // of the one that makes it: the section between two bodies is where every CTA of a normalisation waits at the
        // same time, and each store there costs two words and a global write in front of the next body.  (At most four
        // values wait this way: each keeps its scalar register until the end.)
        int at = fi.level;
        if (at < num_body && deferred_stores < 4) {
          at = num_body;
          ++deferred_stores;
        }
        pro_order[at].push_back(n);
        touch(Canon(n->in[0]), 2 * at);
        continue;
      }
      if (fi.canon != n || n->kind == N_BROADCAST_S) continue;
      pro_order[fi.level].push_back(n);
      if (n->kind == N_REDUCE) continue;
      for (int k = 0; k < 3; ++k)
        if (n->in[k]) touch(Canon(n->in[k]), 2 * fi.level);
    }
    // emit
    VmParam &P = out->param;
    std::vector<const NDObject *> sreg_val(kNumSRegs, nullptr);
    for (int p = 0; p <= num_body; ++p) {
      // ---- PRO_p
      out->bsec[2 * p] = static_cast<uint16_t>(code.size());
      Side ss{this, true, 2 * p};
      ss.reg_val = sreg_val;
      if (p == 0) {
        for (auto n : ops)
          if (n->kind == N_REDUCE && has_reduce) ss.Push0(OP_RINIT, I(n).rslot | (n->sub << 4));
      }
      // free scalar registers whose value is dead by now
      for (int i = 0; i < kNumSRegs; ++i)
        if (ss.reg_val[i] && I(ss.reg_val[i]).last_section < 2 * p) {
          I(ss.reg_val[i]).sreg = -1;
          ss.reg_val[i] = nullptr;
        }
      for (auto n : pro_order[p])
        for (int k = 0; k < 3; ++k)
          if (n->in[k] && n->kind != N_REDUCE) ss.uses(Canon(n->in[k]))++;
      for (auto n : pro_order[p]) {
        if (n->kind == N_STORE) {
          const NDObject *v = Canon(n->in[0]);
          ss.Consume(v);
          ss.ToAcc(v);
          ss.Push0(OP_ST, I(n).slot);
          ss.Release(v);
          continue;
        }
        if (n->kind == N_REDUCE) {
          ss.SaveAcc();
          ss.Push0(OP_RFIN, I(n).rslot | (n->sub << 4));
          ss.acc_val = n;
        } else if (n->kind == N_LOAD) {
          ss.ToAcc(n);
        } else {
          EmitNode(ss, n);
        }
        // a group-constant value read by a later section lives in a scalar register; values consumed
        // inside this section stay in the accumulator until something else needs it
        if (I(n).last_section > ss.section && ss.RegOf(n) < 0) {
          int r = ss.AllocReg(n);
          ss.Push0(OP_MOV, 0, r);
        }
      }
      ss.Push0(OP_END, 0);
      sreg_val = ss.reg_val;
      if (p == num_body) break;
      // ---- BODY_p
      out->bsec[2 * p + 1] = static_cast<uint16_t>(code.size());
      Side vs{this, false, 2 * p + 1};
      CountUses(vs, body_order[p], body_roots[p]);
      // roots are interleaved in program order: emit each as soon as its value exists
      std::vector<const NDObject *> pending = body_roots[p];
      auto flush_roots = [&](const NDObject *just_made) {
        for (auto &r : pending) {
          if (r == nullptr) continue;
          const NDObject *v = Canon(r->in[0]);
          if (v != just_made) continue;
          vs.Consume(v);
          vs.ToAcc(v);
          if (r->kind == N_STORE) {
            vs.Push0(OP_ST, I(r).slot);
          } else {
            vs.Push0(OP_RACC, I(r).rslot | (r->sub << 4));
          }
          vs.Release(v);
          r = nullptr;
        }
      };
      for (auto v : body_order[p]) {
        if (v->kind != N_LOAD && v->kind != N_BROADCAST_S) EmitNode(vs, v);
        flush_roots(v);
      }
      // roots fed by a constant or by a value of the scalar side (a `full`, a broadcast group scalar) have no body node
      for (size_t i = 0; i < pending.size(); ++i)
        if (pending[i] != nullptr) {
          const NDObject *v = Canon(pending[i]->in[0]);
          if (I(v).scalar_space || v->kind == N_BROADCAST_S) flush_roots(v);
        }
      for (auto r : pending)
        if (r != nullptr) throw Fail{"internal: a store or reduction lost its value"};
      vs.Push0(OP_END, 0);
    }
    if (code.size() > static_cast<size_t>(kMaxCodeWords)) throw Fail{"program exceeds the bytecode capacity"};
    // worst case of the lowered program: two micro-ops per operand-taking instruction plus a rounding one
    size_t worst = 0;
    for (uint64_t w : code) worst += DVMB_SCALAR(w) ? 1 : 4;
    if (worst > static_cast<size_t>(kMaxCodeWords)) throw Fail{"program exceeds the micro-op capacity"};
  }

  // ---- step 5: fill VmParam -----------------------------------------------------------------------
  void Fill() {
    VmParam &P = out->param;
    P.num_body = num_body;
    out->bytecode = code;
    int64_t K = 1, G = 1;
    for (auto &a : ckept) K *= a.size;
    for (auto &a : cenum) G *= a.size;
    if (G >= (1ll << 31) || K >= (1ll << 31)) throw Fail{"iteration domain above 2^31 elements"};
    for (int j = 0; j < kMaxKept; ++j) P.kept_size[j] = 1;
    for (int j = 0; j < kMaxEnum; ++j) P.enum_size[j] = 1;
    for (size_t j = 0; j < ckept.size(); ++j)
      P.kept_size[kMaxKept - ckept.size() + j] = static_cast<uint32_t>(ckept[j].size);
    for (size_t j = 0; j < cenum.size(); ++j)
      P.enum_size[kMaxEnum - cenum.size() + j] = static_cast<uint32_t>(cenum[j].size);
    P.num_groups = static_cast<uint32_t>(K);
    P.group_elems = static_cast<uint32_t>(G);
    const int sms = Runtime::Get().sm_count_or_default();
    bool zero = false;
    for (auto n : ops)
      if (n->shape.numel() == 0) zero = true;
    out->idle = zero;

    // ---- thread / chunk geometry
    const int64_t inner = cenum.empty() ? 1 : cenum.back().size;
    // elements of a chunk at most.  With enough groups to fill four CTAs per SM, half-size chunks (128 consumer threads
    // per CTA) run faster: four independent group pipelines per SM overlap each other's barriers and scalar sections
    // (measured 420 -> 345 us on 16384 rows of 4096); with few groups the large CTA keeps more threads on each group.
    uint32_t kChunkCap = kLanes * kVmFlatThreads;
    if (has_reduce && K >= 4ll * sms) kChunkCap /= 2;
    if (const char *env = getenv("DVM_B200_CHUNK_CAP")) kChunkCap = static_cast<uint32_t>(atoi(env));
    bool chunk_in_inner = false;   // every chunk lies inside one run of the innermost iterated axis
    bool packed = false;           // several small groups share a CTA
    if (!has_reduce) {
      P.mode = VM_FLAT;
      // enough chunks for four CTAs per SM: the 128-thread geometry (measured 139 -> 135 us on 2 x 256 MiB of fp32)
      P.tg = G >= 4ll * sms * (kLanes * kVmFlatThreads / 2) ? kVmFlatThreads / 2 : kVmFlatThreads;
      if (const char *env = getenv("DVM_B200_FLAT_THREADS")) P.tg = static_cast<uint32_t>(atoi(env));
      P.groups_per_cta = 1;
      P.chunk_elems = kLanes * P.tg;
      P.chunks = static_cast<uint32_t>((G + P.chunk_elems - 1) / P.chunk_elems);
      chunk_in_inner = cenum.size() <= 1 || (inner % P.chunk_elems == 0);
    } else {
      P.mode = VM_GROUP;
      if (G <= kLanes * 32) {
        uint32_t tg = 1;
        while (kLanes * tg < G) tg <<= 1;
        P.tg = tg;
        P.groups_per_cta = kVmFlatThreads / tg;
        P.chunk_elems = kLanes * tg;
        P.chunks = 1;
        packed = true;
      } else {
        P.groups_per_cta = 1;
        uint32_t ce = 0;
        if (cenum.size() >= 2 && inner % 4 == 0) {
          // cut the innermost axis into equal chunks so that a chunk never straddles two runs
          for (int64_t parts = (inner + kChunkCap - 1) / kChunkCap; parts <= inner / 32 && parts < 4096; ++parts)
            if (inner % parts == 0 && (inner / parts) % 8 == 0) {
              ce = static_cast<uint32_t>(inner / parts);
              break;
            }
        }
        if (ce != 0) {
          P.chunk_elems = ce;
          P.tg = (ce + kLanes - 1) / kLanes;   // every thread of the group holds 16 lanes of the chunk
          chunk_in_inner = true;
        } else {
          const uint32_t chunks = static_cast<uint32_t>((G + kChunkCap - 1) / kChunkCap);
          const uint32_t per = static_cast<uint32_t>((G + 1ll * kLanes * chunks - 1) / (1ll * kLanes * chunks));
          P.tg = (per + 31) / 32 * 32;
          P.chunk_elems = kLanes * P.tg;
          chunk_in_inner = cenum.size() <= 1;
        }
        P.chunks = static_cast<uint32_t>((G + P.chunk_elems - 1) / P.chunk_elems);
      }
    }
    // ---- rounds: a long group's chunk holds several rounds (the chunk sized so far), so that the per-chunk work of
    // the device loop (barrier waits, bookkeeping, the dispatch of single-micro-op bodies) is spread over more elements
    P.rounds = 1;
    P.round_elems = P.chunk_elems;
    // (only the kernels built with the larger register budget carry the round loop: CTAs of 161..256 threads, producer
    // warp included; the many-group geometry keeps its short chunks)
    static const bool no_r128 = getenv("DVM_B200_NO_R128") != nullptr;
    const uint32_t threads_planned = (P.tg * P.groups_per_cta + 31u) / 32u * 32u + 32u;
    if (P.mode == VM_GROUP && !packed && P.chunks >= 2 && K < 4ll * sms && threads_planned > 160 && threads_planned <= 256 && !no_r128) {
      uint64_t round_bytes = 0;
      uint32_t n_in = 0, reads = 0;
      for (int q = 0; q < num_body; ++q) reads |= body_tensor_mask[q];
      for (size_t sidx = 0; sidx < slot_nodes.size(); ++sidx)
        if (slot_nodes[sidx]->kind == N_LOAD && ((reads >> sidx) & 1u) && !I(slot_nodes[sidx]).scalar_space) {
          round_bytes += static_cast<uint64_t>(P.round_elems) * ItemSize(slot_nodes[sidx]->dtype);
          ++n_in;
        }
      uint32_t r = 1;
      // (one producer lane per staged tensor and round; two stages of up to 50 KB fit a CTA that shares its SM with
      // another one; measured on 256 groups of 64 x 6272 B, three passes: 165 us with 1 round per chunk, 133 with 2, 115
      // with 4, 107 with 8)
      while (r < 8 && 2 * r <= P.chunks && 2 * r * std::max(n_in, 1u) <= 32 && 2 * r * round_bytes <= 50u * 1024u) r *= 2;
      if (const char *env = getenv("DVM_B200_ROUNDS")) r = std::max(1, std::min(32 / static_cast<int>(std::max(n_in, 1u)), atoi(env)));
      P.rounds = r;
      P.chunk_elems = r * P.round_elems;
      P.chunks = static_cast<uint32_t>((G + P.chunk_elems - 1) / P.chunk_elems);
    }
    const uint32_t T = (P.tg * P.groups_per_cta + 31u) / 32u * 32u;
    P.tcons = T;

    // ---- tensors
    P.n_tensors = static_cast<uint32_t>(slot_nodes.size());
    P.need_coords = 0;
    out->slot_obj.assign(slot_nodes.begin(), slot_nodes.end());
    out->algo_bytes = 0;
    uint32_t stage_bytes = 0;
    struct RingPlace {
      uint32_t off, size, phases;
    };
    std::vector<RingPlace> ring_placed;
    uint32_t read_mask = 0;
    for (int q = 0; q < num_body; ++q) read_mask |= body_tensor_mask[q];
    for (size_t sidx = 0; sidx < slot_nodes.size(); ++sidx) {
      NDObject *n = slot_nodes[sidx];
      TensorDesc &td = P.tensor[sidx];
      std::memset(&td, 0, sizeof(td));
      td.ring_off = kNoRing;
      td.ptr = reinterpret_cast<uint64_t>(n->addr);
      td.dtype = static_cast<uint8_t>(n->dtype);
      if (n->dtype == kInt64) throw Fail{"int64 tensors are not supported by the vector interpreter"};
      if (n->shape.numel() >= (1ll << 31)) throw Fail{"tensor above 2^31 elements"};
      out->algo_bytes += static_cast<uint64_t>(n->shape.numel()) * ItemSize(n->dtype);
      const int isz = ItemSize(n->dtype);
      bool layout_vec = true, layout_bulk = true;
      for (size_t j = 0; j < ckept.size(); ++j) {
        int64_t st = StrideOn(n, ckept[j].members.back());
        td.kstride[kMaxKept - ckept.size() + j] = static_cast<uint32_t>(st);
        if (st % 4 != 0) layout_vec = false;
        if ((st * isz) % 16 != 0) layout_bulk = false;
      }
      if (I(n).scalar_space) {
        td.mode = AM_SCALAR;
        continue;
      }
      bool dense = true;
      int64_t expect = 1;
      for (int j = static_cast<int>(cenum.size()) - 1; j >= 0; --j) {
        int64_t st = StrideOn(n, cenum[j].members.back());
        td.estride[kMaxEnum - cenum.size() + j] = static_cast<uint32_t>(st);
        if (st != expect) dense = false;
        if (j != static_cast<int>(cenum.size()) - 1) {
          if (st % 4 != 0) layout_vec = false;
          if ((st * isz) % 16 != 0) layout_bulk = false;
        }
        expect *= cenum[j].size;
      }
      const int64_t inner_stride = cenum.empty() ? 1 : StrideOn(n, cenum.back().members.back());
      if (dense) {
        td.mode = AM_DENSE;
      } else if (inner % 4 == 0) {
        td.mode = AM_GRANULE;
        P.need_coords = 1;
      } else {
        td.mode = AM_ELEMENT;
        layout_vec = false;
      }
      if (inner_stride != 1) layout_vec = false;
      td.layout_vec = layout_vec ? 1 : 0;
      // bulk staging: the chunk must be one contiguous, 16-byte aligned run of this tensor
      const bool contiguous_chunk = inner_stride == 1 && (dense || (td.mode == AM_GRANULE && chunk_in_inner));
      td.chunk_contig = contiguous_chunk ? 1 : 0;
      const bool is_input = n->kind == N_LOAD && ((read_mask >> sidx) & 1u);
      if (is_input && !packed && contiguous_chunk && layout_bulk && (static_cast<int64_t>(P.round_elems) * isz) % 16 == 0 &&
          (dense ? true : chunk_in_inner)) {
        td.ring_layout = 1;
        // provisional (Bind() drops it when the address is not 16-byte aligned).  Tensors that no BODY reads together
        // may share bytes of a stage: a stage only ever holds the operands of one BODY's chunk.
        const uint32_t need = (P.chunk_elems * isz + 127u) & ~127u;
        uint32_t phases = 0;
        for (int q = 0; q < num_body; ++q)
          if ((body_tensor_mask[q] >> sidx) & 1u) phases |= 1u << q;
        uint32_t best = 0;
        for (bool moved = true; moved;) {
          moved = false;
          for (auto &pl : ring_placed)
            if ((pl.phases & phases) != 0 && best < pl.off + pl.size && pl.off < best + need) {
              best = pl.off + pl.size;
              moved = true;
            }
        }
        td.ring_off = best;
        ring_placed.push_back({best, need, phases});
        stage_bytes = std::max(stage_bytes, best + need);
      }
    }
    // ---- shared memory plan
    P.num_temps = static_cast<uint32_t>(max_temp);
    // a fast division of the vector side by a group scalar becomes a multiplication by its reciprocal, kept in a
    // scalar register of its own (one per distinct divisor register, as far as registers are left)
    {
      uint32_t divisors = 0;
      for (uint64_t w : code)
        if (!DVMB_SCALAR(w) && DVMB_OPC(w) == OP_BIN && DVMB_SUB(w) == B_DIV_FAST && DVMB_OKIND(w) == K_SREG)
          divisors |= 1u << DVMB_OIDX(w);
      out->sregs_used = static_cast<uint32_t>(max_sreg);
      max_sreg = std::min<int>(kNumSRegs, max_sreg + __builtin_popcount(divisors));
    }
    P.num_sregs = static_cast<uint32_t>(max_sreg);
    // the lowered program's length does not depend on the addresses bound later: lower once now to size its copy
    for (uint32_t t = 0; t < P.n_tensors; ++t) P.tensor[t].vec_ok = P.tensor[t].layout_vec;   // as for aligned addresses
    LowerStage(out);
    out->lowered_for = LoweringKey(*out);
    // (sized for the program without fused handlers: a rebind that takes a tensor off the ring undoes its fusions)
    P.stages_off = VmStagesOffset(P.n_code + out->fused_away);
    const uint32_t fixed = P.stages_off + P.num_temps * T * (4u * kLanes) + P.num_sregs * T * 4u;
    uint32_t stages = 0;
    if (stage_bytes != 0) {
      uint32_t budget = 106 * 1024;   // two CTAs of this size fit one SM
      if (!packed && T <= 128) budget = 52 * 1024;   // four
      if (const char *env = getenv("DVM_B200_RING_KB")) budget = static_cast<uint32_t>(atoi(env)) * 1024u;
      // enough stages to keep about 48 KB per CTA in flight (small tiles need a deep ring to cover the memory
      // latency), at least three; beyond that deeper read-ahead measured slower on large tiles
      const uint32_t want = std::max<uint32_t>(3u, (48u * 1024u + stage_bytes - 1) / stage_bytes + 1);
      stages = fixed + 2 * stage_bytes > budget ? 2 : std::min<uint32_t>(std::min<uint32_t>(want, kVmMaxStages), (budget - fixed) / stage_bytes);
      // the 128-thread CTAs (many-group reduce graphs, long reduce-free ones) run fastest on two stages (a third, when it fits, measured
      // 397 us against 339 us on 16384 rows of 4096)
      if (!packed && T <= 128) stages = std::min<uint32_t>(stages, 2u);
      if (const char *env = getenv("DVM_B200_STAGES")) stages = static_cast<uint32_t>(atoi(env));
      if (fixed + stages * stage_bytes > kVmMaxSmemBytes) {
        // too large to stage even twice: fall back to direct global loads
        stage_bytes = 0;
        stages = 0;
        for (uint32_t t = 0; t < P.n_tensors; ++t) {
          P.tensor[t].ring_layout = 0;
          P.tensor[t].ring_off = kNoRing;
        }
      }
    }
    // ---- resident groups: give every chunk of a group its own slot so that later phases re-read shared memory
    // instead of global memory; a group that does not fit one CTA is shared by a cluster of 2, 4 or 8
    P.resident = 0;
    P.cluster = 1;
    P.cpc = P.chunks;
    P.sets = 1;
    // measured slower than re-streaming from L2 on the shapes tried so far: opt-in until the resident loop is leaner
    static const bool no_resident = getenv("DVM_B200_RESIDENT") == nullptr;
    if (P.mode == VM_GROUP && !packed && stage_bytes != 0 && num_body >= 2 && !no_resident) {
      const uint32_t budget2 = 106 * 1024, budget1 = 210 * 1024;   // shared memory of a CTA at two / one CTA per SM
      for (uint32_t cl = 1; cl <= 8 && !P.resident; cl *= 2) {
        const uint32_t cpc = (P.chunks + cl - 1) / cl;
        if (cl > 1 && (P.chunks < cl || T > static_cast<uint32_t>(kVmFlatThreads))) break;
        const uint64_t one = static_cast<uint64_t>(cpc) * stage_bytes;
        uint32_t sets = 0;
        if (fixed + 2 * one <= budget2) sets = 2;
        else if (fixed + one <= budget2) sets = 1;
        else if (cl == 1 && fixed + 2 * one <= budget1) sets = 2;
        else if (cl >= 8 && fixed + one <= budget1) sets = 1;
        if (sets == 0 || sets * cpc > kVmMaxSlots) continue;
        P.resident = 1;
        P.cluster = cl;
        P.cpc = cpc;
        P.sets = sets;
        stages = sets * cpc;
      }
    }
    // ---- a long group shared by a cluster, streaming: with every CTA on a group of its own, all groups are in flight at
    // once and a pass over a group has left the L2 by the time the next pass comes back to it.  A cluster of CTAs per
    // group (each takes a run of the group's chunks, reductions combined through distributed shared memory) cuts the bytes
    // in flight by the cluster size, so that the later passes of a multi-pass graph are served by the L2.
    if (!P.resident && P.mode == VM_GROUP && !packed && P.rounds > 1 && stage_bytes != 0 && num_body >= 2) {
      const uint64_t group_bytes = static_cast<uint64_t>(P.chunks) * stage_bytes;
      const uint64_t slots = std::min<uint64_t>(static_cast<uint64_t>(K), 2ull * sms);
      // (measured on 256 groups of 400 KB, three passes: 115 us with one CTA per group, 123 us with clusters of two, 147 us
      // with four - the CTAs of a cluster wait for their slowest member at every reduction - so the split is opt-in)
      (void)group_bytes;
      (void)slots;
      uint32_t cl = 1;
      if (const char *env = getenv("DVM_B200_CLUSTER")) cl = static_cast<uint32_t>(std::max(1, std::min(8, atoi(env))));
      while (cl > 1 && P.chunks < 2 * cl) cl /= 2;
      P.cluster = cl;
      P.cpc = (P.chunks + cl - 1) / cl;
    }
    P.stage_bytes = stage_bytes;
    P.num_stages = stages;
    for (int t = 0; t < kMaxTensors; ++t)
      out->ring_plan_off[t] = static_cast<uint32_t>(t) < P.n_tensors ? P.tensor[t].ring_off : kNoRing;
    for (int q = 0; q < kMaxPhases; ++q) P.body_ring_mask[q] = 0;
    out->smem_bytes = fixed + stages * stage_bytes;
    if (out->smem_bytes > kVmMaxSmemBytes) throw Fail{"stage needs more shared memory than one SM has"};
    for (int q = 0; q < num_body; ++q) out->body_tensor_mask[q] = body_tensor_mask[q];
    out->threads = T + (stage_bytes != 0 ? 32u : 0u);

    // ---- grid: persistent CTAs, as many as fit per SM
    uint32_t per_sm_cap = !packed && T <= 128 ? 4u : 2u;
    if (const char *env = getenv("DVM_B200_CTAS_PER_SM")) per_sm_cap = static_cast<uint32_t>(atoi(env));
    uint32_t per_sm = std::max<uint32_t>(1u, std::min<uint32_t>(per_sm_cap, (226u * 1024u) / std::max<uint32_t>(out->smem_bytes + 1024u, 1u)));
    if (T > static_cast<uint32_t>(kVmFlatThreads)) per_sm = 1;
    const uint32_t work = P.mode == VM_FLAT ? P.chunks : (P.num_groups + P.groups_per_cta - 1) / P.groups_per_cta;
    if (P.cluster > 1) {
      const uint32_t units = std::max<uint32_t>(1u, std::min<uint32_t>(work, sms * per_sm / P.cluster));
      out->grid = units * P.cluster;
    } else {
      out->grid = std::max<uint32_t>(1u, std::min<uint32_t>(work, sms * per_sm));
    }
    if (num_body == 0) out->grid = 1;
  }

  // ---- step 5 (MatMul epilogue): tensor table addressed by (batch0, batch1, row, column) -------------
  void FillEpilogue(MatMulStage *mm) {
    MmParam &P = mm->param;
    if (R < 2 || R > 4) throw Fail{"MatMul result rank outside 2..4"};
    if (slot_nodes.size() > static_cast<size_t>(kMmMaxEpiTensors)) throw Fail{"more than 8 tensors in a MatMul epilogue"};
    if (max_temp > kNumTemps) throw Fail{"out of vector registers"};
    // scalar sections must be empty
    for (int p = 0; p <= num_body; ++p)
      if (DVMB_OPC(code[out->bsec[2 * p]]) != OP_END) throw Fail{"group-constant work inside a MatMul epilogue"};
    if (num_body != 1) throw Fail{"MatMul epilogue needs exactly one body"};
    mm->bytecode.clear();
    for (size_t pc = out->bsec[1];; ++pc) {
      mm->bytecode.push_back(code[pc]);
      if (DVMB_OPC(code[pc]) == OP_END) break;
    }
    if (mm->bytecode.size() > static_cast<size_t>(kMmMaxEpilogueWords)) throw Fail{"MatMul epilogue exceeds the program capacity"};
    std::memcpy(P.epilogue, mm->bytecode.data(), mm->bytecode.size() * sizeof(uint64_t));
    P.n_tensors = static_cast<uint32_t>(slot_nodes.size());
    P.num_temps = static_cast<uint32_t>(max_temp);
    P.mma_slot = 0xffffffffu;
    mm->slot_obj.assign(slot_nodes.begin(), slot_nodes.end());
    mm->algo_bytes = 0;
    for (size_t s = 0; s < slot_nodes.size(); ++s) {
      NDObject *n = slot_nodes[s];
      EpiTensor &t = P.tensor[s];
      std::memset(&t, 0, sizeof(t));
      t.dtype = static_cast<uint32_t>(n->dtype);
      if (n->dtype == kInt64) throw Fail{"int64 tensors are not supported"};
      if (n == mma_src) {
        P.mma_slot = static_cast<uint32_t>(s);
        mm->slot_obj[s] = nullptr;
        continue;
      }
      mm->algo_bytes += static_cast<uint64_t>(n->shape.numel()) * ItemSize(n->dtype);
      t.sn = static_cast<int32_t>(StrideOn(n, R - 1));
      t.sm = StrideOn(n, R - 2);
      t.sb1 = R >= 3 ? StrideOn(n, R - 3) : 0;
      t.sb0 = R >= 4 ? StrideOn(n, R - 4) : 0;
    }
  }

  void Run(MatMulStage *mm = nullptr) {
    for (size_t i = 0; i < ops.size(); ++i) ops[i]->cidx = static_cast<int>(i);
    info.assign(ops.size(), Info());
    for (auto n : ops) {
      if (n->kind == N_MATMUL) throw Fail{"MatMul inside a vector stage"};
      if (n->kind == N_ALLREDUCE) throw Fail{"a collective inside a vector stage"};
      if (n->kind == N_VIEW) throw Fail{"a view inside a vector stage"};
      if (n->kind == N_CONCAT) throw Fail{"a concatenation inside a vector stage"};
    }
    AlignAxes();
    Classify();
    MarkExact();
    const bool reduce_free = !has_reduce;
    for (;;) {
      try {
        Geometry();
        break;
      } catch (const Fail &f) {
        // too many iterated axes in a reduce-free graph: one more outer axis (of extent > 1) becomes a group axis
        if (!reduce_free || epilogue || std::string(f.why).find("iterated axes") == std::string::npos) throw;
        int next = -1;
        for (int a = 0; a < R && next < 0; ++a)
          if (!forced_outer[a] && dom[a] != 1) next = a;
        if (next < 0 || num_forced_outer >= R - 1) throw;
        forced_outer[next] = true;
        ++num_forced_outer;
        has_reduce = false;
        Classify();
        MarkExact();
      }
    }
    Emit();
    if (epilogue) {
      FillEpilogue(mm);
    } else {
      Fill();
    }
  }
};

const char *kOpNames[] = {"end", "ld", "st", "copy", "mov", "un", "bin", "cmp", "sel", "cvt", "racc", "rfin", "rinit"};
const char *kUnNames[] = {"Sqrt", "Abs", "Log", "Exp", "Round", "Floor", "Ceil", "Trunc", "IsFinite", "Abs", "ExpFast", "Nop"};
const char *kBinNames[] = {"Add", "Sub", "Mul", "Div", "Max", "Min", "Pow", "RSub", "RDiv",
                           "Add", "Sub", "Mul", "Max", "Min", "RSub", "DivFast", "RDivFast"};
const char *kCmpNames[] = {"Eq", "Ne", "Gt", "Ge", "Lt", "Le"};
const char *kCvtNames[] = {"F2I", "I2F", "NeZ", "NeZ", "Round"};
const char *kRedNames[] = {"Sum", "Max", "Min"};
const char *kModeNames[] = {"dense", "granule", "element", "scalar"};

}  // namespace

bool CompileVectorStage(const std::vector<NDObject *> &ops, VectorStage *out, std::string *why) {
  try {
    std::memset(&out->param, 0, sizeof(out->param));
    Compiler c(ops, out);
    c.Run();
    return true;
  } catch (const Fail &f) {
    if (why) *why = f.why;
    return false;
  }
}

bool CompileEpilogue(const std::vector<NDObject *> &ops, const NDObject *mma_src, MatMulStage *mm, std::string *why) {
  try {
    VectorStage scratch;
    Compiler c(ops, &scratch);
    c.epilogue = true;
    c.mma_src = mma_src;
    c.Run(mm);
    return true;
  } catch (const Fail &f) {
    if (why) *why = f.why;
    return false;
  }
}

namespace {
// `dual`: every BODY is lowered twice, once for chunks in which every lane is valid and once for any chunk; without it
// (programs too long to carry both) the any-chunk variant serves both.  Returns false when the words do not fit.
bool LowerStageAs(VectorStage *st, bool dual) {
  using namespace dvmb;
  VmParam &P = st->param;
  uint32_t n = 0;
  bool overflow = false;
  auto push = [&](uint64_t w) {
    if (n >= static_cast<uint32_t>(kMaxCodeWords)) {
      overflow = true;
      return;
    }
    P.code[n++] = w;
  };
  // fetch of an operand into destination `dest`
  // reciprocal registers: divisor register -> register that holds 1 / divisor (computed at the end of the scalar
  // section in front of every body that divides by it)
  int recip_of[16];
  for (int i = 0; i < 16; ++i) recip_of[i] = -1;
  {
    uint32_t next = st->sregs_used;
    for (uint64_t w : st->bytecode)
      if (!DVMB_SCALAR(w) && DVMB_OPC(w) == OP_BIN && DVMB_SUB(w) == B_DIV_FAST && DVMB_OKIND(w) == K_SREG &&
          recip_of[DVMB_OIDX(w)] < 0 && next < P.num_sregs)
        recip_of[DVMB_OIDX(w)] = static_cast<int>(next++);
  }
  P.body_coords_mask = 0;
  P.pro_skip_mask = 0;
  bool full = true;   // lowering the variant for full chunks
  auto fetch = [&](uint32_t kind, uint32_t idx, uint32_t imm, uint32_t dest) {
    switch (kind) {
      case K_TENSOR: {
        const TensorDesc &td = P.tensor[idx];
        const uint32_t aux = dest | (idx << 2);
        if (full && td.ring_off != kNoRing) {
          static const uint32_t by_dtype[] = {UH_LDR_U8, UH_LDR_F16, UH_LDR_BF16, UH_LDR_F32, UH_LDR_F32};
          push(MakeUop(by_dtype[td.dtype] + (dest == UD_ACC ? UH_LDRA_F32 - UH_LDR_F32 : 0u), aux, td.ring_off >> 4, 0));
        } else {
          push(MakeUop(UH_LDG, aux, 0, 0));
        }
        break;
      }
      case K_TEMP: push(MakeUop(UH_LDT, dest, idx, 0)); break;
      case K_SREG: push(MakeUop(UH_LDS, dest, idx, 0)); break;
      case K_IMM: push(MakeUop(UH_LDI, dest, 0, imm)); break;
      default:
        if (dest != UD_ACC) push(MakeUop(UH_MOVA, dest, 0, 0));
        break;
    }
  };
  auto round = [&](uint32_t rnd) {
    if (rnd == RN_F16) push(MakeUop(UH_RND_F16, 0, 0, 0));
    if (rnd == RN_BF16) push(MakeUop(UH_RND_BF16, 0, 0, 0));
  };
  // Peephole over the micro-ops [begin, n) of a full-chunk body: frequent neighbours become one fused handler (one
  // dispatch instead of two to four).  A fused handler performs its parts' operations in their order, each rounded
  // on its own, so the result is the unfused program's bit for bit.
  uint32_t fused_away = 0;
  auto fuse = [&](uint32_t begin) {
    static const bool off = getenv("DVM_B200_NO_FUSE") != nullptr;
    if (off || overflow) return;
    uint32_t o = begin;
    auto fused_op = [](uint32_t h) -> int {
      if (h == UH_BINV_FIRST + B_ADD) return FO_ADD;
      if (h == UH_BINV_FIRST + B_SUB) return FO_SUB;
      if (h == UH_BINV_FIRST + B_MUL) return FO_MUL;
      return -1;
    };
    for (uint32_t i = begin; i < n;) {
      const uint64_t a = P.code[i];
      const uint32_t ha = DVMB_UH(a), left = n - i;
      const uint64_t b = left >= 2 ? P.code[i + 1] : 0;
      const uint32_t hb = left >= 2 ? DVMB_UH(b) : static_cast<uint32_t>(UH_COUNT);
      uint64_t f = 0;
      uint32_t take = 1;
      const uint32_t hc = left >= 3 ? DVMB_UH(P.code[i + 2]) : static_cast<uint32_t>(UH_COUNT);
      if (((ha == UH_RND_F16 && hb == UH_ST_F16) || (ha == UH_RND_BF16 && hb == UH_ST_BF16)) &&
          (left == 2 || (hc >= UH_LDRA_F32 && hc <= UH_LDRA_U8))) {
        // the vector store rounds the same way, and nothing reads the accumulator before it is loaded again
        ++i;
        ++fused_away;
        continue;
      }
      const uint32_t hd = left >= 4 ? DVMB_UH(P.code[i + 3]) : static_cast<uint32_t>(UH_COUNT);
      const uint32_t he = left >= 5 ? DVMB_UH(P.code[i + 4]) : static_cast<uint32_t>(UH_COUNT);
      const bool centred = ha >= UH_LDRA_F32 && ha <= UH_LDRA_BF16 && hb == UH_BINR_FIRST + B_SUB;
      if (centred && hc == UH_RACCF_FIRST + R_SUM * 4u && hd == UH_SQR && he == UH_RACCF_FIRST + R_SUM * 4u + 1u) {
        f = MakeUop(UH_LDSTATS_FIRST + (ha - UH_LDRA_F32), 0, DVMB_UARG(a), DVMB_UARG(b) & 0xfu);
        take = 5;
      } else if (centred && hc == UH_SQR && (hd == UH_RACCF_FIRST + R_SUM * 4u || hd == UH_RACCF_FIRST + R_SUM * 4u + 1u)) {
        f = MakeUop(UH_LDVAR_FIRST + (hd - (UH_RACCF_FIRST + R_SUM * 4u)) * 3u + (ha - UH_LDRA_F32), 0, DVMB_UARG(a), DVMB_UARG(b) & 0xfu);
        take = 4;
      } else if (centred && hc == UH_BINR_FIRST + B_MUL && hd == UH_BINR_FIRST + B_MUL && he == UH_BINR_FIRST + B_ADD) {
        f = MakeUop(UH_LDNORM_FIRST + (ha - UH_LDRA_F32), 0, DVMB_UARG(a),
                    (DVMB_UARG(b) & 0xfu) | ((DVMB_UARG(P.code[i + 2]) & 0xfu) << 4) | ((DVMB_UARG(P.code[i + 3]) & 0xfu) << 8) |
                      ((DVMB_UARG(P.code[i + 4]) & 0xfu) << 12));
        take = 5;
      } else if (ha >= UH_LDRA_F32 && ha <= UH_LDRA_BF16 && hb == UH_BINS_FIRST + B_MUL && DVMB_UIMM(b) == 0xbf800000u &&
                 hc == UH_UN_FIRST + U_EXP_FAST && hd == UH_BINS_FIRST + B_ADD && DVMB_UIMM(P.code[i + 3]) == 0x3f800000u && he == UH_RCP) {
        f = MakeUop(UH_LDSIGM_FIRST + (ha - UH_LDRA_F32), 0, DVMB_UARG(a), 0);
        take = 5;
      } else if (ha >= UH_LDR_F32 && ha <= UH_LDR_BF16 && hb == UH_BINV_FIRST + B_MUL && hc == ha && hd == UH_BINV_FIRST + B_MUL) {
        f = MakeUop(UH_LDMUL2_FIRST + (ha - UH_LDR_F32), 0, DVMB_UARG(a), DVMB_UARG(P.code[i + 2]));
        take = 4;
      } else if (ha >= UH_LDRA_F32 && ha <= UH_LDRA_BF16 && hb == ha - UH_LDRA_F32 + UH_LDR_F32 && fused_op(hc) >= 0) {
        f = MakeUop(UH_LD2OP_FIRST + static_cast<uint32_t>(fused_op(hc)) * 3u + (ha - UH_LDRA_F32), 0, DVMB_UARG(a), DVMB_UARG(b));
        take = 3;
      } else if (ha == UH_BINR_FIRST + B_MUL && hb == UH_BINR_FIRST + B_MUL && hc == UH_BINR_FIRST + B_ADD) {
        f = MakeUop(UH_MULR_MULR_ADDR, 0, (DVMB_UARG(a) & 0xfu) | ((DVMB_UARG(b) & 0xfu) << 4) | ((DVMB_UARG(P.code[i + 2]) & 0xfu) << 8), 0);
        take = 3;
      } else if (ha >= UH_LDR_F32 && ha <= UH_LDR_BF16 && fused_op(hb) >= 0) {
        f = MakeUop(UH_LDOP_FIRST + static_cast<uint32_t>(fused_op(hb)) * 3u + (ha - UH_LDR_F32), 0, DVMB_UARG(a), 0);
        take = 2;
      } else if (ha >= UH_LDRA_F32 && ha <= UH_LDRA_BF16 && hb == UH_RACCF_FIRST + R_SUM * 4u) {
        f = MakeUop(UH_LDSUM_FIRST + (ha - UH_LDRA_F32), 0, DVMB_UARG(a), 0);
        take = 2;
      } else if (ha >= UH_LDRA_F32 && ha <= UH_LDRA_BF16 && hb == UH_BINR_FIRST + B_SUB) {
        f = MakeUop(UH_LDSUBR_FIRST + (ha - UH_LDRA_F32), 0, DVMB_UARG(a), DVMB_UARG(b));
        take = 2;
      } else if (ha == UH_SQR && (hb == UH_RACCF_FIRST + R_SUM * 4u || hb == UH_RACCF_FIRST + R_SUM * 4u + 1u)) {
        f = MakeUop(hb == UH_RACCF_FIRST + R_SUM * 4u ? UH_SQRSUM0 : UH_SQRSUM1, 0, 0, 0);
        take = 2;
      } else if (left >= 4 && ha == UH_BINS_FIRST + B_MUL && DVMB_UIMM(a) == 0xbf800000u && hb == UH_UN_FIRST + U_EXP_FAST &&
                 DVMB_UH(P.code[i + 2]) == UH_BINS_FIRST + B_ADD && DVMB_UIMM(P.code[i + 2]) == 0x3f800000u &&
                 DVMB_UH(P.code[i + 3]) == UH_RCP) {
        f = MakeUop(UH_SIGMOID_FAST, 0, 0, 0);
        take = 4;
      } else if (ha >= UH_BINR_FIRST && ha <= UH_BINR_LAST && hb >= UH_BINR_FIRST && hb <= UH_BINR_LAST) {
        const uint32_t ka = ha - UH_BINR_FIRST, kb = hb - UH_BINR_FIRST;
        const uint32_t h = ka == B_SUB && kb == B_MUL ? UH_SUBR_MULR : ka == B_MUL && kb == B_ADD ? UH_MULR_ADDR
                           : ka == B_MUL && kb == B_MUL ? UH_MULR_MULR : 0u;
        if (h != 0) {
          f = MakeUop(h, 0, (DVMB_UARG(a) & 0xffu) | ((DVMB_UARG(b) & 0xffu) << 8), 0);
          take = 2;
        }
      }
      P.code[o++] = take > 1 ? f : a;
      i += take;
      fused_away += take - 1;
    }
    // second pass: a normalisation whose result goes straight into a vector store of the operand's own type
    uint32_t o2 = begin;
    for (uint32_t i = begin; i < o; ++i) {
      const uint32_t h = DVMB_UH(P.code[i]);
      if (h >= UH_LDNORM_FIRST && h <= UH_LDNORM_LAST && i + 1 < o) {
        static const uint32_t store_of[] = {UH_ST_F32, UH_ST_F16, UH_ST_BF16};   // by FusedType
        const uint64_t st_op = P.code[i + 1];
        if (DVMB_UH(st_op) == store_of[h - UH_LDNORM_FIRST] && DVMB_UARG(st_op) < 16u) {
          P.code[o2++] = MakeUop(UH_LDNORMST_FIRST + (h - UH_LDNORM_FIRST), 0, DVMB_UARG(P.code[i]),
                                 (DVMB_UIMM(P.code[i]) & 0xffffu) | (DVMB_UARG(st_op) << 16));
          ++i;
          ++fused_away;
          continue;
        }
      }
      // the pieces of a residual RMSNorm + gated activation (ring offsets must fit 12 bits)
      const uint64_t c0 = P.code[i];
      const uint64_t c1 = i + 1 < o ? P.code[i + 1] : 0, c2 = i + 2 < o ? P.code[i + 2] : 0, c3 = i + 3 < o ? P.code[i + 3] : 0;
      const uint32_t h1 = i + 1 < o ? DVMB_UH(c1) : static_cast<uint32_t>(UH_COUNT), h2 = i + 2 < o ? DVMB_UH(c2) : static_cast<uint32_t>(UH_COUNT);
      const uint32_t h3 = i + 3 < o ? DVMB_UH(c3) : static_cast<uint32_t>(UH_COUNT);
      static const uint32_t store_for[] = {UH_ST_F32, UH_ST_F16, UH_ST_BF16};   // by FusedType
      auto small = [](uint32_t off) { return off < 4096u; };
      if (h >= UH_LD2OP_FIRST + FO_ADD * 3u && h <= UH_LD2OP_FIRST + FO_ADD * 3u + 2u && small(DVMB_UARG(c0)) && small(DVMB_UIMM(c0))) {
        const uint32_t ft = h - (UH_LD2OP_FIRST + FO_ADD * 3u);
        if (h1 == UH_SQRSUM0 || h1 == UH_SQRSUM1) {
          P.code[o2++] = MakeUop(UH_LD2ADDSQRSUM_FIRST + (h1 == UH_SQRSUM1 ? 3u : 0u) + ft, 0, DVMB_UARG(c0), DVMB_UIMM(c0));
          i += 1;
          fused_away += 1;
          continue;
        }
        if (h1 == UH_BINR_FIRST + B_MUL && h2 == UH_LDOP_FIRST + FO_MUL * 3u + ft && h3 == store_for[ft] && small(DVMB_UARG(c2)) &&
            DVMB_UARG(c3) < 16u && DVMB_UARG(c1) < 16u) {
          P.code[o2++] = MakeUop(UH_LD2ADDMULRMULST_FIRST + ft, 0, DVMB_UARG(c0),
                                 DVMB_UIMM(c0) | (DVMB_UARG(c2) << 12) | (DVMB_UARG(c3) << 24) | (DVMB_UARG(c1) << 28));
          i += 3;
          fused_away += 3;
          continue;
        }
      }
      if (h >= UH_LDSIGM_FIRST && h <= UH_LDSIGM_LAST && small(DVMB_UARG(c0))) {
        const uint32_t ft = h - UH_LDSIGM_FIRST;
        if (h1 == UH_LDMUL2_FIRST + ft && h2 == store_for[ft] && small(DVMB_UARG(c1)) && small(DVMB_UIMM(c1)) && DVMB_UARG(c2) < 16u) {
          P.code[o2++] = MakeUop(UH_LDSIGMMUL2ST_FIRST + ft, 0, DVMB_UARG(c0), DVMB_UARG(c1) | (DVMB_UIMM(c1) << 12) | (DVMB_UARG(c2) << 24));
          i += 2;
          fused_away += 2;
          continue;
        }
      }
      P.code[o2++] = P.code[i];
    }
    n = o2;
  };
  // every BODY is lowered twice (full chunks, any chunk); PRO sections once
  for (uint32_t pass = 0; pass <= 3 * P.num_body; ++pass) {
    const bool second = pass > 2 * P.num_body;
    const uint32_t sidx = second ? 2 * (pass - 2 * P.num_body - 1) + 1 : pass;
    if (second && !dual) break;
    full = dual && !second;
    if (second) {
      P.sec_any[sidx >> 1] = static_cast<uint16_t>(n);
    } else {
      P.sec[sidx] = static_cast<uint16_t>(n);
      if ((sidx & 1u) && !dual) P.sec_any[sidx >> 1] = static_cast<uint16_t>(n);
    }
    const bool body = (sidx & 1u) != 0;
    for (uint32_t pc = st->bsec[sidx];; ++pc) {
      const uint64_t w = st->bytecode[pc];
      const uint32_t opc = DVMB_OPC(w), sub = DVMB_SUB(w), okind = DVMB_OKIND(w), oidx = DVMB_OIDX(w);
      if (!body) {
        // a sum partial is zero at kernel start and every ReduceSum.fin leaves it at zero again: its init does nothing
        static const bool keep_init = getenv("DVM_B200_NO_FUSE") != nullptr;
        if (opc == OP_RINIT && (sub >> 4) == R_SUM && !keep_init) continue;
        if (opc == OP_END && n == P.sec[sidx]) P.pro_skip_mask |= 1u << (sidx >> 1);
        // scalar sections keep the instruction-word format; the common forms get a flat handler id as opcode
        uint32_t flat = opc;
        const bool plain_operand = okind == K_SREG || okind == K_IMM || okind == K_ACC;
        const bool no_round = DVMB_RND(w) == RN_NONE;
        switch (opc) {
          case OP_COPY: if (plain_operand) flat = SOP_COPY; break;
          case OP_MOV: flat = SOP_MOV; break;
          case OP_RINIT: flat = SOP_RINIT; break;
          case OP_RFIN: flat = SOP_RFIN; break;
          case OP_UN: if (no_round && sub <= U_NOP) flat = SOP_UN_FIRST + sub; break;
          case OP_BIN: if (no_round && plain_operand && sub < B_COUNT) flat = SOP_BIN_FIRST + sub; break;
          case OP_CVT: if (no_round && sub <= V_NEZ_I) flat = SOP_CVT_FIRST + sub; break;
          default: break;
        }
        if (opc == OP_END && sidx < 2 * P.num_body) {
          // reciprocals of the group scalars the next body divides by
          uint32_t done_mask = 0;
          for (uint32_t q = st->bsec[sidx + 1];; ++q) {
            const uint64_t b = st->bytecode[q];
            if (DVMB_OPC(b) == OP_END) break;
            if (DVMB_OPC(b) != OP_BIN || DVMB_SUB(b) != B_DIV_FAST || DVMB_OKIND(b) != K_SREG) continue;
            const uint32_t d = DVMB_OIDX(b);
            if (recip_of[d] < 0 || ((done_mask >> d) & 1u)) continue;
            done_mask |= 1u << d;
            push(Insn::make(SOP_COPY, 0, K_SREG, d, 0, 0, 0, 1, 0));
            push(Insn::make(SOP_BIN_FIRST + B_RDIV_FAST, 0, K_IMM, 0, 0, 0, 0, 1, 0x3f800000u));
            push(Insn::make(SOP_MOV, 0, 0, 0, static_cast<uint32_t>(recip_of[d]), 0, 0, 1, 0));
          }
        }
        if (opc == OP_END && !overflow) {
          // the reciprocal standard deviation chain of a normalisation becomes one word (plus the word that keeps its
          // second immediate); the arithmetic and its order stay the same
          static const bool no_fuse = getenv("DVM_B200_NO_FUSE") != nullptr;
          for (uint32_t q = P.sec[sidx]; !no_fuse && q + 4 <= n; ++q) {
            const uint64_t w0 = P.code[q], w1 = P.code[q + 1], w2 = P.code[q + 2], w3 = P.code[q + 3];
            if (DVMB_OPC(w0) == SOP_BIN_FIRST + B_MUL && DVMB_OKIND(w0) == K_IMM && DVMB_OPC(w1) == SOP_BIN_FIRST + B_ADD &&
                DVMB_OKIND(w1) == K_IMM && DVMB_OPC(w2) == SOP_UN_FIRST + U_SQRT && DVMB_OPC(w3) == SOP_BIN_FIRST + B_RDIV_FAST &&
                DVMB_OKIND(w3) == K_IMM && DVMB_IMM(w3) == 0x3f800000u) {
              P.code[q] = (w0 & ~(0xffull << 32)) | (static_cast<uint64_t>(SOP_RSTD_FAST) << 32);
              for (uint32_t r = q + 4; r < n; ++r) P.code[r - 2] = P.code[r];
              n -= 2;
              fused_away += 2;
              break;
            }
          }
        }
        if (opc == OP_END && !overflow && P.mode == VM_GROUP && P.tg > 32) {
          // two sums finished one after the other share their CTA barrier (not with clusters or resident groups,
          // whose finish also talks to the other CTAs)
          static const bool plain = getenv("DVM_B200_NO_FUSE") == nullptr && getenv("DVM_B200_CLUSTER") == nullptr &&
                                    getenv("DVM_B200_RESIDENT") == nullptr;
          for (uint32_t q = P.sec[sidx]; plain && q + 4 <= n; ++q) {
            const uint64_t w0 = P.code[q], w1 = P.code[q + 1], w2 = P.code[q + 2], w3 = P.code[q + 3];
            if (DVMB_OPC(w0) == SOP_RFIN && DVMB_OPC(w1) == SOP_MOV && DVMB_OPC(w2) == SOP_RFIN && DVMB_OPC(w3) == SOP_MOV &&
                (DVMB_SUB(w0) >> 4) == R_SUM && (DVMB_SUB(w2) >> 4) == R_SUM) {
              P.code[q] = Insn::make(SOP_RFIN2, (DVMB_SUB(w0) & 3u) | ((DVMB_SUB(w2) & 3u) << 2), K_IMM, DVMB_DST(w3), DVMB_DST(w1), 0, 0, 1, 0);
              for (uint32_t r = q + 4; r < n; ++r) P.code[r - 3] = P.code[r];
              n -= 3;
              fused_away += 3;
              break;
            }
          }
        }
        if (opc == OP_END && n > P.sec[sidx] && !overflow) {
          // a section whose last word stores a scalar register or resets a partial ends inside that word's handler
          static const bool no_tail = getenv("DVM_B200_NO_TAIL") != nullptr;
          const uint32_t last = DVMB_OPC(P.code[n - 1]);
          if (!no_tail && (last == SOP_MOV || last == SOP_RINIT)) {
            P.code[n - 1] = (P.code[n - 1] & ~(0xffull << 32)) | (static_cast<uint64_t>(last == SOP_MOV ? SOP_MOV_END : SOP_RINIT_END) << 32);
            ++fused_away;
            break;
          }
        }
        push((w & ~(0xffull << 32)) | (static_cast<uint64_t>(flat) << 32));
        if (opc == OP_END) break;
        continue;
      }
      if (opc == OP_END) {
        if (full) {
          fuse(P.sec[sidx]);
          // a body that ends in a vector store or a reduce accumulation ends inside that handler
          static const bool no_tail = getenv("DVM_B200_NO_TAIL") != nullptr;
          const uint32_t last = n > P.sec[sidx] ? DVMB_UH(P.code[n - 1]) : static_cast<uint32_t>(UH_END);
          const bool ends_body = (last >= UH_ST_F32 && last <= UH_ST_BF16) || (last >= UH_RACCF_FIRST && last <= UH_RACCF_LAST) ||
                                 (last >= UH_LDSUM_FIRST && last <= UH_LDSUM_LAST) || last == UH_SQRSUM0 || last == UH_SQRSUM1 ||
                                 (last >= UH_LDVAR_FIRST && last <= UH_LDVAR_LAST) ||
                                 (last >= UH_LDNORMST_FIRST && last <= UH_LDNORMST_LAST) ||
                                 (last >= UH_LD2ADDSQRSUM_FIRST && last <= UH_LDSIGMMUL2ST_LAST) ||
                                 (last >= UH_LDSTATS_FIRST && last <= UH_LDSTATS_LAST);
          if (ends_body && !no_tail && !overflow) {
            P.code[n - 1] |= static_cast<uint64_t>(UA_LAST) << 8;
            // a body that is one load + reduce micro-op runs all full rounds of a chunk in a single dispatch
            const bool load_reduce = (last >= UH_LDSUM_FIRST && last <= UH_LDSUM_LAST) || (last >= UH_LDVAR_FIRST && last <= UH_LDVAR_LAST) ||
                                     (last >= UH_LDNORMST_FIRST && last <= UH_LDNORMST_LAST) ||
                                     (last >= UH_LD2ADDSQRSUM_FIRST && last <= UH_LDSIGMMUL2ST_LAST) ||
                                     (last >= UH_LDSTATS_FIRST && last <= UH_LDSTATS_LAST);
            if (load_reduce && n - P.sec[sidx] == 1 && P.rounds > 1) P.code[n - 1] |= static_cast<uint64_t>(UA_LOOP) << 8;
            ++fused_away;
            break;
          }
        }
        push(MakeUop(UH_END, 0, 0, 0));
        break;
      }
      const bool splat = okind == K_SREG || okind == K_IMM;
      switch (opc) {
        case OP_COPY: fetch(okind, oidx, DVMB_IMM(w), UD_ACC); break;
        case OP_MOV: push(MakeUop(UH_STT, 0, DVMB_DST(w), 0)); break;
        case OP_UN:
          push(MakeUop(UH_UN_FIRST + sub, 0, 0, 0));
          round(DVMB_RND(w));
          break;
        case OP_BIN:
          if (splat && sub == B_RDIV_FAST && okind == K_IMM && DVMB_IMM(w) == 0x3f800000u) {
            push(MakeUop(UH_RCP, 0, 0, 0));
          } else if (splat && sub == B_DIV_FAST && okind == K_SREG && recip_of[oidx] >= 0) {
            push(MakeUop(UH_BINR_FIRST + B_MUL, 0, static_cast<uint32_t>(recip_of[oidx]), 0));
          } else if (splat) {
            push(MakeUop((okind == K_SREG ? UH_BINR_FIRST : UH_BINS_FIRST) + sub, 0, oidx, DVMB_IMM(w)));
          } else if (okind == K_ACC && sub == B_MUL) {
            push(MakeUop(UH_SQR, 0, 0, 0));
          } else {
            fetch(okind, oidx, 0, UD_B);
            push(MakeUop(UH_BINV_FIRST + sub, 0, 0, 0));
          }
          round(DVMB_RND(w));
          break;
        case OP_CMP:
          if (splat) {
            push(MakeUop(DVMB_ISINT(w) ? UH_CMP_I_S : UH_CMP_F_S, sub | (okind == K_SREG ? UA_CMP_SREG : 0u), oidx, DVMB_IMM(w)));
          } else {
            fetch(okind, oidx, 0, UD_B);
            push(MakeUop(DVMB_ISINT(w) ? UH_CMP_I_V : UH_CMP_F_V, sub, 0, 0));
          }
          break;
        case OP_SEL: {
          // acc holds the condition: keep its lane mask, then false value -> b, true value -> acc
          const bool inv = (DVMB_DST(w) & 1u) != 0;   // the free-form operand is the false value
          push(MakeUop(DVMB_ISINT(w) ? UH_PRED_I : UH_PRED_F, 0, 0, 0));
          if (inv) {
            fetch(okind, oidx, DVMB_IMM(w), UD_B);
            fetch(sub >> 4, sub & 15u, 0, UD_ACC);
          } else {
            fetch(sub >> 4, sub & 15u, 0, UD_B);
            fetch(okind, oidx, DVMB_IMM(w), UD_ACC);
          }
          push(MakeUop(UH_SELM, 0, 0, 0));
          break;
        }
        case OP_CVT: {
          static const uint32_t by_kind[] = {UH_CVT_F2I, UH_CVT_I2F, UH_CVT_NEZ_F, UH_CVT_NEZ_I};
          if (sub != V_RND) push(MakeUop(by_kind[sub], 0, 0, 0));
          if (sub == V_RND && DVMB_OPC(st->bytecode[pc + 1]) == OP_ST) {
            // a store of the same 16-bit type rounds the same way: no separate rounding when nothing else reads acc
            const TensorDesc &td = P.tensor[DVMB_SUB(st->bytecode[pc + 1])];
            const uint32_t after = DVMB_OPC(st->bytecode[pc + 2]);
            const uint32_t rnd = DVMB_RND(w);
            if ((after == OP_END || after == OP_COPY) &&
                ((rnd == RN_F16 && td.dtype == kFloat16) || (rnd == RN_BF16 && td.dtype == kBFloat16)))
              break;
          }
          round(DVMB_RND(w));
          break;
        }
        case OP_RACC:
          if (full) {
            push(MakeUop(UH_RACCF_FIRST + (sub >> 4) * 4u + (sub & 3u), 0, 0, 0));
          } else {
            push(MakeUop(UH_RACC_SUM + (sub >> 4), 0, sub & 3u, 0));
          }
          break;
        case OP_ST: {
          const TensorDesc &td = P.tensor[sub];
          static const uint32_t by_dtype[] = {UH_ST_U8, UH_ST_F16, UH_ST_BF16, UH_ST_F32, UH_ST_F32};
          const bool vec_store = full && td.chunk_contig && td.vec_ok;
          if (vec_store && td.mode != AM_DENSE) P.body_coords_mask |= 1u << (sidx >> 1);
          push(MakeUop(vec_store ? by_dtype[td.dtype] : UH_STG, 0, sub, 0));
          break;
        }
        default: break;
      }
    }
  }
  P.n_code = n;
  st->fused_away = fused_away;
  return !overflow;
}
}  // namespace

void LowerStage(VectorStage *st) {
  if (LowerStageAs(st, true)) return;
  if (!LowerStageAs(st, false)) DvmException("lowered program exceeds the launch capacity");
}


namespace {
// One line of disassembly per instruction word; `dt(slot)` / `ptr(slot)` describe the tensor table.
template <class DT, class PT>
std::string InsnLine(uint32_t pc, uint64_t w, DT dt, PT ptr) {
  using namespace dvmb;
  char buf[256];
  auto operand_text = [&](uint32_t kind, uint32_t idx, uint32_t imm) -> std::string {
    char b[64];
    switch (kind) {
      case K_TENSOR:
        snprintf(b, sizeof(b), "load.%s(0x%llx)", DTypeName(static_cast<DataType>(dt(idx))),
                 static_cast<unsigned long long>(ptr(idx)));
        break;
      case K_TEMP: snprintf(b, sizeof(b), "v%u", idx); break;
      case K_SREG: snprintf(b, sizeof(b), "s%u", idx); break;
      case K_IMM: snprintf(b, sizeof(b), "#0x%08x", imm); break;
      default: snprintf(b, sizeof(b), "acc"); break;
    }
    return b;
  };
  auto operand = [&](uint64_t ww) -> std::string { return operand_text(DVMB_OKIND(ww), DVMB_OIDX(ww), DVMB_IMM(ww)); };
  static const char *rnd_names[] = {"", ".rn_f16", ".rn_bf16", ""};
  const uint32_t opc = DVMB_OPC(w), sub = DVMB_SUB(w), dst = DVMB_DST(w);
  const bool sc = DVMB_SCALAR(w);
  const char *acc = sc ? "sacc" : "acc";
  const char *rp = sc ? "s" : "v";
  const char *ty = DVMB_ISINT(w) ? "int32" : "fp32";
  switch (opc) {
    case OP_END: snprintf(buf, sizeof(buf), "  %u: end\n", pc); break;
    case OP_ST:
      snprintf(buf, sizeof(buf), "  %u: store.%s 0x%llx, %s // t%u\n", pc, DTypeName(static_cast<DataType>(dt(sub))),
               static_cast<unsigned long long>(ptr(sub)), acc, sub);
      break;
    case OP_COPY: snprintf(buf, sizeof(buf), "  %u: copy %s, %s\n", pc, acc, operand(w).c_str()); break;
    case OP_MOV: snprintf(buf, sizeof(buf), "  %u: mov %s%u, %s\n", pc, rp, dst, acc); break;
    case OP_UN:
      snprintf(buf, sizeof(buf), "  %u: %s.%s%s %s, %s\n", pc, kUnNames[sub], sub == U_ABS_I ? "int32" : "fp32",
               rnd_names[DVMB_RND(w)], acc, acc);
      break;
    case OP_BIN:
      snprintf(buf, sizeof(buf), "  %u: %s.%s%s %s, %s, %s\n", pc, kBinNames[sub], (sub >= B_ADD_I && sub <= B_RSUB_I) ? "int32" : "fp32",
               rnd_names[DVMB_RND(w)], acc, acc, operand(w).c_str());
      break;
    case OP_CMP:
      snprintf(buf, sizeof(buf), "  %u: Cmp%s.%s %s, %s, %s\n", pc, kCmpNames[sub], ty, acc, acc, operand(w).c_str());
      break;
    case OP_SEL: {
      std::string second = operand_text(sub >> 4, sub & 15u, 0);
      if (dst & 1u) {
        snprintf(buf, sizeof(buf), "  %u: Select.%s %s, %s ? %s : %s\n", pc, ty, acc, acc, second.c_str(), operand(w).c_str());
      } else {
        snprintf(buf, sizeof(buf), "  %u: Select.%s %s, %s ? %s : %s\n", pc, ty, acc, acc, operand(w).c_str(), second.c_str());
      }
      break;
    }
    case OP_CVT:
      snprintf(buf, sizeof(buf), "  %u: Cvt%s%s %s, %s\n", pc, kCvtNames[sub], rnd_names[DVMB_RND(w)], acc, acc);
      break;
    case OP_RACC: snprintf(buf, sizeof(buf), "  %u: Reduce%s.acc p%u, acc\n", pc, kRedNames[sub >> 4], sub & 3u); break;
    case OP_RFIN: snprintf(buf, sizeof(buf), "  %u: Reduce%s.fin sacc, p%u // bar\n", pc, kRedNames[sub >> 4], sub & 3u); break;
    case OP_RINIT: snprintf(buf, sizeof(buf), "  %u: Reduce%s.init p%u\n", pc, kRedNames[sub >> 4], sub & 3u); break;
    default: snprintf(buf, sizeof(buf), "  %u: ?\n", pc); break;
  }
  return buf;
}
}  // namespace

// Text form of a stage's bytecode (the counterpart of the reference's disassembler, src/code.cc:1093-1498).
// One line per instruction: "<pc>: <Name>.<type> <dst>, <operands>"; loads and stores print as
// "load.<dtype> <dst>, <gm address>" / "store.<dtype> <gm address>, acc".
std::string DisassembleStage(const VectorStage &st) {
  using namespace dvmb;
  const VmParam &P = st.param;
  std::string o;
  char buf[256];
  snprintf(buf, sizeof(buf),
           "vmain.sm100(mode=%s, groups=%u, group_elems=%u, tg=%u, groups_per_cta=%u, chunk_elems=%u, rounds=%u, chunks=%u, grid=%u, "
           "threads=%u, smem=%u, stages=%u x %u B%s, cluster=%u) {\n",
           P.mode == VM_FLAT ? "flat" : "group", P.num_groups, P.group_elems, P.tg, P.groups_per_cta, P.chunk_elems, P.rounds, P.chunks,
           st.grid, st.threads, st.smem_bytes, P.num_stages, P.stage_bytes, P.resident ? " resident" : "", P.cluster);
  o += buf;
  for (uint32_t t = 0; t < P.n_tensors; ++t) {
    const TensorDesc &td = P.tensor[t];
    snprintf(buf, sizeof(buf), "  // t%u: %s %s vec=%d ring=%d kstride=[%u,%u,%u] estride=[%u,%u,%u,%u] @0x%llx\n", t,
             DTypeName(static_cast<DataType>(td.dtype)), kModeNames[td.mode], td.vec_ok, td.ring_off != kNoRing ? 1 : 0,
             td.kstride[0], td.kstride[1],
             td.kstride[2], td.estride[0], td.estride[1], td.estride[2], td.estride[3],
             static_cast<unsigned long long>(td.ptr));
    o += buf;
  }
  if (P.stage_bytes != 0) {
    // tensor slots the producer warp stages for each BODY (what Bind() derived from the bound addresses)
    o += "  // staged:";
    for (uint32_t q = 0; q < P.num_body; ++q) {
      snprintf(buf, sizeof(buf), " body_%u=0x%x", q, P.body_ring_mask[q]);
      o += buf;
    }
    o += "\n";
  }
  auto dt = [&](uint32_t slot) { return static_cast<uint32_t>(P.tensor[slot].dtype); };
  auto ptr = [&](uint32_t slot) { return P.tensor[slot].ptr; };
  for (uint32_t pc = 0; pc < st.bytecode.size(); ++pc) {
    for (uint32_t sidx = 0; sidx <= 2 * P.num_body; ++sidx)
      if (st.bsec[sidx] == pc) {
        snprintf(buf, sizeof(buf), " %s_%u:\n", (sidx & 1) ? "body" : "pro", sidx / 2);
        o += buf;
      }
    o += InsnLine(pc, st.bytecode[pc], dt, ptr);
  }
  // the micro-ops the launch carries for full chunks (what the instruction words above were lowered to)
  auto uop_name = [](uint32_t h) -> std::string {
    static const char *ty[] = {"fp32", "fp16", "bf16", "u8"};
    static const char *fo[] = {"Add", "Sub", "Mul"};
    if (h == UH_END) return "end";
    if (h >= UH_LDR_F32 && h <= UH_LDR_U8) return std::string("ldb.") + ty[h - UH_LDR_F32];
    if (h >= UH_LDRA_F32 && h <= UH_LDRA_U8) return std::string("lda.") + ty[h - UH_LDRA_F32];
    if (h >= UH_BINV_FIRST && h <= UH_BINV_LAST) return std::string(kBinNames[h - UH_BINV_FIRST]) + ".b";
    if (h >= UH_BINS_FIRST && h <= UH_BINS_LAST) return std::string(kBinNames[h - UH_BINS_FIRST]) + ".imm";
    if (h >= UH_BINR_FIRST && h <= UH_BINR_LAST) return std::string(kBinNames[h - UH_BINR_FIRST]) + ".s";
    if (h >= UH_UN_FIRST && h <= UH_UN_LAST) return kUnNames[h - UH_UN_FIRST];
    if (h >= UH_RACCF_FIRST && h <= UH_RACCF_LAST)
      return std::string("Reduce") + kRedNames[(h - UH_RACCF_FIRST) / 4] + ".p" + std::to_string((h - UH_RACCF_FIRST) % 4);
    if (h >= UH_RACC_SUM && h <= UH_RACC_MIN) return std::string("Reduce") + kRedNames[h - UH_RACC_SUM] + ".any";
    if (h >= UH_ST_F32 && h <= UH_ST_U8) return std::string("st.") + ty[h - UH_ST_F32];
    if (h >= UH_LDOP_FIRST && h <= UH_LDOP_LAST)
      return std::string("ldb.") + ty[(h - UH_LDOP_FIRST) % 3] + "+" + fo[(h - UH_LDOP_FIRST) / 3] + ".b";
    if (h >= UH_LD2OP_FIRST && h <= UH_LD2OP_LAST)
      return std::string("lda.") + ty[(h - UH_LD2OP_FIRST) % 3] + "+ldb+" + fo[(h - UH_LD2OP_FIRST) / 3] + ".b";
    if (h >= UH_LDVAR_FIRST && h <= UH_LDVAR_LAST)
      return std::string("lda.") + ty[(h - UH_LDVAR_FIRST) % 3] + "+Sub.s+Sqr+ReduceSum.p" + std::to_string((h - UH_LDVAR_FIRST) / 3);
    if (h >= UH_LDSTATS_FIRST && h <= UH_LDSTATS_LAST)
      return std::string("lda.") + ty[h - UH_LDSTATS_FIRST] + "+Sub.s+ReduceSum.p0+Sqr+ReduceSum.p1";
    if (h >= UH_LDNORM_FIRST && h <= UH_LDNORM_LAST) return std::string("lda.") + ty[h - UH_LDNORM_FIRST] + "+Sub.s+Mul.s+Mul.s+Add.s";
    if (h >= UH_LDSIGM_FIRST && h <= UH_LDSIGM_LAST) return std::string("lda.") + ty[h - UH_LDSIGM_FIRST] + "+SigmoidFast";
    if (h >= UH_LDMUL2_FIRST && h <= UH_LDMUL2_LAST) return std::string("ldb.") + ty[h - UH_LDMUL2_FIRST] + "+Mul.b+ldb+Mul.b";
    if (h >= UH_LDSUM_FIRST && h <= UH_LDSUM_LAST) return std::string("lda.") + ty[h - UH_LDSUM_FIRST] + "+ReduceSum.p0";
    if (h >= UH_LDSUBR_FIRST && h <= UH_LDSUBR_LAST) return std::string("lda.") + ty[h - UH_LDSUBR_FIRST] + "+Sub.s";
    switch (h) {
      case UH_LDG: return "ldg";
      case UH_LDT: return "ldt";
      case UH_LDS: return "lds";
      case UH_LDI: return "ldi";
      case UH_MOVA: return "mova";
      case UH_SQR: return "Sqr";
      case UH_RCP: return "Rcp";
      case UH_STT: return "stt";
      case UH_RND_F16: return "rnd.fp16";
      case UH_RND_BF16: return "rnd.bf16";
      case UH_SELM: return "selm";
      case UH_STG: return "stg";
      case UH_SQRSUM0: return "Sqr+ReduceSum.p0";
      case UH_SQRSUM1: return "Sqr+ReduceSum.p1";
      case UH_SUBR_MULR: return "Sub.s+Mul.s";
      case UH_MULR_ADDR: return "Mul.s+Add.s";
      case UH_MULR_MULR: return "Mul.s+Mul.s";
      case UH_MULR_MULR_ADDR: return "Mul.s+Mul.s+Add.s";
      case UH_LD2ADDSQRSUM_FIRST + 0: case UH_LD2ADDSQRSUM_FIRST + 1: case UH_LD2ADDSQRSUM_FIRST + 2:
        return std::string("lda.") + ty[h - UH_LD2ADDSQRSUM_FIRST] + "+ldb+Add.b+Sqr+ReduceSum.p0";
      case UH_LD2ADDSQRSUM_FIRST + 3: case UH_LD2ADDSQRSUM_FIRST + 4: case UH_LD2ADDSQRSUM_FIRST + 5:
        return std::string("lda.") + ty[h - UH_LD2ADDSQRSUM_FIRST - 3] + "+ldb+Add.b+Sqr+ReduceSum.p1";
      case UH_LD2ADDMULRMULST_FIRST + 0: case UH_LD2ADDMULRMULST_FIRST + 1: case UH_LD2ADDMULRMULST_FIRST + 2:
        return std::string("lda.") + ty[h - UH_LD2ADDMULRMULST_FIRST] + "+ldb+Add.b+Mul.s+ldb+Mul.b+st." + ty[h - UH_LD2ADDMULRMULST_FIRST];
      case UH_LDSIGMMUL2ST_FIRST + 0: case UH_LDSIGMMUL2ST_FIRST + 1: case UH_LDSIGMMUL2ST_FIRST + 2:
        return std::string("lda.") + ty[h - UH_LDSIGMMUL2ST_FIRST] + "+SigmoidFast+ldb+Mul.b+ldb+Mul.b+st." + ty[h - UH_LDSIGMMUL2ST_FIRST];
      case UH_LDNORMST_FIRST + FT_F32: return "lda.fp32+Sub.s+Mul.s+Mul.s+Add.s+st.fp32";
      case UH_LDNORMST_FIRST + FT_F16: return "lda.fp16+Sub.s+Mul.s+Mul.s+Add.s+st.fp16";
      case UH_LDNORMST_FIRST + FT_BF16: return "lda.bf16+Sub.s+Mul.s+Mul.s+Add.s+st.bf16";
      case UH_SIGMOID_FAST: return "SigmoidFast";
      default: return "u" + std::to_string(h);
    }
  };
  for (uint32_t q = 0; q < P.num_body; ++q) {
    o += "  // body_" + std::to_string(q) + " micro-ops:";
    for (uint32_t pc = P.sec[2 * q + 1]; pc < P.n_code; ++pc) {
      const uint32_t h = DVMB_UH(P.code[pc]);
      if (h == UH_END) break;
      o += " " + uop_name(h);
      if (DVMB_UAUX(P.code[pc]) & UA_LAST) {
        o += (DVMB_UAUX(P.code[pc]) & UA_LOOP) ? " (ends the body, loops over the chunk's rounds)" : " (ends the body)";
        break;
      }
    }
    o += "\n";
  }
  o += "}\n";
  return o;
}

}  // namespace dvm

namespace dvm {

// Text form of a MatMul stage: the MatMul itself, then its post-fusion program.
std::string DisassembleEpilogue(const MatMulStage &st) {
  using namespace dvmb;
  const MmParam &P = st.param;
  std::string o;
  char buf[320];
  snprintf(buf, sizeof(buf),
           "mmain.sm100(batch=%ux%u, m=%u, n=%u, k=%u, a=%s, b=%s, %s, engine=%s) {\n", P.batch0, P.batch1, P.M, P.N, P.K,
           P.a_mmajor ? "[k,m]" : "[m,k]", P.b_kmajor ? "[n,k]" : "[k,n]", DTypeName(static_cast<DataType>(P.in_dtype)),
           MatMulUsesTensorCores(P) ? "tcgen05" : "simt");
  o += buf;
  snprintf(buf, sizeof(buf), "  matmul.%s acc, load(0x%llx), load(0x%llx)%s\n", DTypeName(static_cast<DataType>(P.in_dtype)),
           static_cast<unsigned long long>(P.a_ptr), static_cast<unsigned long long>(P.b_ptr), P.bias_ptr ? ", bias" : "");
  o += buf;
  for (uint32_t t = 0; t < P.n_tensors; ++t) {
    const EpiTensor &td = P.tensor[t];
    if (t == P.mma_slot) {
      snprintf(buf, sizeof(buf), "  // t%u: the product\n", t);
    } else {
      snprintf(buf, sizeof(buf), "  // t%u: %s strides=[%lld,%lld,%lld,%d] @0x%llx\n", t, DTypeName(static_cast<DataType>(td.dtype)),
               static_cast<long long>(td.sb0), static_cast<long long>(td.sb1), static_cast<long long>(td.sm), td.sn,
               static_cast<unsigned long long>(td.ptr));
    }
    o += buf;
  }
  auto dt = [&](uint32_t slot) { return P.tensor[slot].dtype; };
  auto ptr = [&](uint32_t slot) { return P.tensor[slot].ptr; };
  o += " post:\n";
  for (uint32_t pc = 0; pc < st.bytecode.size(); ++pc) o += InsnLine(pc, st.bytecode[pc], dt, ptr);
  o += "}\n";
  return o;
}

}  // namespace dvm
