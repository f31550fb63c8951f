// Stage planner: cuts an operator graph that does not fit one vector launch into a sequence of launches -
// vector stages, MatMul stages with their fused post-ops, fused attention - handing values from one stage to
// the next through the kernel's workspace in global memory.
//
// Plays the role of the reference's graph splitter (_SplitKernel::Append/Split/Exchange/AppendCube/BuildKernel,
// src/xkernel.cc:1960-2301) and of the mix kernel's post-fusion collection (MixKernelBase::Append,
// src/xkernel.cc:157-209).  The policy is different: a vector area keeps growing for as long as the vector
// compiler can still fuse it into one launch (reductions followed by elementwise ops stay together), a MatMul
// takes every following elementwise op of its own shape into its epilogue, and the
// MatMul -> softmax -> MatMul pattern becomes one attention launch.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>
#include <unordered_map>
#include <unordered_set>

#include "comm.h"
#include "graph.h"
#include "runtime.h"

namespace dvm {

uint32_t EncodeScalarRefNow(const ScalarRef *ref, DataType dtype);

namespace {

bool IsElementwise(NodeKind k) {
  switch (k) {
    case N_UNARY:
    case N_BINARY:
    case N_BINARY_S:
    case N_COMPARE:
    case N_COMPARE_S:
    case N_SELECT:
    case N_CAST:
    case N_COPY: return true;
    default: return false;
  }
}

// Ops that never get a stage of their own: consumers re-create them from what they read.
bool IsLazy(const NDObject *n) { return n->kind == N_LOAD || n->kind == N_BROADCAST_S || n->kind == N_BROADCAST; }

struct Planner {
  VKernel *vk;
  const std::vector<NDObject *> &ops;
  std::unordered_map<const NDObject *, std::vector<NDObject *>> users;
  std::unordered_map<const NDObject *, int> pos;
  std::unordered_set<const NDObject *> done;
  // where a computed value lives in memory once its stage has run: a planner-made Load
  std::unordered_map<const NDObject *, NDObject *> mem;
  // reductions over an empty extent with a non-empty result: the constant (the reduction's identity) readers see instead
  std::unordered_map<const NDObject *, NDObject *> subst;
  std::vector<NDObject *> cur;   // open vector area, program order
  std::unordered_set<const NDObject *> in_cur;
  size_t ws_top = 0;

  Planner(VKernel *k, const std::vector<NDObject *> &o) : vk(k), ops(o) {
    for (size_t i = 0; i < ops.size(); ++i) {
      pos[ops[i]] = static_cast<int>(i);
      for (int j = 0; j < 3; ++j)
        if (ops[i]->in[j]) users[ops[i]->in[j]].push_back(ops[i]);
    }
  }

  std::unordered_set<const NDObject *> slabbed;   // values that a launch writes straight into their slab of a Concat result

  NDObject *Synth(const NDObject *like) {
    auto n = new NDObject(*like);
    n->origin = nullptr;
    n->ws_off = -1;
    vk->synth_.push_back(n);
    return n;
  }

  NDObject *SynthLoad(const NDObject *value, const Shape &shape) {
    auto n = new NDObject();
    n->kind = N_LOAD;
    n->dtype = value->dtype;
    n->shape = shape;
    n->id = value->id;
    vk->synth_.push_back(n);
    return n;
  }

  size_t AllocWs(const NDObject *value) {
    const size_t bytes = static_cast<size_t>(value->shape.numel()) * ItemSize(value->dtype);
    const size_t off = ws_top;
    ws_top = (ws_top + bytes + 255) & ~static_cast<size_t>(255);
    return off;
  }

  // True when `n` is already addressable in global memory (a user's Load, a view of one, a stored temporary).
  bool InMemory(const NDObject *n) const { return n->kind == N_LOAD || mem.count(n) != 0; }
  // ... and as one contiguous tensor (what the tensor-core stages, collectives and reshapes-as-views need): a strided
  // Load only after it has been copied out to the workspace
  bool InPlainMemory(const NDObject *n) const {
    auto it = mem.find(n);
    if (it != mem.end()) return !it->second->strided;
    return n->kind == N_LOAD && !n->strided;
  }

  // A Load node (planner-made) reading value `n`, which must be InMemory().
  NDObject *MemLoad(const NDObject *n) {
    if (n->kind == N_LOAD && mem.count(n) == 0) {
      NDObject *c = Synth(n);
      c->origin = n->origin ? n->origin : const_cast<NDObject *>(n);
      c->ws_off = n->ws_off;
      return c;
    }
    NDObject *where = mem.at(n);
    NDObject *c = Synth(where);
    c->origin = where->origin;
    c->ws_off = where->ws_off;
    return c;
  }

  // ---- building the op list of one stage out of clones ---------------------------------------------------
  struct Build {
    std::vector<NDObject *> list;
    std::unordered_map<const NDObject *, NDObject *> clone;
    std::vector<std::pair<const NDObject *, NDObject *>> temps;   // (value, planner-made store) to publish in `mem`
  };

  NDObject *InputFor(Build &b, NDObject *v) {
    auto it = b.clone.find(v);
    if (it != b.clone.end()) return it->second;
    NDObject *c = nullptr;
    if (subst.count(v)) {
      c = Synth(subst.at(v));
    } else if (InMemory(v)) {
      c = MemLoad(v);
    } else if (v->kind == N_BROADCAST_S) {
      c = Synth(v);
      c->in[0] = nullptr;
    } else if (v->kind == N_BROADCAST) {
      NDObject *src = InputFor(b, v->in[0]);
      c = Synth(v);
      c->in[0] = src;
    } else {
      DvmException("stage planner: a value is used before the stage that computes it");
    }
    b.clone[v] = c;
    b.list.push_back(c);
    return c;
  }

  NDObject *CloneOp(Build &b, NDObject *n) {
    NDObject *in[3] = {nullptr, nullptr, nullptr};
    for (int j = 0; j < 3; ++j)
      if (n->in[j]) in[j] = InputFor(b, n->in[j]);
    NDObject *c = Synth(n);
    for (int j = 0; j < 3; ++j) c->in[j] = in[j];
    if (n->kind == N_STORE) {
      if (n->ws_off >= 0) {
        c->ws_off = n->ws_off;   // (a store the planner made itself: a Concat slab in the workspace)
      } else {
        c->origin = n;
      }
    }
    b.clone[n] = c;
    b.list.push_back(c);
    return c;
  }

  bool HasOutsideUser(const NDObject *n, const std::unordered_set<const NDObject *> &area) const {
    auto it = users.find(n);
    if (it == users.end()) return false;
    for (auto u : it->second) {
      if (u->kind == N_STORE && !IsLazy(n)) continue;   // stores travel with their value
      if (u->kind == N_CONCAT && slabbed.count(n)) continue;   // (the value goes to its slab of the Concat result instead)
      if (u->kind == N_BROADCAST) {
        if (HasOutsideUser(u, area)) return true;
        continue;
      }
      if (!area.count(u)) return true;
    }
    return false;
  }

  // Clone `nodes` (program order) with their stores; values read outside `area` get a workspace store.
  // With `commit` the workspace is really allocated.
  void CloneArea(Build &b, const std::vector<NDObject *> &nodes, const std::unordered_set<const NDObject *> &area,
                 bool commit) {
    for (auto n : nodes) {
      NDObject *c = b.clone.count(n) ? b.clone.at(n) : CloneOp(b, n);
      if (n->kind == N_STORE) continue;
      auto it = users.find(n);
      if (it != users.end())
        for (auto u : it->second)
          if (u->kind == N_STORE && !area.count(u)) {
            CloneOp(b, u);
            if (commit) done.insert(u);
          }
      if (HasOutsideUser(n, area)) {
        auto st = new NDObject();
        vk->synth_.push_back(st);
        st->kind = N_STORE;
        st->dtype = n->dtype;
        st->shape = n->shape;
        st->in[0] = c;
        st->id = n->id;
        st->ws_off = commit ? static_cast<int64_t>(AllocWs(n)) : 0;
        b.list.push_back(st);
        b.temps.emplace_back(n, st);
      }
    }
  }

  void Publish(const Build &b) {
    for (auto &t : b.temps) {
      NDObject *ld = SynthLoad(t.first, t.first->shape);
      ld->ws_off = t.second->ws_off;
      mem[t.first] = ld;
    }
  }

  // ---- vector areas ----------------------------------------------------------------------------------------
  bool TryVector(const std::vector<NDObject *> &nodes, bool commit, std::string *why) {
    std::unordered_set<const NDObject *> area(nodes.begin(), nodes.end());
    const size_t synth_mark = vk->synth_.size();
    const size_t ws_mark = ws_top;
    Build b;
    CloneArea(b, nodes, area, commit);
    auto st = std::make_unique<Stage>();
    st->kind = STAGE_VECTOR;
    const bool ok = CompileVectorStage(b.list, &st->vec, why);
    if (ok && commit) {
      Publish(b);
      vk->stages_.push_back(std::move(st));
      return true;
    }
    // a trial (or a failure): drop the clones again
    for (size_t i = synth_mark; i < vk->synth_.size(); ++i) delete vk->synth_[i];
    vk->synth_.resize(synth_mark);
    ws_top = ws_mark;
    return ok;
  }

  void CloseCur() {
    if (cur.empty()) return;
    std::string why;
    if (!TryVector(cur, true, &why)) {
      std::string msg = "cannot compile a vector stage: " + why;
      DvmException(msg.c_str());
    }
    for (auto n : cur) done.insert(n);
    cur.clear();
    in_cur.clear();
  }

  void AddVector(NDObject *n) {
    cur.push_back(n);
    std::string why;
    if (TryVector(cur, false, &why)) {
      in_cur.insert(n);
      return;
    }
    cur.pop_back();
    CloseCur();
    cur.push_back(n);
    if (!TryVector(cur, false, &why)) {
      std::string msg = "op #" + std::to_string(n->id) + " cannot run on this backend: " + why;
      DvmException(msg.c_str());
    }
    in_cur.insert(n);
  }

  // The constant that stands for reduction `n` over an empty extent.
  NDObject *EmptyReduce(const NDObject *n) {
    auto c = new NDObject();
    vk->synth_.push_back(c);
    c->kind = N_BROADCAST_S;
    c->dtype = n->dtype;
    c->shape = n->shape;
    c->id = n->id;
    const bool is_int = n->dtype == kInt32;
    if (n->sub == kMax) c->scalar_bits = is_int ? 0x80000000u : 0xff800000u;
    if (n->sub == kMin) c->scalar_bits = is_int ? 0x7fffffffu : 0x7f800000u;
    return c;
  }

  // Write a broadcast out to the workspace in a stage of its own, so that later stages can address it as memory.
  void Materialize(NDObject *v) {
    CloseCur();
    Build b;
    NDObject *c = InputFor(b, v);
    auto st = new NDObject();
    vk->synth_.push_back(st);
    st->kind = N_STORE;
    st->dtype = v->dtype;
    st->shape = v->shape;
    st->in[0] = c;
    st->id = v->id;
    st->ws_off = static_cast<int64_t>(AllocWs(v));
    b.list.push_back(st);
    b.temps.emplace_back(v, st);
    auto stage = std::make_unique<Stage>();
    stage->kind = STAGE_VECTOR;
    std::string why;
    if (!CompileVectorStage(b.list, &stage->vec, &why)) {
      std::string msg = "cannot write a broadcast out to memory: " + why;
      DvmException(msg.c_str());
    }
    Publish(b);
    vk->stages_.push_back(std::move(stage));
  }

  // Make sure `v` is addressable in memory before a tensor-core stage reads it.
  void RequireInMemory(NDObject *v, const char *what) {
    if (InPlainMemory(v)) return;
    if (v->kind == N_BROADCAST || v->kind == N_BROADCAST_S || InMemory(v)) {   // (a strided Load or view is copied out)
      Materialize(v);
      return;
    }
    if (in_cur.count(v)) {
      CloseCur();
      if (InMemory(v)) return;
    }
    std::string msg = std::string(what) + " must be a tensor in memory (a Load or a computed value)";
    DvmException(msg.c_str());
  }

  // ---- MatMul stages ---------------------------------------------------------------------------------------
  static void BatchOf(const Shape &s, uint32_t *b0, uint32_t *b1) {
    *b1 = s.rank >= 3 ? static_cast<uint32_t>(s.d[s.rank - 3]) : 1u;
    *b0 = s.rank >= 4 ? static_cast<uint32_t>(s.d[s.rank - 4]) : 1u;
  }

  bool ExternalOk(const NDObject *x, const NDObject *m) const {
    if (x->kind == N_LOAD || x->kind == N_BROADCAST_S) return true;
    if (x->kind == N_BROADCAST) return ExternalOk(x->in[0], m);
    if (mem.count(x)) return true;
    return in_cur.count(x) != 0;   // computed before the MatMul; its area is closed first
  }

  void PlaceMatMul(NDObject *m) {
    for (int j = 0; j < 3; ++j)
      if (m->in[j]) RequireInMemory(m->in[j], j == 2 ? "MatMul bias" : "MatMul operand");
    // post-fusion area: elementwise ops of the product's own shape that depend on it
    std::vector<NDObject *> area_nodes;
    std::unordered_set<const NDObject *> area{m};
    for (size_t i = pos.at(m) + 1; i < ops.size(); ++i) {
      NDObject *v = ops[i];
      if (done.count(v) || !IsElementwise(v->kind) || !(v->shape == m->shape)) continue;
      if (v->sub_kernel != m->sub_kernel) continue;   // a later sub-kernel of a stacked kernel is a launch of its own
      bool touches = false, ok = true;
      for (int j = 0; j < 3; ++j) {
        if (!v->in[j]) continue;
        if (area.count(v->in[j])) {
          touches = true;
        } else if (!ExternalOk(v->in[j], m)) {
          ok = false;
        }
      }
      if (!touches || !ok) continue;
      area.insert(v);
      area_nodes.push_back(v);
    }
    for (int attempt = 0; attempt < 2; ++attempt) {
      if (attempt == 1) {
        area_nodes.clear();
        area = {m};
      }
      bool need_close = false;
      for (auto v : area_nodes)
        for (int j = 0; j < 3; ++j) {
          const NDObject *x = v->in[j];
          while (x && x->kind == N_BROADCAST) x = x->in[0];
          if (x && in_cur.count(x)) need_close = true;
        }
      if (need_close) CloseCur();
      const size_t synth_mark = vk->synth_.size();
      const size_t ws_mark = ws_top;
      Build b;
      NDObject *src = SynthLoad(m, m->shape);
      b.clone[m] = src;
      b.list.push_back(src);
      std::vector<NDObject *> nodes{m};
      nodes.insert(nodes.end(), area_nodes.begin(), area_nodes.end());
      CloneArea(b, nodes, area, true);
      auto st = std::make_unique<Stage>();
      st->kind = STAGE_MATMUL;
      std::memset(&st->mm.param, 0, sizeof(st->mm.param));
      std::string why;
      if (!CompileEpilogue(b.list, src, &st->mm, &why)) {
        for (size_t i = synth_mark; i < vk->synth_.size(); ++i) delete vk->synth_[i];
        vk->synth_.resize(synth_mark);
        ws_top = ws_mark;
        if (attempt == 1) {
          std::string msg = "cannot compile the MatMul epilogue: " + why;
          DvmException(msg.c_str());
        }
        continue;
      }
      FillMatMul(m, &st->mm);
      Publish(b);
      vk->stages_.push_back(std::move(st));
      done.insert(m);
      for (auto v : area_nodes) {
        done.insert(v);
      }
      for (auto v : nodes) {
        auto it = users.find(v);
        if (it != users.end())
          for (auto u : it->second)
            if (u->kind == N_STORE) done.insert(u);
      }
      return;
    }
  }

  void FillMatMul(NDObject *m, MatMulStage *mm) {
    dvmb::MmParam &P = mm->param;
    const Shape &a = m->in[0]->shape, &bs = m->in[1]->shape, &o = m->shape;
    P.M = static_cast<uint32_t>(o.d[o.rank - 2]);
    P.N = static_cast<uint32_t>(o.d[o.rank - 1]);
    P.K = static_cast<uint32_t>(m->trans_a ? a.d[a.rank - 2] : a.d[a.rank - 1]);
    BatchOf(o, &P.batch0, &P.batch1);
    P.a_mmajor = m->trans_a ? 1 : 0;
    P.b_kmajor = m->trans_b ? 1 : 0;
    P.in_dtype = static_cast<uint32_t>(m->dtype);
    uint32_t ab0, ab1, bb0, bb1;
    BatchOf(a, &ab0, &ab1);
    BatchOf(bs, &bb0, &bb1);
    P.a_mul1 = ab1 > 1 ? 1 : 0;
    P.a_mul0 = ab0 > 1 ? ab1 : 0;
    P.a_batches = ab0 * ab1;
    P.b_mul1 = bb1 > 1 ? 1 : 0;
    P.b_mul0 = bb0 > 1 ? bb1 : 0;
    P.b_batches = bb0 * bb1;
    mm->a = MemLoad(m->in[0]);
    mm->b = MemLoad(m->in[1]);
    mm->bias = m->in[2] ? MemLoad(m->in[2]) : nullptr;
    if (m->in[2]) {
      P.bias_dtype = static_cast<uint32_t>(m->in[2]->dtype);
      if (m->in[2]->shape.numel() != static_cast<int64_t>(P.N)) DvmException("MatMul bias must hold one value per result column");
    }
    mm->idle = o.numel() == 0;
    mm->flops = 2ull * P.M * P.N * P.K * P.batch0 * P.batch1;
    mm->algo_bytes += static_cast<uint64_t>(a.numel() + bs.numel()) * 2 + (m->in[2] ? m->in[2]->shape.numel() * ItemSize(m->in[2]->dtype) : 0);
  }

  // ---- attention -------------------------------------------------------------------------------------------
  std::vector<NDObject *> RealUsers(const NDObject *n) const {
    auto it = users.find(n);
    return it == users.end() ? std::vector<NDObject *>() : it->second;
  }

  static bool ReducesLastDimKeep(const NDObject *r, int kind) {
    if (r->kind != N_REDUCE || r->sub != kind || !r->keepdims || r->shape_ref == nullptr || r->shape_ref->size != 1) return false;
    int64_t d = r->shape_ref->data[0];
    if (d < 0) d += r->in[0]->shape.rank;
    return d == r->in[0]->shape.rank - 1;
  }

  bool TryAttention(NDObject *m1) {
    if (m1->trans_a || !m1->trans_b || m1->in[2]) return false;
    const Shape &qs = m1->in[0]->shape, &ks = m1->in[1]->shape;
    if (qs.rank != ks.rank || qs.rank < 2 || qs.rank > 4) return false;
    for (int i = 0; i < qs.rank - 2; ++i)
      if (qs.d[i] != ks.d[i]) return false;
    std::vector<NDObject *> chain{m1};
    NDObject *x = m1;
    uint32_t scale_bits = 0x3f800000u, round2 = 0;
    auto single_user = [&](NDObject *n) -> NDObject * {
      auto u = RealUsers(n);
      return u.size() == 1 ? u[0] : nullptr;
    };
    NDObject *u = single_user(x);
    if (u && u->kind == N_BINARY_S && u->sub == SB_MUL) {
      scale_bits = u->scalar_ref ? EncodeScalarRefNow(u->scalar_ref, u->dtype) : u->scalar_bits;
      round2 = (u->dtype == kFloat16 || u->dtype == kBFloat16) ? 1 : 0;
      chain.push_back(u);
      x = u;
      u = single_user(x);
    }
    if (u && u->kind == N_CAST && u->dtype == kFloat32) {
      chain.push_back(u);
      x = u;
    }
    if (x->dtype != kFloat32) return false;
    if (x->kind == N_CAST) {
      // an fp32 scale after the cast
      NDObject *u2 = single_user(x);
      if (u2 && u2->kind == N_BINARY_S && u2->sub == SB_MUL && scale_bits == 0x3f800000u) {
        scale_bits = u2->scalar_ref ? EncodeScalarRefNow(u2->scalar_ref, u2->dtype) : u2->scalar_bits;
        chain.push_back(u2);
        x = u2;
      }
    }
    auto ux = RealUsers(x);
    if (ux.size() != 2) return false;
    NDObject *rmax = nullptr, *sub = nullptr;
    for (auto c : ux) {
      if (ReducesLastDimKeep(c, kMax)) rmax = c;
      if (c->kind == N_BINARY && c->sub == kSub && c->in[0] == x) sub = c;
    }
    if (!rmax || !sub || sub->in[1] != rmax || RealUsers(rmax).size() != 1) return false;
    NDObject *e = single_user(sub);
    if (!e || e->kind != N_UNARY || e->sub != kExp) return false;
    auto ue = RealUsers(e);
    if (ue.size() != 2) return false;
    NDObject *rsum = nullptr, *div = nullptr;
    for (auto c : ue) {
      if (ReducesLastDimKeep(c, kSum)) rsum = c;
      if (c->kind == N_BINARY && c->sub == kDiv && c->in[0] == e) div = c;
    }
    if (!rsum || !div || div->in[1] != rsum || RealUsers(rsum).size() != 1) return false;
    NDObject *p = single_user(div);
    if (!p) return false;
    chain.insert(chain.end(), {rmax, sub, e, rsum, div});
    if (p->kind == N_CAST && p->dtype == m1->dtype) {
      chain.push_back(p);
      NDObject *m2 = single_user(p);
      if (!m2) return false;
      p = m2;
    } else {
      return false;
    }
    NDObject *m2 = p;
    if (m2->kind != N_MATMUL || m2->in[0] != chain.back() || m2->trans_a || m2->trans_b || m2->in[2]) return false;
    const Shape &vs = m2->in[1]->shape;
    if (vs.rank != ks.rank) return false;
    for (int i = 0; i < ks.rank - 1; ++i)
      if (vs.d[i] != ks.d[i]) return false;
    if (vs.d[vs.rank - 1] != qs.d[qs.rank - 1]) return false;
    dvmb::AttnParam ap;
    std::memset(&ap, 0, sizeof(ap));
    uint32_t b0, b1;
    BatchOf(qs, &b0, &b1);
    ap.batch = b0 * b1;
    ap.sq = static_cast<uint32_t>(qs.d[qs.rank - 2]);
    ap.skv = static_cast<uint32_t>(ks.d[ks.rank - 2]);
    ap.d = static_cast<uint32_t>(qs.d[qs.rank - 1]);
    ap.dtype = static_cast<uint32_t>(m1->dtype);
    ap.scale_bits = scale_bits;
    ap.scale_first = round2;
    if (!dvmb::AttentionSupported(ap)) return false;
    // every operand must be addressable; only then commit
    NDObject *ins[3] = {m1->in[0], m1->in[1], m2->in[1]};
    for (auto v : ins)
      if (!InPlainMemory(v) && !in_cur.count(v) && !InMemory(v)) return false;
    for (auto v : ins) RequireInMemory(v, "attention operand");
    auto st = std::make_unique<Stage>();
    st->kind = STAGE_ATTENTION;
    st->attn.param = ap;
    st->attn.q = MemLoad(ins[0]);
    st->attn.k = MemLoad(ins[1]);
    st->attn.v = MemLoad(ins[2]);
    auto outs = RealUsers(m2);
    if (outs.size() == 1 && outs[0]->kind == N_STORE) {
      NDObject *o = Synth(outs[0]);
      o->origin = outs[0];
      o->in[0] = nullptr;
      st->attn.o = o;
      done.insert(outs[0]);
    } else {
      NDObject *o = SynthLoad(m2, m2->shape);
      o->ws_off = static_cast<int64_t>(AllocWs(m2));
      st->attn.o = o;
      mem[m2] = o;
    }
    st->attn.idle = m2->shape.numel() == 0;
    st->attn.flops = 4ull * ap.batch * ap.sq * ap.skv * ap.d;
    st->attn.algo_bytes = 2ull * ap.batch * (2ull * ap.sq * ap.d + 2ull * ap.skv * ap.d);
    vk->stages_.push_back(std::move(st));
    for (auto n : chain) done.insert(n);
    done.insert(m2);
    return true;
  }

  // ---- views ------------------------------------------------------------------------------------------------
  // Permute / Slice / Split: no stage, the result is the input's memory read through other strides.  A computed input
  // is stored to the workspace first (closing the open area), a broadcast is written out.
  void PlaceView(NDObject *n) {
    NDObject *src = n->in[0];
    if (!InMemory(src)) {
      if (src->kind == N_BROADCAST || src->kind == N_BROADCAST_S) {
        Materialize(src);
      } else if (in_cur.count(src)) {
        CloseCur();   // the view reads the value from outside the area, so the area stores it to the workspace
      }
      if (!InMemory(src)) DvmException("stage planner: view of a value that is not in memory");
    }
    NDObject *ld = MemLoad(src);
    const Shape &ps = src->shape;
    int64_t pstride[kMaxRank];
    int64_t dense = 1;
    for (int i = ps.rank - 1; i >= 0; --i) {
      pstride[i] = ld->strided ? ld->stride[i] : dense;
      dense *= ps.d[i];
    }
    int64_t off = 0;
    for (int i = 0; i < ps.rank; ++i) off += n->view_start[i] * pstride[i];
    ld->shape = n->shape;
    for (int i = 0; i < n->shape.rank; ++i) ld->stride[i] = pstride[n->view_from[i]];
    ld->strided = true;
    ld->stride_ref = nullptr;
    ld->addr_off += off * ItemSize(n->dtype);
    mem[n] = ld;
    done.insert(n);
  }

  // ---- Concat ----------------------------------------------------------------------------------------------
  // Kernel::Concat arrives as a chain of two-input nodes along one dimension.  The chain's last node writes all its
  // pieces as slabs of one workspace tensor (a strided store each, one launch per piece); the nodes inside the chain do
  // nothing of their own.  Whatever reads the result reads that tensor.
  bool InsideConcatChain(const NDObject *n) const {
    auto it = users.find(n);
    if (it == users.end() || it->second.size() != 1) return false;
    const NDObject *u = it->second[0];
    return u->kind == N_CONCAT && u->in[0] == n && u->in[1] != n && u->view_from[0] == n->view_from[0];
  }

  void PlaceConcat(NDObject *n) {
    if (InsideConcatChain(n)) return;   // (placed with the end of its chain)
    const int d = n->view_from[0];
    std::vector<NDObject *> pieces, inner;
    for (NDObject *c = n;;) {
      pieces.insert(pieces.begin(), c->in[1]);
      NDObject *a = c->in[0];
      if (a->kind == N_CONCAT && InsideConcatChain(a) && !done.count(a)) {
        inner.push_back(a);
        c = a;
        continue;
      }
      pieces.insert(pieces.begin(), a);
      break;
    }
    NDObject *dst = SynthLoad(n, n->shape);
    dst->ws_off = static_cast<int64_t>(AllocWs(n));
    int64_t stride[kMaxRank];
    int64_t dense = 1;
    for (int i = n->shape.rank - 1; i >= 0; --i) {
      stride[i] = dense;
      dense *= n->shape.d[i];
    }
    auto slab_store = [&](NDObject *value, const Shape &shape, int64_t at) {
      auto st = new NDObject();
      vk->synth_.push_back(st);
      st->kind = N_STORE;
      st->dtype = n->dtype;
      st->shape = shape;
      st->in[0] = value;
      st->id = n->id;
      st->ws_off = dst->ws_off;
      st->addr_off = at * stride[d] * static_cast<int64_t>(ItemSize(n->dtype));
      st->strided = true;
      for (int i = 0; i < n->shape.rank; ++i) st->stride[i] = stride[i];
      return st;
    };
    // a piece the open area computes goes to its slab from the launch that makes it, when that launch can hold the
    // strided store; anything else is copied from where it lives
    std::vector<int64_t> starts;
    int64_t at = 0;
    for (auto p : pieces) {
      starts.push_back(at);
      at += p->shape.d[d];
    }
    std::vector<char> placed(pieces.size(), 0);
    for (size_t i = 0; i < pieces.size(); ++i) {
      NDObject *p = pieces[i];
      if (!in_cur.count(p) || slabbed.count(p) || p->shape.numel() == 0) continue;
      NDObject *st = slab_store(p, p->shape, starts[i]);
      users[p].push_back(st);
      slabbed.insert(p);
      std::string why;
      if (TryVector(cur, false, &why)) {
        placed[i] = 1;
      } else {
        users[p].pop_back();
        slabbed.erase(p);
      }
    }
    for (size_t i = 0; i < pieces.size(); ++i) {
      NDObject *p = pieces[i];
      if (placed[i] || InMemory(p)) continue;
      if (p->kind == N_BROADCAST || p->kind == N_BROADCAST_S) {
        Materialize(p);
      } else {
        CloseCur();   // the open area stores the piece to the workspace: the chain reads it from outside the area
      }
      if (!InMemory(p)) DvmException("Concat of a value that is not in memory");
    }
    CloseCur();
    for (size_t i = 0; i < pieces.size(); ++i) {
      NDObject *p = pieces[i];
      if (placed[i] || p->shape.numel() == 0) continue;
      Build b;
      NDObject *src = InputFor(b, p);
      b.list.push_back(slab_store(src, p->shape, starts[i]));
      auto stage = std::make_unique<Stage>();
      stage->kind = STAGE_VECTOR;
      std::string why;
      if (!CompileVectorStage(b.list, &stage->vec, &why)) {
        std::string msg = "cannot write a Concat input to its slab: " + why;
        DvmException(msg.c_str());
      }
      vk->stages_.push_back(std::move(stage));
    }
    mem[n] = dst;
    done.insert(n);
    for (auto c : inner) done.insert(c);
  }

  // ---- collectives -----------------------------------------------------------------------------------------
  void PushCollective(uint32_t kind, const NDObject *n, NDObject *send, int64_t send_off, NDObject *recv, int64_t recv_off,
                      uint64_t count, uint64_t wire_bytes) {
    auto st = std::make_unique<Stage>();
    st->kind = STAGE_COLLECTIVE;
    CollStage &c = st->coll;
    c.kind = kind;
    c.reduce_type = n->kind == N_ALLREDUCE ? n->sub : 0;
    c.dtype = static_cast<int>(send->dtype);
    c.comm = n->comm;
    c.send = send;
    c.recv = recv;
    c.send_off = send_off;
    c.recv_off = recv_off;
    c.count = count;
    c.wire_bytes = wire_bytes;
    vk->stages_.push_back(std::move(st));
  }

  // True when `x` (not yet computed) can be recomputed inside a row-block stage: an elementwise chain without a row axis
  // (or with a row extent of 1) over scalars and tensors in memory.  Collects the chain in `extra`.
  bool PullRowFree(const NDObject *x, std::unordered_set<const NDObject *> &extra) {
    while (x->kind == N_BROADCAST) x = x->in[0];
    if (x->kind == N_BROADCAST_S || InMemory(x) || extra.count(x)) return true;
    if (done.count(x) || !IsElementwise(x->kind)) return false;
    const Shape &xs = x->shape;
    if (!(xs.rank < 2 || xs.d[xs.rank - 2] == 1)) return false;
    for (int j = 0; j < 3; ++j)
      if (x->in[j] && !PullRowFree(x->in[j], extra)) return false;
    extra.insert(x);
    return true;
  }

  // All transitive users of `root`, in program order, when they form a tail that can run on a row block: elementwise ops
  // and stores only, every other operand a scalar, a row-free value (no row axis or a row extent of 1: a tensor in memory
  // or an elementwise chain over such, which the stage then computes itself) or a full [M, N] tensor in memory.  Empty
  // when the tail does not qualify.
  std::vector<NDObject *> RowBlockTail(const NDObject *root) {
    const Shape &rs = root->shape;
    std::unordered_set<const NDObject *> in_tail{root}, extra;
    for (size_t i = pos.at(root) + 1; i < ops.size(); ++i) {
      NDObject *v = ops[i];
      bool touches = false;
      for (int j = 0; j < 3; ++j)
        if (v->in[j] && in_tail.count(v->in[j])) touches = true;
      if (!touches) continue;
      if (done.count(v)) return {};
      if (v->kind == N_STORE) {
        if (!(v->shape == rs)) return {};
      } else if (!IsElementwise(v->kind) || !(v->shape == rs)) {
        return {};
      }
      for (int j = 0; j < 3; ++j) {
        const NDObject *x = v->in[j];
        if (!x || in_tail.count(x)) continue;
        while (x->kind == N_BROADCAST) x = x->in[0];
        if (x->kind == N_BROADCAST_S) continue;
        if (InMemory(x)) {
          const Shape &xs = x->shape;
          const bool row_free = xs.rank < 2 || xs.d[xs.rank - 2] == 1;
          if (!row_free && !(xs == rs)) return {};
          if (!row_free && !InPlainMemory(x)) return {};   // (the row block of a strided tensor is not a plain offset)
        } else if (!PullRowFree(x, extra)) {
          return {};
        }
      }
      in_tail.insert(v);
    }
    std::vector<NDObject *> nodes;
    bool stores = false;
    for (size_t i = 0; i < ops.size(); ++i) {
      NDObject *v = ops[i];
      if (v == root || (!in_tail.count(v) && !extra.count(v))) continue;
      nodes.push_back(v);
      stores |= v->kind == N_STORE && in_tail.count(v);
    }
    // (every user of a tail value is in the tail by construction; a tail that stores nothing is not worth a special plan)
    return stores ? nodes : std::vector<NDObject *>();
  }

  // Clone of load-like node `x` (a Load or a value in memory) restricted to the rank's row block.
  void ToRowBlock(NDObject *c, int64_t rows_all, int64_t rows, int rank_id) {
    Shape &s = c->shape;
    if (s.rank < 2 || s.d[s.rank - 2] != rows_all) return;
    int64_t row_bytes = ItemSize(c->dtype);
    for (int i = s.rank - 1; i < s.rank; ++i) row_bytes *= s.d[i];
    s.d[s.rank - 2] = rows;
    if (c->kind == N_LOAD || c->kind == N_STORE) c->addr_off += rank_id * rows * row_bytes;
  }

  // AllReduce(sum) of an [M, N] value that sits in a workspace temporary of its own, followed by a row-independent tail:
  // reduce-scatter in place (each rank ends up with the sum of its own M / size rows), the tail on that row block only,
  // all-gather of every stored result.  Same results on every rank as all-reduce + tail everywhere, with the second half of
  // the exchange in the (narrower) result type and the tail's work divided by the number of ranks (src/ops_c.cc:366-645 is
  // the reference's fused MatMul + all-reduce this stands in for).
  bool TryShardedTail(NDObject *n) {
    static const bool off = getenv("DVM_B200_NO_SHARDED_TAIL") != nullptr;
    const Communicator *comm = n->comm;
    const Shape &rs = n->shape;
    if (off || comm->size <= 1 || n->sub != kSum || rs.rank != 2 || rs.d[0] % comm->size != 0 || rs.numel() == 0) return false;
    NDObject *v = n->in[0];
    auto where = mem.find(v);
    if (where == mem.end() || where->second->ws_off < 0) return false;   // (a caller's buffer must not be overwritten)
    auto uv = users.find(v);
    if (uv == users.end() || uv->second.size() != 1) return false;
    std::vector<NDObject *> tail = RowBlockTail(n);
    if (tail.empty()) return false;
    const int64_t rows_all = rs.d[0];
    const int64_t isz = ItemSize(n->dtype);
    // Row chunks (DVM_B200_TP_CHUNKS=n).  When the stage in front is the MatMul that makes the temporary (and nothing
    // else), the product can be cut into row chunks: chunk c's reduce-scatter, tail and all-gather run while the MatMul works on chunk c + 1, the
    // collectives on a second stream (Stage::lane).  Rank r then owns rows [c Mc + r Mc / size, ...) of every chunk instead
    // of one block of M / size rows: the same results, since the tail is row-independent.
    int chunks = 1;
    Stage *mm_stage = nullptr;
    int ws_slot = -1;
    if (!vk->stages_.empty() && vk->stages_.back()->kind == STAGE_MATMUL) {
      MatMulStage &m0 = vk->stages_.back()->mm;
      bool other = false;
      for (size_t sl = 0; sl < m0.slot_obj.size(); ++sl) {
        NDObject *o = m0.slot_obj[sl];
        if (!o) continue;
        if (o->kind == N_STORE && o->ws_off >= 0 && o->ws_off == where->second->ws_off && o->shape == rs) {
          ws_slot = static_cast<int>(sl);
        } else {
          other = true;
        }
      }
      const dvmb::MmParam &mp = m0.param;
      if (ws_slot >= 0 && !other && !mp.a_mmajor && mp.batch0 * mp.batch1 == 1 && mp.M == static_cast<uint32_t>(rows_all) &&
          m0.a->shape.rank == 2 && !m0.idle)
        mm_stage = vk->stages_.back().get();
    }
    if (mm_stage) {
      // (off unless asked for: on 8 GPUs the [16384, 8192] product measured 1.57 ms in one chunk, 1.57 in two and 1.65-1.71
      // in four - the collectives lose more by sharing the GPU with the MatMul and by their smaller messages than the
      // overlap wins; on 2 GPUs, where the MatMul is the longer part, four chunks measured 1.81 against 1.89 ms)
      int want = 1;
      if (const char *env = getenv("DVM_B200_TP_CHUNKS")) want = std::max(1, atoi(env));
      // every chunk keeps whole MatMul tiles (256 rows per CTA pair) and whole rows per rank
      while (want > 1 && (rows_all % (static_cast<int64_t>(want) * comm->size) != 0 || (rows_all / want) % 256 != 0)) --want;
      chunks = want;
    }
    const int64_t rows_chunk = rows_all / chunks, rows = rows_chunk / comm->size;   // rows of a chunk, of a rank's block in it
    const int64_t blk_elems = rows * rs.d[1];
    auto copy_node = [&](const NDObject *like) {
      auto c = new NDObject(*like);
      vk->synth_.push_back(c);
      return c;
    };
    // the stages of every chunk, pushed in pipeline order further down
    std::vector<std::unique_ptr<Stage>> mm_c, rs_c, tail_c;
    std::vector<std::vector<std::unique_ptr<Stage>>> ag_c(chunks);
    std::unique_ptr<Stage> mm_base;
    if (chunks > 1) {
      mm_base = std::move(vk->stages_.back());
      vk->stages_.pop_back();
      for (int c = 0; c < chunks; ++c) {
        auto st = std::make_unique<Stage>(*mm_base);
        MatMulStage &mc = st->mm;
        mc.a = copy_node(mm_base->mm.a);
        ToRowBlock(mc.a, rows_all, rows_chunk, c);
        mc.slot_obj[ws_slot] = copy_node(mm_base->mm.slot_obj[ws_slot]);
        ToRowBlock(mc.slot_obj[ws_slot], rows_all, rows_chunk, c);
        mc.param.M = static_cast<uint32_t>(rows_chunk);
        mc.param.leave_sms = 16;   // room for the collective that runs beside this launch
        mc.flops = mm_base->mm.flops / chunks;
        mc.algo_bytes = mm_base->mm.algo_bytes / chunks;
        mm_c.push_back(std::move(st));
      }
    }
    auto take_last = [&]() {
      std::unique_ptr<Stage> st = std::move(vk->stages_.back());
      vk->stages_.pop_back();
      return st;
    };
    std::unordered_set<const NDObject *> area(tail.begin(), tail.end());
    area.insert(n);
    for (int c = 0; c < chunks; ++c) {
      const int64_t chunk_off = static_cast<int64_t>(c) * rows_chunk * rs.d[1];   // elements in front of the chunk
      // 1. reduce-scatter, in place on the chunk's rows of the temporary
      NDObject *w = MemLoad(v);
      PushCollective(dvmb::COLL_REDUCE_SCATTER, n, w, chunk_off * isz, w, (chunk_off + comm->rank * blk_elems) * isz,
                     static_cast<uint64_t>(blk_elems), static_cast<uint64_t>(blk_elems * isz) * (comm->size - 1));
      rs_c.push_back(take_last());
      // 2. the tail on the rank's rows of the chunk
      Build b;
      NDObject *src = MemLoad(v);
      src->shape = rs;
      b.clone[n] = src;
      b.list.push_back(src);
      const size_t first_clone = vk->synth_.size() - 1;
      CloneArea(b, tail, area, c == 0);
      if (c > 0 && !b.temps.empty()) DvmException("stage planner: a row-block tail with a temporary cannot be cut into chunks");
      for (size_t i = first_clone; i < vk->synth_.size(); ++i)
        ToRowBlock(vk->synth_[i], rows_all, rows, c * comm->size + comm->rank);
      auto st = std::make_unique<Stage>();
      st->kind = STAGE_VECTOR;
      std::string why;
      if (!CompileVectorStage(b.list, &st->vec, &why)) {
        std::string msg = "cannot compile the row-block tail of an all-reduce: " + why;
        DvmException(msg.c_str());
      }
      tail_c.push_back(std::move(st));
      // 3. all-gather of every result, in place on the caller's buffer
      for (auto t : tail) {
        if (c == 0) {
          // (a recomputed row-free chain that something else reads as well stays open for the stage that needs it)
          bool inside = true;
          auto ut = users.find(t);
          if (ut != users.end())
            for (auto u : ut->second) inside &= area.count(u) != 0;
          if (inside) done.insert(t);
        }
        if (t->kind != N_STORE) continue;
        NDObject *whole = Synth(t);
        whole->origin = t;
        whole->in[0] = nullptr;
        const int64_t osz = ItemSize(t->dtype);
        PushCollective(dvmb::COLL_ALL_GATHER, n, whole, (chunk_off + comm->rank * blk_elems) * osz, whole, chunk_off * osz,
                       static_cast<uint64_t>(blk_elems), static_cast<uint64_t>(blk_elems * osz) * (comm->size - 1));
        vk->stages_.back()->coll.dtype = static_cast<int>(t->dtype);
        ag_c[c].push_back(take_last());
      }
    }
    // pipeline order.  Launch stream: mm_0, mm_1, tail_0, mm_2, tail_1, ...; second stream: rs_0, rs_1, ag_0, rs_2, ag_1, ...
    std::vector<int> at_mm(chunks, -1), at_rs(chunks, -1), at_tail(chunks, -1);
    auto push = [&](std::unique_ptr<Stage> st, int lane, int after) {
      st->lane = chunks > 1 ? lane : 0;
      st->after = chunks > 1 ? after : -1;
      vk->stages_.push_back(std::move(st));
      return static_cast<int>(vk->stages_.size()) - 1;
    };
    if (chunks > 1) {
      at_mm[0] = push(std::move(mm_c[0]), 0, -1);
      at_mm[1] = push(std::move(mm_c[1]), 0, -1);
    }
    at_rs[0] = push(std::move(rs_c[0]), 1, chunks > 1 ? at_mm[0] : -1);
    for (int c = 0; c < chunks; ++c) {
      if (c + 1 < chunks) at_rs[c + 1] = push(std::move(rs_c[c + 1]), 1, at_mm[c + 1]);
      at_tail[c] = push(std::move(tail_c[c]), 0, at_rs[c]);
      if (c + 2 < chunks) at_mm[c + 2] = push(std::move(mm_c[c + 2]), 0, -1);
      for (auto &ag : ag_c[c]) push(std::move(ag), 1, at_tail[c]);
    }
    done.insert(n);
    return true;
  }

  void PlaceAllReduce(NDObject *n) {
    NDObject *v = n->in[0];
    if (!InPlainMemory(v)) {
      if (v->kind == N_BROADCAST || v->kind == N_BROADCAST_S || InMemory(v)) {
        Materialize(v);
      } else {
        CloseCur();   // the open area stores v to the workspace: this node reads it from outside the area
      }
      if (!InMemory(v)) DvmException("AllReduce of a value that is not in memory");
    } else {
      CloseCur();
    }
    if (n->coll == 0 && TryShardedTail(n)) return;
    // general form: the result goes to a workspace temporary
    NDObject *src = MemLoad(v);
    NDObject *dst = SynthLoad(n, n->shape);
    dst->ws_off = static_cast<int64_t>(AllocWs(n));
    const uint64_t ranks = static_cast<uint64_t>(n->comm->size);
    if (n->coll == 1) {   // reduce-scatter: this rank's block of the sum
      const uint64_t blk = static_cast<uint64_t>(n->shape.numel());
      PushCollective(dvmb::COLL_REDUCE_SCATTER, n, src, 0, dst, 0, blk, blk * ItemSize(n->dtype) * (ranks - 1));
    } else if (n->coll == 2) {   // all-gather: every rank's tensor, stacked
      const uint64_t blk = static_cast<uint64_t>(v->shape.numel());
      PushCollective(dvmb::COLL_ALL_GATHER, n, src, 0, dst, 0, blk, blk * ItemSize(n->dtype) * (ranks - 1));
    } else {
      const uint64_t count = static_cast<uint64_t>(n->shape.numel());
      const uint64_t bytes = count * ItemSize(n->dtype);
      PushCollective(dvmb::COLL_ALL_REDUCE, n, src, 0, dst, 0, count, ranks > 1 ? 2 * bytes * (ranks - 1) / ranks : 0);
    }
    mem[n] = dst;
    done.insert(n);
  }

  // ---- driver ------------------------------------------------------------------------------------------------
  void Run() {
    // Sub-kernels of a kSequence / kParallel kernel (Kernel::SequenceAdd / ParallelAdd; the reference's SequenceKernel
    // and ParallelKernel, src/xkernel.cc:1226-1468, 1009-1151): the open vector area is closed where the sub-kernel
    // changes, so each sub-kernel becomes launches of its own, enqueued in the order of the adds, and a value that a
    // later sub-kernel reads crosses through the workspace.
    int sub = ops.empty() ? 0 : ops.front()->sub_kernel;
    for (auto n : ops) {
      if (n->sub_kernel != sub) {
        CloseCur();
        sub = n->sub_kernel;
      }
      if (done.count(n)) continue;
      if (n->shape.numel() == 0) {   // nothing to compute or to write
        done.insert(n);
        continue;
      }
      if (n->kind == N_REDUCE && n->in[0]->shape.numel() == 0) {
        subst[n] = EmptyReduce(n);
        done.insert(n);
        continue;
      }
      switch (n->kind) {
        case N_LOAD:
        case N_BROADCAST_S:
        case N_BROADCAST: break;
        case N_STORE: {
          NDObject *v = n->in[0];
          if (IsLazy(v) || mem.count(v) || subst.count(v)) AddVector(n);   // a plain copy of something already in memory
          break;
        }
        case N_RESHAPE: {
          NDObject *src = n->in[0];
          if (in_cur.count(src)) {
            // try the reshape inside the open area (it can stay there when it only adds or drops unit dims)
            cur.push_back(n);
            std::string why;
            if (TryVector(cur, false, &why)) {
              in_cur.insert(n);
              break;
            }
            cur.pop_back();
            CloseCur();
          }
          if (!InPlainMemory(src)) {
            if (src->kind != N_BROADCAST && src->kind != N_BROADCAST_S && !InMemory(src))
              DvmException("stage planner: reshape of a value that is not in memory");
            // a broadcast is re-created by its readers: a reshape that only adds or drops unit dims joins an area,
            // any other one needs the broadcast written out first
            std::string why;
            cur.push_back(n);
            if (TryVector(cur, false, &why)) {
              in_cur.insert(n);
              break;
            }
            cur.pop_back();
            CloseCur();
            cur.push_back(n);
            if (TryVector(cur, false, &why)) {
              in_cur.insert(n);
              break;
            }
            cur.pop_back();
            Materialize(src);
          }
          // a view of memory: same bytes, new shape
          NDObject *ld = MemLoad(src);
          ld->shape = n->shape;
          mem[n] = ld;
          done.insert(n);
          break;
        }
        case N_MATMUL:
          if (!TryAttention(n)) PlaceMatMul(n);
          break;
        case N_ALLREDUCE: PlaceAllReduce(n); break;
        case N_VIEW: PlaceView(n); break;
        case N_CONCAT: PlaceConcat(n); break;
        default: AddVector(n); break;
      }
    }
    CloseCur();
  }
};

}  // namespace

void VKernel::PlanStages(const std::vector<NDObject *> &ops) {
  Planner p(this, ops);
  p.Run();
  ws_bytes_ = p.ws_top;
}

}  // namespace dvm
