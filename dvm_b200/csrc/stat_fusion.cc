// Sums of squared deviations without a pass of their own.
//
// A normalisation written the textbook way reads its input three times: sum(x) for the mean m, sum((x - m)^2) for the
// variance, then the normalised result.  The middle pass exists only because m is not known while the first one runs.
// With a reference value s per group that IS known up front (the group's first element), the first pass can also
// accumulate  T = sum(x - s)  and  Q = sum((x - s)^2),  and for ANY group scalar m
//
//     sum(x)          = T + n s
//     sum((x - m)^2)  = Q - 2 e T + n e^2          with e = m - s   (exact in real arithmetic)
//
// so the second pass disappears: one read of the tensor less.  Where m is the mean itself, m = sum(x) / n (the usual
// case), the two collapse to  m = s + T / n  and  sum((x - m)^2) = Q - T (T / n).
// In fp32 the identity costs a little accuracy where (m - s)^2 is large against the variance (cancellation between Q
// and n e^2); for a 16-bit input, whose values are a few thousand steps apart at most, the relative error of the
// result stays near 1e-6 * (1 + (m - s)^2 / var), far inside the 1e-2 / 1e-3 tolerance class of reductions over
// 16-bit data.  The rewrite is therefore applied only to a
// 16-bit tensor widened to fp32, and DVM_B200_EXACT_MATH=1 (which also keeps exact divisions) switches it off.
//
// No counterpart in the reference, whose vector kernels run each reduction as written (src/vm_gpu.cu:1552-1617: seven
// kernels for this graph).
#include <cstdlib>
#include <cstring>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "graph.h"

namespace dvm {
namespace {

bool SameDims(const NDObject *a, const NDObject *b) {
  if (a->shape_ref == nullptr || b->shape_ref == nullptr) return false;
  const int rank = a->in[0]->shape.rank;
  if (rank != b->in[0]->shape.rank) return false;
  bool da[kMaxRank] = {false}, db[kMaxRank] = {false};
  for (size_t i = 0; i < a->shape_ref->size; ++i) {
    int64_t d = a->shape_ref->data[i];
    if (d < 0) d += rank;
    if (d < 0 || d >= rank) return false;
    da[d] = true;
  }
  for (size_t i = 0; i < b->shape_ref->size; ++i) {
    int64_t d = b->shape_ref->data[i];
    if (d < 0) d += rank;
    if (d < 0 || d >= rank) return false;
    db[d] = true;
  }
  for (int i = 0; i < rank; ++i)
    if (da[i] != db[i]) return false;
  return true;
}

bool IsSumKeep(const NDObject *n) { return n->kind == N_REDUCE && n->sub == kSum && n->keepdims; }

// `m` is computed from `root` through group scalars only (values of the reduction's own shape).
bool DependsOn(const NDObject *m, const NDObject *root, int depth = 0) {
  if (m == root) return true;
  if (depth > 16 || !(m->shape == root->shape)) return false;
  for (int k = 0; k < 3; ++k)
    if (m->in[k] && DependsOn(m->in[k], root, depth + 1)) return true;
  return false;
}

uint32_t FloatBits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}

struct Match {
  NDObject *r1, *r2, *sq, *m, *x, *load;
  int64_t n;
  bool mean_form;   // m = r1 * (1 / n) and nothing else reads r1
};

}  // namespace

std::vector<NDObject *> VKernel::FuseDeviationSums(const std::vector<NDObject *> &ops) {
  static const bool off = getenv("DVM_B200_EXACT_MATH") != nullptr;
  if (off) return ops;
  std::unordered_map<const NDObject *, std::vector<NDObject *>> users;
  std::unordered_map<const NDObject *, size_t> pos;
  for (size_t i = 0; i < ops.size(); ++i) {
    pos[ops[i]] = i;
    for (int k = 0; k < 3; ++k)
      if (ops[i]->in[k]) users[ops[i]->in[k]].push_back(ops[i]);
  }
  std::vector<Match> found;
  std::unordered_set<const NDObject *> taken;
  for (auto r2 : ops) {
    if (!IsSumKeep(r2)) continue;
    NDObject *sq = r2->in[0];
    if (sq->kind != N_BINARY || sq->sub != kMul || sq->in[0] != sq->in[1] || users[sq].size() != 1) continue;
    NDObject *d = sq->in[0];
    if (d->kind != N_BINARY || d->sub != kSub) continue;
    NDObject *x = d->in[0], *m = d->in[1];
    if (x->kind != N_CAST || x->dtype != kFloat32 || x->in[0]->kind != N_LOAD) continue;
    NDObject *load = x->in[0];
    if (load->dtype != kFloat16 && load->dtype != kBFloat16) continue;
    if (!(m->shape == r2->shape) || m->dtype != kFloat32 || r2->shape.rank != x->shape.rank) continue;
    NDObject *r1 = nullptr;
    for (auto u : users[x])
      if (u != r2 && IsSumKeep(u) && !taken.count(u) && SameDims(u, r2) && pos[u] < pos[m] && DependsOn(m, u)) r1 = u;
    if (r1 == nullptr || !(r1->shape == r2->shape)) continue;
    const int64_t groups = r1->shape.numel();
    if (groups <= 0 || x->shape.numel() % groups != 0) continue;
    const int64_t n = x->shape.numel() / groups;
    if (n < 2 || n > (1 << 24)) continue;
    taken.insert(r1);
    const bool mean_form = m->kind == N_BINARY_S && m->sub == SB_MUL && m->in[0] == r1 && m->scalar_ref == nullptr &&
                           m->scalar_bits == FloatBits(static_cast<float>(1.0 / static_cast<double>(n))) && users[r1].size() == 1;
    found.push_back(Match{r1, r2, sq, m, x, load, n, mean_form});
  }
  if (found.empty()) return ops;

  auto make = [&](NodeKind kind, const NDObject *like, uint8_t sub, NDObject *a, NDObject *b) {
    auto n = new NDObject();
    n->kind = kind;
    n->dtype = kFloat32;
    n->sub = sub;
    n->shape = like->shape;
    n->id = like->id;
    n->sub_kernel = like->sub_kernel;
    n->in[0] = a;
    n->in[1] = b;
    synth_.push_back(n);
    return n;
  };
  auto copy_of = [&](const NDObject *n) {
    auto c = new NDObject(*n);
    synth_.push_back(c);
    return c;
  };

  std::unordered_map<const NDObject *, NDObject *> repl;
  std::unordered_map<const NDObject *, const Match *> at_r1, at_r2;
  std::unordered_set<const NDObject *> dead;
  for (auto &mt : found) {
    at_r1[mt.r1] = &mt;
    at_r2[mt.r2] = &mt;
    dead.insert(mt.sq);
  }
  struct Sums {
    NDObject *s, *t, *q, *tn;   // tn = T / n (mean form only)
  };
  std::unordered_map<const NDObject *, const Match *> at_mean;
  for (auto &mt : found)
    if (mt.mean_form) at_mean[mt.m] = &mt;
  std::unordered_map<const Match *, Sums> sums;
  std::vector<NDObject *> out;
  auto mapped = [&](NDObject *v) {
    auto it = repl.find(v);
    return it == repl.end() ? v : it->second;
  };
  for (auto n : ops) {
    if (dead.count(n)) continue;
    if (at_r1.count(n)) {
      const Match *mt = at_r1.at(n);
      // s: the first element of every group, read through a strided view of the input
      NDObject *sl = copy_of(mt->load);
      sl->origin = mt->load->origin ? mt->load->origin : mt->load;
      sl->shape = mt->r1->shape;
      int64_t dense = 1;
      for (int i = mt->load->shape.rank - 1; i >= 0; --i) {
        sl->stride[i] = mt->load->strided ? mt->load->stride[i] : dense;
        dense *= mt->load->shape.d[i];
      }
      sl->strided = true;
      sl->stride_ref = nullptr;
      sl->shape_ref = nullptr;
      NDObject *s = copy_of(mt->x);
      s->in[0] = sl;
      s->shape = sl->shape;
      NDObject *d0 = make(N_BINARY, mt->x, kSub, mapped(mt->x), s);
      NDObject *t = copy_of(mt->r1);
      t->in[0] = d0;
      NDObject *sq0 = make(N_BINARY, mt->x, kMul, d0, d0);
      NDObject *q = copy_of(mt->r2);
      q->in[0] = sq0;
      for (NDObject *v : {sl, s, d0, t, sq0, q}) out.push_back(v);
      if (mt->mean_form) {
        sums[mt] = Sums{s, t, q, nullptr};   // the mean itself is made where the graph makes it
        continue;
      }
      NDObject *ns = make(N_BINARY_S, mt->r1, SB_MUL, s, nullptr);
      ns->scalar_bits = FloatBits(static_cast<float>(mt->n));
      NDObject *sum = make(N_BINARY, mt->r1, kAdd, t, ns);
      out.push_back(ns);
      out.push_back(sum);
      repl[n] = sum;
      sums[mt] = Sums{s, t, q, nullptr};
      continue;
    }
    if (at_mean.count(n)) {
      const Match *mt = at_mean.at(n);
      Sums &sm = sums.at(mt);
      sm.tn = make(N_BINARY_S, mt->r1, SB_MUL, sm.t, nullptr);
      sm.tn->scalar_bits = n->scalar_bits;
      NDObject *mean = make(N_BINARY, mt->r1, kAdd, sm.tn, sm.s);
      out.push_back(sm.tn);
      out.push_back(mean);
      repl[n] = mean;
      continue;
    }
    if (at_r2.count(n)) {
      const Match *mt = at_r2.at(n);
      const Sums &sm = sums.at(mt);
      if (mt->mean_form) {
        NDObject *ttn = make(N_BINARY, mt->r2, kMul, sm.t, sm.tn);
        NDObject *res = make(N_BINARY, mt->r2, kSub, sm.q, ttn);
        out.push_back(ttn);
        out.push_back(res);
        repl[n] = res;
        continue;
      }
      NDObject *e = make(N_BINARY, mt->r2, kSub, mapped(mt->m), sm.s);
      NDObject *et = make(N_BINARY, mt->r2, kMul, e, sm.t);
      NDObject *et2 = make(N_BINARY_S, mt->r2, SB_MUL, et, nullptr);
      et2->scalar_bits = FloatBits(2.0f);
      NDObject *ne = make(N_BINARY_S, mt->r2, SB_MUL, e, nullptr);
      ne->scalar_bits = FloatBits(static_cast<float>(mt->n));
      NDObject *nee = make(N_BINARY, mt->r2, kMul, ne, e);
      NDObject *t1 = make(N_BINARY, mt->r2, kSub, sm.q, et2);
      NDObject *res = make(N_BINARY, mt->r2, kAdd, t1, nee);
      for (NDObject *v : {e, et, et2, ne, nee, t1, res}) out.push_back(v);
      repl[n] = res;
      continue;
    }
    bool changed = false;
    for (int k = 0; k < 3; ++k) changed |= n->in[k] && repl.count(n->in[k]);
    if (!changed) {
      out.push_back(n);
      continue;
    }
    NDObject *c = copy_of(n);
    for (int k = 0; k < 3; ++k)
      if (c->in[k]) c->in[k] = mapped(c->in[k]);
    if (n->kind == N_STORE || n->kind == N_LOAD) c->origin = n->origin ? n->origin : n;
    repl[n] = c;
    out.push_back(c);
  }
  return out;
}

}  // namespace dvm
