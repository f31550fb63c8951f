// Shape inference for graph nodes (the counterpart of the NDObject::Normalize family in the reference:
// Load src/ops.cc:1117-1123, binary broadcast 2398-2464, Select 2578-2622, Broadcast 2683-2695,
// Reduce 3080-3123, Reshape 1799-1827, MatMul src/ops_m.cc:271-305).  Shapes are kept in API order
// (outermost first); NumPy right-aligned broadcasting rules apply.
#include <string>

#include <algorithm>

#include "comm.h"
#include "graph.h"

namespace dvm {

int ItemSize(DataType t) {
  switch (t) {
    case kBool: return 1;
    case kFloat16:
    case kBFloat16: return 2;
    case kFloat32:
    case kInt32: return 4;
    default: return 8;
  }
}

const char *DTypeName(DataType t) {
  static const char *names[] = {"bool", "fp16", "bf16", "fp32", "int32", "int64"};
  return t >= 0 && t < kDataTypeEnd ? names[t] : "?";
}

namespace {

[[noreturn]] void Fail(const NDObject *n, const char *what) {
  std::string msg = "shape inference failed at op #" + std::to_string(n->id) + ": " + what;
  DvmException(msg.c_str());
}

Shape FromRef(const NDObject *n, const IntArrayRef *ref) {
  if (ref == nullptr || (ref->size > 0 && ref->data == nullptr)) Fail(n, "missing shape");
  if (ref->size > static_cast<size_t>(kMaxRank)) Fail(n, "rank above 10");
  Shape s;
  s.rank = static_cast<int>(ref->size);
  for (int i = 0; i < s.rank; ++i) s.d[i] = ref->data[i];
  return s;
}

Shape BroadcastShapes(const NDObject *n, const Shape &a, const Shape &b) {
  Shape o;
  o.rank = a.rank > b.rank ? a.rank : b.rank;
  for (int p = 0; p < o.rank; ++p) {   // p counts from the innermost dim
    int64_t da = p < a.rank ? a.d[a.rank - 1 - p] : 1;
    int64_t db = p < b.rank ? b.d[b.rank - 1 - p] : 1;
    if (da != db && da != 1 && db != 1) Fail(n, "operands are not broadcast-compatible");
    o.d[o.rank - 1 - p] = da == 1 ? db : da;
  }
  return o;
}

}  // namespace

// A view's element strides, one per dim of the node's shape (borrowed reference, re-read at every Normalize).
static void ReadStrides(NDObject *n) {
  n->strided = false;
  if (n->stride_ref == nullptr) return;
  if (static_cast<int>(n->stride_ref->size) != n->shape.rank) Fail(n, "a view needs one stride per dimension");
  int64_t dense = 1;
  bool same = true;
  for (int i = n->shape.rank - 1; i >= 0; --i) {
    const int64_t st = n->stride_ref->data[i];
    if (st < 0) Fail(n, "negative strides are not supported");
    n->stride[i] = st;
    if (n->shape.d[i] != 1 && st != dense) same = false;
    dense *= n->shape.d[i];
  }
  n->strided = !same;   // (strides that describe a contiguous tensor need no special handling)
}

void InferShape(NDObject *n) {
  switch (n->kind) {
    case N_LOAD:
      n->shape = FromRef(n, n->shape_ref);
      for (int i = 0; i < n->shape.rank; ++i)
        if (n->shape.d[i] < 0) Fail(n, "negative dimension");
      if (n->slice_mode != 0) {
        const Shape full = n->shape;
        const int r = full.rank;
        if (n->slice_a == nullptr || n->slice_b == nullptr || static_cast<int>(n->slice_a->size) != r ||
            static_cast<int>(n->slice_b->size) != r || (n->slice_mode == 2 && (n->slice_c == nullptr || static_cast<int>(n->slice_c->size) != r)))
          Fail(n, "a slice load needs one start, one size (or end and step) per dimension");
        int64_t dense = 1, off = 0;
        for (int i = r - 1; i >= 0; --i) {
          int64_t b = n->slice_a->data[i], len = 0, step = 1;
          if (n->slice_mode == 1) {
            len = n->slice_b->data[i];
            if (b < 0 || len < 0 || b + len > full.d[i]) Fail(n, "slice outside its tensor");
          } else {   // start / end as Python slices read them
            int64_t e = n->slice_b->data[i];
            step = n->slice_c->data[i];
            if (step <= 0) Fail(n, "slice steps must be positive");
            if (b < 0) b += full.d[i];
            if (e < 0) e += full.d[i];
            b = std::min<int64_t>(std::max<int64_t>(b, 0), full.d[i]);
            e = std::min<int64_t>(std::max<int64_t>(e, b), full.d[i]);
            len = (e - b + step - 1) / step;
          }
          n->shape.d[i] = len;
          n->stride[i] = dense * step;
          off += b * dense;
          dense *= full.d[i];
        }
        n->strided = true;
        n->addr_off = off * static_cast<int64_t>(ItemSize(n->dtype));
        break;
      }
      ReadStrides(n);
      break;
    case N_STORE:
      n->shape = n->in[0]->shape;
      if (n->pad_size > 0 && n->shape.rank > 0) {
        int64_t dense = 1;
        for (int i = n->shape.rank - 1; i >= 0; --i) {
          n->stride[i] = dense;
          dense *= n->shape.d[i] + (i == n->shape.rank - 1 ? n->pad_size : 0);
        }
        n->strided = true;
        break;
      }
      ReadStrides(n);
      break;
    case N_UNARY:
    case N_BINARY_S:
    case N_COMPARE_S:
    case N_CAST:
    case N_COPY: n->shape = n->in[0]->shape; break;
    case N_BINARY:
    case N_COMPARE: n->shape = BroadcastShapes(n, n->in[0]->shape, n->in[1]->shape); break;
    case N_SELECT:
      n->shape = BroadcastShapes(n, BroadcastShapes(n, n->in[0]->shape, n->in[1]->shape), n->in[2]->shape);
      break;
    case N_BROADCAST: {
      Shape t = FromRef(n, n->shape_ref);
      const Shape &s = n->in[0]->shape;
      if (t.rank < s.rank) Fail(n, "broadcast target has lower rank than its input");
      for (int i = 0; i < t.rank; ++i) {
        int si = i - (t.rank - s.rank);
        int64_t in_dim = si >= 0 ? s.d[si] : 1;
        if (t.d[i] == -1) t.d[i] = in_dim;   // -1 keeps the input dimension
        if (in_dim != 1 && in_dim != t.d[i]) Fail(n, "broadcast target does not match its input");
      }
      n->shape = t;
      break;
    }
    case N_BROADCAST_S: n->shape = n->in[0] ? n->in[0]->shape : FromRef(n, n->shape_ref); break;
    case N_RESHAPE: {
      Shape t = FromRef(n, n->shape_ref);
      if (t.numel() != n->in[0]->shape.numel()) Fail(n, "reshape changes the element count");
      n->shape = t;
      break;
    }
    case N_REDUCE: {
      const Shape &s = n->in[0]->shape;
      bool red[kMaxRank] = {false};
      if (n->reduce_all) {
        for (int i = 0; i < s.rank; ++i) n->all_dims[i] = i;
        n->all_ref.data = n->all_dims;
        n->all_ref.size = static_cast<size_t>(s.rank);
        n->shape_ref = &n->all_ref;
      }
      if (n->shape_ref == nullptr) Fail(n, "missing reduce dims");
      for (size_t i = 0; i < n->shape_ref->size; ++i) {
        int64_t d = n->shape_ref->data[i];
        if (d < 0) d += s.rank;
        if (d < 0 || d >= s.rank) Fail(n, "reduce dim out of range");
        red[d] = true;
      }
      Shape o;
      o.rank = 0;
      for (int i = 0; i < s.rank; ++i) {
        if (red[i]) {
          if (n->keepdims) o.d[o.rank++] = 1;
        } else {
          o.d[o.rank++] = s.d[i];
        }
      }
      n->shape = o;
      break;
    }
    case N_CONCAT: {
      const Shape &a = n->in[0]->shape, &b = n->in[1]->shape;
      if (a.rank != b.rank || a.rank == 0) Fail(n, "concat inputs must have one rank");
      int d = n->view_dim;
      if (d < 0) d += a.rank;
      if (d < 0 || d >= a.rank) Fail(n, "concat dimension out of range");
      Shape o = a;
      for (int i = 0; i < a.rank; ++i)
        if (i != d && a.d[i] != b.d[i]) Fail(n, "concat inputs differ outside the concatenated dimension");
      o.d[d] = a.d[d] + b.d[d];
      n->view_from[0] = d;   // (the normalised dimension, for the planner)
      n->shape = o;
      break;
    }
    case N_VIEW: {
      const Shape &in = n->in[0]->shape;
      Shape o = in;
      for (int i = 0; i < in.rank; ++i) {
        n->view_from[i] = i;
        n->view_start[i] = 0;
      }
      auto norm_dim = [&](int d) {
        if (d < 0) d += in.rank;
        if (d < 0 || d >= in.rank) Fail(n, "view dimension out of range");
        return d;
      };
      auto scalar_int = [&](const ScalarRef *r) -> int64_t {
        if (r == nullptr) Fail(n, "slice bound missing");
        return r->type == kFloat32 ? static_cast<int64_t>(r->f32) : (r->type == kInt32 ? r->i32 : r->i64);
      };
      switch (n->sub) {
        case VIEW_PERMUTE: {   // result dim i walks input dim dims[i] (ref: include/dvm.h:428-434)
          if (n->shape_ref == nullptr || static_cast<int>(n->shape_ref->size) != in.rank) Fail(n, "permute needs one axis per dim");
          bool seen[kMaxRank] = {false};
          for (int i = 0; i < in.rank; ++i) {
            const int d = norm_dim(static_cast<int>(n->shape_ref->data[i]));
            if (seen[d]) Fail(n, "permute axes repeat");
            seen[d] = true;
            n->view_from[i] = d;
            o.d[i] = in.d[d];
          }
          break;
        }
        case VIEW_SLICE: {     // ref: include/dvm.h:436-443
          if (n->shape_ref == nullptr || n->aux_ref == nullptr || static_cast<int>(n->shape_ref->size) != in.rank ||
              static_cast<int>(n->aux_ref->size) != in.rank)
            Fail(n, "slice needs a start and a size per dim");
          for (int i = 0; i < in.rank; ++i) {
            const int64_t st = n->shape_ref->data[i], sz = n->aux_ref->data[i];
            if (st < 0 || sz < 0 || st + sz > in.d[i]) Fail(n, "slice outside its input");
            n->view_start[i] = st;
            o.d[i] = sz;
          }
          break;
        }
        case VIEW_SLICE_DIM: { // begin / end along one dim, negative indices count from the end (ref: include/dvm.h:445-453)
          const int d = norm_dim(n->view_dim);
          int64_t b = scalar_int(n->scalar_ref), e = scalar_int(n->scalar_ref2);
          if (b < 0) b += in.d[d];
          if (e < 0) e += in.d[d];
          b = std::min<int64_t>(std::max<int64_t>(b, 0), in.d[d]);
          e = std::min<int64_t>(std::max<int64_t>(e, b), in.d[d]);
          n->view_start[d] = b;
          o.d[d] = e - b;
          break;
        }
        default: {             // VIEW_SPLIT: chunk `view_index` of size `view_arg` along a dim, the last one may be smaller
          const int d = norm_dim(n->view_dim);
          const int64_t b = n->view_index * n->view_arg;
          if (n->view_arg <= 0 || b >= in.d[d]) Fail(n, "split chunk outside its input");
          n->view_start[d] = b;
          o.d[d] = std::min<int64_t>(n->view_arg, in.d[d] - b);
          break;
        }
      }
      n->shape = o;
      break;
    }
    case N_ALLREDUCE: {
      n->shape = n->in[0]->shape;
      const int ranks = n->comm ? n->comm->size : 1;
      Shape &s = n->shape;
      if (n->coll == 2) {   // all-gather: the ranks' tensors stacked along the leading dim (src/ops_c.cc:951-962)
        if (s.rank < 1) Fail(n, "all-gather of a scalar");
        s.d[0] *= ranks;
      } else if (n->coll == 1) {   // reduce-scatter: rank r keeps block r of the leading dim (src/ops_c.cc:90-111)
        if (s.rank < 1 || s.d[0] % ranks != 0) Fail(n, "reduce-scatter needs a leading dim divisible by the number of ranks");
        if (s.d[0] == ranks) {
          s.d[0] = 1;
        } else {
          if (s.rank >= kMaxRank) Fail(n, "reduce-scatter result exceeds the rank limit");
          for (int i = s.rank; i > 1; --i) s.d[i] = s.d[i - 1];
          s.d[1] = s.d[0] / ranks;
          s.d[0] = 1;
          s.rank += 1;
        }
      }
      break;
    }
    case N_MATMUL: {
      const Shape &a = n->in[0]->shape, &b = n->in[1]->shape;
      if (a.rank < 2 || b.rank < 2) Fail(n, "matmul operands need rank >= 2");
      int64_t m = n->trans_a ? a.d[a.rank - 1] : a.d[a.rank - 2];
      int64_t ka = n->trans_a ? a.d[a.rank - 2] : a.d[a.rank - 1];
      int64_t kb = n->trans_b ? b.d[b.rank - 1] : b.d[b.rank - 2];
      int64_t nn = n->trans_b ? b.d[b.rank - 2] : b.d[b.rank - 1];
      if (ka != kb) Fail(n, "matmul inner dimensions differ");
      Shape ba, bb;
      ba.rank = a.rank - 2;
      bb.rank = b.rank - 2;
      for (int i = 0; i < ba.rank; ++i) ba.d[i] = a.d[i];
      for (int i = 0; i < bb.rank; ++i) bb.d[i] = b.d[i];
      Shape o = BroadcastShapes(n, ba, bb);
      if (o.rank > 2) Fail(n, "matmul supports at most two batch dims");
      o.d[o.rank++] = m;
      o.d[o.rank++] = nn;
      n->shape = o;
      break;
    }
  }
}

}  // namespace dvm
