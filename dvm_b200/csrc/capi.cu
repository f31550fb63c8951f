// C ABI over the C++ builder (include/dvm_c.h).  Exceptions never cross this boundary: they are turned
// into an error return plus a thread-local message.
#include <cuda_runtime.h>

#include <chrono>
#include <cstring>
#include <exception>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/dvm.h"
#include "../../include/dvm_c.h"
#include "comm.h"
#include "graph.h"
#include "runtime.h"
#include "vm_launch.h"
#include "mm_launch.h"

struct dvm_int_array {
  std::vector<int64_t> data;
  dvm::IntArrayRef ref;
  void sync() {
    ref.data = data.data();
    ref.size = data.size();
  }
};

struct dvm_scalar {
  dvm::ScalarRef ref;
};

struct dvm_comm : dvm::Comm {
  dvm::Communicator *&impl() { return comm_; }   // (comm_ is the protected member of dvm::Comm)
};

struct dvm_kernel {
  dvm::Kernel kernel;
  double last_jit_us = 0.0;
};

// Kernel::Clone's helper over the C handles: registered pairs first, copies owned by the map for everything else
struct dvm_clone_map : dvm::CloneHelper {
  std::unordered_map<const void *, void *> refs;
  std::unordered_map<const dvm::NDObject *, dvm::NDObject *> ops;
  std::vector<std::unique_ptr<dvm_int_array>> own_arrays;
  std::vector<std::unique_ptr<dvm_scalar>> own_scalars;
  dvm::IntArrayRef *GetClone(dvm::IntArrayRef *r) override {
    auto it = refs.find(r);
    if (it != refs.end()) return static_cast<dvm::IntArrayRef *>(it->second);
    auto a = std::make_unique<dvm_int_array>();
    a->data.assign(r->data, r->data + r->size);
    a->sync();
    dvm::IntArrayRef *out = &a->ref;
    refs[r] = out;
    own_arrays.push_back(std::move(a));
    return out;
  }
  dvm::ScalarRef *GetClone(dvm::ScalarRef *r) override {
    auto it = refs.find(r);
    if (it != refs.end()) return static_cast<dvm::ScalarRef *>(it->second);
    auto s = std::make_unique<dvm_scalar>();
    s->ref = *r;
    dvm::ScalarRef *out = &s->ref;
    refs[r] = out;
    own_scalars.push_back(std::move(s));
    return out;
  }
  dvm::NDObject *GetClone(dvm::NDObject *op) override {
    auto it = ops.find(op);
    return it == ops.end() ? nullptr : it->second;
  }
  void SetClone(dvm::NDObject *op, dvm::NDObject *clone) override { ops[op] = clone; }
};

namespace {

thread_local std::string g_error;

template <typename F>
auto Guard(F &&f, decltype(f()) fail) -> decltype(f()) {
  try {
    g_error.clear();
    return f();
  } catch (const std::exception &e) {
    g_error = e.what();
  } catch (...) {
    g_error = "unknown error";
  }
  return fail;
}

inline dvm::NDObject *N(dvm_object *o) { return reinterpret_cast<dvm::NDObject *>(o); }
inline dvm_object *O(dvm::NDObject *n) { return reinterpret_cast<dvm_object *>(n); }

struct CallbackAlloc : dvm::WsAllocator {
  dvm_ws_alloc_fn fn;
  void *user;
  size_t asked = 0;
  void *Alloc(size_t size) override {
    asked = size;
    return fn ? fn(size, user) : nullptr;
  }
};

// Scratch for dvm_launch_static_scratch(): lives in the library's device image, so every GPU that loads the
// library holds these bytes until the process exits.  Host code may not pass the symbol itself to a kernel;
// the device address is looked up once per device with cudaGetSymbolAddress.
constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
void *g_static_scratch_addr[64] = {nullptr};

int CudaCheck(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return 0;
  g_error = std::string(what) + ": " + cudaGetErrorString(e);
  return static_cast<int>(e);
}

template <typename S>
dvm::NDObject *BinaryScalarDispatch(dvm::Kernel &k, int op, dvm::NDObject *x, S v, bool scalar_is_lhs) {
  return scalar_is_lhs ? k.Binary(op, v, x) : k.Binary(op, x, v);
}

}  // namespace

extern "C" {

const char *dvm_last_error(void) { return g_error.c_str(); }
const char *dvm_version(void) { return "dvm-b200 0.1 (sm_100a)"; }

dvm_int_array *dvm_int_array_new(const int64_t *data, size_t size) {
  auto a = new dvm_int_array();
  if (size) a->data.assign(data, data + size);
  a->sync();
  return a;
}
int dvm_int_array_update(dvm_int_array *a, const int64_t *data, size_t size) {
  a->data.assign(data, data + size);
  a->sync();
  return 0;
}
size_t dvm_int_array_size(const dvm_int_array *a) { return a->data.size(); }
const int64_t *dvm_int_array_data(const dvm_int_array *a) { return a->data.data(); }
void dvm_int_array_free(dvm_int_array *a) { delete a; }

dvm_scalar *dvm_scalar_new(void) {
  auto s = new dvm_scalar();
  s->ref.type = dvm::kDataTypeEnd;
  s->ref.i64 = 0;
  return s;
}
void dvm_scalar_set_f32(dvm_scalar *s, float v) { s->ref = v; }
void dvm_scalar_set_i64(dvm_scalar *s, int64_t v) { s->ref = v; }
void dvm_scalar_free(dvm_scalar *s) { delete s; }

dvm_kernel *dvm_kernel_new(int kernel_type, uint32_t flags) {
  return Guard(
    [&]() {
      auto k = std::make_unique<dvm_kernel>();
      k->kernel.Reset(static_cast<dvm::KernelType>(kernel_type), flags);
      return k.release();
    },
    static_cast<dvm_kernel *>(nullptr));
}
int dvm_kernel_reset(dvm_kernel *k, int kernel_type, uint32_t flags) {
  return Guard([&]() { k->kernel.Reset(static_cast<dvm::KernelType>(kernel_type), flags); return 0; }, 1);
}
void dvm_kernel_free(dvm_kernel *k) { delete k; }
int dvm_set_name_hint(dvm_kernel *k, const char *name) {
  return Guard([&]() { k->kernel.SetNameHint(name, name); return 0; }, 1);
}

#define DVM_OBJ_GUARD(EXPR) Guard([&]() { return O(EXPR); }, static_cast<dvm_object *>(nullptr))

dvm_object *dvm_load(dvm_kernel *k, void *addr, dvm_int_array *shape, int dtype) {
  return DVM_OBJ_GUARD(k->kernel.Load(addr, &shape->ref, static_cast<dvm::DataType>(dtype)));
}
dvm_object *dvm_store(dvm_kernel *k, void *addr, dvm_object *input) { return DVM_OBJ_GUARD(k->kernel.Store(addr, N(input))); }
dvm_object *dvm_load_strided(dvm_kernel *k, void *addr, dvm_int_array *shape, dvm_int_array *stride, int dtype) {
  return DVM_OBJ_GUARD(k->kernel.Load(addr, &shape->ref, &stride->ref, static_cast<dvm::DataType>(dtype)));
}
dvm_object *dvm_slice_load(dvm_kernel *k, void *addr, dvm_int_array *shape, dvm_int_array *start, dvm_int_array *size, int dtype) {
  return DVM_OBJ_GUARD(k->kernel.SliceLoad(addr, &shape->ref, &start->ref, &size->ref, static_cast<dvm::DataType>(dtype)));
}
dvm_object *dvm_strided_slice_load(dvm_kernel *k, void *addr, dvm_int_array *shape, dvm_int_array *start, dvm_int_array *end,
                                   dvm_int_array *step, int dtype) {
  return DVM_OBJ_GUARD(
    k->kernel.StridedSliceLoad(addr, &shape->ref, &start->ref, &end->ref, &step->ref, static_cast<dvm::DataType>(dtype)));
}
dvm_object *dvm_elem_any(dvm_kernel *k, dvm_object *input) { return DVM_OBJ_GUARD(k->kernel.ElemAny(N(input))); }
dvm_object *dvm_pad_store(dvm_kernel *k, void *addr, dvm_object *input, int64_t pad_size) {
  return DVM_OBJ_GUARD(k->kernel.PadStore(addr, N(input), pad_size));
}
dvm_object *dvm_store_strided(dvm_kernel *k, void *addr, dvm_object *input, dvm_int_array *stride) {
  return DVM_OBJ_GUARD(k->kernel.Store(addr, N(input), &stride->ref));
}
dvm_object *dvm_unary(dvm_kernel *k, int unary_type, dvm_object *input) {
  return DVM_OBJ_GUARD(k->kernel.Unary(unary_type, N(input)));
}
dvm_object *dvm_binary(dvm_kernel *k, int binary_type, dvm_object *lhs, dvm_object *rhs) {
  return DVM_OBJ_GUARD(k->kernel.Binary(binary_type, N(lhs), N(rhs)));
}
dvm_object *dvm_binary_f32(dvm_kernel *k, int binary_type, dvm_object *x, float v, int scalar_is_lhs) {
  return DVM_OBJ_GUARD(BinaryScalarDispatch(k->kernel, binary_type, N(x), v, scalar_is_lhs != 0));
}
dvm_object *dvm_binary_i64(dvm_kernel *k, int binary_type, dvm_object *x, int64_t v, int scalar_is_lhs) {
  return DVM_OBJ_GUARD(BinaryScalarDispatch(k->kernel, binary_type, N(x), v, scalar_is_lhs != 0));
}
dvm_object *dvm_binary_ref(dvm_kernel *k, int binary_type, dvm_object *x, dvm_scalar *v, int scalar_is_lhs) {
  return DVM_OBJ_GUARD(BinaryScalarDispatch(k->kernel, binary_type, N(x), &v->ref, scalar_is_lhs != 0));
}
dvm_object *dvm_reduce(dvm_kernel *k, int reduce_type, dvm_object *input, dvm_int_array *dims, int keepdims) {
  return DVM_OBJ_GUARD(k->kernel.Reduce(reduce_type, N(input), &dims->ref, keepdims != 0));
}
dvm_object *dvm_select(dvm_kernel *k, dvm_object *cond, dvm_object *lhs, dvm_object *rhs) {
  return DVM_OBJ_GUARD(k->kernel.Select(N(cond), N(lhs), N(rhs)));
}
dvm_object *dvm_cast(dvm_kernel *k, dvm_object *input, int dtype) {
  return DVM_OBJ_GUARD(k->kernel.Cast(N(input), static_cast<dvm::DataType>(dtype)));
}
dvm_object *dvm_broadcast(dvm_kernel *k, dvm_object *input, dvm_int_array *shape) {
  return DVM_OBJ_GUARD(k->kernel.Broadcast(N(input), &shape->ref));
}
dvm_object *dvm_full_f32(dvm_kernel *k, float v, dvm_int_array *shape, int dtype) {
  return DVM_OBJ_GUARD(k->kernel.Broadcast(v, &shape->ref, static_cast<dvm::DataType>(dtype)));
}
dvm_object *dvm_full_i64(dvm_kernel *k, int64_t v, dvm_int_array *shape, int dtype) {
  return DVM_OBJ_GUARD(k->kernel.Broadcast(v, &shape->ref, static_cast<dvm::DataType>(dtype)));
}
dvm_object *dvm_full_ref(dvm_kernel *k, dvm_scalar *v, dvm_int_array *shape, int dtype) {
  return DVM_OBJ_GUARD(k->kernel.Broadcast(&v->ref, &shape->ref, static_cast<dvm::DataType>(dtype)));
}
dvm_object *dvm_reshape(dvm_kernel *k, dvm_object *input, dvm_int_array *shape) {
  return DVM_OBJ_GUARD(k->kernel.Reshape(N(input), &shape->ref));
}
dvm_object *dvm_permute(dvm_kernel *k, dvm_object *input, dvm_int_array *dims) {
  return DVM_OBJ_GUARD(k->kernel.Permute(N(input), &dims->ref));
}
dvm_object *dvm_slice(dvm_kernel *k, dvm_object *input, dvm_int_array *start, dvm_int_array *size) {
  return DVM_OBJ_GUARD(k->kernel.Slice(N(input), &start->ref, &size->ref));
}
dvm_object *dvm_slice_dim(dvm_kernel *k, dvm_object *input, int dim, dvm_scalar *begin, dvm_scalar *end) {
  return DVM_OBJ_GUARD(k->kernel.Slice(N(input), dim, &begin->ref, &end->ref));
}
dvm_object *dvm_split_chunk(dvm_kernel *k, dvm_object *input, int dim, int64_t split_size, size_t split_num, size_t index) {
  return Guard(
    [&]() {
      if (index >= split_num) dvm::DvmException("dvm_split_chunk: index outside the split");
      // one Kernel::Split call per distinct (input, dim, size, num) would do; a front-end asks chunk by chunk
      return O(k->kernel.Split(N(input), dim, split_size, split_num)[index]);
    },
    static_cast<dvm_object *>(nullptr));
}
dvm_clone_map *dvm_clone_map_new(void) { return new (std::nothrow) dvm_clone_map(); }
void dvm_clone_map_free(dvm_clone_map *m) { delete m; }
int dvm_clone_map_int_array(dvm_clone_map *m, dvm_int_array *base, dvm_int_array *clone) {
  return Guard([&]() {
    clone->data = base->data;
    clone->sync();
    m->refs[&base->ref] = &clone->ref;
    return 0;
  }, 1);
}
int dvm_clone_map_scalar(dvm_clone_map *m, dvm_scalar *base, dvm_scalar *clone) {
  return Guard([&]() {
    clone->ref = base->ref;
    m->refs[&base->ref] = &clone->ref;
    return 0;
  }, 1);
}
int dvm_kernel_clone(dvm_kernel *dst, dvm_kernel *base, dvm_clone_map *m) {
  return Guard([&]() {
    dst->kernel.Clone(base->kernel, *m);
    return 0;
  }, 1);
}
dvm_object *dvm_clone_map_object(dvm_clone_map *m, dvm_object *base) { return O(m->GetClone(N(base))); }
dvm_object *dvm_concat(dvm_kernel *k, dvm_object **inputs, size_t input_num, int dim) {
  return Guard(
    [&]() {
      std::vector<dvm::NDObject *> in(input_num);
      for (size_t i = 0; i < input_num; ++i) in[i] = N(inputs[i]);
      return O(k->kernel.Concat(in.data(), input_num, dim));
    },
    static_cast<dvm_object *>(nullptr));
}
dvm_object *dvm_copy(dvm_kernel *k, dvm_object *input) { return DVM_OBJ_GUARD(k->kernel.Copy(N(input))); }
dvm_object *dvm_matmul(dvm_kernel *k, dvm_object *lhs, dvm_object *rhs, int trans_a, int trans_b, dvm_object *bias) {
  return DVM_OBJ_GUARD(k->kernel.MatMul(N(lhs), N(rhs), trans_a != 0, trans_b != 0, bias ? N(bias) : nullptr));
}

dvm_comm *dvm_comm_new(void) { return new dvm_comm(); }
void dvm_comm_free(dvm_comm *c) { delete c; }
size_t dvm_comm_id_bytes(void) { return dvmb::kCommIdBytes; }
int dvm_comm_unique_id(void *id, size_t bytes) {
  if (bytes < dvmb::kCommIdBytes) {
    g_error = "the id buffer is smaller than dvm_comm_id_bytes()";
    return 1;
  }
  g_error.clear();
  return dvmb::CommUniqueId(id, &g_error);
}
int dvm_comm_init_rank(dvm_comm *c, const void *id, size_t bytes, int rank, int size) {
  if (bytes < dvmb::kCommIdBytes || rank < 0 || rank >= size) {
    g_error = "dvm_comm_init_rank: bad id size or rank";
    return 1;
  }
  g_error.clear();
  if (c->impl() == nullptr) c->impl() = new dvm::Communicator();
  return dvmb::CommInitRank(c->impl(), id, rank, size, &g_error);
}
int dvm_comm_init_dummy(dvm_comm *c, int rank, int size) {
  return Guard([&]() { return c->Init(rank, size, dvm::Comm::kDummy) ? 0 : 1; }, 1);
}
int dvm_comm_adopt(dvm_comm *c, void *nccl_comm) {
  return Guard([&]() { c->Init(nccl_comm); return 0; }, 1);
}
int dvm_comm_rank(const dvm_comm *c) { return c->GetImpl() ? c->GetImpl()->rank : 0; }
int dvm_comm_size(const dvm_comm *c) { return c->GetImpl() ? c->GetImpl()->size : 1; }
dvm_object *dvm_allreduce(dvm_kernel *k, int reduce_type, dvm_object *input, dvm_comm *c) {
  return DVM_OBJ_GUARD(k->kernel.AllReduce(reduce_type, N(input), c));
}

dvm_object *dvm_allgather(dvm_kernel *k, dvm_object *input, dvm_comm *c) { return DVM_OBJ_GUARD(k->kernel.AllGather(N(input), c)); }
dvm_object *dvm_reducescatter(dvm_kernel *k, dvm_object *input, dvm_comm *c) {
  return DVM_OBJ_GUARD(k->kernel.ReduceScatter(N(input), c));
}

int dvm_sequence_add(dvm_kernel *k, int kernel_type, uint32_t flags) {
  return Guard([&]() { k->kernel.SequenceAdd(static_cast<dvm::KernelType>(kernel_type), flags); return 0; }, 1);
}
int dvm_parallel_add(dvm_kernel *k, int kernel_type, uint32_t flags, size_t thread_limit) {
  return Guard([&]() { k->kernel.ParallelAdd(static_cast<dvm::KernelType>(kernel_type), flags, thread_limit); return 0; }, 1);
}
int dvm_spec_next(dvm_kernel *k) {
  return Guard([&]() { k->kernel.SpecNext(); return 0; }, 1);
}
int dvm_set_store_inplace(dvm_kernel *k, dvm_object *store) {
  return Guard([&]() { k->kernel.SetStoreInplace(N(store)); return 0; }, 1);
}

int dvm_normalize(dvm_kernel *k) {
  return Guard([&]() { k->kernel.Normalize(); return 0; }, 1);
}

int dvm_pre_codegen(dvm_kernel *k, size_t *workspace_bytes) {
  return Guard(
    [&]() {
      auto t0 = std::chrono::steady_clock::now();
      size_t ws = k->kernel.PreCodeGen();
      k->last_jit_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
      if (workspace_bytes) *workspace_bytes = ws;
      return 0;
    },
    1);
}

int dvm_codegen(dvm_kernel *k, const dvm_reloc *relocs, size_t reloc_size, dvm_ws_alloc_fn alloc, void *user) {
  return Guard(
    [&]() {
      static_assert(sizeof(dvm_reloc) == sizeof(dvm::RelocEntry), "dvm_reloc must match dvm::RelocEntry");
      CallbackAlloc cb;
      cb.fn = alloc;
      cb.user = user;
      auto t0 = std::chrono::steady_clock::now();
      k->kernel.Normalize();
      k->kernel.CodeGen(reinterpret_cast<const dvm::RelocEntry *>(relocs), reloc_size, &cb);
      k->last_jit_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
      return 0;
    },
    1);
}

int dvm_launch(dvm_kernel *k, void *stream) {
  return Guard([&]() { return k->kernel.Launch(stream); }, -1);
}

int dvm_launch_reloc(dvm_kernel *k, const dvm_reloc *relocs, size_t reloc_size, void *workspace, void *stream) {
  return Guard(
    [&]() { return k->kernel.Launch(reinterpret_cast<const dvm::RelocEntry *>(relocs), reloc_size, workspace, stream); },
    -1);
}

size_t dvm_static_scratch_capacity(void) { return kStaticScratchBytes; }

int dvm_launch_static_scratch(dvm_kernel *k, const dvm_reloc *relocs, size_t reloc_size, void *stream) {
  return Guard(
    [&]() {
      // the workspace the program compiled for the CURRENT shapes needs (any call that compiles - code generation, a
      // listing, an inspection after a shape update - may have changed it, so it is read here and never cached)
      const dvm::VKernel *vk = k->kernel.GetImpl();
      if (vk == nullptr || !vk->compiled_) {
        g_error = "dvm_launch_static_scratch needs dvm_pre_codegen() or dvm_codegen() for the current shapes first";
        return -5;
      }
      if (vk->ws_bytes_ > kStaticScratchBytes) {
        char buf[160];
        snprintf(buf, sizeof(buf), "this kernel needs %zu bytes of workspace; the static scratch holds %zu", vk->ws_bytes_,
                 kStaticScratchBytes);
        g_error = buf;
        return -2;
      }
      int dev = -1;
      if (CudaCheck(cudaGetDevice(&dev), "cudaGetDevice") != 0) return -3;
      if (dev < 0 || dev >= 64) {
        g_error = "device index outside 0..63";
        return -3;
      }
      if (g_static_scratch_addr[dev] == nullptr) {
        // first call on this device: resolve the device address of the scratch array
        void *p = nullptr;
        if (CudaCheck(cudaGetSymbolAddress(&p, g_static_scratch), "cudaGetSymbolAddress(static scratch)") != 0) return -4;
        g_static_scratch_addr[dev] = p;
      }
      return k->kernel.Launch(reinterpret_cast<const dvm::RelocEntry *>(relocs), reloc_size, g_static_scratch_addr[dev], stream);
    },
    -1);
}

double dvm_last_jit_us(const dvm_kernel *k) { return k->last_jit_us; }

int dvm_object_rank(const dvm_object *o) { return reinterpret_cast<const dvm::NDObject *>(o)->shape.rank; }
int64_t dvm_object_dim(const dvm_object *o, int i) {
  const dvm::NDObject *n = reinterpret_cast<const dvm::NDObject *>(o);
  // (a PadStore reports the shape of its buffer: rows longer by the pad)
  return n->shape.d[i] + (n->kind == dvm::N_STORE && i == n->shape.rank - 1 ? n->pad_size : 0);
}
int dvm_object_dtype(const dvm_object *o) { return reinterpret_cast<const dvm::NDObject *>(o)->dtype; }

const char *dvm_dump(dvm_kernel *k) { return Guard([&]() { return k->kernel.Dump(); }, ""); }
const char *dvm_dump_r(dvm_kernel *k) { return Guard([&]() { return k->kernel.DumpR(); }, ""); }
const char *dvm_das(dvm_kernel *k) { return Guard([&]() { return k->kernel.Das(); }, ""); }
const char *dvm_inspect(dvm_kernel *k) { return Guard([&]() { return k->kernel.Inspect(); }, ""); }

int dvm_rt_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
int dvm_rt_set_device(int dev) { return CudaCheck(cudaSetDevice(dev), "cudaSetDevice"); }
int dvm_rt_sm_count(void) {
  return Guard(
    [&]() {
      dvmb::Runtime::Get().EnsureInit();
      return dvmb::Runtime::Get().sm_count();
    },
    0);
}
void *dvm_rt_malloc(size_t bytes) {
  void *p = nullptr;
  if (CudaCheck(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc") != 0) return nullptr;
  return p;
}
int dvm_rt_free(void *p) { return CudaCheck(cudaFree(p), "cudaFree"); }
int dvm_rt_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream) {
  return CudaCheck(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)), "H2D copy");
}
int dvm_rt_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream) {
  return CudaCheck(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)), "D2H copy");
}
int dvm_rt_memset(void *dst, int value, size_t bytes, void *stream) {
  return CudaCheck(cudaMemsetAsync(dst, value, bytes, static_cast<cudaStream_t>(stream)), "memset");
}
// Reads (and clears) the status records of the device interpreters: a bounded device wait that expired (the kernel
// then ran to its end with wrong results) is reported here as an error.  Does not wait for anything.
int dvm_rt_check_status(void) {
  const unsigned int sv = dvmb::ReadVectorStatus(), sm = dvmb::ReadMatMulStatus(), sa = dvmb::ReadAttentionStatus();
  if ((sv | sm | sa) != 0) {
    char buf[160];
    snprintf(buf, sizeof(buf), "a bounded device wait expired (vector 0x%08x, matmul 0x%08x, attention 0x%08x)", sv, sm, sa);
    g_error = buf;
    return -1;
  }
  return 0;
}
// Waits for the stream, then reports like dvm_rt_check_status().
int dvm_rt_sync(void *stream) {
  int rc = CudaCheck(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), "stream sync");
  if (rc != 0) return rc;
  return dvm_rt_check_status();
}
int dvm_rt_selftest_wait_expiry(unsigned int limit_ms, void *stream) {
  return Guard(
    [&]() {
      dvmb::Runtime::Get().EnsureInit();
      return dvmb::LaunchWaitSelfTest(limit_ms, stream);
    },
    -1);
}
void *dvm_rt_host_alloc(size_t bytes) {
  void *p = nullptr;
  if (CudaCheck(cudaMallocHost(&p, bytes ? bytes : 1), "cudaMallocHost") != 0) return nullptr;
  return p;
}
int dvm_rt_host_free(void *p) { return CudaCheck(cudaFreeHost(p), "cudaFreeHost"); }

int dvm_perf(dvm_kernel *k, int warmup, int reps, void *stream, float *min_us, float *max_us, float *mean_us) {
  return Guard(
    [&]() {
      cudaStream_t s = static_cast<cudaStream_t>(stream);
      cudaEvent_t e0, e1;
      if (CudaCheck(cudaEventCreate(&e0), "event") || CudaCheck(cudaEventCreate(&e1), "event")) return 1;
      for (int i = 0; i < warmup; ++i) {
        int rc = k->kernel.Launch(stream);
        if (rc != 0) return rc;
      }
      float lo = 1e30f, hi = 0.0f, sum = 0.0f;
      for (int i = 0; i < reps; ++i) {
        cudaEventRecord(e0, s);
        int rc = k->kernel.Launch(stream);
        cudaEventRecord(e1, s);
        if (rc != 0) return rc;
        if (CudaCheck(cudaEventSynchronize(e1), "event sync")) return 1;
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, e0, e1);
        float us = ms * 1000.0f;
        lo = us < lo ? us : lo;
        hi = us > hi ? us : hi;
        sum += us;
      }
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
      if (min_us) *min_us = lo;
      if (max_us) *max_us = hi;
      if (mean_us) *mean_us = reps > 0 ? sum / reps : 0.0f;
      return 0;
    },
    1);
}

// Per-stage device times of one kernel: every launch / collective of the plan bracketed by its own pair of events.
int dvm_perf_stages(dvm_kernel *k, int warmup, int reps, void *stream, float *mean_us, size_t capacity, size_t *stages) {
  return Guard(
    [&]() {
      dvm::VKernel *vk = k->kernel.GetImpl();
      if (vk == nullptr || !vk->compiled_) dvm::DvmException("dvm_perf_stages needs a generated kernel");
      const size_t n = vk->stages_.size();
      if (stages) *stages = n;
      if (n > capacity) dvm::DvmException("dvm_perf_stages: the output array is too small");
      cudaStream_t s = static_cast<cudaStream_t>(stream);
      std::vector<cudaEvent_t> ev(n + 1);
      for (auto &e : ev)
        if (CudaCheck(cudaEventCreate(&e), "event")) return 1;
      std::vector<double> sum(n, 0.0);
      for (int it = 0; it < warmup + reps; ++it) {
        cudaEventRecord(ev[0], s);
        for (size_t i = 0; i < n; ++i) {
          int rc = vk->LaunchStage(i, stream);
          if (rc != 0) return rc;
          cudaEventRecord(ev[i + 1], s);
        }
        if (CudaCheck(cudaEventSynchronize(ev[n]), "event sync")) return 1;
        if (it < warmup) continue;
        for (size_t i = 0; i < n; ++i) {
          float ms = 0.0f;
          cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
          sum[i] += ms * 1000.0;
        }
      }
      for (auto &e : ev) cudaEventDestroy(e);
      for (size_t i = 0; i < n; ++i) mean_us[i] = reps > 0 ? static_cast<float>(sum[i] / reps) : 0.0f;
      return 0;
    },
    1);
}

}  // extern "C"
