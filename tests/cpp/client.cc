// A client of the C++ builder API as a user of the reference writes it (docs/tutorial.md:59-67 of mindspore-ai/dvm):
// Reset -> build -> CodeGen(relocs, workspace allocator) -> Launch(stream).  Built by tests/test_cpp_api.py against
// include/dvm.h and linked with libdvm_b200.so.
//   client dry    builds two graphs, infers shapes, compiles them and prints the disassembly; needs no GPU
//   client run    also launches them on device 0 and checks the results against host arithmetic
#include <cmath>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "dvm.h"

#ifdef WITH_CUDA
#include <cuda_runtime.h>
#define CK(x)                                                             \
  do {                                                                    \
    cudaError_t e_ = (x);                                                 \
    if (e_ != cudaSuccess) {                                              \
      std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); \
      return 2;                                                           \
    }                                                                     \
  } while (0)
#endif

namespace {
struct Workspace : dvm::WsAllocator {
  void *base = nullptr;
  size_t asked = 0;
  void *Alloc(size_t size) override {
    asked = size;
#ifdef WITH_CUDA
    if (size != 0 && base == nullptr) cudaMalloc(&base, size);
#endif
    return base;
  }
};
}  // namespace

int main(int argc, char **argv) {
  const bool run = argc > 1 && std::strcmp(argv[1], "run") == 0;
  const int64_t rows = 37, cols = 515;
  std::vector<int64_t> shape{rows, cols}, dims{1};
  dvm::IntArrayRef shape_ref(shape), dims_ref(dims);

  // graph 1: z = exp(x) * y + 0.5, and the row sums of z (a reduction with a fused elementwise producer)
  dvm::Kernel k;
  k.Reset(dvm::kVector, 0);
  dvm::NDObject *x = k.Load(nullptr, &shape_ref, dvm::kFloat32);
  dvm::NDObject *y = k.Load(nullptr, &shape_ref, dvm::kFloat32);
  dvm::NDObject *z = k.Binary<dvm::kAdd>(k.Binary<dvm::kMul>(k.Unary<dvm::kExp>(x), y), 0.5f);
  dvm::NDObject *sz = k.Store(nullptr, z);
  dvm::NDObject *ss = k.Store(nullptr, k.Reduce<dvm::kSum>(z, &dims_ref, true));
  k.Normalize();
  dvm::IntArrayRef *out_shape = dvm::Kernel::GetShape(ss);
  if (out_shape->size != 2 || out_shape->data[0] != rows || out_shape->data[1] != 1) {
    std::printf("FAIL: inferred shape of the row sums\n");
    return 1;
  }
  // an op outside this backend's path links and throws, as the reference's unsupported combinations do
  bool threw = false;
  try {
    dvm::Kernel bad;
    bad.Reset(dvm::kVector, 0);
    bad.MultiLoad(nullptr, &shape_ref, dvm::kFloat32, nullptr);
  } catch (const std::runtime_error &e) {
    threw = std::strstr(e.what(), "DVM EXCEPTION") != nullptr;
  }
  if (!threw) {
    std::printf("FAIL: MultiLoad did not raise DvmException\n");
    return 1;
  }
  {
    // Concat: two inputs one after the other along the rows (planned as two slabs of one workspace tensor)
    dvm::Kernel c;
    c.Reset(dvm::kVector, 0);
    dvm::NDObject *parts[2] = {c.Load(nullptr, &shape_ref, dvm::kFloat32), c.Load(nullptr, &shape_ref, dvm::kFloat32)};
    dvm::NDObject *cat = c.Concat(parts, 2, 0);
    c.Store(nullptr, c.Binary<dvm::kAdd>(cat, 1.0f));
    c.Normalize();
    dvm::IntArrayRef *cs = dvm::Kernel::GetShape(cat);
    if (cs->size != 2 || cs->data[0] != 2 * rows) {
      std::printf("FAIL: inferred shape of a Concat\n");
      return 1;
    }
    if (c.PreCodeGen() == 0) {
      std::printf("FAIL: a Concat result needs a workspace\n");
      return 1;
    }
  }
  {
    // a view: the transpose of a Load is its memory read through permuted strides (no copy, no workspace)
    dvm::Kernel v;
    v.Reset(dvm::kVector, 0);
    std::vector<int64_t> perm{1, 0};
    dvm::IntArrayRef perm_ref(perm);
    auto t = v.Permute(v.Load(nullptr, &shape_ref, dvm::kFloat32), &perm_ref);
    v.Store(nullptr, v.Binary<dvm::kAdd>(t, 1.0f));
    if (v.PreCodeGen() != 0) {
      std::printf("FAIL: a permuted Load needed a workspace\n");
      return 1;
    }
    dvm::IntArrayRef *ts = v.GetShape(t);
    if (ts->size != 2 || ts->data[0] != cols || ts->data[1] != rows) {
      std::printf("FAIL: inferred shape of the transpose\n");
      return 1;
    }
  }

  std::vector<float> hx(rows * cols), hy(rows * cols), hz(rows * cols), hs(rows);
  for (size_t i = 0; i < hx.size(); ++i) {
    hx[i] = std::sin(0.37f * static_cast<float>(i));
    hy[i] = std::cos(0.11f * static_cast<float>(i));
  }
  void *dx = nullptr, *dy = nullptr, *dz = nullptr, *ds = nullptr;
#ifdef WITH_CUDA
  if (run) {
    CK(cudaSetDevice(0));
    CK(cudaMalloc(&dx, hx.size() * 4));
    CK(cudaMalloc(&dy, hy.size() * 4));
    CK(cudaMalloc(&dz, hz.size() * 4));
    CK(cudaMalloc(&ds, hs.size() * 4));
    CK(cudaMemcpy(dx, hx.data(), hx.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dy, hy.data(), hy.size() * 4, cudaMemcpyHostToDevice));
  }
#endif
  if (!run) {   // any distinct, aligned values stand in for addresses
    dx = reinterpret_cast<void *>(0x10000);
    dy = reinterpret_cast<void *>(0x20000);
    dz = reinterpret_cast<void *>(0x30000);
    ds = reinterpret_cast<void *>(0x40000);
  }
  dvm::RelocEntry relocs[] = {{x, dx}, {y, dy}, {sz, dz}, {ss, ds}};
  Workspace ws;
  k.CodeGen(relocs, 4, &ws);
  const char *das = k.Das();
  if (das == nullptr || std::strstr(das, "Exp") == nullptr) {
    std::printf("FAIL: disassembly misses the graph\n");
    return 1;
  }
  std::printf("%s", das);
  if (!run) {
    std::printf("DRY OK\n");
    return 0;
  }
#ifdef WITH_CUDA
  if (k.Launch(nullptr) != 0) {
    std::printf("FAIL: launch\n");
    return 1;
  }
  CK(cudaDeviceSynchronize());
  CK(cudaMemcpy(hz.data(), dz, hz.size() * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(hs.data(), ds, hs.size() * 4, cudaMemcpyDeviceToHost));
  for (int64_t r = 0; r < rows; ++r) {
    double sum = 0;
    for (int64_t c = 0; c < cols; ++c) {
      const size_t i = r * cols + c;
      const float want = std::exp(hx[i]) * hy[i] + 0.5f;
      if (std::fabs(hz[i] - want) > 1e-5f * (1.0f + std::fabs(want))) {
        std::printf("FAIL: z[%zu] = %g, want %g\n", i, hz[i], want);
        return 1;
      }
      sum += want;
    }
    if (std::fabs(hs[r] - sum) > 1e-4 * (1.0 + std::fabs(sum))) {
      std::printf("FAIL: row sum %lld = %g, want %g\n", static_cast<long long>(r), hs[r], sum);
      return 1;
    }
  }
  // re-launch with new addresses through the relocating Launch overload (include/dvm.h, Launch(relocs, n, workspace, stream))
  void *dz2 = nullptr;
  CK(cudaMalloc(&dz2, hz.size() * 4));
  dvm::RelocEntry again[] = {{x, dy}, {y, dx}, {sz, dz2}, {ss, ds}};
  if (k.Launch(again, 4, ws.base, nullptr) != 0) {
    std::printf("FAIL: relocating launch\n");
    return 1;
  }
  CK(cudaDeviceSynchronize());
  CK(cudaMemcpy(hz.data(), dz2, hz.size() * 4, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < hz.size(); ++i) {
    const float want = std::exp(hy[i]) * hx[i] + 0.5f;
    if (std::fabs(hz[i] - want) > 1e-5f * (1.0f + std::fabs(want))) {
      std::printf("FAIL: after relocation z[%zu] = %g, want %g\n", i, hz[i], want);
      return 1;
    }
  }
  std::printf("RUN OK\n");
  return 0;
#else
  std::printf("built without CUDA\n");
  return 3;
#endif
}
