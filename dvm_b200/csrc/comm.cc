// NCCL binding and the collective launcher (see comm.h).
#include "comm.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include "isa.h"

namespace dvmb {
namespace {

struct NcclApi {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommCount)(const ncclComm_t, int *) = nullptr;
  ncclResult_t (*CommUserRank)(const ncclComm_t, int *) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  std::string why;
};

template <typename F>
bool Bind(void *h, const char *name, F *fn, std::string *why) {
  *fn = reinterpret_cast<F>(dlsym(h, name));
  if (*fn == nullptr) *why = std::string("NCCL symbol missing: ") + name;
  return *fn != nullptr;
}

NcclApi *Api(std::string *err) {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, []() {
    // A copy that the process already holds (a framework's own build) is used first: two NCCL builds in one process
    // clash, because the loader resolves a later library's dependency on "libnccl.so.2" to whichever copy came first.
    // For the same reason a process that will load such a framework later must load it before its first communicator
    // (the Python front-end does that for torch).  DVM_B200_NCCL_LIB names a specific library file.
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_NOLOAD);
      if (api.handle) break;
    }
    if (!api.handle)
      if (const char *path = getenv("DVM_B200_NCCL_LIB")) api.handle = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    for (const char *n : names) {
      if (api.handle) break;
      api.handle = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    }
    if (!api.handle) {
      api.why = std::string("NCCL is not available: ") + dlerror();
      return;
    }
    void *h = api.handle;
    const bool ok = Bind(h, "ncclGetUniqueId", &api.GetUniqueId, &api.why) && Bind(h, "ncclCommInitRank", &api.CommInitRank, &api.why) &&
                    Bind(h, "ncclCommDestroy", &api.CommDestroy, &api.why) && Bind(h, "ncclCommCount", &api.CommCount, &api.why) &&
                    Bind(h, "ncclCommUserRank", &api.CommUserRank, &api.why) && Bind(h, "ncclAllReduce", &api.AllReduce, &api.why) &&
                    Bind(h, "ncclReduceScatter", &api.ReduceScatter, &api.why) && Bind(h, "ncclAllGather", &api.AllGather, &api.why) &&
                    Bind(h, "ncclGetErrorString", &api.GetErrorString, &api.why);
    if (!ok) api.handle = nullptr;
  });
  if (!api.handle) {
    if (err) *err = api.why;
    return nullptr;
  }
  return &api;
}

int Check(NcclApi *api, ncclResult_t r, const char *what, std::string *err) {
  if (r == ncclSuccess) return 0;
  if (err) *err = std::string(what) + ": " + api->GetErrorString(r);
  return 1000 + static_cast<int>(r);
}

bool NcclType(int dtype, ncclDataType_t *t) {
  switch (dtype) {
    case T_F16: *t = ncclFloat16; return true;
    case T_BF16: *t = ncclBfloat16; return true;
    case T_F32: *t = ncclFloat32; return true;
    case T_I32: *t = ncclInt32; return true;
    case T_BOOL: *t = ncclUint8; return true;
    default: return false;
  }
}

size_t ItemBytes(int dtype) { return dtype == T_F32 || dtype == T_I32 ? 4 : (dtype == T_BOOL ? 1 : 2); }

}  // namespace

int CommUniqueId(void *id, std::string *err) {
  NcclApi *api = Api(err);
  if (!api) return 1;
  static_assert(sizeof(ncclUniqueId) == kCommIdBytes, "rendezvous id size");
  return Check(api, api->GetUniqueId(reinterpret_cast<ncclUniqueId *>(id)), "ncclGetUniqueId", err);
}

int CommInitRank(dvm::Communicator *c, const void *id, int rank, int size, std::string *err) {
  NcclApi *api = Api(err);
  if (!api) return 1;
  if (c->nccl && c->owns) api->CommDestroy(static_cast<ncclComm_t>(c->nccl));
  c->nccl = nullptr;
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  ncclComm_t comm = nullptr;
  int rc = Check(api, api->CommInitRank(&comm, size, uid, rank), "ncclCommInitRank", err);
  if (rc != 0) return rc;
  c->nccl = comm;
  c->owns = true;
  c->rank = rank;
  c->size = size;
  c->type = dvm::Comm::kHccl;
  return 0;
}

int CommAdopt(dvm::Communicator *c, void *nccl_comm, std::string *err) {
  NcclApi *api = Api(err);
  if (!api) return 1;
  if (c->nccl && c->owns) api->CommDestroy(static_cast<ncclComm_t>(c->nccl));
  c->nccl = nccl_comm;
  c->owns = false;
  c->type = dvm::Comm::kHccl;
  int rc = Check(api, api->CommCount(static_cast<ncclComm_t>(nccl_comm), &c->size), "ncclCommCount", err);
  if (rc == 0) rc = Check(api, api->CommUserRank(static_cast<ncclComm_t>(nccl_comm), &c->rank), "ncclCommUserRank", err);
  return rc;
}

int RunCollective(const dvm::Communicator *c, CollKind kind, int reduce_type, int dtype, const void *send, void *recv,
                  size_t count, void *stream, std::string *err) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (c == nullptr || c->size <= 1) {
    // one rank: every collective is a copy of the rank's own data (or nothing, in place)
    if (send != recv && count != 0) {
      cudaError_t e = cudaMemcpyAsync(recv, send, count * ItemBytes(dtype), cudaMemcpyDeviceToDevice, s);
      if (e != cudaSuccess) {
        if (err) *err = std::string("collective copy: ") + cudaGetErrorString(e);
        return static_cast<int>(e);
      }
    }
    return 0;
  }
  if (c->nccl == nullptr) {
    if (err) *err = "this communicator has no NCCL communicator behind it (Comm::kDummy plans but cannot launch)";
    return 1;
  }
  NcclApi *api = Api(err);
  if (!api) return 1;
  ncclDataType_t t;
  if (!NcclType(dtype, &t)) {
    if (err) *err = "collective on an unsupported element type";
    return 1;
  }
  const ncclRedOp_t op = reduce_type == dvm::kMax ? ncclMax : (reduce_type == dvm::kMin ? ncclMin : ncclSum);
  ncclComm_t comm = static_cast<ncclComm_t>(c->nccl);
  switch (kind) {
    case COLL_ALL_REDUCE: return Check(api, api->AllReduce(send, recv, count, t, op, comm, s), "ncclAllReduce", err);
    case COLL_REDUCE_SCATTER: return Check(api, api->ReduceScatter(send, recv, count, t, op, comm, s), "ncclReduceScatter", err);
    default: return Check(api, api->AllGather(send, recv, count, t, comm, s), "ncclAllGather", err);
  }
}

}  // namespace dvmb

namespace dvm {

Communicator::~Communicator() {
  if (nccl && owns) {
    std::string err;
    if (auto api = dvmb::Api(&err)) api->CommDestroy(static_cast<ncclComm_t>(nccl));
  }
}

Comm::~Comm() { delete comm_; }

// ref: Comm::Init, src/dvm.cc:1130-1147.  kDummy records rank and size only (plans, never launches).  The other
// types create an NCCL communicator; the ranks of one job find each other through a file that rank 0 writes: its path
// comes from DVM_B200_COMM_ID_FILE (every rank sets the same path, the file must not exist beforehand).  Callers that
// already own a communicator, or another way to pass 128 bytes around, use Init(void *) or the C ABI instead.
bool Comm::Init(int rank_id, int rank_size, int comm_type, const uint32_t *) {
  if (comm_ == nullptr) comm_ = new Communicator();
  comm_->rank = rank_id;
  comm_->size = rank_size;
  comm_->type = comm_type;
  if (comm_type == kDummy) return true;
  std::string err;
  unsigned char id[dvmb::kCommIdBytes];
  if (rank_size > 1) {
    const char *path = getenv("DVM_B200_COMM_ID_FILE");
    if (path == nullptr) return false;
    if (rank_id == 0) {
      if (dvmb::CommUniqueId(id, &err) != 0) return false;
      const std::string tmp = std::string(path) + ".tmp";
      FILE *f = fopen(tmp.c_str(), "wb");
      if (!f) return false;
      const bool ok = fwrite(id, 1, sizeof(id), f) == sizeof(id);
      fclose(f);
      if (!ok || rename(tmp.c_str(), path) != 0) return false;
    } else {
      bool got = false;
      for (int i = 0; i < 6000 && !got; ++i) {   // up to a minute
        if (FILE *f = fopen(path, "rb")) {
          got = fread(id, 1, sizeof(id), f) == sizeof(id);
          fclose(f);
        }
        if (!got) std::this_thread::sleep_for(std::chrono::milliseconds(10));
      }
      if (!got) return false;
    }
  } else if (dvmb::CommUniqueId(id, &err) != 0) {
    return false;
  }
  return dvmb::CommInitRank(comm_, id, rank_id, rank_size, &err) == 0;
}

// ref: Comm::Init(void *hccl_comm), src/dvm.cc:1149-1156: use the caller's communicator (here an ncclComm_t).
void Comm::Init(void *nccl_comm) {
  if (comm_ == nullptr) comm_ = new Communicator();
  std::string err;
  if (dvmb::CommAdopt(comm_, nccl_comm, &err) != 0) DvmException(err.c_str());
}

}  // namespace dvm
