// Collectives of the hot path: the K-split MatMul's all-reduce (and the reduce-scatter / all-gather pair it is
// lowered to), on NCCL over NVLink.  Stands in for the reference's Communicator family (MemoryComm / HcclComm,
// src/comm.cc:406-587, include/dvm.h:219-231) and its collective ops (src/ops_c.cc:90-645).
//
// NCCL is bound at run time (dlopen of libnccl.so.2 at the first communicator), not at link time: loading this
// library alone never pulls a second NCCL into a process whose framework already carries its own, and hosts
// without NCCL can still build, plan and run single-device kernels.
#ifndef DVM_B200_COMM_H_
#define DVM_B200_COMM_H_

#include <cstddef>
#include <cstdint>
#include <string>

#include "../../include/dvm.h"

namespace dvm {

class Communicator {
 public:
  int rank = 0, size = 1, type = Comm::kDummy;
  void *nccl = nullptr;   // ncclComm_t; null for a dummy communicator (planning only)
  bool owns = false;      // created here (destroyed with the object) or adopted from the caller
  ~Communicator();
};

}  // namespace dvm

namespace dvmb {

enum CollKind : uint32_t { COLL_ALL_REDUCE = 0, COLL_REDUCE_SCATTER, COLL_ALL_GATHER };
constexpr size_t kCommIdBytes = 128;   // sizeof(ncclUniqueId)

// Fills `id` (kCommIdBytes) with a fresh rendezvous id; rank 0 calls it and hands the bytes to the other ranks.
int CommUniqueId(void *id, std::string *err);
// Creates the NCCL communicator of `rank` out of `size` on the current device (collective over all ranks).
int CommInitRank(dvm::Communicator *c, const void *id, int rank, int size, std::string *err);
// Uses a communicator the caller owns (an ncclComm_t of its framework).
int CommAdopt(dvm::Communicator *c, void *nccl_comm, std::string *err);
// Enqueues one collective on `stream`.  `count` is the element count NCCL's call takes (all-reduce: elements of the
// tensor; reduce-scatter / all-gather: elements per rank).  A communicator of size 1 copies (or does nothing in place).
int RunCollective(const dvm::Communicator *c, CollKind kind, int reduce_type, int dtype, const void *send, void *recv,
                  size_t count, void *stream, std::string *err);

}  // namespace dvmb

#endif  // DVM_B200_COMM_H_
