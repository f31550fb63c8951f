/* dvm-b200 C ABI: the drop-in boundary of the fused-operator path.
 *
 * Plain C entry points (opaque handles, pointers and sizes only) over the C++ builder in dvm.h.  These are
 * the functions a foreign-function binding of the reference's operator path would bind: each one cites the
 * reference interface it replaces, either the C++ builder (`include/dvm.h:<line>` of mindspore-ai/dvm) or
 * the method of its Python extension module (`src/pybind_api.cc:<line>`, `include/dvm_py.h:<line>`).
 *
 * Error convention: functions returning a pointer return NULL on failure, functions returning int return
 * 0 on success and non-zero on failure; dvm_last_error() then gives the message of the DvmException that
 * was raised (thread-local).  A NULL result from dvm_reduce() with an empty error string mirrors the
 * reference's "unsupported dtype" null result (src/dvm.cc:1538-1540).
 *
 * There is no CPU execution path behind this ABI: compute entry points fail when no sm_100 device is
 * usable.
 */
#ifndef DVM_B200_DVM_C_H_
#define DVM_B200_DVM_C_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DVM_C_API __attribute__((visibility("default")))

typedef struct dvm_kernel dvm_kernel;         /* a dvm::Kernel plus what it borrowed through this ABI */
typedef struct dvm_object dvm_object;         /* dvm::NDObject, owned by its kernel */
typedef struct dvm_int_array dvm_int_array;   /* owning int64 array with a stable dvm::IntArrayRef */
typedef struct dvm_scalar dvm_scalar;         /* owning dvm::ScalarRef */

/* (load/store object, device address): same layout as dvm::RelocEntry (include/dvm.h:201-206). */
typedef struct dvm_reloc {
  dvm_object *io;
  void *addr;
} dvm_reloc;

/* Workspace callback, the C form of dvm::WsAllocator (include/dvm.h:208-210). */
typedef void *(*dvm_ws_alloc_fn)(size_t size, void *user);

DVM_C_API const char *dvm_last_error(void);
DVM_C_API const char *dvm_version(void);

/* ---- borrowed shape / scalar holders (IntArrayRefPy and ScalarRefPy, include/dvm_py.h:40-92) ---- */
DVM_C_API dvm_int_array *dvm_int_array_new(const int64_t *data, size_t size);
DVM_C_API int dvm_int_array_update(dvm_int_array *a, const int64_t *data, size_t size);
DVM_C_API size_t dvm_int_array_size(const dvm_int_array *a);
DVM_C_API const int64_t *dvm_int_array_data(const dvm_int_array *a);
DVM_C_API void dvm_int_array_free(dvm_int_array *a);
DVM_C_API dvm_scalar *dvm_scalar_new(void);
DVM_C_API void dvm_scalar_set_f32(dvm_scalar *s, float v);
DVM_C_API void dvm_scalar_set_i64(dvm_scalar *s, int64_t v);
DVM_C_API void dvm_scalar_free(dvm_scalar *s);

/* ---- kernel lifecycle: Kernel::Kernel / Reset / ~Kernel (include/dvm.h:238-252) ---- */
DVM_C_API dvm_kernel *dvm_kernel_new(int kernel_type, uint32_t flags);
DVM_C_API int dvm_kernel_reset(dvm_kernel *k, int kernel_type, uint32_t flags);
DVM_C_API void dvm_kernel_free(dvm_kernel *k);
DVM_C_API int dvm_set_name_hint(dvm_kernel *k, const char *name);               /* include/dvm.h:266 */

/* ---- graph building ---- */
DVM_C_API dvm_object *dvm_load(dvm_kernel *k, void *addr, dvm_int_array *shape, int dtype);  /* dvm.h:276 */
DVM_C_API dvm_object *dvm_store(dvm_kernel *k, void *addr, dvm_object *input);               /* dvm.h:331 */
/* views: a tensor that is not contiguous in memory, one element stride per dim of its shape (dvm.h:294, 339) */
DVM_C_API dvm_object *dvm_load_strided(dvm_kernel *k, void *addr, dvm_int_array *shape, dvm_int_array *stride, int dtype);
DVM_C_API dvm_object *dvm_store_strided(dvm_kernel *k, void *addr, dvm_object *input, dvm_int_array *stride);
DVM_C_API dvm_object *dvm_unary(dvm_kernel *k, int unary_type, dvm_object *input);           /* dvm.h:372 */
DVM_C_API dvm_object *dvm_binary(dvm_kernel *k, int binary_type, dvm_object *lhs, dvm_object *rhs); /* dvm.h:381 */
/* tensor (op) scalar; scalar_is_lhs selects `scalar op tensor` (KernelPy::Binary, include/dvm_py.h:113-133) */
DVM_C_API dvm_object *dvm_binary_f32(dvm_kernel *k, int binary_type, dvm_object *x, float v, int scalar_is_lhs);
DVM_C_API dvm_object *dvm_binary_i64(dvm_kernel *k, int binary_type, dvm_object *x, int64_t v, int scalar_is_lhs);
DVM_C_API dvm_object *dvm_binary_ref(dvm_kernel *k, int binary_type, dvm_object *x, dvm_scalar *v, int scalar_is_lhs);
DVM_C_API dvm_object *dvm_reduce(dvm_kernel *k, int reduce_type, dvm_object *input, dvm_int_array *dims,
                                 int keepdims);                                               /* dvm.h:391 */
DVM_C_API dvm_object *dvm_select(dvm_kernel *k, dvm_object *cond, dvm_object *lhs, dvm_object *rhs); /* dvm.h:401 */
DVM_C_API dvm_object *dvm_cast(dvm_kernel *k, dvm_object *input, int dtype);                  /* dvm.h:409 */
DVM_C_API dvm_object *dvm_broadcast(dvm_kernel *k, dvm_object *input, dvm_int_array *shape);  /* dvm.h:417 */
/* scalar -> tensor (KernelPy::Full, include/dvm_py.h:146-162; dvm.h:426) */
DVM_C_API dvm_object *dvm_full_f32(dvm_kernel *k, float v, dvm_int_array *shape, int dtype);
DVM_C_API dvm_object *dvm_full_i64(dvm_kernel *k, int64_t v, dvm_int_array *shape, int dtype);
DVM_C_API dvm_object *dvm_full_ref(dvm_kernel *k, dvm_scalar *v, dvm_int_array *shape, int dtype);
DVM_C_API dvm_object *dvm_reshape(dvm_kernel *k, dvm_object *input, dvm_int_array *shape);    /* dvm.h:434 */
/* Kernel::ElemAny (dvm.h:496): one fp32 element, 1 when any element of the input differs from 0 */
DVM_C_API dvm_object *dvm_elem_any(dvm_kernel *k, dvm_object *input);
/* Kernel::PadStore (dvm.h:344): rows of the result lie `pad_size` elements further apart than the tensor's own */
DVM_C_API dvm_object *dvm_pad_store(dvm_kernel *k, void *addr, dvm_object *input, int64_t pad_size);
/* a window of a tensor in memory (Kernel::SliceLoad dvm.h:312, StridedSliceLoad :317): `shape` is the whole tensor's */
DVM_C_API dvm_object *dvm_slice_load(dvm_kernel *k, void *addr, dvm_int_array *shape, dvm_int_array *start,
                                     dvm_int_array *size, int dtype);
DVM_C_API dvm_object *dvm_strided_slice_load(dvm_kernel *k, void *addr, dvm_int_array *shape, dvm_int_array *start,
                                             dvm_int_array *end, dvm_int_array *step, int dtype);
/* views of the input's memory: Kernel::Permute (dvm.h:434), Slice (:443, :453), one chunk of Kernel::Split (:479) */
DVM_C_API dvm_object *dvm_permute(dvm_kernel *k, dvm_object *input, dvm_int_array *dims);
DVM_C_API dvm_object *dvm_slice(dvm_kernel *k, dvm_object *input, dvm_int_array *start, dvm_int_array *size);
DVM_C_API dvm_object *dvm_slice_dim(dvm_kernel *k, dvm_object *input, int dim, dvm_scalar *begin, dvm_scalar *end);
DVM_C_API dvm_object *dvm_split_chunk(dvm_kernel *k, dvm_object *input, int dim, int64_t split_size, size_t split_num,
                                      size_t index);
/* Kernel::Concat (dvm.h:469): the inputs one after the other along `dim` */
DVM_C_API dvm_object *dvm_concat(dvm_kernel *k, dvm_object **inputs, size_t input_num, int dim);
DVM_C_API dvm_object *dvm_copy(dvm_kernel *k, dvm_object *input);                             /* dvm.h:466 */
DVM_C_API dvm_object *dvm_matmul(dvm_kernel *k, dvm_object *lhs, dvm_object *rhs, int trans_a, int trans_b,
                                 dvm_object *bias);                                           /* dvm.h:509 */

/* ---- Kernel::Clone (dvm.h:255-259, CloneHelper dvm.h:212-217) ----
 * dvm_kernel_clone makes `dst` a copy of `base`'s graph (same kernel type and flags).  The map says what every borrowed
 * dvm_int_array / dvm_scalar of `base` becomes in the copy: pairs registered beforehand are used as given (the caller
 * keeps updating the clone's shapes and scalars through them), every other one is copied into an object the map owns -
 * so the map must live as long as `dst` does.  After the call dvm_clone_map_object gives the copy of any op of `base`
 * (its loads and stores, for binding), NULL for an op the base kernel does not hold. */
typedef struct dvm_clone_map dvm_clone_map;
DVM_C_API dvm_clone_map *dvm_clone_map_new(void);
DVM_C_API void dvm_clone_map_free(dvm_clone_map *m);
DVM_C_API int dvm_clone_map_int_array(dvm_clone_map *m, dvm_int_array *base, dvm_int_array *clone);
DVM_C_API int dvm_clone_map_scalar(dvm_clone_map *m, dvm_scalar *base, dvm_scalar *clone);
DVM_C_API int dvm_kernel_clone(dvm_kernel *dst, dvm_kernel *base, dvm_clone_map *m);
DVM_C_API dvm_object *dvm_clone_map_object(dvm_clone_map *m, dvm_object *base);

/* ---- collectives (Comm, include/dvm.h:219-231; Kernel::AllReduce, dvm.h:531) ----
 * The communicator is NCCL's; it is bound at run time, so a host without NCCL can still use everything else.
 * Rank 0 makes a rendezvous id (dvm_comm_id_bytes() bytes) and hands it to the other ranks by any means the job has
 * (a torch.distributed / MPI broadcast, a file); then every rank calls dvm_comm_init_rank with the device it will launch
 * on current.  dvm_comm_adopt uses an ncclComm_t the caller owns (Comm::Init(void *), dvm.h:228).  A dummy communicator
 * (Comm::kDummy) carries rank and size for planning and listings and cannot launch. */
typedef struct dvm_comm dvm_comm;
DVM_C_API dvm_comm *dvm_comm_new(void);
DVM_C_API void dvm_comm_free(dvm_comm *c);
DVM_C_API size_t dvm_comm_id_bytes(void);
DVM_C_API int dvm_comm_unique_id(void *id, size_t bytes);
DVM_C_API int dvm_comm_init_rank(dvm_comm *c, const void *id, size_t bytes, int rank, int size);
DVM_C_API int dvm_comm_init_dummy(dvm_comm *c, int rank, int size);
DVM_C_API int dvm_comm_adopt(dvm_comm *c, void *nccl_comm);
DVM_C_API int dvm_comm_rank(const dvm_comm *c);
DVM_C_API int dvm_comm_size(const dvm_comm *c);
/* the value of `input` combined (reduce_type: 0 sum, 1 max, 2 min) over the ranks of `c` (KernelPy::AllReduce,
 * include/dvm_py.h; python/dvm/_dvm_py.pyi:166) */
DVM_C_API dvm_object *dvm_allreduce(dvm_kernel *k, int reduce_type, dvm_object *input, dvm_comm *c);
/* every rank's tensor stacked along the leading dim (Kernel::AllGather, dvm.h:225); this rank's block of the sum along the
 * leading dim, shape [1, d0 / ranks, ...] or [1, d1, ...] when d0 equals the number of ranks (Kernel::ReduceScatter, :227) */
DVM_C_API dvm_object *dvm_allgather(dvm_kernel *k, dvm_object *input, dvm_comm *c);
DVM_C_API dvm_object *dvm_reducescatter(dvm_kernel *k, dvm_object *input, dvm_comm *c);

/* ---- stacked kernels and marks ---- */
/* start the next stage of a kSequence kernel (Kernel::SequenceAdd, dvm.h:559; KernelPy::SeqAdd, include/dvm_py.h) */
DVM_C_API int dvm_sequence_add(dvm_kernel *k, int kernel_type, uint32_t flags);
/* start the next independent sub-kernel of a kParallel kernel (Kernel::ParallelAdd, dvm.h:552) */
DVM_C_API int dvm_parallel_add(dvm_kernel *k, int kernel_type, uint32_t flags, size_t thread_limit);
/* stage hint of a speculative vector kernel (Kernel::SpecNext, dvm.h:544) */
DVM_C_API int dvm_spec_next(dvm_kernel *k);
/* mark a store whose buffer also feeds the kernel (Kernel::SetStoreInplace, dvm.h:350) */
DVM_C_API int dvm_set_store_inplace(dvm_kernel *k, dvm_object *store);

/* ---- shape inference, code generation, launch ---- */
DVM_C_API int dvm_normalize(dvm_kernel *k);                                                   /* dvm.h:566 */
DVM_C_API int dvm_pre_codegen(dvm_kernel *k, size_t *workspace_bytes);                        /* dvm.h:590 */
DVM_C_API int dvm_codegen(dvm_kernel *k, const dvm_reloc *relocs, size_t reloc_size, dvm_ws_alloc_fn alloc,
                          void *user);                                                        /* dvm.h:572 */
DVM_C_API int dvm_launch(dvm_kernel *k, void *stream);                                        /* dvm.h:578 */
DVM_C_API int dvm_launch_reloc(dvm_kernel *k, const dvm_reloc *relocs, size_t reloc_size, void *workspace,
                               void *stream);                                                 /* dvm.h:599 */
/* No counterpart in the reference.  Launch like dvm_launch_reloc(), but with the kernel's workspace (the
 * global-memory temporaries that hand values from one stage of a split graph to the next) taken from a fixed
 * array inside the library's device image instead of a buffer the caller allocates.  It is meant for callers
 * that cannot call cudaMalloc at the point of launch: code running inside a framework's allocator hooks, inside a
 * memory-pool region that forbids new allocations, or on a serving path where an allocation could stall the
 * device.  The entry point itself calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - dvm_pre_codegen() or dvm_codegen() must have run for the current shapes; `relocs` supplies every input
 *     and output address, exactly as for dvm_launch_reloc().
 *   - Limit: kernels whose workspace exceeds dvm_static_scratch_capacity() bytes (16 MiB) are refused with a
 *     non-zero return and a message in dvm_last_error(); nothing is launched.
 *   - Every GPU that loads the library holds the array until the process exits.
 *   - The first call on a device resolves the array's device address (cudaGetSymbolAddress, with that device
 *     current) and, like the first launch of any kernel of this library, sets function attributes; make that first call
 *     before starting any stream capture, and from one thread (the per-device address is cached without a lock; later
 *     calls only read it).
 *   - All calls share the one array, which keeps whatever the last call left in it.  A kernel's temporaries are
 *     always written before they are read, so nothing needs clearing; but two such launches that overlap on the
 *     GPU (different streams) race on the array - serialise them. */
DVM_C_API int dvm_launch_static_scratch(dvm_kernel *k, const dvm_reloc *relocs, size_t reloc_size, void *stream);
DVM_C_API size_t dvm_static_scratch_capacity(void);
/* Host microseconds spent by the last dvm_codegen / dvm_pre_codegen (shape inference + planning + emission). */
DVM_C_API double dvm_last_jit_us(const dvm_kernel *k);

/* ---- introspection (NDObjectPy::GetShape/GetDType include/dvm_py.h:28-38; Dump/DumpR/Das/Inspect dvm.h:619-637) ---- */
DVM_C_API int dvm_object_rank(const dvm_object *o);
DVM_C_API int64_t dvm_object_dim(const dvm_object *o, int i);
DVM_C_API int dvm_object_dtype(const dvm_object *o);
DVM_C_API const char *dvm_dump(dvm_kernel *k);
DVM_C_API const char *dvm_dump_r(dvm_kernel *k);
DVM_C_API const char *dvm_das(dvm_kernel *k);
DVM_C_API const char *dvm_inspect(dvm_kernel *k);

/* ---- device runtime used by the Python runner (DevRunner, src/pybind_api.cc:195-271; Device, :1100-1116) ---- */
DVM_C_API int dvm_rt_device_count(void);
DVM_C_API int dvm_rt_set_device(int dev);
DVM_C_API int dvm_rt_sm_count(void);
DVM_C_API void *dvm_rt_malloc(size_t bytes);
DVM_C_API int dvm_rt_free(void *p);
DVM_C_API int dvm_rt_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream);
DVM_C_API int dvm_rt_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream);
DVM_C_API int dvm_rt_memset(void *dst, int value, size_t bytes, void *stream);
/* Waits for `stream`, then reports like dvm_rt_check_status(). */
DVM_C_API int dvm_rt_sync(void *stream);
/* No counterpart in the reference (its device waits are unbounded).  Every wait inside the device kernels is bounded
 * (about two seconds); a kernel whose wait ran out records that, finishes with wrong results and leaves the context
 * usable.  This call reads and clears the record of the current device without waiting for anything: 0 = no wait has
 * expired since the last check, -1 = one has (details in dvm_last_error()).  Callers that synchronise their own streams
 * (cudaStreamSynchronize, events) instead of dvm_rt_sync() - C++ clients of include/dvm.h link the same symbol - call it
 * after they have synchronised.  An expiry is tied to the launch it happened in: it does not shorten the waits of later
 * launches or of launches on other streams. */
DVM_C_API int dvm_rt_check_status(void);
/* No counterpart in the reference.  Enqueues a one-thread kernel whose only wait can never be satisfied and gives up
 * after `limit_ms` milliseconds (clamped to 1000), so that the reporting path above can be exercised without a hang or
 * a fault: after a synchronisation dvm_rt_check_status() returns -1 once and 0 afterwards. */
DVM_C_API int dvm_rt_selftest_wait_expiry(unsigned int limit_ms, void *stream);
DVM_C_API void *dvm_rt_host_alloc(size_t bytes);   /* pinned host memory */
DVM_C_API int dvm_rt_host_free(void *p);
/* warmup launches, then `reps` launches timed one by one with device events on `stream`
 * (RtKernelPy::Perf, src/pybind_api.cc:751-767: 1 warm-up + 10 timed runs, min/max/mean in us). */
DVM_C_API int dvm_perf(dvm_kernel *k, int warmup, int reps, void *stream, float *min_us, float *max_us,
                       float *mean_us);

/* No counterpart in the reference.  Like dvm_perf(), but with one pair of device events around every launch or
 * collective of the kernel's plan (the order of dvm_das()): mean_us[i] is the mean device time of stage i over `reps`
 * runs; *stages receives the number of stages, which must not exceed `capacity`. */
DVM_C_API int dvm_perf_stages(dvm_kernel *k, int warmup, int reps, void *stream, float *mean_us, size_t capacity,
                              size_t *stages);

#ifdef __cplusplus
}
#endif

#endif /* DVM_B200_DVM_C_H_ */
