"""Python front-end over the C ABI: DataType, NDObject, IntArrayRef, ScalarRef, Kernel, PyKernel, Device.

Mirrors the classes the reference's extension module registers (include/dvm_py.h:277-387,
src/pybind_api.cc:1066-1116, python/dvm/_dvm_py.pyi): same class names, method names, argument order and
error behaviour (failures surface as RuntimeError).  Device buffers are managed through the runtime
helpers of the C ABI, like the reference's DevRunner (src/pybind_api.cc:195-271): ``input`` allocates and
copies host -> device, ``output`` copies device -> host.
"""
import ctypes

import numpy as np

from . import _capi
from ._capi import DvmError, check_ptr, check_rc

try:  # bfloat16 arrays are carried as ml_dtypes.bfloat16 when available, else as raw uint16
    import ml_dtypes
    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    ml_dtypes = None
    _BF16 = None


class DataType(int):
    """Element types, numbered like dvm::DataType (include/dvm.h:27-35)."""
    _names = ["bool", "float16", "bfloat16", "float32", "int32", "int64"]

    def __repr__(self):
        return "DataType.%s" % self._names[int(self)]

    __str__ = __repr__


for _i, _n in enumerate(DataType._names):
    setattr(DataType, _n, DataType(_i))

ITEM_SIZE = [1, 2, 2, 4, 4, 8]


def np_dtype_of(dtype):
    return [np.dtype(np.bool_), np.dtype(np.float16), _BF16 if _BF16 is not None else np.dtype(np.uint16),
            np.dtype(np.float32), np.dtype(np.int32), np.dtype(np.int64)][int(dtype)]


def dvm_dtype_of(np_dt):
    np_dt = np.dtype(np_dt)
    if _BF16 is not None and np_dt == _BF16:
        return DataType.bfloat16
    table = {np.dtype(np.bool_): DataType.bool, np.dtype(np.float16): DataType.float16,
             np.dtype(np.float32): DataType.float32, np.dtype(np.int32): DataType.int32,
             np.dtype(np.int64): DataType.int64}
    if np_dt not in table:
        raise DvmError("unsupported numpy dtype %s" % np_dt)
    return table[np_dt]


class NDObject:
    def __init__(self, handle, owner):
        self._h = handle
        self._owner = owner  # keeps the kernel alive

    def shape(self):
        lib = _capi.load()
        return tuple(int(lib.dvm_object_dim(self._h, i)) for i in range(lib.dvm_object_rank(self._h)))

    def dtype(self):
        return DataType(_capi.load().dvm_object_dtype(self._h))


class IntArrayRef:
    def __init__(self, shape=None):
        lib = _capi.load()
        vals = [int(v) for v in (shape or [])]
        arr = (ctypes.c_int64 * max(1, len(vals)))(*vals)
        self._h = check_ptr(lib.dvm_int_array_new(arr, len(vals)), "int array")

    def shape(self):
        lib = _capi.load()
        n = lib.dvm_int_array_size(self._h)
        data = lib.dvm_int_array_data(self._h)
        return tuple(int(data[i]) for i in range(n))

    def update(self, shape):
        vals = [int(v) for v in shape]
        arr = (ctypes.c_int64 * max(1, len(vals)))(*vals)
        _capi.load().dvm_int_array_update(self._h, arr, len(vals))

    def __del__(self):
        try:
            _capi.load().dvm_int_array_free(self._h)
        except Exception:
            pass


class ScalarRef:
    def __init__(self, dtype=None):
        self._h = check_ptr(_capi.load().dvm_scalar_new(), "scalar")

    def update(self, value):
        lib = _capi.load()
        if isinstance(value, (bool, np.bool_)):
            lib.dvm_scalar_set_i64(self._h, int(value))
        elif isinstance(value, (int, np.integer)):
            lib.dvm_scalar_set_i64(self._h, int(value))
        elif isinstance(value, (float, np.floating)):
            lib.dvm_scalar_set_f32(self._h, float(value))
        else:
            raise DvmError("Unsupported scalar value type for current data type.")

    def __del__(self):
        try:
            _capi.load().dvm_scalar_free(self._h)
        except Exception:
            pass


_UNARY = ["sqrt", "abs", "log", "exp", "reciprocal", "isfinite", "logical_not", "round", "floor", "ceil", "trunc"]
_BINARY = ["equal", "not_equal", "greater", "greater_equal", "less", "less_equal", "add", "sub", "mul", "div", "pow",
           "maximum", "minimum", "logical_and", "logical_or"]
_KERNEL_TYPES = {"": 0, "vector": 0, "cube": 1, "mix": 2, "parallel": 3, "seq": 4, "split": 5, "eager": 6}
_KERNEL_FLAGS = {"dyn": 0x1, "unify_ws": 0x2, "spec": 0x4, "lazy": 0x8, "opt_fractal": 1 << 29, "priv1": 1 << 30,
                 "priv2": 1 << 31}


def parse_kernel_type(ker_type):
    """'type[:flag,flag...]' -> (KernelType, flags); ref: ParseKernelType, src/pybind_api.cc:117-154."""
    name, _, flag_str = ker_type.partition(":")
    flags = 0
    if flag_str:
        for f in flag_str.split(","):
            if f not in _KERNEL_FLAGS:
                raise DvmError("DVM EXCEPTION. reason: kernel flag error")
            flags |= _KERNEL_FLAGS[f]
    if name not in _KERNEL_TYPES:
        raise DvmError("DVM EXCEPTION. reason: kernel type error")
    return _KERNEL_TYPES[name], flags


class Kernel:
    """Graph-builder methods (KernelPy, include/dvm_py.h:97-268)."""
    K_VEC, K_CUBE, K_MIX, K_PARAL, K_SEQ, K_SPLIT, K_EAGER = range(7)
    F_DYN, F_UWS, F_SPEC, F_PRIV1 = 0x1, 0x2, 0x4, 1 << 30

    def __init__(self, kernel_type=0, flags=0):
        self._lib = _capi.load()
        self._k = check_ptr(self._lib.dvm_kernel_new(int(kernel_type), int(flags)), "kernel")
        self._ktype = int(kernel_type)
        self._flags = int(flags)
        self._keep = []  # shape / scalar holders the graph borrows

    def __del__(self):
        try:
            self._lib.dvm_kernel_free(self._k)
        except Exception:
            pass

    # -- helpers
    def _shape_ref(self, shape):
        if isinstance(shape, IntArrayRef):
            return shape
        ref = IntArrayRef(list(shape))
        self._keep.append(ref)
        return ref

    def _obj(self, handle, what):
        if not handle:
            err = _capi.last_error()
            if err:
                raise DvmError("%s failed: %s" % (what, err))
            return None  # the reference returns a null object for unsupported builder combinations
        return NDObject(handle, self)

    def is_dynamic(self):
        return bool(self._flags & 0x1)

    # -- inputs / outputs
    def load(self, shape, type):
        ref = self._shape_ref(shape)
        op = self._obj(self._lib.dvm_load(self._k, None, ref._h, int(type)), "load")
        op._shape_ref = ref
        return op

    def store(self, obj, type=None):
        if type is not None and int(type) < len(DataType._names):
            obj = self.cast(obj, type)
        return self._obj(self._lib.dvm_store(self._k, None, obj._h), "store")

    def view_load(self, shape, stride, type):
        """A tensor that is not contiguous in memory: one element stride per dim (KernelPy::ViewLoad, include/dvm_py.h:104)."""
        ref, sref = self._shape_ref(shape), self._shape_ref(stride)
        op = self._obj(self._lib.dvm_load_strided(self._k, None, ref._h, sref._h, int(type)), "view_load")
        op._shape_ref = ref
        return op

    def element_any(self, input):
        """KernelPy::ElementAny: one element, 1 when any element of the input differs from 0."""
        return self._obj(self._lib.dvm_elem_any(self._k, input._h), "element_any")

    def pad_store(self, obj, pad_size):
        """KernelPy::PadStore: the result in a buffer whose rows are `pad_size` elements longer (shape() of the store)."""
        return self._obj(self._lib.dvm_pad_store(self._k, None, obj._h, int(pad_size)), "pad_store")

    def slice_load(self, shape, start, size, type):
        """A window (start + size per dim) of a tensor in memory whose whole shape is `shape` (KernelPy::SliceLoad)."""
        ref = self._shape_ref(shape)
        op = self._obj(self._lib.dvm_slice_load(self._k, None, ref._h, self._shape_ref(list(start))._h,
                                                self._shape_ref(list(size))._h, int(type)), "slice_load")
        op._shape_ref = ref
        return op

    def stridedslice_load(self, shape, start, end, step, type):
        """The same with start / end / step per dim, read as Python slices are (KernelPy::StridedSliceLoad)."""
        ref = self._shape_ref(shape)
        op = self._obj(self._lib.dvm_strided_slice_load(self._k, None, ref._h, self._shape_ref(list(start))._h,
                                                        self._shape_ref(list(end))._h, self._shape_ref(list(step))._h,
                                                        int(type)), "stridedslice_load")
        op._shape_ref = ref
        return op

    def view_store(self, obj, stride, type=None):
        """Store with element strides; what lies between the written elements keeps its content (KernelPy::ViewStore,
        include/dvm_py.h:107)."""
        if type is not None and int(type) < len(DataType._names):
            obj = self.cast(obj, type)
        return self._obj(self._lib.dvm_store_strided(self._k, None, obj._h, self._shape_ref(stride)._h), "view_store")

    def scalar(self, dtype=None):
        ref = ScalarRef(dtype)
        self._keep.append(ref)
        return ref

    def int_array(self):
        ref = IntArrayRef()
        self._keep.append(ref)
        return ref

    # -- element-wise
    def _unary(self, code, x):
        return self._obj(self._lib.dvm_unary(self._k, code, x._h), _UNARY[code])

    def _binary(self, code, lhs, rhs):
        name = _BINARY[code]

        def scalar_call(x, v, scalar_is_lhs):
            if isinstance(v, ScalarRef):
                return self._lib.dvm_binary_ref(self._k, code, x._h, v._h, scalar_is_lhs)
            if isinstance(v, (bool, np.bool_, int, np.integer)):
                return self._lib.dvm_binary_i64(self._k, code, x._h, int(v), scalar_is_lhs)
            if isinstance(v, (float, np.floating)):
                return self._lib.dvm_binary_f32(self._k, code, x._h, float(v), scalar_is_lhs)
            raise DvmError("unsupported operand type for %s: %r" % (name, type(v)))

        if not isinstance(lhs, NDObject):
            return self._obj(scalar_call(rhs, lhs, 1), name)
        if not isinstance(rhs, NDObject):
            return self._obj(scalar_call(lhs, rhs, 0), name)
        return self._obj(self._lib.dvm_binary(self._k, code, lhs._h, rhs._h), name)

    def cast(self, input, type):
        return self._obj(self._lib.dvm_cast(self._k, input._h, int(type)), "cast")

    def select(self, cond, lhs, rhs):
        return self._obj(self._lib.dvm_select(self._k, cond._h, lhs._h, rhs._h), "select")

    def broadcast(self, input, shape):
        return self._obj(self._lib.dvm_broadcast(self._k, input._h, self._shape_ref(shape)._h), "broadcast")

    def full(self, scalar, shape, dtype):
        ref = self._shape_ref(shape)
        if isinstance(scalar, ScalarRef):
            h = self._lib.dvm_full_ref(self._k, scalar._h, ref._h, int(dtype))
        elif isinstance(scalar, (bool, np.bool_, int, np.integer)):
            h = self._lib.dvm_full_i64(self._k, int(scalar), ref._h, int(dtype))
        elif isinstance(scalar, (float, np.floating)):
            h = self._lib.dvm_full_f32(self._k, float(scalar), ref._h, int(dtype))
        else:
            raise DvmError("Unsupported scalar type for full: expected bool, int, float, or ScalarRef.")
        return self._obj(h, "full")

    def reshape(self, input, shape):
        return self._obj(self._lib.dvm_reshape(self._k, input._h, self._shape_ref(shape)._h), "reshape")

    # -- views of the input's memory (KernelPy::Permute / Slice / SliceDim / Split, include/dvm_py.h:163-186)
    def permute(self, input, dims):
        return self._obj(self._lib.dvm_permute(self._k, input._h, self._shape_ref(list(dims))._h), "permute")

    def slice(self, input, begin, size):
        return self._obj(self._lib.dvm_slice(self._k, input._h, self._shape_ref(list(begin))._h,
                                             self._shape_ref(list(size))._h), "slice")

    def _index_ref(self, v):
        if isinstance(v, ScalarRef):
            return v
        ref = ScalarRef()
        ref.update(int(v))
        self._keep.append(ref)
        return ref

    def slice_dim(self, input, dim, begin, end):
        return self._obj(self._lib.dvm_slice_dim(self._k, input._h, int(dim), self._index_ref(begin)._h,
                                                 self._index_ref(end)._h), "slice_dim")

    def split(self, input, dim, split_size, split_num):
        return [self._obj(self._lib.dvm_split_chunk(self._k, input._h, int(dim), int(split_size), int(split_num), i), "split")
                for i in range(int(split_num))]

    def concat(self, inputs, dim):
        """KernelPy::Concat (include/dvm_py.h): the inputs one after the other along `dim`."""
        import ctypes
        arr = (ctypes.c_void_p * len(inputs))(*[x._h for x in inputs])
        return self._obj(self._lib.dvm_concat(self._k, arr, len(inputs), int(dim)), "concat")

    def copy(self, input):
        return self._obj(self._lib.dvm_copy(self._k, input._h), "copy")

    def _reduce(self, code, input, dims, keepdims):
        ref = self._shape_ref(dims)
        return self._obj(self._lib.dvm_reduce(self._k, code, input._h, ref._h, 1 if keepdims else 0), "reduce")

    def sum(self, input, dims, keepdims=False):
        return self._reduce(0, input, dims, keepdims)

    def max(self, input, dims, keepdims=False):
        return self._reduce(1, input, dims, keepdims)

    def min(self, input, dims, keepdims=False):
        return self._reduce(2, input, dims, keepdims)

    def matmul(self, lhs, rhs, trans_a, trans_b, bias=None):
        return self._obj(self._lib.dvm_matmul(self._k, lhs._h, rhs._h, int(bool(trans_a)), int(bool(trans_b)),
                                              bias._h if bias is not None else None), "matmul")

    # -- text
    def tile(self, start, end, num, factor=0):
        """Tiling hint of the reference's runner (src/pybind_api.cc:1093); the tile geometry here follows from the shapes
        alone, so the hint is accepted and has no effect."""
        return None

    def das(self):
        return self._lib.dvm_das(self._k).decode()

    def dump(self):
        return self._lib.dvm_dump(self._k).decode()

    def dump_r(self):
        return self._lib.dvm_dump_r(self._k).decode()

    def inspect(self):
        return self._lib.dvm_inspect(self._k).decode()

    def spec_next(self):
        """Stage hint of a speculative vector kernel (KernelPy::SpecNext, include/dvm_py.h)."""
        check_rc(self._lib.dvm_spec_next(self._k), "spec_next")

    def seq_add(self, ktype, flags=0):
        """Start the next stage of a "seq" kernel (KernelPy::SequenceAdd, include/dvm_py.h:371)."""
        check_rc(self._lib.dvm_sequence_add(self._k, int(ktype), int(flags)), "seq_add")

    def parallel_add(self, ktype, flags=0, core_limit=0):
        """Start the next independent sub-kernel of a "parallel" kernel (KernelPy::ParallelAdd, include/dvm_py.h:214)."""
        check_rc(self._lib.dvm_parallel_add(self._k, int(ktype), int(flags), int(core_limit)), "parallel_add")

    def clear_store_memory(self, store):
        """RtKernelPy::ClearStoreMemory zeroes a buffer that the reference's kernels accumulate into; stores here write
        every element of their result, so there is nothing to clear."""
        self._find(self._stores, store)

    def set_store_inplace(self, store):
        """Mark a store whose buffer also feeds the kernel (KernelPy::SetStoreInplace, include/dvm_py.h:206)."""
        check_rc(self._lib.dvm_set_store_inplace(self._k, store._h), "set_store_inplace")

    @staticmethod
    def set_deterministic(enable):
        pass  # reductions always use a fixed tree on this backend

    @staticmethod
    def set_online_tuning(enable):
        pass

    @staticmethod
    def set_vf_fusion(mode):
        pass

    @staticmethod
    def set_cube_store_type(type):
        pass  # (a tuning switch of the reference's MatMul store path; results do not depend on it)

    @staticmethod
    def set_lazy_tuning(enable):
        pass


def _make_unary(code):
    def f(self, input):
        return self._unary(code, input)
    f.__name__ = _UNARY[code]
    return f


def _make_binary(code):
    def f(self, lhs, rhs):
        return self._binary(code, lhs, rhs)
    f.__name__ = _BINARY[code]
    return f


for _c, _name in enumerate(_UNARY):
    setattr(Kernel, _name, _make_unary(_c))
for _c, _name in enumerate(_BINARY):
    setattr(Kernel, _name, _make_binary(_c))


class _DevBuf:
    """One device allocation owned by a PyKernel."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)
        self.ptr = check_ptr(_capi.load().dvm_rt_malloc(self.nbytes), "device allocation of %d bytes" % nbytes)

    def free(self):
        if self.ptr:
            _capi.load().dvm_rt_free(self.ptr)
            self.ptr = None


class _ExternalBuf:
    """Device memory owned by the caller (e.g. a torch tensor) bound to a load or store."""

    def __init__(self, ptr, nbytes):
        self.ptr = int(ptr)
        self.nbytes = int(nbytes)

    def free(self):
        self.ptr = None


class _ProcessComm:
    """The process-wide communicator of the Python runner (g_mpc.comm, src/pybind_api.cc:675-687)."""
    handle = None
    rank = 0
    size = 1


def _framework_nccl_first():
    """Two NCCL builds in one process clash (the loader hands the copy that came first to every later library that asks
    for "libnccl.so.2").  torch ships its own build, so when torch is installed it is imported before this library binds
    NCCL; the library then finds and uses the copy torch loaded."""
    import importlib.util
    import sys
    if "torch" not in sys.modules and importlib.util.find_spec("torch") is not None:
        import torch  # noqa: F401


def comm_unique_id():
    """A fresh rendezvous id (bytes): rank 0 makes it, every rank passes the same bytes to init_comm_with_id()."""
    _framework_nccl_first()
    lib = _capi.load()
    n = lib.dvm_comm_id_bytes()
    buf = ctypes.create_string_buffer(n)
    check_rc(lib.dvm_comm_unique_id(buf, n), "comm_unique_id")
    return buf.raw


def init_comm_with_id(rank_id, rank_size, id_bytes):
    """Create this process's NCCL communicator from a rendezvous id the ranks have shared by their own means
    (collective over all ranks; the device this rank launches on must be current)."""
    _framework_nccl_first()
    lib = _capi.load()
    if _ProcessComm.handle is None:
        _ProcessComm.handle = check_ptr(lib.dvm_comm_new(), "comm")
    check_rc(lib.dvm_comm_init_rank(_ProcessComm.handle, id_bytes, len(id_bytes), int(rank_id), int(rank_size)), "init_comm")
    _ProcessComm.rank, _ProcessComm.size = int(rank_id), int(rank_size)


class PyKernel(Kernel):
    """Kernel plus a device runner (RtKernelPy, src/pybind_api.h:27-119)."""

    @staticmethod
    def init_comm(rank_id, rank_size, comm_type="memory"):
        """RtKernelPy::InitComm (src/pybind_api.cc:675-687).  "dummy" records rank and size only (plans and listings);
        any other type creates an NCCL communicator, the ranks meeting through the file named by DVM_B200_COMM_ID_FILE
        (rank 0 writes the rendezvous id there)."""
        lib = _capi.load()
        if _ProcessComm.handle is None:
            _ProcessComm.handle = check_ptr(lib.dvm_comm_new(), "comm")
        if comm_type == "dummy":
            check_rc(lib.dvm_comm_init_dummy(_ProcessComm.handle, int(rank_id), int(rank_size)), "init_comm")
        else:
            import os
            path = os.environ.get("DVM_B200_COMM_ID_FILE")
            if int(rank_size) > 1 and not path:
                raise DvmError("init_comm: set DVM_B200_COMM_ID_FILE to a path all ranks share, or use init_comm_with_id()")
            if int(rank_id) == 0 or int(rank_size) == 1:
                uid = comm_unique_id()
                if int(rank_size) > 1:
                    with open(path + ".tmp", "wb") as f:
                        f.write(uid)
                    os.replace(path + ".tmp", path)
            else:
                import time
                deadline = time.time() + 60
                while not os.path.exists(path):
                    if time.time() > deadline:
                        raise DvmError("init_comm: no rendezvous id appeared at %s" % path)
                    time.sleep(0.01)
                with open(path, "rb") as f:
                    uid = f.read()
            init_comm_with_id(rank_id, rank_size, uid)
            return
        _ProcessComm.rank, _ProcessComm.size = int(rank_id), int(rank_size)

    def allreduce(self, type, input):
        """RtKernelPy::AllReduce (src/pybind_api.cc:562-572): "sum" or "max" over the ranks of the process's communicator."""
        codes = {"sum": 0, "max": 1}
        if type not in codes:
            raise ValueError("Unsupported AllReduce type: " + str(type))
        if _ProcessComm.handle is None:
            raise DvmError("allreduce before init_comm()")
        return self._obj(self._lib.dvm_allreduce(self._k, codes[type], input._h, _ProcessComm.handle), "allreduce")

    def allgather(self, input):
        """RtKernelPy::AllGather (src/pybind_api.cc:578): every rank's tensor stacked along the leading dim."""
        if _ProcessComm.handle is None:
            raise DvmError("allgather before init_comm()")
        return self._obj(self._lib.dvm_allgather(self._k, input._h, _ProcessComm.handle), "allgather")

    def reducescatter(self, input):
        """RtKernelPy::ReduceScatter (src/pybind_api.cc:574-576): this rank's block of the sum over the ranks."""
        if _ProcessComm.handle is None:
            raise DvmError("reducescatter before init_comm()")
        return self._obj(self._lib.dvm_reducescatter(self._k, input._h, _ProcessComm.handle), "reducescatter")

    def __init__(self, ker_type="", run_type="dev", dev_id=0):
        ktype, flags = parse_kernel_type(ker_type)
        Kernel.__init__(self, ktype, flags)
        if run_type not in ("dev", "das"):
            raise DvmError("run type '%s' is not available on this backend" % run_type)
        self._run_type = run_type
        self._dev_id = int(dev_id)
        self._loads = []   # [op, dev buffer, host array]
        self._stores = []  # [op, dev buffer, host array]
        self._ws = None
        self._ws_cb = None
        if run_type == "dev":
            check_rc(self._lib.dvm_rt_set_device(self._dev_id), "set device")

    def clone(self, base, remap):
        """RtKernelPy::Clone (src/pybind_api.cc:918-997): this kernel becomes a copy of `base`'s graph with its own
        shapes and scalars.  `remap` lists ops, IntArrayRefs and ScalarRefs of `base`; their counterparts in the copy
        come back in the same order."""
        lib = self._lib
        m = check_ptr(lib.dvm_clone_map_new(), "clone map")

        class _Map:   # the copy borrows what the map owns: it lives as long as this kernel does
            def __init__(self, h):
                self.h = h

            def __del__(self):
                try:
                    lib.dvm_clone_map_free(self.h)
                except Exception:
                    pass

        self._keep.append(_Map(m))
        load_refs = []
        for rec in base._loads:
            ref = IntArrayRef(rec[0]._shape_ref.shape())
            check_rc(lib.dvm_clone_map_int_array(m, rec[0]._shape_ref._h, ref._h), "clone")
            self._keep.append(ref)
            load_refs.append(ref)
        out = [None] * len(remap)
        for i, x in enumerate(remap):
            if isinstance(x, IntArrayRef):
                ref = IntArrayRef(x.shape())
                check_rc(lib.dvm_clone_map_int_array(m, x._h, ref._h), "clone")
            elif isinstance(x, ScalarRef):
                ref = ScalarRef()
                check_rc(lib.dvm_clone_map_scalar(m, x._h, ref._h), "clone")
            else:
                continue
            self._keep.append(ref)
            out[i] = ref
        check_rc(lib.dvm_kernel_clone(self._k, base._k, m), "clone")
        self._ktype, self._flags = base._ktype, base._flags
        self._loads, self._stores = [], []
        for rec, ref in zip(base._loads, load_refs):
            op = self._obj(lib.dvm_clone_map_object(m, rec[0]._h), "clone")
            op._shape_ref = ref
            self._loads.append([op, None, None])
        for rec in base._stores:
            self._stores.append([self._obj(lib.dvm_clone_map_object(m, rec[0]._h), "clone"), None, None])
        known = {rec[0]._h: rec[0] for rec in self._loads + self._stores}
        for i, x in enumerate(remap):
            if isinstance(x, NDObject):
                h = lib.dvm_clone_map_object(m, x._h)
                out[i] = known.get(h) or self._obj(h, "clone")
        return tuple(out)

    # bookkeeping wrappers
    def load(self, shape, type):
        op = Kernel.load(self, shape, type)
        self._loads.append([op, None, None])
        return op

    def store(self, obj, type=None):
        op = Kernel.store(self, obj, type)
        self._stores.append([op, None, None])
        return op

    def view_load(self, shape, stride, type):
        op = Kernel.view_load(self, shape, stride, type)
        self._loads.append([op, None, None])
        return op

    def pad_store(self, obj, pad_size):
        op = Kernel.pad_store(self, obj, pad_size)
        self._stores.append([op, None, None])
        return op

    def slice_load(self, shape, start, size, type):
        op = Kernel.slice_load(self, shape, start, size, type)
        self._loads.append([op, None, None])
        return op

    def stridedslice_load(self, shape, start, end, step, type):
        op = Kernel.stridedslice_load(self, shape, start, end, step, type)
        self._loads.append([op, None, None])
        return op

    def view_store(self, obj, stride, type=None):
        op = Kernel.view_store(self, obj, stride, type)
        self._stores.append([op, None, None])
        return op

    def set_output(self, store, array, offset=0):
        """The host array a store's result lives in (RtKernelPy::SetOutput, src/pybind_api.cc:867-872): its size is the
        size of the device buffer and its content is what the buffer holds before the kernel runs - a strided store writes
        only some of the elements.  `offset` (elements; not in the reference) is where in the array the stored tensor
        starts, the counterpart of input()'s offset."""
        rec = self._find(self._stores, store)
        rec[2] = np.ascontiguousarray(array)
        self._preset = getattr(self, "_preset", {})
        self._preset[store._h] = (rec[2], int(offset) * rec[2].dtype.itemsize)

    def _find(self, table, op):
        for rec in table:
            if rec[0] is op or rec[0]._h == op._h:
                return rec
        raise DvmError("object does not belong to this kernel")

    @staticmethod
    def convert_to_bf16(array):
        """fp32 array -> bfloat16 storage (round to nearest even), ref: src/pybind_api.cc:580-595."""
        a = np.ascontiguousarray(array, dtype=np.float32)
        if _BF16 is not None:
            return a.astype(_BF16)
        u = a.view(np.uint32)
        r = ((u >> 16) & 1) + 0x7FFF
        return ((u + r) >> 16).astype(np.uint16)

    @staticmethod
    def convert_from_bf16(array):
        a = np.asarray(array)
        if _BF16 is not None and a.dtype == _BF16:
            return a.astype(np.float32)
        return (a.astype(np.uint32) << 16).view(np.float32)

    def input(self, obj, val, offset=0):
        if isinstance(obj, IntArrayRef):
            obj.update(val)
            return
        if isinstance(obj, ScalarRef):
            obj.update(val)
            return
        rec = self._find(self._loads, obj)
        arr = np.ascontiguousarray(val)
        if self.is_dynamic():
            obj._shape_ref.update(arr.shape)
        if self._run_type != "dev":
            rec[2] = arr
            return
        if rec[1] is None or rec[1].nbytes < arr.nbytes:
            if rec[1] is not None:
                rec[1].free()
            rec[1] = _DevBuf(max(arr.nbytes, 1))
        rec[2] = arr
        self._load_offset = getattr(self, "_load_offset", {})
        self._load_offset[obj._h] = int(offset) * arr.dtype.itemsize   # the tensor starts `offset` elements into the array
        if arr.nbytes:
            check_rc(self._lib.dvm_rt_memcpy_h2d(rec[1].ptr, arr.ctypes.data, arr.nbytes, None), "H2D copy")

    def bind_device(self, obj, ptr, nbytes):
        """Use caller-owned device memory for a load or store (no counterpart in the reference's Python API, which
        always copies through NumPy; the C++ API takes device pointers through RelocEntry, include/dvm.h:201-206)."""
        for recs in (self._loads, self._stores):
            for rec in recs:
                if rec[0]._h == obj._h:
                    if rec[1] is not None:
                        rec[1].free()
                    rec[1] = _ExternalBuf(ptr, nbytes)
                    return
        raise DvmError("bind_device: not a load or store of this kernel")

    def codegen(self, pass_names=None):
        check_rc(self._lib.dvm_normalize(self._k), "normalize")
        relocs = []
        for rec in self._stores:
            op = rec[0]
            shape = op.shape()
            dt = np_dtype_of(op.dtype())
            nbytes = int(np.prod(shape, dtype=np.int64)) * dt.itemsize if len(shape) else dt.itemsize
            preset, preset_off = getattr(self, "_preset", {}).get(op._h, (None, 0))
            if preset is not None:
                rec[2] = preset
                nbytes = preset.nbytes
            else:
                rec[2] = np.empty(shape, dtype=dt)
            if self._run_type == "dev":
                if rec[1] is None or rec[1].nbytes < nbytes:
                    if rec[1] is not None:
                        rec[1].free()
                    rec[1] = _DevBuf(max(nbytes, 1))
                if preset is not None and nbytes:
                    check_rc(self._lib.dvm_rt_memcpy_h2d(rec[1].ptr, preset.ctypes.data, nbytes, None), "H2D copy")
                relocs.append((op._h, rec[1].ptr + preset_off))
            else:
                relocs.append((op._h, 0x1000 * (len(relocs) + 1)))
        for rec in self._loads:
            if self._run_type == "dev":
                if rec[1] is None:
                    raise DvmError("load has no input bound; call input() first")
                relocs.append((rec[0]._h, rec[1].ptr + getattr(self, "_load_offset", {}).get(rec[0]._h, 0)))
            else:
                relocs.append((rec[0]._h, 0x1000 * (len(relocs) + 1)))
        arr = (_capi.Reloc * max(1, len(relocs)))()
        for i, (h, p) in enumerate(relocs):
            arr[i].io = h
            arr[i].addr = p

        def alloc(size, _user):
            if self._run_type != "dev":
                return 0x100000
            if self._ws is None or self._ws.nbytes < size:
                if self._ws is not None:
                    self._ws.free()
                self._ws = _DevBuf(size)
            return self._ws.ptr

        self._ws_cb = _capi.WS_ALLOC_FN(alloc)
        self._reloc_args = (arr, len(relocs))   # what the last code generation was given (kept for repeat_codegen_launch)
        check_rc(self._lib.dvm_codegen(self._k, arr, len(relocs), self._ws_cb, None), "codegen")

    def repeat_codegen_launch(self, stream=None):
        """Shape inference + planning + emission + binding + launch once more, with the addresses of the last codegen():
        the three C calls a framework makes when a new shape arrives (dvm_normalize is part of dvm_codegen), without this
        front-end's own bookkeeping around them."""
        arr, n = self._reloc_args
        check_rc(self._lib.dvm_codegen(self._k, arr, n, self._ws_cb, None), "codegen")
        check_rc(self._lib.dvm_launch(self._k, stream), "launch")

    def run(self):
        if self._run_type != "dev":
            raise DvmError("run() needs run_type 'dev'")
        check_rc(self._lib.dvm_launch(self._k, None), "launch")
        check_rc(self._lib.dvm_rt_sync(None), "synchronize")

    def launch(self, stream=None):
        """Enqueue without synchronising (no counterpart in the reference's Python API)."""
        check_rc(self._lib.dvm_launch(self._k, stream), "launch")

    def output(self, store):
        rec = self._find(self._stores, store)
        host = rec[2]
        if host is None:
            raise DvmError("output() before codegen()")
        if host.nbytes:
            check_rc(self._lib.dvm_rt_memcpy_d2h(host.ctypes.data, rec[1].ptr, host.nbytes, None), "D2H copy")
            check_rc(self._lib.dvm_rt_sync(None), "synchronize")
        return host

    def perf(self, warmup=1, reps=10):
        lo, hi, mean = ctypes.c_float(), ctypes.c_float(), ctypes.c_float()
        check_rc(self._lib.dvm_perf(self._k, warmup, reps, None, ctypes.byref(lo), ctypes.byref(hi),
                                    ctypes.byref(mean)), "perf")
        return (lo.value, hi.value, mean.value)

    def perf_stages(self, warmup=1, reps=10):
        """Mean device microseconds of every launch / collective of the plan, in the order of das()."""
        cap = 64
        arr = (ctypes.c_float * cap)()
        n = ctypes.c_size_t(0)
        check_rc(self._lib.dvm_perf_stages(self._k, warmup, reps, None, arr, cap, ctypes.byref(n)), "perf_stages")
        return [arr[i] for i in range(n.value)]

    def jit_us(self):
        return float(self._lib.dvm_last_jit_us(self._k))

    def reset(self):
        """RtKernelPy::Reset (src/pybind_api.cc:909-922): an eager kernel drops its graph, loads and stores so that the
        next graph can be built on the same object; other kernel types keep theirs."""
        if self._ktype != Kernel.K_EAGER:
            return
        self.release_io()
        check_rc(self._lib.dvm_kernel_reset(self._k, self._ktype, self._flags), "reset")
        self._loads = []
        self._stores = []
        self._keep = []

    def release_io(self):
        for rec in self._loads + self._stores:
            if rec[1] is not None:
                rec[1].free()
                rec[1] = None

    def device_ptr(self, op):
        for rec in self._loads + self._stores:
            if rec[0]._h == op._h:
                return rec[1].ptr if rec[1] is not None else None
        return None

    def __del__(self):
        try:
            self.release_io()
            if self._ws is not None:
                self._ws.free()
        except Exception:
            pass
        Kernel.__del__(self)

    # multi-process helpers of the reference (fork/join/barrier) are not part of this backend
    @staticmethod
    def barrier():
        pass

    @staticmethod
    def rank_id():
        return 0

    @staticmethod
    def rank_size():
        return 1


class Device:
    @staticmethod
    def arch():
        return "sm_100a"

    @staticmethod
    def core_num():
        return int(_capi.load().dvm_rt_sm_count())

    @staticmethod
    def soc_name():
        return "B200"
