"""ctypes binding of the C ABI declared in include/dvm_c.h.

The library is the product: if it is missing this module raises at import of the first symbol, and
there is no Python or CPU fallback for any compute entry point.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libdvm_b200.so")

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_size_t = ctypes.c_size_t
c_int64 = ctypes.c_int64
c_char_p = ctypes.c_char_p


class Reloc(ctypes.Structure):
    _fields_ = [("io", c_void_p), ("addr", c_void_p)]


WS_ALLOC_FN = ctypes.CFUNCTYPE(c_void_p, c_size_t, c_void_p)

# name -> (restype, argtypes); every symbol include/dvm_c.h declares
SIGNATURES = {
    "dvm_last_error": (c_char_p, []),
    "dvm_version": (c_char_p, []),
    "dvm_int_array_new": (c_void_p, [ctypes.POINTER(c_int64), c_size_t]),
    "dvm_int_array_update": (c_int, [c_void_p, ctypes.POINTER(c_int64), c_size_t]),
    "dvm_int_array_size": (c_size_t, [c_void_p]),
    "dvm_int_array_data": (ctypes.POINTER(c_int64), [c_void_p]),
    "dvm_int_array_free": (None, [c_void_p]),
    "dvm_scalar_new": (c_void_p, []),
    "dvm_scalar_set_f32": (None, [c_void_p, ctypes.c_float]),
    "dvm_scalar_set_i64": (None, [c_void_p, c_int64]),
    "dvm_scalar_free": (None, [c_void_p]),
    "dvm_kernel_new": (c_void_p, [c_int, ctypes.c_uint32]),
    "dvm_kernel_reset": (c_int, [c_void_p, c_int, ctypes.c_uint32]),
    "dvm_kernel_free": (None, [c_void_p]),
    "dvm_set_name_hint": (c_int, [c_void_p, c_char_p]),
    "dvm_load": (c_void_p, [c_void_p, c_void_p, c_void_p, c_int]),
    "dvm_store": (c_void_p, [c_void_p, c_void_p, c_void_p]),
    "dvm_load_strided": (c_void_p, [c_void_p, c_void_p, c_void_p, c_void_p, c_int]),
    "dvm_slice_load": (c_void_p, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int]),
    "dvm_strided_slice_load": (c_void_p, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int]),
    "dvm_elem_any": (c_void_p, [c_void_p, c_void_p]),
    "dvm_pad_store": (c_void_p, [c_void_p, c_void_p, c_void_p, c_int64]),
    "dvm_store_strided": (c_void_p, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "dvm_unary": (c_void_p, [c_void_p, c_int, c_void_p]),
    "dvm_binary": (c_void_p, [c_void_p, c_int, c_void_p, c_void_p]),
    "dvm_binary_f32": (c_void_p, [c_void_p, c_int, c_void_p, ctypes.c_float, c_int]),
    "dvm_binary_i64": (c_void_p, [c_void_p, c_int, c_void_p, c_int64, c_int]),
    "dvm_binary_ref": (c_void_p, [c_void_p, c_int, c_void_p, c_void_p, c_int]),
    "dvm_reduce": (c_void_p, [c_void_p, c_int, c_void_p, c_void_p, c_int]),
    "dvm_select": (c_void_p, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "dvm_cast": (c_void_p, [c_void_p, c_void_p, c_int]),
    "dvm_broadcast": (c_void_p, [c_void_p, c_void_p, c_void_p]),
    "dvm_full_f32": (c_void_p, [c_void_p, ctypes.c_float, c_void_p, c_int]),
    "dvm_full_i64": (c_void_p, [c_void_p, c_int64, c_void_p, c_int]),
    "dvm_full_ref": (c_void_p, [c_void_p, c_void_p, c_void_p, c_int]),
    "dvm_reshape": (c_void_p, [c_void_p, c_void_p, c_void_p]),
    "dvm_permute": (c_void_p, [c_void_p, c_void_p, c_void_p]),
    "dvm_slice": (c_void_p, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "dvm_slice_dim": (c_void_p, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "dvm_split_chunk": (c_void_p, [c_void_p, c_void_p, c_int, c_int64, c_size_t, c_size_t]),
    "dvm_clone_map_new": (c_void_p, []),
    "dvm_clone_map_free": (None, [c_void_p]),
    "dvm_clone_map_int_array": (c_int, [c_void_p, c_void_p, c_void_p]),
    "dvm_clone_map_scalar": (c_int, [c_void_p, c_void_p, c_void_p]),
    "dvm_kernel_clone": (c_int, [c_void_p, c_void_p, c_void_p]),
    "dvm_clone_map_object": (c_void_p, [c_void_p, c_void_p]),
    "dvm_concat": (c_void_p, [c_void_p, ctypes.POINTER(c_void_p), c_size_t, c_int]),
    "dvm_copy": (c_void_p, [c_void_p, c_void_p]),
    "dvm_matmul": (c_void_p, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "dvm_comm_new": (c_void_p, []),
    "dvm_comm_free": (None, [c_void_p]),
    "dvm_comm_id_bytes": (c_size_t, []),
    "dvm_comm_unique_id": (c_int, [c_void_p, c_size_t]),
    "dvm_comm_init_rank": (c_int, [c_void_p, c_void_p, c_size_t, c_int, c_int]),
    "dvm_comm_init_dummy": (c_int, [c_void_p, c_int, c_int]),
    "dvm_comm_adopt": (c_int, [c_void_p, c_void_p]),
    "dvm_comm_rank": (c_int, [c_void_p]),
    "dvm_comm_size": (c_int, [c_void_p]),
    "dvm_allreduce": (c_void_p, [c_void_p, c_int, c_void_p, c_void_p]),
    "dvm_allgather": (c_void_p, [c_void_p, c_void_p, c_void_p]),
    "dvm_reducescatter": (c_void_p, [c_void_p, c_void_p, c_void_p]),
    "dvm_sequence_add": (c_int, [c_void_p, c_int, ctypes.c_uint32]),
    "dvm_parallel_add": (c_int, [c_void_p, c_int, ctypes.c_uint32, c_size_t]),
    "dvm_spec_next": (c_int, [c_void_p]),
    "dvm_set_store_inplace": (c_int, [c_void_p, c_void_p]),
    "dvm_normalize": (c_int, [c_void_p]),
    "dvm_pre_codegen": (c_int, [c_void_p, ctypes.POINTER(c_size_t)]),
    "dvm_codegen": (c_int, [c_void_p, ctypes.POINTER(Reloc), c_size_t, WS_ALLOC_FN, c_void_p]),
    "dvm_launch": (c_int, [c_void_p, c_void_p]),
    "dvm_launch_reloc": (c_int, [c_void_p, ctypes.POINTER(Reloc), c_size_t, c_void_p, c_void_p]),
    "dvm_launch_static_scratch": (c_int, [c_void_p, ctypes.POINTER(Reloc), c_size_t, c_void_p]),
    "dvm_static_scratch_capacity": (c_size_t, []),
    "dvm_last_jit_us": (ctypes.c_double, [c_void_p]),
    "dvm_object_rank": (c_int, [c_void_p]),
    "dvm_object_dim": (c_int64, [c_void_p, c_int]),
    "dvm_object_dtype": (c_int, [c_void_p]),
    "dvm_dump": (c_char_p, [c_void_p]),
    "dvm_dump_r": (c_char_p, [c_void_p]),
    "dvm_das": (c_char_p, [c_void_p]),
    "dvm_inspect": (c_char_p, [c_void_p]),
    "dvm_rt_device_count": (c_int, []),
    "dvm_rt_set_device": (c_int, [c_int]),
    "dvm_rt_sm_count": (c_int, []),
    "dvm_rt_malloc": (c_void_p, [c_size_t]),
    "dvm_rt_free": (c_int, [c_void_p]),
    "dvm_rt_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "dvm_rt_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "dvm_rt_memset": (c_int, [c_void_p, c_int, c_size_t, c_void_p]),
    "dvm_rt_sync": (c_int, [c_void_p]),
    "dvm_rt_check_status": (c_int, []),
    "dvm_rt_selftest_wait_expiry": (c_int, [ctypes.c_uint, c_void_p]),
    "dvm_rt_host_alloc": (c_void_p, [c_size_t]),
    "dvm_rt_host_free": (c_int, [c_void_p]),
    "dvm_perf": (c_int, [c_void_p, c_int, c_int, c_void_p, ctypes.POINTER(ctypes.c_float),
                         ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float)]),
    "dvm_perf_stages": (c_int, [c_void_p, c_int, c_int, c_void_p, ctypes.POINTER(ctypes.c_float), c_size_t,
                                ctypes.POINTER(c_size_t)]),
}

_lib = None


def load():
    """Load libdvm_b200.so and set every prototype; raise if the library was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "dvm_b200: %s is missing; build it with `python -m dvm_b200.build` "
            "(there is no fallback implementation)" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


class DvmError(RuntimeError):
    pass


def last_error():
    return load().dvm_last_error().decode("utf-8", "replace")


def check_ptr(p, what):
    if not p:
        raise DvmError("%s failed: %s" % (what, last_error()))
    return p


def check_rc(rc, what):
    if rc != 0:
        raise DvmError("%s failed (code %d): %s" % (what, rc, last_error()))
