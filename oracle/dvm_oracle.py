"""CPU oracle for the fused-operator path: a NumPy restatement of the reference's per-op semantics.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; only tests/, the smoke
check and the CPU-baseline legs of bench.py use it, and only as the checker.

It restates, in NumPy, what mindspore-ai/dvm computes for a graph built through its Python API:
  * the API-level dtype lowering of src/dvm.cc (which ops are promoted through fp16/fp32, how scalars are
    encoded, which casts chain through which type) - each method cites the lines it follows;
  * the device arithmetic of the CUDA interpreter src/vm_gpu.cu:147-329 - fp32 math, fp16/bf16 results
    rounded to storage precision after every op, float->int by truncation, compares producing 1/0 in the
    operand dtype, max/min as ``a > b ? a : b``, sums accumulated in double (src/vm_gpu.cu:796-835).
One deliberate difference: fp32->bf16 keeps NaN as NaN (the host encoder's rule, src/dvm.cc:173-186); the
reference's device routine (src/vm_gpu.cu:155-160) has no NaN guard.

Parity pinning: the reference stores no golden vectors for this path - every expectation in its tests is
recomputed with NumPy from a seed (tests/ut/*.py).  tests/test_oracle_pins.py checks this oracle against
those same NumPy formulas and tests/golden/ holds vectors produced by it with the generating script.
"""
import numpy as np

try:
    import ml_dtypes
    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    _BF16 = None

BOOL, F16, BF16, F32, I32, I64 = range(6)
DTYPE_NAMES = ["bool", "float16", "bfloat16", "float32", "int32", "int64"]


def round_bf16(x):
    """fp32 -> nearest-even bf16 precision, returned as fp32 (src/dvm.cc:173-186)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u >> 16) & 1) + 0x7FFF
    out = (((u + r) >> 16) << 16).astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), np.float32(np.nan), out).astype(np.float32)


def round_f16(x):
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_to(dtype, x):
    if dtype == F16:
        return round_f16(x)
    if dtype == BF16:
        return round_bf16(x)
    return np.asarray(x, dtype=np.float32)


def to_storage(dtype, a):
    """Register-form array -> array in the tensor's storage dtype."""
    if dtype == BOOL:
        return a.astype(np.bool_)
    if dtype == F16:
        return a.astype(np.float16)
    if dtype == BF16:
        return a.astype(_BF16) if _BF16 is not None else (a.view(np.uint32) >> 16).astype(np.uint16)
    if dtype == F32:
        return a.astype(np.float32)
    if dtype == I32:
        return a.astype(np.int32)
    raise ValueError("unsupported dtype")


def from_storage(dtype, a):
    """Storage array -> register form (fp32 for float types, int32 for int32/bool)."""
    a = np.asarray(a)
    if dtype in (BOOL, I32):
        return a.astype(np.int32)
    if dtype == BF16 and a.dtype == np.uint16:
        return (a.astype(np.uint32) << 16).view(np.float32)
    return a.astype(np.float32)


def dtype_of_array(a):
    if _BF16 is not None and a.dtype == _BF16:
        return BF16
    return {np.dtype(np.bool_): BOOL, np.dtype(np.float16): F16, np.dtype(np.float32): F32,
            np.dtype(np.int32): I32}[a.dtype]


# next hop of the cast chain (g_cast_staff_type, src/dvm.cc:416-423)
def cast_hop(cur, target):
    if cur == target:
        return target
    if cur == BOOL:
        return F16
    if target == BOOL:
        if cur in (F16, I64):
            return BOOL
        return F32 if cur == BF16 else F16
    if cur in (F16, BF16):
        return I32 if target == I32 else F32
    if cur == F32:
        return target
    if cur == I32:
        return F16 if target == F16 else (I64 if target == I64 else F32)
    return I32 if target == I32 else F32


class OVal:
    """A value of the oracle: dtype + register-form array (+ how it was made, for promotion peeling)."""

    def __init__(self, dtype, a, noloss_src=None):
        self.dt = dtype
        self.a = a
        self.noloss_src = noloss_src  # set when this value is a promotion cast of `noloss_src`

    def shape(self):
        return tuple(self.a.shape)

    def dtype(self):
        return self.dt


def _is_int(dt):
    return dt in (BOOL, I32)


class OracleKernel:
    """Evaluates eagerly; method names and argument order follow the reference's Python Kernel."""

    # ---- inputs / outputs ----------------------------------------------------------------------
    def load(self, array, dtype=None):
        array = np.asarray(array)
        dt = dtype_of_array(array) if dtype is None else int(dtype)
        if dt == BF16 and array.dtype == np.float32:
            array = round_bf16(array)
        if dt == F16 and array.dtype == np.float32:
            array = round_f16(array)
        return OVal(dt, from_storage(dt, array))

    def store(self, x, dtype=None):
        """Returns the stored tensor in its storage dtype (Store, src/dvm.cc:1546-1561)."""
        if dtype is not None:
            x = self.cast(x, dtype)
        return to_storage(x.dt, x.a)

    # ---- single cast step (device casts, src/vm_gpu.cu:293-329) ---------------------------------
    def _cast_step(self, x, to, noloss=False):
        frm = x.dt
        a = x.a
        if to == BOOL:
            out = (a != 0).astype(np.int32)
        elif _is_int(frm) and not _is_int(to):
            out = round_to(to, a.astype(np.float32))
        elif not _is_int(frm) and to == I32:
            with np.errstate(invalid="ignore"):
                out = np.trunc(a).astype(np.int32)
        elif _is_int(frm):
            out = a.astype(np.int32)
        else:
            out = round_to(to, a)
        return OVal(to, out, noloss_src=x if noloss else None)

    def _noloss_cast(self, x, to):
        """NoLossCast, src/dvm.cc:425-443: undo a previous promotion instead of stacking a new cast."""
        cur = x.dt
        while cur != to:
            hop = cast_hop(cur, to)
            if x.noloss_src is not None and x.noloss_src.dt == hop:
                x = x.noloss_src
            else:
                x = self._cast_step(x, hop, noloss=True)
            cur = hop
        return x

    def cast(self, x, to):
        """Kernel::Cast, src/dvm.cc:1429-1447."""
        to = int(to)
        if x.dt == to:
            return x
        if to == BOOL:
            x = self.not_equal(x, 0)
        cur = x.dt
        while cur != to:
            hop = cast_hop(cur, to)
            x = self._cast_step(x, hop)
            cur = hop
        return x

    # ---- scalars --------------------------------------------------------------------------------
    @staticmethod
    def _encode(v, dt):
        """EncodeScalar, src/dvm.cc:188-223: scalar -> register-form value of the tensor dtype."""
        is_float = isinstance(v, (float, np.floating))
        f = np.float32(v) if is_float else np.float32(int(v))
        if dt == F16:
            return round_f16(f)[()]
        if dt == BF16:
            return round_bf16(np.array(f))[()]
        if dt == F32:
            return f
        if dt == I32:
            return np.int32(int(np.float32(v))) if is_float else np.int32(int(v))
        return np.int32(1 if v != 0 else 0)

    # ---- unary (Kernel::Unary, src/dvm.cc:1245-1283) --------------------------------------------
    def _unary(self, name, x):
        if x.dt == BOOL:
            r = self._unary(name, self._noloss_cast(x, F16))
            return self._noloss_cast(r, BOOL)
        if x.dt == BF16:
            return self.cast(self._unary(name, self.cast(x, F32)), BF16)
        if x.dt == F16 and name in ("round", "floor", "ceil", "trunc"):
            return self.cast(self._unary(name, self.cast(x, F32)), F16)
        if name == "logical_not":
            return self.sub(1, x)
        if name == "reciprocal":
            return self.div(1, x)
        a = x.a
        with np.errstate(all="ignore"):
            if name == "abs" and x.dt == I32:
                return OVal(I32, np.where(a < 0, (0 - a.astype(np.int64)).astype(np.int32), a).astype(np.int32))
            fn = {"sqrt": np.sqrt, "abs": np.abs, "log": np.log, "exp": np.exp, "round": np.rint,
                  "floor": np.floor, "ceil": np.ceil, "trunc": np.trunc,
                  "isfinite": lambda t: np.isfinite(t).astype(np.float32)}[name]
            out = fn(a.astype(np.float32)).astype(np.float32)
        return OVal(x.dt, round_to(x.dt, out))

    def sqrt(self, x): return self._unary("sqrt", x)
    def abs(self, x): return self._unary("abs", x)
    def log(self, x): return self._unary("log", x)
    def exp(self, x): return self._unary("exp", x)
    def reciprocal(self, x): return self._unary("reciprocal", x)
    def isfinite(self, x): return self._unary("isfinite", x)
    def logical_not(self, x): return self._unary("logical_not", x)
    def round(self, x): return self._unary("round", x)
    def floor(self, x): return self._unary("floor", x)
    def ceil(self, x): return self._unary("ceil", x)
    def trunc(self, x): return self._unary("trunc", x)

    # ---- binary ---------------------------------------------------------------------------------
    @staticmethod
    def _arith(name, dt, a, b):
        """Device functors, src/vm_gpu.cu:198-254 (fp16/bf16: fp32 math then round to storage)."""
        with np.errstate(all="ignore"):
            if _is_int(dt):
                a64, b64 = a.astype(np.int64), b.astype(np.int64)
                if name == "add": r = a64 + b64
                elif name == "sub": r = a64 - b64
                elif name == "mul": r = a64 * b64
                elif name in ("maximum", "logical_or"): r = np.where(a64 > b64, a64, b64)
                elif name in ("minimum", "logical_and"): r = np.where(a64 < b64, a64, b64)
                else: raise ValueError("int op " + name)
                return (r & 0xFFFFFFFF).astype(np.uint32).view(np.int32) if r.ndim else np.int32(np.uint32(int(r) & 0xFFFFFFFF).view(np.int32))
            a = np.asarray(a, dtype=np.float32)
            b = np.asarray(b, dtype=np.float32)
            if name == "add": r = a + b
            elif name == "sub": r = a - b
            elif name == "mul": r = a * b
            elif name == "div": r = a / b
            elif name == "pow": r = np.power(a, b)
            elif name in ("maximum", "logical_or"): r = np.where(a > b, a, b)
            elif name in ("minimum", "logical_and"): r = np.where(a < b, a, b)
            else: raise ValueError(name)
            return round_to(dt, r.astype(np.float32))

    @staticmethod
    def _compare(name, dt, a, b):
        """CompareValue, src/vm_gpu.cu:331-349: 1/0 written in the operand dtype."""
        with np.errstate(invalid="ignore"):
            r = {"equal": a == b, "not_equal": a != b, "greater": a > b, "greater_equal": a >= b,
                 "less": a < b, "less_equal": a <= b}[name]
        return r.astype(np.int32) if _is_int(dt) else r.astype(np.float32)

    _CMP = ("equal", "not_equal", "greater", "greater_equal", "less", "less_equal")
    _MIRROR = {"equal": "equal", "not_equal": "not_equal", "greater": "less", "greater_equal": "less_equal",
               "less": "greater", "less_equal": "greater_equal"}

    def _tensor_binary(self, name, x, y):
        """Kernel::Binary tensor-tensor branch, src/dvm.cc:1317-1381."""
        if x.dt == BOOL:
            r = self._tensor_binary(name, self._noloss_cast(x, F16), self._noloss_cast(y, F16))
            return self._noloss_cast(r, BOOL)
        if (x.dt == BF16 and name in ("pow", "div")) or (x.dt == F16 and name == "pow"):
            r = self._tensor_binary(name, self.cast(x, F32), self.cast(y, F32))
            return self.cast(r, x.dt)
        a, b = np.broadcast_arrays(x.a, y.a)
        if name in self._CMP:
            return self._noloss_cast(OVal(x.dt, self._compare(name, x.dt, a, b)), BOOL)
        return OVal(x.dt, self._arith(name, x.dt, a, b))

    def _full_like(self, v, x):
        if x.dt == BOOL:
            return self.cast(OVal(F16, np.full(x.a.shape, self._encode(v, F16), np.float32)), BOOL)
        enc = self._encode(v, x.dt)
        return OVal(x.dt, np.full(x.a.shape, enc, np.int32 if _is_int(x.dt) else np.float32))

    def _scalar_binary(self, name, v, x, scalar_rhs):
        """GetBinaryS, src/dvm.cc:586-676; None when the table has no scalar form."""
        is_int_scalar = isinstance(v, (int, np.integer)) and not isinstance(v, (bool, np.bool_))
        if name in ("add", "mul", "minimum", "maximum"):
            return OVal(x.dt, self._arith(name, x.dt, x.a, self._encode(v, x.dt)))
        if name == "div":
            if x.dt == BF16:
                r = self._scalar_binary(name, v, self.cast(x, F32), scalar_rhs)
                return self.cast(r, BF16)
            s = self._encode(v, x.dt)
            return OVal(x.dt, self._arith("div", x.dt, x.a, s) if scalar_rhs else self._arith("div", x.dt, s, x.a))
        if name in self._CMP:
            if x.dt == I32:
                return None
            op = name if scalar_rhs else self._MIRROR[name]
            r = OVal(x.dt, self._compare(op, x.dt, x.a, self._encode(v, x.dt)))
            return self._noloss_cast(r, BOOL)
        if name == "pow":
            if scalar_rhs:
                if is_int_scalar or (isinstance(v, (float, np.floating)) and np.floor(v) == v):
                    return self._pow_int(x, v)
                return None
            if v > 0:
                if x.dt != F32:
                    r = self._scalar_binary("pow", float(np.float32(v)), self.cast(x, F32), False)
                    return self.cast(r, x.dt)
                t = self._scalar_binary("mul", float(np.log(np.float32(v))), x, True)
                return self.exp(t)
            return None
        if name == "sub":
            if scalar_rhs:
                return self._scalar_binary("add", -v, x, True)
            neg = self._scalar_binary("mul", -1 if is_int_scalar else -1.0, x, True)
            return self._scalar_binary("add", v, neg, True)
        return None

    def _pow_int(self, x, v):
        """PowS, src/dvm.cc:255-279: integer exponent as a multiply chain."""
        n = abs(int(v))
        if n == 0:
            return self._full_like(1 if isinstance(v, (int, np.integer)) else 1.0, x)
        res = None
        if n == 1:
            res = x
        else:
            base = x
            while n:
                if n & 1:
                    res = base if res is None else self.mul(res, base)
                if n != 1:
                    base = self.mul(base, base)
                n >>= 1
        if v < 0:
            res = self.reciprocal(res)
        return res

    def _binary(self, name, lhs, rhs):
        if not isinstance(lhs, OVal):
            return self._scalar_tensor(name, lhs, rhs, False)
        if not isinstance(rhs, OVal):
            return self._scalar_tensor(name, rhs, lhs, True)
        return self._tensor_binary(name, lhs, rhs)

    def _scalar_tensor(self, name, v, x, scalar_rhs):
        """Kernel::Binary scalar branches, src/dvm.cc:1300-1316."""
        if x.dt == BOOL:
            r = self._scalar_tensor(name, v, self._noloss_cast(x, F16), scalar_rhs)
            return self._noloss_cast(r, BOOL)
        r = self._scalar_binary(name, v, x, scalar_rhs)
        if r is not None:
            return r
        full = self._full_like(v, x)
        return self._tensor_binary(name, x, full) if scalar_rhs else self._tensor_binary(name, full, x)

    def equal(self, a, b): return self._binary("equal", a, b)
    def not_equal(self, a, b): return self._binary("not_equal", a, b)
    def greater(self, a, b): return self._binary("greater", a, b)
    def greater_equal(self, a, b): return self._binary("greater_equal", a, b)
    def less(self, a, b): return self._binary("less", a, b)
    def less_equal(self, a, b): return self._binary("less_equal", a, b)
    def add(self, a, b): return self._binary("add", a, b)
    def sub(self, a, b): return self._binary("sub", a, b)
    def mul(self, a, b): return self._binary("mul", a, b)
    def div(self, a, b): return self._binary("div", a, b)
    def pow(self, a, b): return self._binary("pow", a, b)
    def maximum(self, a, b): return self._binary("maximum", a, b)
    def minimum(self, a, b): return self._binary("minimum", a, b)
    def logical_and(self, a, b): return self._binary("logical_and", a, b)
    def logical_or(self, a, b): return self._binary("logical_or", a, b)

    # ---- select / broadcast / reshape / copy ------------------------------------------------------
    def select(self, cond, lhs, rhs):
        """Kernel::Select src/dvm.cc:1415-1427; device SelectOp src/vm_gpu.cu:401-410."""
        if cond.dt != lhs.dt:
            cond = self._noloss_cast(cond, lhs.dt)
        c, a, b = np.broadcast_arrays(cond.a, lhs.a, rhs.a)
        return OVal(lhs.dt, np.where(c != 0, a, b))

    def broadcast(self, x, shape):
        shape = list(shape)
        src = list(x.a.shape)
        for i, s in enumerate(shape):
            if s == -1:
                shape[i] = src[len(src) + i - len(shape)]
        return OVal(x.dt, np.broadcast_to(x.a, shape).copy())

    def full(self, scalar, shape, dtype):
        dtype = int(dtype)
        if dtype == BOOL:
            return self.cast(self.full(scalar, shape, F16), BOOL)
        enc = self._encode(scalar, dtype)
        return OVal(dtype, np.full(list(shape), enc, np.int32 if _is_int(dtype) else np.float32))

    def reshape(self, x, shape):
        return OVal(x.dt, x.a.reshape(list(shape)))

    def copy(self, x):
        return OVal(x.dt, x.a.copy())

    # ---- reductions (fp32 only for sum, src/dvm.cc:1537-1544; double accumulation) -----------------
    def _reduce(self, kind, x, dims, keepdims):
        if kind == "sum" and x.dt != F32:
            return None
        if _is_int(x.dt):
            return None
        axes = tuple(int(d) % x.a.ndim for d in dims)
        if kind == "sum":
            r = np.sum(x.a.astype(np.float64), axis=axes, keepdims=keepdims).astype(np.float32)
        elif kind == "max":
            r = np.max(x.a, axis=axes, keepdims=keepdims)
        else:
            r = np.min(x.a, axis=axes, keepdims=keepdims)
        return OVal(x.dt, np.asarray(r, dtype=np.float32))

    def sum(self, x, dims, keepdims=False): return self._reduce("sum", x, dims, keepdims)
    def max(self, x, dims, keepdims=False): return self._reduce("max", x, dims, keepdims)
    def min(self, x, dims, keepdims=False): return self._reduce("min", x, dims, keepdims)

    # ---- matmul (CubeOp semantics, src/ops_m.h:29-141: fp32 accumulate, result in the input dtype) ----
    def matmul(self, lhs, rhs, trans_a, trans_b, bias=None):
        a = lhs.a.astype(np.float32)
        b = rhs.a.astype(np.float32)
        if trans_a:
            a = np.swapaxes(a, -1, -2)
        if trans_b:
            b = np.swapaxes(b, -1, -2)
        c = np.matmul(a, b)
        if bias is not None:
            c = c + bias.a.astype(np.float32)
        return OVal(lhs.dt, round_to(lhs.dt, c.astype(np.float32)))
