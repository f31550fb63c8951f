"""The five benchmark graphs, written against the builder API (any object with the Kernel method names).

Each function takes a builder ``k`` and already-loaded operands and returns the value(s) to store, so the
same definition drives the device kernel (Tester / PyKernel) and any other evaluator of the API.
Formulas follow the reference's own examples and tests: examples/01_add.py:19-25 (scaled up),
examples/02_batchnorm.py:25-45, tests/ut/test_spec_vector.py:133-160 (RMSNorm),
examples/04_matmul_post_fusion.py:19-40 (SiLU chain), examples/03_attention.py:31-52,
tests/ut/test_composite_ops.py:25-65 (tanh-GeLU through exp).
"""
F32 = 3  # dvm::kFloat32
F16 = 1
BF16 = 2


def fused_elementwise(k, x, y):
    """C1: z = exp(x) * y + 0.5."""
    return k.add(k.mul(k.exp(x), y), 0.5)


def batchnorm_train(k, x, gamma, beta, count, eps=1e-5):
    """C2: per-channel training batch-norm of NCHW fp16 x; returns (y fp16, mean fp32, var fp32).

    gamma/beta are fp32 of shape [1, C, 1, 1]; statistics are reduced over (N, H, W) in fp32.
    """
    xf = k.cast(x, F32)
    rec = 1.0 / float(count)
    mean = k.mul(k.sum(xf, (0, 2, 3), True), rec)
    xc = k.sub(xf, mean)
    var = k.mul(k.sum(k.mul(xc, xc), (0, 2, 3), True), rec)
    std = k.sqrt(k.add(var, eps))
    y = k.add(k.mul(k.div(xc, std), gamma), beta)
    return k.cast(y, F16), mean, var


def rmsnorm_swiglu(k, h, r, w, g, u, hidden, eps=1e-6):
    """C3: out1 = rmsnorm(h + r) * w, out2 = silu(g) * u; bf16 in/out, fp32 math."""
    s = k.add(k.cast(h, F32), k.cast(r, F32))
    ss = k.sum(k.mul(s, s), (1,), True)
    inv = k.div(1.0, k.sqrt(k.add(k.mul(ss, 1.0 / float(hidden)), eps)))
    out1 = k.cast(k.mul(k.mul(s, inv), k.cast(w, F32)), BF16)
    gf = k.cast(g, F32)
    sig = k.div(1.0, k.add(k.exp(k.mul(gf, -1.0)), 1.0))
    out2 = k.cast(k.mul(k.mul(gf, sig), k.cast(u, F32)), BF16)
    return out1, out2


def gelu_tanh(k, x):
    """0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x^3))) written as x / (1 + exp(-2*sqrt(2/pi)*(x+0.044715x^3)))."""
    x3 = k.mul(k.mul(x, x), x)
    inner = k.add(x, k.mul(x3, 0.044715))
    e = k.exp(k.mul(inner, -1.5957691216057308))
    return k.div(x, k.add(e, 1.0))


def matmul_bias_gelu(k, a, b, bias):
    """C5: C = gelu_tanh(A @ B + bias), fp32 epilogue, bf16 result."""
    c = k.matmul(a, b, False, False, bias)
    return k.cast(gelu_tanh(k, k.cast(c, F32)), BF16)


def attention(k, q, kmat, v, scale, dtype=BF16):
    """C4: softmax(Q K^T * scale) V, non-causal, fp32 softmax, result in the operand type `dtype`."""
    s = k.mul(k.matmul(q, kmat, False, True), scale)
    s = k.cast(s, F32)
    m = k.max(s, (-1,), True)
    e = k.exp(k.sub(s, m))
    p = k.div(e, k.sum(e, (-1,), True))
    return k.matmul(k.cast(p, dtype), v, False, False)
