"""CPU oracle for the training-step path: numpy front end over oracle/mc_oracle.c
plus a small define-by-run tape, Adam and GradScaler that follow the reference's
host logic.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU
baseline leg of the benchmark.  The shipped package never imports it.

Reference files followed (paths relative to the reference project root):
  tape walker      crates/modern-chainer-autograd/src/variable.rs:150-217
  apply / OpNode   crates/modern-chainer-autograd/src/node.rs:26-79
  op backward      crates/modern-chainer-autograd/src/ops.rs, host_ops.rs
  Adam, zero_grad  crates/modern-chainer-optim/src/lib.rs:17-120
  GradScaler       crates/modern-chainer-optim/src/amp.rs:8-113
  nn initialisers  crates/modern-chainer-nn/src/lib.rs:38-73,141-147,185-191,246-271
  decoder layout   crates/modern-chainer-llm/src/decoder.rs:98-140,213-241
"""
import ctypes as C
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
F32, I64, I32, U8, F16, BF16 = 0, 1, 2, 3, 4, 5
_NP2DT = {np.dtype(np.int64): I64, np.dtype(np.int32): I32, np.dtype(np.uint8): U8}


class OracleError(Exception):
    def __init__(self, status):
        super().__init__(f"oracle status {status}")
        self.status = status


def build():
    subprocess.check_call(["make", "-s", "-f", os.path.join(_HERE, "Makefile")], cwd=_HERE)


_libs = {}


def lib(fast=False):
    """Load the checker build (gcc -O2, single thread) or the OpenMP build (-O3 -fopenmp)."""
    name = "libmc_oracle_fast.so" if fast else "libmc_oracle.so"
    if name not in _libs:
        path = os.path.join(_HERE, name)
        if not os.path.exists(path):
            build()
        l = C.CDLL(path)
        l.mco_sum_all.restype = C.c_float
        l.mco_count_non_finite.restype = C.c_int64
        l.mco_rng_normal.restype = C.c_double
        l.mco_rng_next_f64.restype = C.c_double
        l.mco_rng_next_u64.restype = C.c_uint64
        l.mco_f32_to_bf16_bits.restype = C.c_uint16
        l.mco_f32_to_bf16_bits.argtypes = [C.c_float]
        l.mco_bf16_bits_to_f32.restype = C.c_float
        l.mco_bf16_bits_to_f32.argtypes = [C.c_uint16]
        _libs[name] = l
    return _libs[name]


# "checker": one thread, big GEMMs summed in f64 (the parity reference)
# "threaded": the same arithmetic, operation for operation, with independent loop iterations spread
#             over OpenMP threads (bit-identical to "checker"; for full-size parity cases)
# "fast": f32 blocked threaded GEMM (different summation order; the timed CPU baseline only)
_MODE = "checker"


def set_mode(mode):
    global _MODE
    assert mode in ("checker", "threaded", "fast")
    _MODE = mode


def use_fast(on=True):
    """Route every kernel through the threaded timing build (CPU baseline runs)."""
    set_mode("fast" if on else "checker")


class threaded:
    """`with threaded():` runs the checker arithmetic on all host cores (same bits, less waiting)."""

    def __enter__(self):
        self.prev = _MODE
        set_mode("threaded")

    def __exit__(self, *a):
        set_mode(self.prev)


def _l():
    if _MODE == "checker":
        return lib(False)
    l = lib(True)
    l.mco_set_fast_gemm(1 if _MODE == "fast" else 0)
    l.mco_set_parallel(1)
    return l


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _dims(shape):
    return (C.c_int64 * max(len(shape), 1))(*shape)


def _i(v):
    return C.c_int64(int(v))


def _chk(st):
    if st:
        raise OracleError(st)


# ---------------------------------------------------------------- RNG / init
class Rng:
    class _S(C.Structure):
        _fields_ = [("state", C.c_uint64), ("has_spare", C.c_int), ("spare", C.c_double)]

    def __init__(self, seed):
        self.s = Rng._S()
        lib().mco_rng_seed(C.byref(self.s), C.c_uint64(seed))

    def next_u64(self):
        return lib().mco_rng_next_u64(C.byref(self.s))

    def next_f64(self):
        return lib().mco_rng_next_f64(C.byref(self.s))

    def normal(self):
        return lib().mco_rng_normal(C.byref(self.s))

    def normal_vec(self, n, mean, std):
        out = np.empty(n, np.float32)
        lib().mco_rng_normal_fill(C.byref(self.s), _i(n), C.c_double(mean), C.c_double(std), _p(out))
        return out


def he_normal(shape, fan_in, seed):
    n = int(np.prod(shape))
    out = np.empty(n, np.float32)
    lib().mco_he_normal(_i(n), _i(fan_in), C.c_uint64(seed), _p(out))
    return out.reshape(shape)


# ---------------------------------------------------------------- dtype helpers
def f32_to_bf16_bits(x):
    x = _f(x)
    out = np.empty(x.shape, np.uint16)
    lib().mco_f32_to_bf16(_p(x), _p(out), _i(x.size))
    return out


def bf16_bits_to_f32(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def round_bf16(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def f32_to_f16_bits(x):
    """core/src/dtype.rs:75-108 (see mco_f32_to_f16_bits for the subnormal range)."""
    x = _f(x)
    out = np.empty(x.shape, np.uint16)
    lib().mco_f32_to_f16(_p(x), _p(out), _i(x.size))
    return out


def f16_bits_to_f32(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    out = np.empty(b.shape, np.float32)
    lib().mco_f16_to_f32(_p(b), _p(out), _i(b.size))
    return out


def round_f16(x):
    return f16_bits_to_f32(f32_to_f16_bits(x))


# ---------------------------------------------------------------- low-precision (AMP) oracle
# The reference's CPU backend ignores autocast (only cuda/src/ops.rs reads it), so it has no
# low-precision arithmetic to restate.  Under `with amp(BF16)` / `amp(F16)` this oracle keeps every
# formula, accumulation type and loop order of the f32 oracle and rounds (to nearest even,
# core/src/dtype.rs:75-146) each tensor that a 16-bit training path stores in 16 bits, at the point
# where it is stored: LayerNorm outputs, Linear / linear_activation outputs and pre-activations,
# attention outputs, and in backward the gradients of those tensors.  GEMM operands are therefore
# 16-bit values, products are exact in f32 and sums are f32/f64 as before.  What stays in f32:
# parameters' master copies, the residual stream, LayerNorm / softmax / loss arithmetic, weight and
# bias gradients, optimizer state.  Comparing a 16-bit GPU step with this oracle isolates kernel
# error (summation order, on-chip roundings) from the format error both sides share.
_AMP = [None]


class amp:
    def __init__(self, dtype=BF16):
        assert dtype in (BF16, F16)
        self.dtype = dtype

    def __enter__(self):
        self.prev = _AMP[0]
        _AMP[0] = self.dtype

    def __exit__(self, *a):
        _AMP[0] = self.prev


def _lp(x, mode=None):
    mode = _AMP[0] if mode is None else mode
    if mode is None or x is None:
        return x
    return round_bf16(x) if mode == BF16 else round_f16(x)


# ---------------------------------------------------------------- kernels
def binary(op, a, b):
    a, b = _f(a), _f(b)
    out = np.empty(np.broadcast_shapes(a.shape, b.shape), np.float32)
    _chk(_l().mco_binary(op, _p(a), _dims(a.shape), a.ndim, _p(b), _dims(b.shape), b.ndim, _p(out)))
    return out


def add(a, b):
    return binary(0, a, b)


def sub(a, b):
    return binary(1, a, b)


def mul(a, b):
    return binary(2, a, b)


def div(a, b):
    return binary(3, a, b)


def scale(x, factor):
    x = _f(x)
    out = np.empty_like(x)
    _l().mco_scale(_p(x), C.c_double(factor), _p(out), _i(x.size))
    return out


def _map1(fn, x):
    x = _f(x)
    out = np.empty_like(x)
    fn(_p(x), _p(out), _i(x.size))
    return out


def relu(x):
    return _map1(_l().mco_relu, x)


def gelu(x):
    return _map1(_l().mco_gelu, x)


def unary(op, x):
    x = _f(x)
    out = np.empty_like(x)
    _l().mco_unary(op, _p(x), _p(out), _i(x.size))
    return out


def relu_backward(x, g):
    x, g = _f(x), _f(g)
    out = np.empty_like(x)
    _l().mco_relu_backward(_p(x), _p(g), _p(out), _i(x.size))
    return out


def gelu_backward(x, g):
    x, g = _f(x), _f(g)
    out = np.empty_like(x)
    _l().mco_gelu_backward(_p(x), _p(g), _p(out), _i(x.size))
    return out


def sum_all(x):
    x = _f(x)
    return np.float32(_l().mco_sum_all(_p(x), _i(x.size)))


def sum_to(a, shape):
    a = _f(a)
    shape = tuple(shape)
    out = np.empty(shape, np.float32)
    _chk(_l().mco_sum_to(_p(a), _dims(a.shape), a.ndim, _dims(shape), len(shape), _p(out)))
    return out


def matmul(a, b):
    a, b = _f(a), _f(b)
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), np.float32)
    _l().mco_matmul(_p(a), _p(b), _p(out), _i(m), _i(k), _i(n))
    return out


def linear(x, w, bias=None):
    x, w = _f(x), _f(w)
    m, k = x.shape
    n = w.shape[0]
    out = np.empty((m, n), np.float32)
    b = _f(bias) if bias is not None else None
    _l().mco_linear(_p(x), _p(w), _p(b) if b is not None else None, _p(out), _i(m), _i(k), _i(n))
    return out


def linear_backward(g, x, w, need_bias=True):
    g, x, w = _f(g), _f(x), _f(w)
    m, k = x.shape
    n = w.shape[0]
    dx, dw = np.empty((m, k), np.float32), np.empty((n, k), np.float32)
    db = np.empty(n, np.float32) if need_bias else None
    _l().mco_linear_backward(_p(g), _p(x), _p(w), _p(dx), _p(dw), _p(db) if need_bias else None, _i(m), _i(k), _i(n))
    return dx, dw, db


def softmax(x):
    x = _f(x)
    out = np.empty_like(x)
    _l().mco_softmax(_p(x), _p(out), _i(x.shape[0]), _i(x.shape[1]))
    return out


def softmax_backward(x, g):
    x, g = _f(x), _f(g)
    out = np.empty_like(x)
    _l().mco_softmax_backward(_p(x), _p(g), _p(out), _i(x.shape[0]), _i(x.shape[1]))
    return out


def layer_norm(x, gamma, beta, eps):
    x, gamma, beta = _f(x), _f(gamma), _f(beta)
    dim = x.shape[-1]
    out = np.empty_like(x)
    _l().mco_layer_norm(_p(x), _p(gamma), _p(beta), C.c_double(eps), _p(out), _i(x.size // dim), _i(dim))
    return out


def layer_norm_backward(x, gamma, g, eps):
    x, gamma, g = _f(x), _f(gamma), _f(g)
    dim = x.shape[-1]
    dx, dg, db = np.empty_like(x), np.empty(dim, np.float32), np.empty(dim, np.float32)
    _l().mco_layer_norm_backward(_p(x), _p(gamma), _p(g), C.c_double(eps), _p(dx), _p(dg), _p(db),
                                 _i(x.size // dim), _i(dim))
    return dx, dg, db


def _labels(t):
    t = np.ascontiguousarray(t)
    if t.dtype not in _NP2DT:
        raise OracleError(4)
    return t, _NP2DT[t.dtype]


def softmax_cross_entropy(x, labels):
    x = _f(x)
    lab, dt = _labels(labels)
    if lab.size != x.shape[0]:
        raise OracleError(5)
    out = C.c_float(0)
    _chk(_l().mco_softmax_cross_entropy(_p(x), _p(lab), dt, _i(x.shape[0]), _i(x.shape[1]), C.byref(out)))
    return np.float32(out.value)


def softmax_cross_entropy_backward(x, labels):
    x = _f(x)
    lab, dt = _labels(labels)
    if lab.size != x.shape[0]:
        raise OracleError(5)
    out = np.zeros_like(x)
    _chk(_l().mco_softmax_cross_entropy_backward(_p(x), _p(lab), dt, _i(x.shape[0]), _i(x.shape[1]), _p(out)))
    return out


def embedding(ids, weight):
    weight = _f(weight)
    ids_c, dt = _labels(ids)
    out = np.empty(ids_c.shape + (weight.shape[1],), np.float32)
    _chk(_l().mco_embedding(_p(ids_c), dt, _i(ids_c.size), _p(weight), _i(weight.shape[0]), _i(weight.shape[1]), _p(out)))
    return out


def embedding_backward(ids, weight_shape, g):
    g = _f(g)
    ids_c, dt = _labels(ids)
    out = np.empty(weight_shape, np.float32)
    _chk(_l().mco_embedding_backward(_p(ids_c), dt, _i(ids_c.size), _p(g), _i(weight_shape[0]), _i(weight_shape[1]), _p(out)))
    return out


def adam_update(p, g, m, v, lr, beta1, beta2, eps, step):
    p, g, m, v = _f(p), _f(g), _f(m), _f(v)
    np_, nm, nv = np.empty_like(p), np.empty_like(p), np.empty_like(p)
    _l().mco_adam_update(_p(p), _p(g), _p(m), _p(v), _p(np_), _p(nm), _p(nv), _i(p.size), C.c_double(lr),
                         C.c_double(beta1), C.c_double(beta2), C.c_double(eps), C.c_int32(step))
    return np_, nm, nv


def count_non_finite(g):
    g = _f(g)
    return int(_l().mco_count_non_finite(_p(g), _i(g.size)))


def _out_extent(i, k, s, p):
    return (i + 2 * p - k) // s + 1


def conv2d(x, w, bias, stride, pad):
    x, w = _f(x), _f(w)
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    out = np.empty((n, o, _out_extent(h, kh, stride, pad), _out_extent(wd, kw, stride, pad)), np.float32)
    b = _f(bias) if bias is not None else None
    _l().mco_conv2d(_p(x), _p(w), _p(b) if b is not None else None, _p(out), _i(n), _i(c), _i(h), _i(wd), _i(o),
                    _i(kh), _i(kw), _i(stride), _i(pad))
    return out


def conv2d_backward(x, w, g, stride, pad, need_bias=True):
    x, w, g = _f(x), _f(w), _f(g)
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    dx, dw = np.empty_like(x), np.empty_like(w)
    db = np.empty(o, np.float32) if need_bias else None
    _l().mco_conv2d_backward(_p(x), _p(w), _p(g), _p(dx), _p(dw), _p(db) if need_bias else None, _i(n), _i(c), _i(h),
                             _i(wd), _i(o), _i(kh), _i(kw), _i(stride), _i(pad))
    return dx, dw, db


def max_pool2d(x, kernel, stride, pad):
    x = _f(x)
    n, c, h, w = x.shape
    out = np.empty((n, c, _out_extent(h, kernel, stride, pad), _out_extent(w, kernel, stride, pad)), np.float32)
    _l().mco_max_pool2d(_p(x), _p(out), _i(n), _i(c), _i(h), _i(w), _i(kernel), _i(stride), _i(pad))
    return out


def max_pool2d_backward(x, g, kernel, stride, pad):
    x, g = _f(x), _f(g)
    n, c, h, w = x.shape
    dx = np.empty_like(x)
    _l().mco_max_pool2d_backward(_p(x), _p(g), _p(dx), _i(n), _i(c), _i(h), _i(w), _i(kernel), _i(stride), _i(pad))
    return dx


def attention(q, k, v, heads, causal):
    q, k, v = _f(q), _f(k), _f(v)
    n, s, d = q.shape
    out = np.empty_like(q)
    _l().mco_attention(_p(q), _p(k), _p(v), _p(out), _i(n), _i(s), _i(d), _i(heads), int(bool(causal)))
    return out


def attention_backward(q, k, v, g, heads, causal):
    q, k, v, g = _f(q), _f(k), _f(v), _f(g)
    n, s, d = q.shape
    dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(q)
    _l().mco_attention_backward(_p(q), _p(k), _p(v), _p(g), _p(dq), _p(dk), _p(dv), _i(n), _i(s), _i(d), _i(heads),
                                int(bool(causal)))
    return dq, dk, dv


# ---------------------------------------------------------------- tape
_grad_enabled = [True]


class no_grad:
    def __enter__(self):
        self.prev = _grad_enabled[0]
        _grad_enabled[0] = False

    def __exit__(self, *a):
        _grad_enabled[0] = self.prev


class Variable:
    """Mirror of autograd::Variable: data, grad, creator node, requires_grad."""

    def __init__(self, data, requires_grad=True, node=None):
        data = np.asarray(data)
        self.data = np.ascontiguousarray(data, np.float32) if data.dtype.kind == "f" else np.ascontiguousarray(data)
        self.grad = None
        self.node = node
        self.requires_grad = requires_grad

    @staticmethod
    def constant(data):
        return Variable(np.ascontiguousarray(data), requires_grad=False)

    def cleargrad(self):
        self.grad = None

    def unchain_backward(self):
        self.node = None

    def is_leaf(self):
        return self.node is None

    def backward(self):
        if not self.requires_grad or not _grad_enabled[0]:
            return
        order, seen, stack = [], set(), [(self, False)]
        while stack:
            var, expanded = stack.pop()
            if expanded:
                order.append(var)
                continue
            if id(var) in seen:
                continue
            seen.add(id(var))
            stack.append((var, True))
            if var.node is not None:
                for inp in var.node[1]:
                    stack.append((inp, False))
        grads = {id(self): np.ones_like(self.data, dtype=np.float32)}
        for var in reversed(order):
            g = grads.pop(id(var), None)
            if g is None:
                continue
            var.grad = g if var.grad is None else add(var.grad, g)
            if var.node is not None:
                bwd, inputs = var.node
                for inp, ig in zip(inputs, bwd(g)):
                    if ig is None or not inp.requires_grad:
                        continue
                    grads[id(inp)] = add(grads[id(inp)], ig) if id(inp) in grads else ig


def _apply(out_data, inputs, backward):
    if _grad_enabled[0] and any(i.requires_grad for i in inputs):
        return Variable(out_data, True, (backward, list(inputs)))
    return Variable(out_data, False)


class F:
    """Free functions named like crates/modern-chainer-autograd/src/ops.rs and host_ops.rs."""

    @staticmethod
    def add(a, b):
        return _apply(add(a.data, b.data), [a, b], lambda g: [sum_to(g, a.data.shape), sum_to(g, b.data.shape)])

    @staticmethod
    def sub(a, b):
        return _apply(sub(a.data, b.data), [a, b],
                      lambda g: [sum_to(g, a.data.shape), sum_to(scale(g, -1.0), b.data.shape)])

    @staticmethod
    def mul(a, b):
        return _apply(mul(a.data, b.data), [a, b],
                      lambda g: [sum_to(mul(g, b.data), a.data.shape), sum_to(mul(g, a.data), b.data.shape)])

    @staticmethod
    def div(a, b):
        def bwd(g):
            ga = div(g, b.data)
            gb = scale(div(mul(g, a.data), mul(b.data, b.data)), -1.0)
            return [sum_to(ga, a.data.shape), sum_to(gb, b.data.shape)]
        return _apply(div(a.data, b.data), [a, b], bwd)

    @staticmethod
    def scale(x, factor):
        return _apply(scale(x.data, factor), [x], lambda g: [scale(g, factor)])

    @staticmethod
    def sum(x):
        def bwd(g):
            return [np.full(x.data.shape, np.float32(float(g.reshape(-1)[0]) * 1.0), np.float32)]
        return _apply(np.asarray(sum_all(x.data), np.float32).reshape(()), [x], bwd)

    @staticmethod
    def mean(x):
        n = max(x.data.size, 1)

        def bwd(g):
            return [np.full(x.data.shape, np.float32(float(g.reshape(-1)[0]) * (1.0 / n)), np.float32)]
        out = scale(np.asarray(sum_all(x.data), np.float32).reshape(1), 1.0 / n).reshape(())
        return _apply(out, [x], bwd)

    @staticmethod
    def relu(x):
        return _apply(relu(x.data), [x], lambda g: [relu_backward(x.data, g)])

    @staticmethod
    def gelu(x):
        return _apply(gelu(x.data), [x], lambda g: [gelu_backward(x.data, g)])

    @staticmethod
    def exp(x):
        y = unary(0, x.data)
        return _apply(y, [x], lambda g: [mul(g, y)])

    @staticmethod
    def log(x):
        return _apply(unary(1, x.data), [x], lambda g: [div(g, x.data)])

    @staticmethod
    def sigmoid(x):
        y = unary(2, x.data)
        return _apply(y, [x], lambda g: [mul(g, mul(y, sub(np.ones_like(y), y)))])

    @staticmethod
    def sqrt(x):
        y = unary(3, x.data)
        return _apply(y, [x], lambda g: [div(g, scale(y, 2.0))])

    @staticmethod
    def matmul(a, b):
        def bwd(g):
            return [matmul(g, np.ascontiguousarray(b.data.T)), matmul(np.ascontiguousarray(a.data.T), g)]
        return _apply(matmul(a.data, b.data), [a, b], bwd)

    @staticmethod
    def linear(x, w, b=None):
        mode = _AMP[0]
        xs, ws = _lp(x.data, mode), _lp(w.data, mode)

        def bwd(g):
            dx, dw, db = linear_backward(_lp(g, mode), xs, ws, b is not None)
            return [_lp(dx, mode), dw] + ([db] if b is not None else [])
        ins = [x, w] + ([b] if b is not None else [])
        return _apply(_lp(linear(xs, ws, None if b is None else b.data), mode), ins, bwd)

    @staticmethod
    def linear_activation(x, w, b, act):
        fwd = {"relu": relu, "gelu": gelu}[act]
        mode = _AMP[0]
        xs, ws = _lp(x.data, mode), _lp(w.data, mode)

        def bwd(g):
            # the reference recomputes the pre-activation with a second forward product (ops.rs:936-1045)
            pre = _lp(linear(xs, ws, None if b is None else b.data), mode)
            gp = relu_backward(pre, _lp(g, mode)) if act == "relu" else gelu_backward(pre, _lp(g, mode))
            dx, dw, db = linear_backward(_lp(gp, mode), xs, ws, b is not None)
            return [_lp(dx, mode), dw] + ([db] if b is not None else [])
        ins = [x, w] + ([b] if b is not None else [])
        return _apply(_lp(fwd(linear(xs, ws, None if b is None else b.data)), mode), ins, bwd)

    @staticmethod
    def softmax(x):
        return _apply(softmax(x.data), [x], lambda g: [softmax_backward(x.data, g)])

    @staticmethod
    def layer_norm(x, gamma, beta, eps):
        mode = _AMP[0]

        def bwd(g):
            return list(layer_norm_backward(x.data, gamma.data, _lp(g, mode), eps))
        return _apply(_lp(layer_norm(x.data, gamma.data, beta.data, eps), mode), [x, gamma, beta], bwd)

    @staticmethod
    def softmax_cross_entropy(logits, target):
        mode = _AMP[0]

        def bwd(g):
            base = softmax_cross_entropy_backward(logits.data, target.data)
            return [_lp(scale(base, float(g.reshape(-1)[0])), mode), None]
        loss = softmax_cross_entropy(logits.data, target.data)
        return _apply(np.asarray(loss, np.float32).reshape(()), [logits, target], bwd)

    @staticmethod
    def embedding(ids, weight):
        def bwd(g):
            return [None, embedding_backward(ids.data, weight.data.shape, g.reshape(-1, weight.data.shape[1]))]
        return _apply(embedding(ids.data, weight.data), [ids, weight], bwd)

    @staticmethod
    def reshape(x, shape):
        return _apply(x.data.reshape(shape), [x], lambda g: [g.reshape(x.data.shape)])

    @staticmethod
    def transpose(x):
        """Transpose2d (autograd/src/ops.rs:235-255, cpu/src/kernels.rs:306-330): 2-D only; the
        gradient is the transposed upstream gradient.  Pure data movement, so numpy is exact."""
        if x.data.ndim != 2:
            raise ValueError("transpose2d expects a 2-D tensor, got rank %d" % x.data.ndim)
        return _apply(np.ascontiguousarray(x.data.T), [x], lambda g: [np.ascontiguousarray(g.T)])

    @staticmethod
    def permute(x, axes):
        """PermuteOp (autograd/src/host_ops.rs:690-777): output dim d takes source axis axes[d];
        backward applies the inverse permutation.  Errors follow permute_data (703-715)."""
        axes = [int(a) for a in axes]
        if len(axes) != x.data.ndim:
            raise ValueError("permute rank mismatch")
        if sorted(axes) != list(range(len(axes))):
            raise ValueError("invalid permute axes")
        inverse = [0] * len(axes)
        for i, a in enumerate(axes):
            inverse[a] = i
        return _apply(np.ascontiguousarray(np.transpose(x.data, axes)), [x],
                      lambda g: [np.ascontiguousarray(np.transpose(g, inverse))])

    @staticmethod
    def conv2d(x, w, b, stride, pad):
        def bwd(g):
            dx, dw, db = conv2d_backward(x.data, w.data, g, stride, pad, b is not None)
            return [dx, dw] + ([db] if b is not None else [])
        ins = [x, w] + ([b] if b is not None else [])
        return _apply(conv2d(x.data, w.data, None if b is None else b.data, stride, pad), ins, bwd)

    @staticmethod
    def max_pool2d(x, kernel, stride, pad):
        return _apply(max_pool2d(x.data, kernel, stride, pad), [x],
                      lambda g: [max_pool2d_backward(x.data, g, kernel, stride, pad)])

    @staticmethod
    def multi_head_attention(q, k, v, heads, causal):
        mode = _AMP[0]
        qs, ks, vs = _lp(q.data, mode), _lp(k.data, mode), _lp(v.data, mode)

        def bwd(g):
            return [_lp(t, mode) for t in attention_backward(qs, ks, vs, _lp(g, mode), heads, causal)]
        return _apply(_lp(attention(qs, ks, vs, heads, causal), mode), [q, k, v], bwd)


# ---------------------------------------------------------------- optimizers / AMP
def zero_grad(params):
    for p in params:
        p.cleargrad()


class SGD:
    def __init__(self, lr):
        self.lr = lr

    def update(self, params):
        for p in params:
            if p.grad is None:
                continue
            p.data = sub(p.data, scale(p.grad, self.lr))


class Adam:
    """optim/src/lib.rs:53-120: per-parameter state and step counter."""

    def __init__(self, lr, beta1=0.9, beta2=0.999, eps=1e-8):
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.state = {}

    def update(self, params):
        for p in params:
            if p.grad is None:
                continue
            st = self.state.setdefault(id(p), {"m": np.zeros_like(p.data), "v": np.zeros_like(p.data), "t": 0})
            st["t"] += 1
            p.data, st["m"], st["v"] = adam_update(p.data, p.grad, st["m"], st["v"], self.lr, self.beta1, self.beta2,
                                                   self.eps, st["t"])


_MCN_TAGS = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.float16): 2, np.dtype(np.int32): 4,
             np.dtype(np.int64): 5, np.dtype(np.uint8): 6, np.dtype(np.bool_): 7}


def mcn_save(path, entries):
    """serial/src/lib.rs:14-33: "MCHN0001", u32 count, then per (name, array): u32 name length, name,
    u8 dtype tag, u32 rank, u64 dims, u64 byte length, bytes; all little-endian."""
    import struct
    with open(path, "wb") as f:
        f.write(b"MCHN0001")
        f.write(struct.pack("<I", len(entries)))
        for name, arr in entries:
            arr = np.ascontiguousarray(arr)
            nb = name.encode("utf-8")
            f.write(struct.pack("<I", len(nb)) + nb)
            f.write(bytes([_MCN_TAGS[arr.dtype]]))
            f.write(struct.pack("<I", arr.ndim))
            for d in arr.shape:
                f.write(struct.pack("<Q", d))
            raw = arr.astype(arr.dtype.newbyteorder("<"), copy=False).tobytes()
            f.write(struct.pack("<Q", len(raw)))
            f.write(raw)


def mcn_load(path):
    """serial/src/lib.rs:35-62; returns [(name, array)] in file order."""
    import struct
    inv = {v: k for k, v in _MCN_TAGS.items()}
    out = []
    with open(path, "rb") as f:
        if f.read(8) != b"MCHN0001":
            raise ValueError("not a Modern Chainer .mcn file")
        (count,) = struct.unpack("<I", f.read(4))
        for _ in range(count):
            (nl,) = struct.unpack("<I", f.read(4))
            name = f.read(nl).decode("utf-8")
            tag = f.read(1)[0]
            if tag == 3:
                dt = np.dtype(np.uint16)  # bf16 bit patterns
            elif tag in inv:
                dt = inv[tag]
            else:
                raise ValueError("unknown dtype tag %d" % tag)
            (rank,) = struct.unpack("<I", f.read(4))
            dims = [struct.unpack("<Q", f.read(8))[0] for _ in range(rank)]
            (nbytes,) = struct.unpack("<Q", f.read(8))
            out.append((name, np.frombuffer(f.read(nbytes), dt.newbyteorder("<")).astype(dt).reshape(dims)))
    return out


class MomentumSGD:
    """optim/src/lib.rs:122-160: velocity = previous*momentum + grad (the gradient itself on the first
    update of a parameter), p += velocity * (-lr); every product narrows its factor to f32 first."""

    def __init__(self, lr, momentum):
        self.lr, self.momentum = lr, momentum
        self.velocity = {}

    def update(self, params):
        for p in params:
            if p.grad is None:
                continue
            prev = self.velocity.get(id(p))
            vel = p.grad.copy() if prev is None else add(scale(prev, self.momentum), p.grad)
            self.velocity[id(p)] = vel
            p.data = add(p.data, scale(vel, -self.lr))


class AdamW:
    """optim/src/lib.rs:162-214: the Adam step, then next - scale(p_old, weight_decay*lr)."""

    def __init__(self, lr, weight_decay, beta1=0.9, beta2=0.999, eps=1e-8):
        self.lr, self.weight_decay, self.beta1, self.beta2, self.eps = lr, weight_decay, beta1, beta2, eps
        self.state = {}

    def update(self, params):
        for p in params:
            if p.grad is None:
                continue
            st = self.state.setdefault(id(p), {"m": np.zeros_like(p.data), "v": np.zeros_like(p.data), "t": 0})
            st["t"] += 1
            nxt, st["m"], st["v"] = adam_update(p.data, p.grad, st["m"], st["v"], self.lr, self.beta1, self.beta2, self.eps, st["t"])
            p.data = sub(nxt, scale(p.data, self.weight_decay * self.lr))


def clip_grad_norm(params, max_norm):
    """optim/src/lib.rs:216-243: per parameter sum_all(g*g) (an f32 scalar), added up in f64; sqrt in f64;
    if norm > max_norm the gradients are scaled by max_norm/norm (narrowed to f32).  Returns the pre-clip norm."""
    if max_norm <= 0.0:
        raise ValueError("max_norm must be positive")
    total = 0.0
    for p in params:
        if p.grad is not None:
            total += float(sum_all(mul(p.grad, p.grad)))
    norm = float(np.sqrt(np.float64(total)))
    if norm > max_norm and norm > 0.0:
        f = max_norm / norm
        for p in params:
            if p.grad is not None:
                p.grad = scale(p.grad, f)
    return norm


def _powi_f64(a, b):
    """f64::powi (binary exponentiation, as compiler-rt's __powidf2)."""
    recip, r = b < 0, 1.0
    b = abs(int(b))
    while True:
        if b & 1:
            r *= a
        b //= 2
        if b == 0:
            break
        a *= a
    return 1.0 / r if recip else r


class LinearWarmupCosineLR:
    """optim/src/lib.rs:247-270."""

    def __init__(self, warmup_steps, total_steps, base_lr, min_lr):
        self.warmup_steps, self.total_steps, self.base_lr, self.min_lr = warmup_steps, total_steps, base_lr, min_lr

    def get_lr(self, step):
        import math
        if step < self.warmup_steps:
            if self.warmup_steps == 0:
                return self.base_lr
            return self.base_lr * float(step) / float(self.warmup_steps)
        if step >= self.total_steps:
            return self.min_lr
        denom = float(max(self.total_steps - self.warmup_steps, 1))
        progress = float(step - self.warmup_steps) / denom
        c = math.cos(math.pi * progress) * 0.5 + 0.5
        return self.min_lr + (self.base_lr - self.min_lr) * c


class StepLR:
    """optim/src/lib.rs:272-284."""

    def __init__(self, base_lr, step_size, gamma):
        self.base_lr, self.step_size, self.gamma = base_lr, step_size, gamma

    def get_lr(self, step):
        return self.base_lr * _powi_f64(self.gamma, step // max(self.step_size, 1))


class ConstantLR:
    def __init__(self, lr):
        self.lr = lr

    def get_lr(self, step):
        return self.lr


class PolynomialLR:
    """optim/src/lib.rs:297-311."""

    def __init__(self, base_lr, total_steps, power, min_lr):
        self.base_lr, self.total_steps, self.power, self.min_lr = base_lr, total_steps, power, min_lr

    def get_lr(self, step):
        if step == 0:
            return self.base_lr
        progress = min(max(float(step) / float(max(self.total_steps, 1)), 0.0), 1.0)
        return self.min_lr + (self.base_lr - self.min_lr) * (1.0 - progress) ** self.power


class GradScaler:
    """optim/src/amp.rs:8-113."""

    def __init__(self, scale=65536.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000):
        self.scale = max(float(scale), 1.0)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval = growth_interval
        self.growth_tracker = 0

    def scale_loss(self, loss):
        return F.scale(loss, self.scale)

    def unscale_(self, params):
        if abs(self.scale - 1.0) < np.finfo(np.float64).eps:
            return
        inv = 1.0 / self.scale
        for p in params:
            if p.grad is not None:
                p.grad = scale(p.grad, inv)

    def has_non_finite_grad(self, params):
        return any(p.grad is not None and count_non_finite(p.grad) > 0 for p in params)

    def step(self, optimizer, params):
        if self.has_non_finite_grad(params):
            self.scale = max(self.scale * self.backoff_factor, 1.0)
            self.growth_tracker = 0
            zero_grad(params)
            return False
        self.unscale_(params)
        optimizer.update(params)
        self.growth_tracker += 1
        if self.growth_tracker >= self.growth_interval:
            self.scale *= self.growth_factor
            self.growth_tracker = 0
        return True


# ---------------------------------------------------------------- nn modules
class Linear:
    def __init__(self, in_features, out_features, seed):
        self.W = Variable(he_normal((out_features, in_features), in_features, seed))
        self.b = Variable(np.zeros(out_features, np.float32))

    def __call__(self, x):
        return F.linear(x, self.W, self.b)

    def parameters(self):
        return [self.W, self.b]


class LayerNorm:
    def __init__(self, dim, eps=1e-5):
        self.gamma = Variable(np.ones(dim, np.float32))
        self.beta = Variable(np.zeros(dim, np.float32))
        self.eps = eps

    def __call__(self, x):
        return F.layer_norm(x, self.gamma, self.beta, self.eps)

    def parameters(self):
        return [self.gamma, self.beta]


class MultiHeadAttention:
    """nn/src/lib.rs:430-481: four Linear layers seeded 1..4 around the attention host op."""

    def __init__(self, dim, heads, causal):
        self.wq, self.wk, self.wv, self.wo = (Linear(dim, dim, s) for s in (1, 2, 3, 4))
        self.heads, self.causal = heads, causal

    def __call__(self, x):
        b, s, d = x.data.shape
        flat = F.reshape(x, (b * s, d))
        q = F.reshape(self.wq(flat), (b, s, d))
        k = F.reshape(self.wk(flat), (b, s, d))
        v = F.reshape(self.wv(flat), (b, s, d))
        ctx = F.reshape(F.multi_head_attention(q, k, v, self.heads, self.causal), (b * s, d))
        return F.reshape(self.wo(ctx), (b, s, d))

    def parameters(self):
        return self.wq.parameters() + self.wk.parameters() + self.wv.parameters() + self.wo.parameters()


class Conv2d:
    """nn/src/lib.rs:246-271: He-normal weight with fan_in = C*KH*KW, zero bias."""

    def __init__(self, cin, cout, kernel, stride, pad, seed):
        self.W = Variable(he_normal((cout, cin, kernel, kernel), cin * kernel * kernel, seed))
        self.b = Variable(np.zeros(cout, np.float32))
        self.stride, self.pad = stride, pad

    def __call__(self, x):
        return F.conv2d(x, self.W, self.b, self.stride, self.pad)

    def parameters(self):
        return [self.W, self.b]


# ---------------------------------------------------------------- the benchmark models
class MLP:
    """Linear(784,100)-ReLU-Linear(100,10); seeds 0 and 1."""

    def __init__(self, sizes=(784, 100, 10)):
        self.l1, self.l2 = Linear(sizes[0], sizes[1], 0), Linear(sizes[1], sizes[2], 1)

    def parameters(self):
        return self.l1.parameters() + self.l2.parameters()

    def loss(self, x, labels):
        return F.softmax_cross_entropy(self.l2(F.relu(self.l1(x))), labels)


class EncoderBlock:
    """Pre-LN block: x + MHA(LN(x)); then x + W2 gelu(W1 LN(x)). FFN seeds 5 and 6."""

    def __init__(self, d, heads, ff, causal=False):
        self.ln1, self.ln2 = LayerNorm(d), LayerNorm(d)
        self.attn = MultiHeadAttention(d, heads, causal)
        self.w1, self.w2 = Linear(d, ff, 5), Linear(ff, d, 6)

    def parameters(self):
        return (self.ln1.parameters() + self.attn.parameters() + self.ln2.parameters() + self.w1.parameters() +
                self.w2.parameters())

    def __call__(self, x):
        b, s, d = x.data.shape
        x = F.add(x, self.attn(self.ln1(x)))
        flat = F.reshape(self.ln2(x), (b * s, d))
        h = F.linear_activation(flat, self.w1.W, self.w1.b, "gelu")
        return F.add(x, F.reshape(self.w2(h), (b, s, d)))

    def loss(self, x, target):
        diff = F.sub(self(x), target)
        return F.mean(F.mul(diff, diff))


class CNN:
    """conv3x3(3,32)-ReLU-pool2-conv3x3(32,64)-ReLU-pool2-Linear(4096,10); seeds 0,1,2."""

    def __init__(self, cin=3, c1=32, c2=64, hw=32, classes=10):
        self.c1, self.c2 = Conv2d(cin, c1, 3, 1, 1, 0), Conv2d(c1, c2, 3, 1, 1, 1)
        self.fc = Linear(c2 * (hw // 4) * (hw // 4), classes, 2)

    def parameters(self):
        return self.c1.parameters() + self.c2.parameters() + self.fc.parameters()

    def loss(self, x, labels):
        h = F.max_pool2d(F.relu(self.c1(x)), 2, 2, 0)
        h = F.max_pool2d(F.relu(self.c2(h)), 2, 2, 0)
        h = F.reshape(h, (h.data.shape[0], -1))
        return F.softmax_cross_entropy(self.fc(h), labels)


class Decoder:
    """Training-side mirror of llm/src/decoder.rs: token embedding (std 0.02), per layer
    LN-QKVO-LN-FFN with one RNG stream in the order of Decoder::new, final LN, untied
    lm_head (std 0.02, no bias), causal attention, no positional table."""

    def __init__(self, vocab, d, heads, ff, layers, seed=0):
        rng = Rng(seed)
        mat = lambda r, c, std: Variable(rng.normal_vec(r * c, 0.0, std).reshape(r, c))
        vec = lambda n, v: Variable(np.full(n, v, np.float32))
        self.heads = heads
        self.tok_emb = mat(vocab, d, 0.02)
        self.layers = []
        for _ in range(layers):
            std = math.sqrt(2.0 / d)
            L = {}
            L["ln1_g"], L["ln1_b"] = vec(d, 1.0), vec(d, 0.0)
            for nm in ("q", "k", "v", "o"):
                L["w" + nm], L["b" + nm] = mat(d, d, std), vec(d, 0.0)
            L["ln2_g"], L["ln2_b"] = vec(d, 1.0), vec(d, 0.0)
            L["w1"], L["b1"] = mat(ff, d, math.sqrt(2.0 / d)), vec(ff, 0.0)
            L["w2"], L["b2"] = mat(d, ff, math.sqrt(2.0 / ff)), vec(d, 0.0)
            self.layers.append(L)
        self.ln_f_g, self.ln_f_b = vec(d, 1.0), vec(d, 0.0)
        self.lm_head = mat(vocab, d, 0.02)

    ORDER = ("ln1_g", "ln1_b", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "ln2_g", "ln2_b", "w1", "b1", "w2", "b2")

    def parameters(self):
        out = [self.tok_emb]
        for L in self.layers:
            out += [L[k] for k in self.ORDER]
        return out + [self.ln_f_g, self.ln_f_b, self.lm_head]

    def loss(self, ids, targets, eps=1e-5):
        b, s = ids.data.shape
        x = F.embedding(Variable.constant(ids.data.reshape(-1)), self.tok_emb)
        d = x.data.shape[-1]
        for L in self.layers:
            n = F.layer_norm(x, L["ln1_g"], L["ln1_b"], eps)
            q = F.reshape(F.linear(n, L["wq"], L["bq"]), (b, s, d))
            k = F.reshape(F.linear(n, L["wk"], L["bk"]), (b, s, d))
            v = F.reshape(F.linear(n, L["wv"], L["bv"]), (b, s, d))
            a = F.reshape(F.multi_head_attention(q, k, v, self.heads, True), (b * s, d))
            x = F.add(x, F.linear(a, L["wo"], L["bo"]))
            n = F.layer_norm(x, L["ln2_g"], L["ln2_b"], eps)
            h = F.linear_activation(n, L["w1"], L["b1"], "gelu")
            x = F.add(x, F.linear(h, L["w2"], L["b2"]))
        x = F.layer_norm(x, self.ln_f_g, self.ln_f_b, eps)
        logits = F.linear(x, self.lm_head, None)
        return F.softmax_cross_entropy(logits, Variable.constant(targets.data.reshape(-1)))
