"""Functional operations (`F.*`) with the names and argument order of the reference's Python module
(python/chainer/functions.py, python/chainer/_chainer.pyi:95-141).  Each forwards to the tape entry
point of the library (`mcb_f_*`); functions outside the training-step path raise NotImplementedError."""
from . import Variable, _api, _wrap

_F = _api.F


def _u(x):
    return x._v if isinstance(x, Variable) else x


def add(a, b):
    return _wrap(_F.add(a._v, b._v), a)


def sub(a, b):
    return _wrap(_F.sub(a._v, b._v), a)


def mul(a, b):
    return _wrap(_F.mul(a._v, b._v), a)


def div(a, b):
    return _wrap(_F.div(a._v, b._v), a)


def scale(x, factor):
    return _wrap(_F.scale(x._v, factor), x)


def exp(x):
    return _wrap(_F.exp(x._v), x)


def log(x):
    return _wrap(_F.log(x._v), x)


def sigmoid(x):
    return _wrap(_F.sigmoid(x._v), x)


def sqrt(x):
    return _wrap(_F.sqrt(x._v), x)


def neg(x):
    return _wrap(_F.neg(x._v), x)


def silu(x):
    return _wrap(_F._un(4, x._v), x)


def abs(x):
    return _wrap(_F._un(5, x._v), x)


def relu(x):
    return _wrap(_F.relu(x._v), x)


def gelu(x):
    return _wrap(_F.gelu(x._v), x)


def sum(x):
    return _wrap(_F.sum(x._v), x)


def mean(x):
    return _wrap(_F.mean(x._v), x)


def softmax(x):
    return _wrap(_F.softmax(x._v), x)


def matmul(a, b):
    return _wrap(_F.matmul(a._v, b._v), a)


def transpose(x):
    return _wrap(_F.transpose(x._v), x)


def permute(x, axes):
    return _wrap(_F.permute(x._v, list(axes)), x)


def reshape(x, shape):
    return _wrap(_F.reshape(x._v, list(shape)), x)


def linear(x, weight, bias=None):
    return _wrap(_F.linear(x._v, weight._v, bias._v if bias is not None else None), x)


def layer_norm(x, gamma, beta, eps=1e-5):
    return _wrap(_F.layer_norm(x._v, gamma._v, beta._v, eps), x)


def softmax_cross_entropy(logits, target):
    return _wrap(_F.softmax_cross_entropy(logits._v, target._v), logits)


def embedding(ids, weight):
    return _wrap(_F.embedding(ids._v, weight._v), weight)


def conv2d(x, weight, bias, stride=1, padding=0):
    return _wrap(_F.conv2d(x._v, weight._v, bias._v if bias is not None else None, stride, padding), x)


def max_pool2d(x, kernel, stride=1, padding=0):
    return _wrap(_F.max_pool2d(x._v, kernel, stride, padding), x)


def multi_head_attention(q, k, v, heads, causal=False):
    return _wrap(_F.multi_head_attention(q._v, k._v, v._v, heads, causal), q)


def _outside(name):
    def f(*a, **k):
        raise NotImplementedError(f"F.{name} lies outside the training-step path this backend implements")
    f.__name__ = name
    return f


def batch_norm(x, gamma, beta, eps=1e-5):
    """Batch statistics per channel over (N, spatial...), as host_ops.rs:488-532 (a host op in the reference).  Composed
    from ops of the path: with channels moved to the rows of a [C, N * spatial] matrix it is a LayerNorm of each row
    with unit scale, then a per-row scale and shift; the tape differentiates the composition."""
    import numpy as np
    from . import Tensor
    dims = list(x.shape)
    if len(dims) < 2:
        raise ValueError("batch_norm expects rank >= 2")
    n, c = dims[0], dims[1]
    if list(gamma.shape) != [c] or list(beta.shape) != [c]:
        raise ValueError("batch_norm gamma/beta size mismatch")
    m = int(np.prod([n] + dims[2:]))
    axes = [1, 0] + list(range(2, len(dims)))
    rows = reshape(permute(x, axes), [c, m])
    one = Variable.constant(Tensor(np.ones(m, np.float32), x.device))
    zero = Variable.constant(Tensor(np.zeros(m, np.float32), x.device))
    y = add(mul(layer_norm(rows, one, zero, eps), reshape(gamma, [c, 1])), reshape(beta, [c, 1]))
    return permute(reshape(y, [c, n] + dims[2:]), axes)


average_pool2d = _outside("average_pool2d")
clamp = _outside("clamp")
conv_transpose2d = _outside("conv_transpose2d")
dropout = _outside("dropout")
rms_norm = _outside("rms_norm")

__all__ = ["abs", "add", "average_pool2d", "batch_norm", "clamp", "conv2d", "conv_transpose2d", "div", "dropout", "embedding", "exp",
           "gelu", "layer_norm", "linear", "log", "matmul", "max_pool2d", "mean", "multi_head_attention", "mul", "neg", "permute",
           "relu", "reshape", "rms_norm", "scale", "sigmoid", "silu", "softmax", "softmax_cross_entropy", "sqrt", "sub", "sum",
           "transpose"]
