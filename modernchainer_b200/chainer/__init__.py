"""`chainer` facade over libmcb.so: the Python surface of the reference (python/chainer/__init__.py,
python/chainer/_chainer.pyi, crates/modern-chainer-python/src/lib.rs) with the same class, function and
argument names, so that code written against the reference's package runs on this backend:

    PYTHONPATH=<repo>/modernchainer_b200 python -c "import chainer, chainer.functions as F"
    # or: import modernchainer_b200.chainer as chainer

There is one compute backend here, the sm_100a library.  Device strings ("cpu", "cuda", "cuda:0") are
accepted and remembered for source compatibility, but every operation executes on the GPU of the
process-wide context; nothing is computed on the host.  Parts of the reference's surface that lie
outside the training-step path (ConvTranspose2d, RMSNorm, dropout, clamp, average pooling,
Vulkan) raise NotImplementedError.
"""
from contextlib import contextmanager

import numpy as np

try:
    from .. import api as _api
except ImportError:  # imported as the top-level package `chainer` (PYTHONPATH=<repo>/modernchainer_b200)
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from modernchainer_b200 import api as _api

__version__ = "0.1.0+mcb200"

_ctx = None


def _context():
    """The process-wide device context (created on first use; fails loudly without a GPU)."""
    global _ctx
    if _ctx is None:
        _ctx = _api.Context(0)
    return _ctx


def cuda_available():
    try:
        return _api.device_count() > 0
    except Exception:
        return False


def vulkan_available():
    return False


def vulkan_devices():
    return []


def synchronize(device="cpu"):
    if _ctx is not None:
        _ctx.sync()


def version():
    return __version__


_DTYPE_NAMES = {np.dtype(np.float32): "f32", np.dtype(np.int64): "i64", np.dtype(np.int32): "i32", np.dtype(np.uint8): "u8"}
_DTYPES = {"f32": np.float32, "float32": np.float32, "i64": np.int64, "int64": np.int64, "i32": np.int32, "int32": np.int32,
           "u8": np.uint8, "uint8": np.uint8}


class Tensor:
    """Host-visible value with a shape, a dtype name and a device label (_chainer.pyi:5-25)."""

    def __init__(self, array, device="cpu"):
        self._a = np.ascontiguousarray(array)
        if self._a.dtype == np.float64:
            self._a = self._a.astype(np.float32)
        self._device = device

    @staticmethod
    def zeros(shape, device="cpu"):
        return Tensor(np.zeros(tuple(shape), np.float32), device)

    @staticmethod
    def from_list(data, shape, device="cpu"):
        return Tensor(np.asarray(data, np.float32).reshape(tuple(shape)), device)

    @staticmethod
    def from_numpy(array, device="cpu"):
        return Tensor(np.array(array), device)

    @property
    def shape(self):
        return list(self._a.shape)

    @property
    def dtype(self):
        return _DTYPE_NAMES[self._a.dtype]

    @property
    def device(self):
        return self._device

    @property
    def ndim(self):
        return self._a.ndim

    def numel(self):
        return int(self._a.size)

    def to(self, device):
        return Tensor(self._a, device)

    def astype(self, dtype):
        return Tensor(self._a.astype(_DTYPES[dtype]), self._device)

    def contiguous(self):
        return self

    def tolist(self):
        return self._a.reshape(-1).tolist()

    def numpy(self):
        return self._a.copy()

    def __repr__(self):
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, device={self._device})"


class Variable:
    """Node of the define-by-run graph (_chainer.pyi:27-54) over an `mcb_var` handle."""

    def __init__(self, tensor, _v=None, _requires_grad=True, _device=None):
        if _v is not None:
            self._v = _v
            self._device = _device or "cpu"
            return
        if not isinstance(tensor, Tensor):
            tensor = Tensor(tensor)
        self._device = tensor.device
        self._v = _api.Variable(_context(), tensor._a, requires_grad=_requires_grad)

    @staticmethod
    def constant(tensor):
        return Variable(tensor, _requires_grad=False)

    @property
    def data(self):
        return Tensor(self._v.data, self._device)

    @property
    def array(self):
        return self._v.data

    @property
    def grad(self):
        g = self._v.grad
        return None if g is None else Tensor(g, self._device)

    @property
    def shape(self):
        return list(self._v.shape)

    @property
    def device(self):
        return self._device

    @property
    def grad_fn(self):
        return None if self._v.is_leaf() else "Op"

    @property
    def requires_grad(self):
        return bool(self._v.requires_grad)

    def backward(self):
        self._v.backward()

    def to(self, device):
        self._device = device
        return self

    def cleargrad(self):
        self._v.cleargrad()

    def unchain_backward(self):
        self._v.unchain_backward()

    def __repr__(self):
        return f"Variable(shape={self.shape}, device={self._device}, requires_grad={self.requires_grad})"


def _wrap(v, like=None):
    return Variable(None, _v=v, _device=like._device if like is not None else "cpu")


def _he_normal(shape, fan_in, seed):
    import ctypes as C
    out = np.empty(int(np.prod(shape)), np.float32)
    st = _api._lib.load().mcb_he_normal(out.ctypes.data_as(C.c_void_p), out.size, int(fan_in), int(seed))
    if st:
        raise _api.McbError(st, "he_normal")
    return out.reshape(shape)


class _Link:
    def parameters(self):
        return list(self._params)

    def cleargrads(self):
        for p in self._params:
            p.cleargrad()

    def __call__(self, x):
        return self.forward(x)


class Linear(_Link):
    """nn::Linear (nn/src/lib.rs:38-73): W he_normal([out, in], in, seed), zero bias."""

    def __init__(self, in_features, out_features, seed=0, device="cpu"):
        self.W = Variable(Tensor(_he_normal((out_features, in_features), in_features, seed), device))
        self.b = Variable(Tensor(np.zeros(out_features, np.float32), device))
        self._params = [self.W, self.b]

    def forward(self, x):
        from . import functions as F
        return F.linear(x, self.W, self.b)


class Conv2d(_Link):
    """nn::Conv2d (nn/src/lib.rs:246-271): W he_normal([O, C, K, K], C*K*K, seed), zero bias."""

    def __init__(self, in_channels, out_channels, kernel, stride=1, padding=0, seed=0, device="cpu"):
        fan_in = in_channels * kernel * kernel
        self.W = Variable(Tensor(_he_normal((out_channels, in_channels, kernel, kernel), fan_in, seed), device))
        self.b = Variable(Tensor(np.zeros(out_channels, np.float32), device))
        self.stride, self.padding = stride, padding
        self._params = [self.W, self.b]

    def forward(self, x):
        from . import functions as F
        return F.conv2d(x, self.W, self.b, self.stride, self.padding)


class LayerNorm(_Link):
    """nn::LayerNorm (nn/src/lib.rs:141-147): gamma ones, beta zeros."""

    def __init__(self, dim, eps=1e-5, device="cpu"):
        self.gamma = Variable(Tensor(np.ones(dim, np.float32), device))
        self.beta = Variable(Tensor(np.zeros(dim, np.float32), device))
        self.eps = eps
        self._params = [self.gamma, self.beta]

    def forward(self, x):
        from . import functions as F
        return F.layer_norm(x, self.gamma, self.beta, self.eps)


class Embedding(_Link):
    """nn::Embedding (nn/src/lib.rs:185-191): he_normal([vocab, dim], dim, seed)."""

    def __init__(self, vocab, dim, seed=0, device="cpu"):
        self.W = Variable(Tensor(_he_normal((vocab, dim), dim, seed), device))
        self._params = [self.W]

    def forward(self, ids):
        from . import functions as F
        return F.embedding(ids, self.W)


class MultiHeadAttention(_Link):
    """nn::MultiHeadAttention (nn/src/lib.rs:430-481): four Linear(dim, dim) with seeds 1..4 around the fused op."""

    def __init__(self, dim, heads, causal=False, device="cpu"):
        self.wq, self.wk, self.wv, self.wo = (Linear(dim, dim, s, device) for s in (1, 2, 3, 4))
        self.heads, self.causal = heads, causal
        self._params = self.wq.parameters() + self.wk.parameters() + self.wv.parameters() + self.wo.parameters()

    def forward(self, x):
        from . import functions as F
        if len(x.shape) != 3:
            raise _api.McbError(5, "MultiHeadAttention expects [N, S, D]")
        n, s, d = x.shape
        flat = F.reshape(x, [n * s, d])
        q, k, v = (F.reshape(w(flat), [n, s, d]) for w in (self.wq, self.wk, self.wv))
        ctxt = F.reshape(F.multi_head_attention(q, k, v, self.heads, self.causal), [n * s, d])
        return F.reshape(self.wo(ctxt), [n, s, d])


def _outside(name):
    class _Missing:
        def __init__(self, *a, **k):
            raise NotImplementedError(f"{name} lies outside the training-step path this backend implements")
    _Missing.__name__ = name
    return _Missing


class BatchNorm(_Link):
    """nn::BatchNorm (nn/src/lib.rs:395-423): gamma ones, beta zeros, batch statistics."""

    def __init__(self, channels, eps=1e-5, device="cpu"):
        self.gamma = Variable(Tensor(np.ones(channels, np.float32), device))
        self.beta = Variable(Tensor(np.zeros(channels, np.float32), device))
        self.eps = eps
        self._params = [self.gamma, self.beta]

    def forward(self, x):
        from . import functions as F
        return F.batch_norm(x, self.gamma, self.beta, self.eps)


ConvTranspose2d = _outside("ConvTranspose2d")
RMSNorm = _outside("RMSNorm")


class _Optimizer:
    """setup / update / zero_grad of the reference's Python optimizers (_chainer.pyi:66-93)."""

    def _make(self, ctx):
        raise NotImplementedError

    def setup(self, params):
        self._params = list(params)
        self._opt = self._make(_context())

    def update(self):
        self._opt.update([p._v for p in self._params])

    def zero_grad(self):
        for p in self._params:
            p.cleargrad()


class SGD(_Optimizer):
    def __init__(self, lr):
        self.lr = lr

    def _make(self, ctx):
        return _api.SGD(ctx, self.lr)


class MomentumSGD(_Optimizer):
    def __init__(self, lr=0.01, momentum=0.9):
        self.lr, self.momentum = lr, momentum

    def _make(self, ctx):
        return _api.MomentumSGD(ctx, self.lr, self.momentum)


class Adam(_Optimizer):
    def __init__(self, lr=0.001):
        self.lr = lr

    def _make(self, ctx):
        return _api.Adam(ctx, self.lr)


class AdamW(_Optimizer):
    def __init__(self, lr=0.001, weight_decay=0.01):
        self.lr, self.weight_decay = lr, weight_decay

    def _make(self, ctx):
        return _api.AdamW(ctx, self.lr, self.weight_decay)


class LinearWarmupCosineLR(_api.LinearWarmupCosineLR):
    def __init__(self, warmup_steps=100, total_steps=1000, base_lr=0.001, min_lr=0.0):
        super().__init__(warmup_steps, total_steps, base_lr, min_lr)


_LINKS = (Linear, Conv2d, LayerNorm, Embedding, MultiHeadAttention)


class Chain:
    """Minimal Chainer-style container for links (python/chainer/__init__.py:44-88)."""

    def __init__(self):
        object.__setattr__(self, "_children", {})

    @contextmanager
    def init_scope(self):
        yield

    def __setattr__(self, name, value):
        object.__setattr__(self, name, value)
        if isinstance(value, _LINKS + (Chain,)):
            self._children[name] = value

    def add_link(self, name, link):
        setattr(self, name, link)
        return link

    def children(self):
        return dict(self._children)

    def parameters(self):
        params = []
        for link in self._children.values():
            params.extend(link.parameters())
        return params

    def cleargrads(self):
        for parameter in self.parameters():
            parameter.cleargrad()

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def forward(self, *args, **kwargs):
        raise NotImplementedError


from . import functions, links, optimizers  # noqa: E402

__all__ = ["Adam", "BatchNorm", "Chain", "Conv2d", "ConvTranspose2d", "Embedding", "LayerNorm", "Linear", "MultiHeadAttention",
           "SGD", "Tensor", "Variable", "__version__", "cuda_available", "synchronize", "vulkan_available", "vulkan_devices",
           "functions", "links", "optimizers"]
