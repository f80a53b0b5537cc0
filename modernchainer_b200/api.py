"""Python classes over the C ABI (include/mcb.h).  Host data are numpy arrays; bf16 host
data are uint16 bit patterns.  Nothing here computes: every method forwards to libmcb.so."""
import ctypes as C
import os

import numpy as np

from . import _lib

F32, I64, I32, U8, F16, BF16 = 0, 1, 2, 3, 4, 5
_NP_OF = {F32: np.float32, I64: np.int64, I32: np.int32, U8: np.uint8, F16: np.float16, BF16: np.uint16}
_DT_OF = {np.dtype(np.float32): F32, np.dtype(np.int64): I64, np.dtype(np.int32): I32, np.dtype(np.uint8): U8,
          np.dtype(np.float16): F16}
STATUS_NAMES = {0: "Ok", 1: "ShapeMismatch", 2: "Broadcast", 3: "DTypeMismatch", 4: "UnsupportedDType",
                5: "InvalidArgument", 6: "OutOfBounds", 7: "Unsupported", 8: "Backend", 9: "Io"}


GUARD_BYTE = 0xA5  # canary pattern of Context.guard


class McbError(RuntimeError):
    """Mirrors core::Error of the reference; `.status` is the C status code."""

    def __init__(self, status, message=""):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


def device_count():
    return _lib.load().mcb_device_count()


def f32_to_bf16_bits(x):
    """Round-to-nearest-even narrowing on the host (same rule the device kernels use)."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def _dims(shape):
    return (C.c_int64 * max(len(shape), 1))(*shape)


class Context:
    """One device, one stream, one caching allocator (CudaBackend::new in the reference)."""

    def __init__(self, ordinal=0):
        self.lib = _lib.load()
        h = C.c_void_p()
        st = self.lib.mcb_ctx_create(ordinal, C.byref(h))
        if st:
            raise McbError(st, f"no usable CUDA device {ordinal}; this backend has no CPU fallback")
        self.h = h

    def check(self, st):
        if st:
            raise McbError(st, (self.lib.mcb_last_error(self.h) or b"").decode())

    def close(self):
        if self.h:
            self.lib.mcb_ctx_destroy(self.h)
            self.h = None

    def sync(self):
        self.check(self.lib.mcb_sync(self.h))

    def launch_count(self):
        return self.lib.mcb_launch_count(self.h)

    def set_knob(self, name, value=1):
        """Sets (value >= 0) or clears (value < 0 or None) one test / tuning knob of this context, by the name of its
        environment variable.  The library reads the environment only while a context is created."""
        self.check(self.lib.mcb_set_knob(self.h, name.encode(), -1 if value is None else int(value)))

    def knob(self, name, value=1):
        """`with ctx.knob("MCB_UNFUSED_BWD"):` -- the knob is set inside the block and cleared after it."""
        ctx = self

        class _Scope:
            def __enter__(self):
                ctx.set_knob(name, value)

            def __exit__(self, *exc):
                ctx.set_knob(name, None)
                return False
        return _Scope()

    def set_compute_type(self, compute):
        self.check(self.lib.mcb_set_compute_type(self.h, compute))

    # ---- timing
    def event(self):
        e = C.c_void_p()
        self.check(self.lib.mcb_event_create(self.h, C.byref(e)))
        return e

    def record(self, e):
        self.check(self.lib.mcb_event_record(self.h, e))

    def elapsed_ms(self, a, b):
        ms = C.c_float()
        self.check(self.lib.mcb_event_elapsed_ms(self.h, a, b, C.byref(ms)))
        return ms.value

    # ---- canary bands around every array made from here on (a debugging aid: out-of-bounds writes of a kernel show
    # up as a changed band; the library itself is not involved)
    def guard(self, nbytes=256, shift=0):
        self.guard_bytes, self.guard_shift, self.guard_checked, self.guard_broken = int(nbytes), int(shift), 0, []

    def check_guards(self):
        """Number of guarded arrays checked so far (each when it was released); raises if a band of any was written."""
        if self.guard_broken:
            raise AssertionError(f"a kernel wrote outside arrays (shape, dtype): {self.guard_broken}")
        return self.guard_checked

    # ---- memory
    def empty(self, shape, dtype=F32):
        return DeviceArray(self, tuple(int(s) for s in shape), dtype)

    def array(self, host, dtype=None):
        host = np.ascontiguousarray(host)
        if dtype is None:
            if host.dtype == np.float64:
                host = host.astype(np.float32)
            dtype = _DT_OF[host.dtype]
        elif dtype == BF16 and host.dtype != np.uint16:
            host = f32_to_bf16_bits(host)
        d = DeviceArray(self, host.shape, dtype)
        d.upload(host)
        return d

    def zeros(self, shape, dtype=F32):
        d = self.empty(shape, dtype)
        self.check(self.lib.mcb_memset(self.h, d.ptr, 0, d.nbytes))
        return d


class DeviceArray:
    def __init__(self, ctx, shape, dtype):
        self.ctx, self.shape, self.dtype = ctx, tuple(shape), dtype
        self.size = int(np.prod(self.shape)) if self.shape else 1
        self.nbytes = self.size * np.dtype(_NP_OF[dtype]).itemsize
        p = C.c_void_p()
        guard = getattr(ctx, "guard_bytes", 0)
        if not guard:
            ctx.check(ctx.lib.mcb_alloc(ctx.h, max(self.nbytes, 1), C.byref(p)))
            self.ptr = self._base = p
            self._guard = None
            return
        # canary bands: `guard` bytes of a fixed pattern before and after the array (and `guard_shift` bytes of it in
        # front, to move the array off its 16-byte alignment); Context.check_guards() reads them back
        item = np.dtype(_NP_OF[dtype]).itemsize
        shift = (ctx.guard_shift + item - 1) // item * item  # never below the element's own alignment
        total = guard + shift + self.nbytes + guard
        ctx.check(ctx.lib.mcb_alloc(ctx.h, total, C.byref(p)))
        band = np.full(total, GUARD_BYTE, np.uint8)
        ctx.check(ctx.lib.mcb_memcpy_h2d(ctx.h, p, band.ctypes.data_as(C.c_void_p), total))
        ctx.sync()
        self._base = p
        self.ptr = C.c_void_p(p.value + guard + shift)
        self._guard = (guard + shift, guard)

    def guards_intact(self):
        front, back = self._guard
        for start, n in ((self._base.value, front), (self.ptr.value + self.nbytes, back)):
            got = np.empty(n, np.uint8)
            self.ctx.check(self.ctx.lib.mcb_memcpy_d2h(self.ctx.h, got.ctypes.data_as(C.c_void_p), C.c_void_p(start), n))
            if not (got == GUARD_BYTE).all():
                return False
        return True

    def __del__(self):
        try:
            if self._base and self.ctx.h:
                if self._guard:  # the bands are read when the array dies; Context.check_guards() reports
                    self.ctx.sync()
                    self.ctx.guard_checked += 1
                    if not self.guards_intact():
                        self.ctx.guard_broken.append((self.shape, self.dtype))
                self.ctx.lib.mcb_free(self.ctx.h, self._base)
        except Exception:
            pass

    def upload(self, host):
        host = np.asarray(host)
        if self.dtype == F16 and host.dtype == np.uint16:
            host = host.view(np.float16)  # f16 bit patterns, like the uint16 form of bf16
        host = np.ascontiguousarray(host, _NP_OF[self.dtype])
        assert host.size == self.size
        self.ctx.check(self.ctx.lib.mcb_memcpy_h2d(self.ctx.h, self.ptr, host.ctypes.data_as(C.c_void_p), self.nbytes))
        self.ctx.sync()

    def numpy(self):
        """Host copy; bf16 is widened to f32.  Raises if a kernel flagged a bad label or index."""
        out = np.empty(self.shape, _NP_OF[self.dtype])
        self.ctx.check(self.ctx.lib.mcb_memcpy_d2h(self.ctx.h, out.ctypes.data_as(C.c_void_p), self.ptr, self.nbytes))
        if self.dtype == BF16:
            return bf16_bits_to_f32(out).reshape(self.shape)
        return out.astype(np.float32) if self.dtype == F16 else out


class _Ops:
    """Host-array front end of the op-level entry points (one call = upload, kernel, download).
    Used by the parity tests; the names are the `Ops` trait methods of the reference."""

    def __init__(self, ctx):
        self.ctx, self.lib = ctx, ctx.lib

    def _a(self, x, dt=None):
        return self.ctx.array(x, dt)

    def binary(self, op, a, b):
        a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
        try:
            oshape = np.broadcast_shapes(a.shape, b.shape)
        except ValueError:
            oshape = a.shape  # let the library report the broadcast error
        out = self.ctx.empty(oshape)
        da, db = self._a(a), self._a(b)
        self.ctx.check(self.lib.mcb_binary(self.ctx.h, op, da.ptr, _dims(a.shape), a.ndim, db.ptr, _dims(b.shape), b.ndim, out.ptr))
        return out.numpy()

    def scale(self, x, f):
        d = self._a(np.asarray(x, np.float32))
        out = self.ctx.empty(d.shape)
        self.ctx.check(self.lib.mcb_scale(self.ctx.h, d.ptr, float(f), out.ptr, d.size))
        return out.numpy()

    def unary(self, op, x):
        d = self._a(np.asarray(x, np.float32))
        out = self.ctx.empty(d.shape)
        self.ctx.check(self.lib.mcb_unary(self.ctx.h, op, d.ptr, out.ptr, d.size))
        return out.numpy()

    def _map1(self, fn, x, dt):
        d = self._a(np.asarray(x, np.float32), dt)
        out = self.ctx.empty(d.shape, dt)
        self.ctx.check(fn(self.ctx.h, d.ptr, out.ptr, d.size, dt))
        return out.numpy()

    def _map2(self, fn, x, g, dt):
        d, e = self._a(np.asarray(x, np.float32), dt), self._a(np.asarray(g, np.float32), dt)
        out = self.ctx.empty(d.shape, dt)
        self.ctx.check(fn(self.ctx.h, d.ptr, e.ptr, out.ptr, d.size, dt))
        return out.numpy()

    def relu(self, x, dt=F32):
        return self._map1(self.lib.mcb_relu, x, dt)

    def gelu(self, x, dt=F32):
        return self._map1(self.lib.mcb_gelu, x, dt)

    def relu_backward(self, x, g, dt=F32):
        return self._map2(self.lib.mcb_relu_backward, x, g, dt)

    def gelu_backward(self, x, g, dt=F32):
        return self._map2(self.lib.mcb_gelu_backward, x, g, dt)

    def cast(self, x, src_dt, dst_dt):
        d = self._a(x, src_dt)
        out = self.ctx.empty(d.shape, dst_dt)
        self.ctx.check(self.lib.mcb_cast(self.ctx.h, d.ptr, src_dt, out.ptr, dst_dt, d.size))
        return out

    def add_inplace(self, dst, src, dt=F32):
        d, s = self._a(np.asarray(dst, np.float32), dt), self._a(np.asarray(src, np.float32), dt)
        self.ctx.check(self.lib.mcb_add_inplace(self.ctx.h, d.ptr, s.ptr, d.size, dt))
        return d.numpy()

    def sum_all(self, x):
        d = self._a(np.asarray(x, np.float32))
        out = self.ctx.empty(())
        self.ctx.check(self.lib.mcb_sum_all(self.ctx.h, d.ptr, d.size, out.ptr))
        return out.numpy()

    def sum_to(self, a, shape):
        a = np.asarray(a, np.float32)
        d = self._a(a)
        out = self.ctx.empty(shape)
        self.ctx.check(self.lib.mcb_sum_to(self.ctx.h, d.ptr, _dims(a.shape), a.ndim, _dims(shape), len(shape), out.ptr))
        return out.numpy()

    def col_sum(self, a, dt=F32):
        a = np.asarray(a, np.float32)
        d = self._a(a, dt)
        out = self.ctx.empty((a.shape[1],))
        self.ctx.check(self.lib.mcb_col_sum(self.ctx.h, d.ptr, dt, a.shape[0], a.shape[1], out.ptr))
        return out.numpy()

    def softmax(self, x):
        d = self._a(np.asarray(x, np.float32))
        out = self.ctx.empty(d.shape)
        self.ctx.check(self.lib.mcb_softmax(self.ctx.h, d.ptr, out.ptr, d.shape[0], d.shape[1]))
        return out.numpy()

    def softmax_backward(self, x, g):
        d, e = self._a(np.asarray(x, np.float32)), self._a(np.asarray(g, np.float32))
        out = self.ctx.empty(d.shape)
        self.ctx.check(self.lib.mcb_softmax_backward(self.ctx.h, d.ptr, e.ptr, out.ptr, d.shape[0], d.shape[1]))
        return out.numpy()

    def softmax_backward_from_output(self, y, g):
        d, e = self._a(np.asarray(y, np.float32)), self._a(np.asarray(g, np.float32))
        out = self.ctx.empty(d.shape)
        self.ctx.check(self.lib.mcb_softmax_backward_from_output(self.ctx.h, d.ptr, e.ptr, out.ptr, d.shape[0], d.shape[1]))
        return out.numpy()

    def layer_norm(self, x, gamma, beta, eps, out_dt=F32, with_stats=False):
        x = np.asarray(x, np.float32)
        dim = x.shape[-1]
        rows = x.size // dim
        d, g, b = self._a(x), self._a(np.asarray(gamma, np.float32)), self._a(np.asarray(beta, np.float32))
        out, mean, rstd = self.ctx.empty(x.shape, out_dt), self.ctx.empty((rows,)), self.ctx.empty((rows,))
        self.ctx.check(self.lib.mcb_layer_norm(self.ctx.h, d.ptr, g.ptr, b.ptr, float(eps), out.ptr, out_dt, mean.ptr, rstd.ptr, rows, dim))
        return (out.numpy(), mean.numpy(), rstd.numpy()) if with_stats else out.numpy()

    def layer_norm_backward(self, x, gamma, g, eps, g_dt=F32, stats=None):
        x = np.asarray(x, np.float32)
        dim = x.shape[-1]
        rows = x.size // dim
        d, ga, gr = self._a(x), self._a(np.asarray(gamma, np.float32)), self._a(np.asarray(g, np.float32), g_dt)
        mean = self._a(stats[0]) if stats else None
        rstd = self._a(stats[1]) if stats else None
        dx, dg, db = self.ctx.empty(x.shape), self.ctx.empty((dim,)), self.ctx.empty((dim,))
        self.ctx.check(self.lib.mcb_layer_norm_backward(self.ctx.h, d.ptr, ga.ptr, gr.ptr, g_dt, float(eps),
                                                        mean.ptr if mean else None, rstd.ptr if rstd else None, dx.ptr, dg.ptr,
                                                        db.ptr, rows, dim))
        return dx.numpy(), dg.numpy(), db.numpy()

    def softmax_cross_entropy(self, logits, labels):
        d = self._a(np.asarray(logits, np.float32))
        lab = self._a(np.ascontiguousarray(labels))
        out = self.ctx.empty(())
        self.ctx.check(self.lib.mcb_softmax_cross_entropy(self.ctx.h, d.ptr, lab.ptr, lab.dtype, d.shape[0], d.shape[1], out.ptr))
        return out.numpy()

    def softmax_cross_entropy_backward(self, logits, labels):
        d = self._a(np.asarray(logits, np.float32))
        lab = self._a(np.ascontiguousarray(labels))
        out = self.ctx.empty(d.shape)
        self.ctx.check(self.lib.mcb_softmax_cross_entropy_backward(self.ctx.h, d.ptr, lab.ptr, lab.dtype, d.shape[0], d.shape[1], out.ptr))
        return out.numpy()

    def softmax_ce_fused(self, logits, labels, dt=F32, upstream=None):
        d = self._a(np.asarray(logits, np.float32), dt)
        lab = self._a(np.ascontiguousarray(labels))
        loss = self.ctx.empty(())
        up = self._a(np.asarray([upstream], np.float32)) if upstream is not None else None
        self.ctx.check(self.lib.mcb_softmax_ce_fused(self.ctx.h, d.ptr, dt, lab.ptr, lab.dtype, d.shape[0], d.shape[1], loss.ptr,
                                                     up.ptr if up else None))
        return loss.numpy(), d.numpy()

    def embedding(self, ids, weight):
        w = self._a(np.asarray(weight, np.float32))
        i = self._a(np.ascontiguousarray(ids))
        out = self.ctx.empty(i.shape + (w.shape[1],))
        self.ctx.check(self.lib.mcb_embedding(self.ctx.h, i.ptr, i.dtype, i.size, w.ptr, w.shape[0], w.shape[1], out.ptr))
        return out.numpy()

    def embedding_backward(self, ids, weight_shape, g, g_dt=F32):
        i = self._a(np.ascontiguousarray(ids))
        gr = self._a(np.asarray(g, np.float32), g_dt)
        out = self.ctx.empty(weight_shape)
        self.ctx.check(self.lib.mcb_embedding_backward(self.ctx.h, i.ptr, i.dtype, i.size, gr.ptr, g_dt, weight_shape[0], weight_shape[1], out.ptr, 0))
        return out.numpy()

    def matmul(self, a, b):
        a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
        da, db = self._a(a), self._a(b)
        out = self.ctx.empty((a.shape[0], b.shape[1]))
        self.ctx.check(self.lib.mcb_matmul(self.ctx.h, da.ptr, db.ptr, out.ptr, a.shape[0], a.shape[1], b.shape[1]))
        return out.numpy()

    def transpose2d(self, a):
        a = np.asarray(a, np.float32)
        if a.ndim != 2:
            raise McbError(5, "transpose2d expects a 2-D tensor, got rank %d" % a.ndim)
        da = self._a(a)
        out = self.ctx.empty((a.shape[1], a.shape[0]))
        self.ctx.check(self.lib.mcb_transpose2d(self.ctx.h, da.ptr, out.ptr, a.shape[0], a.shape[1]))
        return out.numpy()

    def permute(self, a, axes):
        a = np.asarray(a, np.float32)
        if len(axes) != a.ndim:
            raise McbError(5, "permute rank mismatch")
        da = self._a(a)
        ax = (C.c_int32 * max(1, len(axes)))(*[int(v) for v in axes])
        ok = sorted(int(v) for v in axes) == list(range(a.ndim))
        out = self.ctx.empty(tuple(a.shape[int(v)] for v in axes) if ok else a.shape)
        self.ctx.check(self.lib.mcb_permute(self.ctx.h, da.ptr, _dims(a.shape), a.ndim, ax, out.ptr))
        return out.numpy()

    def linear(self, x, w, bias=None, act=0):
        x, w = np.asarray(x, np.float32), np.asarray(w, np.float32)
        dx, dw = self._a(x), self._a(w)
        db = self._a(np.asarray(bias, np.float32)) if bias is not None else None
        out = self.ctx.empty((x.shape[0], w.shape[0]))
        self.ctx.check(self.lib.mcb_linear(self.ctx.h, dx.ptr, dw.ptr, db.ptr if db else None, out.ptr, x.shape[0], x.shape[1], w.shape[0], act))
        return out.numpy()

    def linear_backward(self, g, x, w):
        g, x, w = (np.asarray(t, np.float32) for t in (g, x, w))
        dg, dx_, dw_ = self._a(g), self._a(x), self._a(w)
        m, k, n = x.shape[0], x.shape[1], w.shape[0]
        gx, gw, gb = self.ctx.empty((m, k)), self.ctx.empty((n, k)), self.ctx.empty((n,))
        self.ctx.check(self.lib.mcb_linear_backward(self.ctx.h, dg.ptr, dx_.ptr, dw_.ptr, gx.ptr, gw.ptr, gb.ptr, m, k, n))
        return gx.numpy(), gw.numpy(), gb.numpy()

    def gemm_bf16(self, a, a_mn, b, b_mn, m, n, k, out_dt=F32, bias=None, accumulate=False, split_k=1, init=None):
        """a, b: f32 host arrays in their stored layout (rounded to bf16 on upload)."""
        return self.gemm_lowp(BF16, a, a_mn, b, b_mn, m, n, k, out_dt, bias, accumulate, split_k, init)

    def gemm_lowp(self, in_dt, a, a_mn, b, b_mn, m, n, k, out_dt=F32, bias=None, accumulate=False, split_k=1, init=None):
        """The tensor-core GEMM with bf16 or f16 operands (in_dt); a, b are rounded to in_dt on upload."""
        da, db = self._a(np.asarray(a, np.float32), in_dt), self._a(np.asarray(b, np.float32), in_dt)
        dbias = self._a(np.asarray(bias, np.float32)) if bias is not None else None
        out = self.ctx.array(np.asarray(init, np.float32)) if init is not None else self.ctx.zeros((m, n), out_dt)
        self.ctx.check(self.lib.mcb_gemm_lowp(self.ctx.h, in_dt, da.ptr, int(a_mn), db.ptr, int(b_mn), out.ptr, out_dt,
                                              dbias.ptr if dbias else None, m, n, k, int(accumulate), split_k))
        return out.numpy()

    def attention(self, q, k, v, heads, causal, dt=F32):
        q = np.asarray(q, np.float32)
        n, s, d = q.shape
        dq, dk, dv = self._a(q, dt), self._a(np.asarray(k, np.float32), dt), self._a(np.asarray(v, np.float32), dt)
        out, lse = self.ctx.empty(q.shape, dt), self.ctx.empty((n, heads, s))
        self.ctx.check(self.lib.mcb_attention(self.ctx.h, dq.ptr, dk.ptr, dv.ptr, out.ptr, lse.ptr, n, s, d, heads, int(causal), dt))
        return out.numpy(), lse.numpy()

    def attention_backward(self, q, k, v, g, heads, causal, dt=F32):
        q = np.asarray(q, np.float32)
        n, s, d = q.shape
        dq, dk, dv, dg = (self._a(np.asarray(t, np.float32), dt) for t in (q, k, v, g))
        out, lse = self.ctx.empty(q.shape, dt), self.ctx.empty((n, heads, s))
        self.ctx.check(self.lib.mcb_attention(self.ctx.h, dq.ptr, dk.ptr, dv.ptr, out.ptr, lse.ptr, n, s, d, heads, int(causal), dt))
        gq, gk, gv = self.ctx.empty(q.shape, dt), self.ctx.empty(q.shape, dt), self.ctx.empty(q.shape, dt)
        self.ctx.check(self.lib.mcb_attention_backward(self.ctx.h, dq.ptr, dk.ptr, dv.ptr, out.ptr, dg.ptr, lse.ptr, gq.ptr, gk.ptr, gv.ptr,
                                                       n, s, d, heads, int(causal), dt))
        return gq.numpy(), gk.numpy(), gv.numpy()

    def conv2d(self, x, w, bias, stride, pad):
        x, w = np.asarray(x, np.float32), np.asarray(w, np.float32)
        n, c, h, wd = x.shape
        o, _, kh, kw = w.shape
        dx, dw = self._a(x), self._a(w)
        db = self._a(np.asarray(bias, np.float32)) if bias is not None else None
        out = self.ctx.empty((n, o, (h + 2 * pad - kh) // stride + 1, (wd + 2 * pad - kw) // stride + 1))
        self.ctx.check(self.lib.mcb_conv2d(self.ctx.h, dx.ptr, dw.ptr, db.ptr if db else None, out.ptr, n, c, h, wd, o, kh, kw, stride, pad))
        return out.numpy()

    def conv2d_backward(self, x, w, g, stride, pad):
        x, w, g = (np.asarray(t, np.float32) for t in (x, w, g))
        n, c, h, wd = x.shape
        o, _, kh, kw = w.shape
        dx, dw, dg = self._a(x), self._a(w), self._a(g)
        gx, gw, gb = self.ctx.empty(x.shape), self.ctx.empty(w.shape), self.ctx.empty((o,))
        self.ctx.check(self.lib.mcb_conv2d_backward(self.ctx.h, dx.ptr, dw.ptr, dg.ptr, gx.ptr, gw.ptr, gb.ptr, n, c, h, wd, o, kh, kw, stride, pad))
        return gx.numpy(), gw.numpy(), gb.numpy()

    def max_pool2d(self, x, kernel, stride, pad):
        x = np.asarray(x, np.float32)
        n, c, h, w = x.shape
        d = self._a(x)
        out = self.ctx.empty((n, c, (h + 2 * pad - kernel) // stride + 1, (w + 2 * pad - kernel) // stride + 1))
        self.ctx.check(self.lib.mcb_max_pool2d(self.ctx.h, d.ptr, out.ptr, n, c, h, w, kernel, stride, pad))
        return out.numpy()

    def max_pool2d_backward(self, x, g, kernel, stride, pad):
        x, g = np.asarray(x, np.float32), np.asarray(g, np.float32)
        n, c, h, w = x.shape
        d, e = self._a(x), self._a(g)
        out = self.ctx.empty(x.shape)
        self.ctx.check(self.lib.mcb_max_pool2d_backward(self.ctx.h, d.ptr, e.ptr, out.ptr, n, c, h, w, kernel, stride, pad))
        return out.numpy()

    def adam_update(self, p, g, m, v, lr, beta1, beta2, eps, step):
        dp, dg, dm, dv = (self._a(np.asarray(t, np.float32)) for t in (p, g, m, v))
        np_, nm, nv = self.ctx.empty(dp.shape), self.ctx.empty(dp.shape), self.ctx.empty(dp.shape)
        self.ctx.check(self.lib.mcb_adam_update(self.ctx.h, dp.ptr, dg.ptr, dm.ptr, dv.ptr, np_.ptr, nm.ptr, nv.ptr, dp.size, lr, beta1, beta2, eps, step))
        return np_.numpy(), nm.numpy(), nv.numpy()

    def adam_flat(self, p, g, m, v, lr, beta1, beta2, eps, step, inv_scale=1.0, g_dt=F32, shadow=False, skip=None):
        dp, dm, dv = (self._a(np.asarray(t, np.float32)) for t in (p, m, v))
        dg = self._a(g, g_dt) if g_dt == BF16 and np.asarray(g).dtype == np.uint16 else self._a(np.asarray(g, np.float32), g_dt)
        sh = self.ctx.empty(dp.shape, BF16) if shadow else None
        flag = self._a(np.asarray([skip], np.int32)) if skip is not None else None
        self.ctx.check(self.lib.mcb_adam_flat(self.ctx.h, dp.ptr, dg.ptr, g_dt, dm.ptr, dv.ptr, sh.ptr if sh else None, dp.size, lr, beta1, beta2,
                                              eps, step, inv_scale, flag.ptr if flag else None))
        return dp.numpy(), dm.numpy(), dv.numpy(), (sh.numpy() if sh else None)

    def check_finite(self, g, g_dt=F32):
        dg = self._a(g, g_dt) if np.asarray(g).dtype == np.uint16 else self._a(np.asarray(g, np.float32), g_dt)
        flag = self.ctx.zeros((1,), I32)
        self.ctx.check(self.lib.mcb_check_finite(self.ctx.h, dg.ptr, g_dt, dg.size, flag.ptr))
        return int(flag.numpy()[0])


def ops(ctx):
    return _Ops(ctx)


# ------------------------------------------------------------------ tape front end
class no_grad:
    def __enter__(self):
        lib = _lib.load()
        self.prev = lib.mcb_is_grad_enabled()
        lib.mcb_set_grad_enabled(0)

    def __exit__(self, *a):
        _lib.load().mcb_set_grad_enabled(self.prev)


class autocast:
    """`with autocast(BF16):` / `with autocast(F16):` lowers linear / attention of the calling thread to
    tensor-core kernels with operands of that type (core/src/autocast.rs:10-44); scopes nest."""

    def __init__(self, dtype=BF16):
        self.dtype = dtype

    def __enter__(self):
        lib = _lib.load()
        self.prev = lib.mcb_get_autocast()
        lib.mcb_set_autocast(self.dtype)

    def __exit__(self, *a):
        _lib.load().mcb_set_autocast(self.prev)


class Variable:
    def __init__(self, ctx, data=None, requires_grad=True, dtype=None, _h=None):
        self.ctx, self.lib = ctx, ctx.lib
        if _h is not None:
            self.h = _h
            return
        data = np.ascontiguousarray(data)
        if data.dtype == np.float64:
            data = data.astype(np.float32)
        if dtype is None:
            dtype = _DT_OF[data.dtype]
        elif dtype == BF16 and data.dtype != np.uint16:
            data = f32_to_bf16_bits(data)
        h = C.c_void_p()
        ctx.check(self.lib.mcb_var_new(ctx.h, data.ctypes.data_as(C.c_void_p), dtype, _dims(data.shape), data.ndim, int(requires_grad), C.byref(h)))
        self.h = h

    @staticmethod
    def constant(ctx, data, dtype=None):
        return Variable(ctx, data, requires_grad=False, dtype=dtype)

    def __del__(self):
        try:
            if self.h and self.ctx.h:
                self.lib.mcb_var_release(self.h)
        except Exception:
            pass

    @property
    def shape(self):
        r = C.c_int32()
        self.lib.mcb_var_rank(self.h, C.byref(r))
        d = (C.c_int64 * max(r.value, 1))()
        self.lib.mcb_var_dims(self.h, d)
        return tuple(d[i] for i in range(r.value))

    @property
    def dtype(self):
        d = C.c_int32()
        self.lib.mcb_var_dtype(self.h, C.byref(d))
        return d.value

    @property
    def data(self):
        dt = self.dtype
        out = np.empty(self.shape, np.float32 if dt in (BF16, F16) else _NP_OF[dt])
        self.ctx.check(self.lib.mcb_var_data(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    @property
    def grad(self):
        has = C.c_int32()
        self.ctx.check(self.lib.mcb_var_grad(self.h, None, C.byref(has)))
        if not has.value:
            return None
        out = np.empty(self.shape, np.float32)
        self.ctx.check(self.lib.mcb_var_grad(self.h, out.ctypes.data_as(C.c_void_p), C.byref(has)))
        return out

    def set_data(self, host):
        host = np.ascontiguousarray(host, _NP_OF[self.dtype])
        self.ctx.check(self.lib.mcb_var_set_data(self.h, host.ctypes.data_as(C.c_void_p)))

    def set_grad(self, host):
        if host is None:
            self.ctx.check(self.lib.mcb_var_set_grad(self.h, None))
        else:
            host = np.ascontiguousarray(host, np.float32)
            self.ctx.check(self.lib.mcb_var_set_grad(self.h, host.ctypes.data_as(C.c_void_p)))

    def cleargrad(self):
        self.lib.mcb_var_cleargrad(self.h)

    def is_leaf(self):
        o = C.c_int32()
        self.lib.mcb_var_is_leaf(self.h, C.byref(o))
        return bool(o.value)

    @property
    def requires_grad(self):
        o = C.c_int32()
        self.lib.mcb_var_requires_grad(self.h, C.byref(o))
        return bool(o.value)

    def unchain_backward(self):
        self.lib.mcb_var_unchain_backward(self.h)

    def backward(self):
        self.ctx.check(self.lib.mcb_var_backward(self.h))


def _out(ctx, st, h):
    ctx.check(st)
    return Variable(ctx, _h=h)


class _F:
    """Free functions named like crates/modern-chainer-autograd/src/ops.rs and host_ops.rs."""

    def _bin(self, op, a, b):
        h = C.c_void_p()
        return _out(a.ctx, a.lib.mcb_f_binary(op, a.h, b.h, C.byref(h)), h)

    def add(self, a, b):
        return self._bin(0, a, b)

    def sub(self, a, b):
        return self._bin(1, a, b)

    def mul(self, a, b):
        return self._bin(2, a, b)

    def div(self, a, b):
        return self._bin(3, a, b)

    def scale(self, x, f):
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_scale(x.h, float(f), C.byref(h)), h)

    def _un(self, op, x):
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_unary(op, x.h, C.byref(h)), h)

    def exp(self, x):
        return self._un(0, x)

    def log(self, x):
        return self._un(1, x)

    def sigmoid(self, x):
        return self._un(2, x)

    def sqrt(self, x):
        return self._un(3, x)

    def neg(self, x):
        return self._un(6, x)

    def _1(self, fn, x):
        h = C.c_void_p()
        return _out(x.ctx, fn(x.h, C.byref(h)), h)

    def relu(self, x):
        return self._1(x.lib.mcb_f_relu, x)

    def gelu(self, x):
        return self._1(x.lib.mcb_f_gelu, x)

    def sum(self, x):
        return self._1(x.lib.mcb_f_sum, x)

    def mean(self, x):
        return self._1(x.lib.mcb_f_mean, x)

    def softmax(self, x):
        return self._1(x.lib.mcb_f_softmax, x)

    def matmul(self, a, b):
        h = C.c_void_p()
        return _out(a.ctx, a.lib.mcb_f_matmul(a.h, b.h, C.byref(h)), h)

    def linear(self, x, w, b=None):
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_linear(x.h, w.h, b.h if b is not None else None, C.byref(h)), h)

    def linear_activation(self, x, w, b, act):
        code = {"relu": 1, "gelu": 2}[act] if isinstance(act, str) else act
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_linear_activation(x.h, w.h, b.h if b is not None else None, code, C.byref(h)), h)

    def layer_norm(self, x, gamma, beta, eps):
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_layer_norm(x.h, gamma.h, beta.h, float(eps), C.byref(h)), h)

    def softmax_cross_entropy(self, logits, target):
        h = C.c_void_p()
        return _out(logits.ctx, logits.lib.mcb_f_softmax_cross_entropy(logits.h, target.h, C.byref(h)), h)

    def embedding(self, ids, weight):
        h = C.c_void_p()
        return _out(ids.ctx, ids.lib.mcb_f_embedding(ids.h, weight.h, C.byref(h)), h)

    def reshape(self, x, shape):
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_reshape(x.h, _dims(shape), len(shape), C.byref(h)), h)

    def transpose(self, x):
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_transpose(x.h, C.byref(h)), h)

    def permute(self, x, axes):
        h = C.c_void_p()
        ax = (C.c_int32 * max(1, len(axes)))(*[int(v) for v in axes])
        return _out(x.ctx, x.lib.mcb_f_permute(x.h, ax, len(axes), C.byref(h)), h)

    def multi_head_attention(self, q, k, v, heads, causal):
        h = C.c_void_p()
        return _out(q.ctx, q.lib.mcb_f_multi_head_attention(q.h, k.h, v.h, heads, int(causal), C.byref(h)), h)

    def conv2d(self, x, w, b, stride, pad):
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_conv2d(x.h, w.h, b.h if b is not None else None, stride, pad, C.byref(h)), h)

    def max_pool2d(self, x, kernel, stride, pad):
        h = C.c_void_p()
        return _out(x.ctx, x.lib.mcb_f_max_pool2d(x.h, kernel, stride, pad, C.byref(h)), h)


F = _F()


def _handles(params):
    return (C.c_void_p * max(len(params), 1))(*[p.h.value for p in params]), len(params)


def zero_grad(params):
    if params:
        arr, n = _handles(params)
        params[0].lib.mcb_zero_grad(arr, n)


class Arena:
    """Moves parameters into one flat p/grad/m/v allocation (fused optimizer, bucketed all-reduce)."""

    def __init__(self, ctx, params):
        self.ctx, self.params = ctx, list(params)
        arr, n = _handles(self.params)
        h = C.c_void_p()
        ctx.check(ctx.lib.mcb_arena_create(ctx.h, arr, n, C.byref(h)))
        self.h = h

    @property
    def numel(self):
        o = C.c_int64()
        self.ctx.lib.mcb_arena_numel(self.h, C.byref(o))
        return o.value


class Adam:
    def __init__(self, ctx, lr, beta1=0.9, beta2=0.999, eps=1e-8):
        self.ctx = ctx
        h = C.c_void_p()
        ctx.check(ctx.lib.mcb_adam_create(ctx.h, lr, beta1, beta2, eps, C.byref(h)))
        self.h = h

    def update(self, params):
        arr, n = _handles(params)
        self.ctx.check(self.ctx.lib.mcb_adam_step(self.h, arr, n))

    @property
    def lr(self):
        v = C.c_double()
        self.ctx.check(self.ctx.lib.mcb_opt_get_lr(self.h, C.byref(v)))
        return v.value

    @lr.setter
    def lr(self, value):
        self.ctx.check(self.ctx.lib.mcb_opt_set_lr(self.h, float(value)))


class _Opt(Adam):
    """The other members of the Optimizer family (optim/src/lib.rs:23-51, 122-214) on the same handle."""
    KIND = 0

    def _create(self, ctx, lr, beta1, beta2, eps, weight_decay):
        self.ctx = ctx
        h = C.c_void_p()
        ctx.check(ctx.lib.mcb_opt_create(ctx.h, self.KIND, lr, beta1, beta2, eps, weight_decay, C.byref(h)))
        self.h = h


class AdamW(_Opt):
    KIND = 1

    def __init__(self, ctx, lr, weight_decay, beta1=0.9, beta2=0.999, eps=1e-8):
        self._create(ctx, lr, beta1, beta2, eps, weight_decay)


class SGD(_Opt):
    KIND = 2

    def __init__(self, ctx, lr):
        self._create(ctx, lr, 0.0, 0.0, 0.0, 0.0)


class MomentumSGD(_Opt):
    KIND = 3

    def __init__(self, ctx, lr, momentum):
        self._create(ctx, lr, momentum, 0.0, 0.0, 0.0)


def clip_grad_norm(params, max_norm):
    """clip_grad_norm (optim/src/lib.rs:216-243): returns the norm before clipping."""
    arr, n = _handles(params)
    ctx = params[0].ctx
    out = C.c_double()
    ctx.check(ctx.lib.mcb_clip_grad_norm(arr, n, float(max_norm), C.byref(out)))
    return out.value


def _named(named_params):
    names = [str(k).encode("utf-8") for k, _ in named_params]
    arr, n = _handles([v for _, v in named_params])
    cn = (C.c_char_p * max(1, n))(*names)
    return cn, arr, n


def save_checkpoint(path, named_params, optimizer=None, scaler=None):
    """Parameters (and optimizer / GradScaler state) into one `.mcn` file, the reference's container
    (crates/modern-chainer-serial/src/lib.rs:12-62).  named_params: [(name, Variable), ...]."""
    cn, arr, n = _named(named_params)
    ctx = named_params[0][1].ctx
    ctx.check(ctx.lib.mcb_checkpoint_save(ctx.h, os.fsencode(path), cn, arr, n, optimizer.h if optimizer else None,
                                          scaler.h if scaler else None))


def load_checkpoint(path, named_params, optimizer=None, scaler=None):
    cn, arr, n = _named(named_params)
    ctx = named_params[0][1].ctx
    ctx.check(ctx.lib.mcb_checkpoint_load(ctx.h, os.fsencode(path), cn, arr, n, optimizer.h if optimizer else None,
                                          scaler.h if scaler else None))


class LinearWarmupCosineLR:
    def __init__(self, warmup_steps, total_steps, base_lr, min_lr):
        self.a = (int(warmup_steps), int(total_steps), float(base_lr), float(min_lr))

    def get_lr(self, step):
        return _lib.load().mcb_lr_linear_warmup_cosine(int(step), *self.a)


class StepLR:
    def __init__(self, base_lr, step_size, gamma):
        self.a = (float(base_lr), int(step_size), float(gamma))

    def get_lr(self, step):
        return _lib.load().mcb_lr_step(int(step), *self.a)


class ConstantLR:
    def __init__(self, lr):
        self.lr = float(lr)

    def get_lr(self, step):
        return self.lr


class PolynomialLR:
    def __init__(self, base_lr, total_steps, power, min_lr):
        self.a = (float(base_lr), int(total_steps), float(power), float(min_lr))

    def get_lr(self, step):
        return _lib.load().mcb_lr_polynomial(int(step), *self.a)


class GradScaler:
    def __init__(self, ctx, scale=65536.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000):
        self.ctx = ctx
        h = C.c_void_p()
        ctx.check(ctx.lib.mcb_scaler_create(ctx.h, scale, growth_factor, backoff_factor, growth_interval, C.byref(h)))
        self.h = h

    def scale_loss(self, loss):
        h = C.c_void_p()
        return _out(self.ctx, self.ctx.lib.mcb_scaler_scale_loss(self.h, loss.h, C.byref(h)), h)

    def step(self, optimizer, params):
        arr, n = _handles(params)
        applied = C.c_int32()
        self.ctx.check(self.ctx.lib.mcb_scaler_step(self.h, optimizer.h, arr, n, C.byref(applied)))
        return bool(applied.value)

    def step_async(self, optimizer, params):
        arr, n = _handles(params)
        self.ctx.check(self.ctx.lib.mcb_scaler_step_async(self.h, optimizer.h, arr, n))

    def _state(self):
        s, t, f = C.c_double(), C.c_int32(), C.c_int32()
        self.ctx.check(self.ctx.lib.mcb_scaler_state(self.h, C.byref(s), C.byref(t), C.byref(f)))
        return s.value, t.value, f.value

    @property
    def scale(self):
        return self._state()[0]

    @property
    def growth_tracker(self):
        return self._state()[1]

    @property
    def last_found_inf(self):
        return bool(self._state()[2])


class Model:
    """The benchmark models built inside the library (kinds: 'mlp', 'encoder', 'cnn', 'decoder')."""
    KINDS = {"mlp": 0, "encoder": 1, "cnn": 2, "decoder": 3}

    def __init__(self, ctx, kind, cfg):
        self.ctx = ctx
        h = C.c_void_p()
        arr = (C.c_int64 * len(cfg))(*cfg)
        ctx.check(ctx.lib.mcb_model_create(ctx.h, self.KINDS[kind], arr, len(cfg), C.byref(h)))
        self.h = h
        n = C.c_int32()
        ctx.lib.mcb_model_num_params(self.h, C.byref(n))
        self._params = []
        for i in range(n.value):
            p = C.c_void_p()
            ctx.check(ctx.lib.mcb_model_param(self.h, i, C.byref(p)))
            self._params.append(Variable(ctx, _h=p))

    def parameters(self):
        return self._params

    def loss(self, x, target):
        h = C.c_void_p()
        return _out(self.ctx, self.ctx.lib.mcb_model_loss(self.h, x.h, target.h, C.byref(h)), h)


class StaticStep:
    """One whole training step (zero_grad, loss, backward, optimizer update) captured as a CUDA Graph and
    replayed with a single launch (the reference's CudaStaticStep, cuda/src/static_run.rs:1875-2096).
    x_like / y_like give the shape and dtype of the fixed input buffers."""

    def __init__(self, model, optimizer, x_like, y_like, scaler=None, autocast_dtype=None):
        self.ctx = model.ctx
        x_like, y_like = np.asarray(x_like), np.asarray(y_like)
        self._xs, self._ys = (x_like.shape, x_like.dtype), (y_like.shape, y_like.dtype)
        h = C.c_void_p()
        self.ctx.check(self.ctx.lib.mcb_static_step_create(
            model.h, optimizer.h, scaler.h if scaler else None, -1 if autocast_dtype is None else autocast_dtype,
            _dims(x_like.shape), x_like.ndim, _DT_OF[x_like.dtype], _dims(y_like.shape), y_like.ndim, _DT_OF[y_like.dtype], C.byref(h)))
        self.h = h
        self._keep = (model, optimizer, scaler)

    def _host(self, a, spec):
        a = np.ascontiguousarray(a, spec[1])
        if a.shape != tuple(spec[0]):
            raise McbError(1, "static step input has shape %s, captured %s" % (a.shape, tuple(spec[0])))
        return a

    def run(self, x=None, y=None):
        """Copies x / y (host arrays; None keeps the buffer's contents) and launches the graph; asynchronous,
        but the host arrays may be reused as soon as this returns only if they are pageable (pinned: sync first)."""
        hx = self._host(x, self._xs) if x is not None else None
        hy = self._host(y, self._ys) if y is not None else None
        self.ctx.check(self.ctx.lib.mcb_static_step_run(self.h, hx.ctypes.data if hx is not None else None,
                                                        hy.ctypes.data if hy is not None else None))
        self._last = (hx, hy)

    def loss(self):
        v = C.c_float()
        self.ctx.check(self.ctx.lib.mcb_static_step_loss(self.h, C.byref(v)))
        return v.value

    def run_pipelined(self, x=None, y=None):
        """Launches this step and returns the loss of the PREVIOUS pipelined run (None on the first call), waiting only
        for that one; `drain()` returns the last run's loss.  The host arrays of a call may be rewritten once the next
        call has returned."""
        hx = self._host(x, self._xs) if x is not None else None
        hy = self._host(y, self._ys) if y is not None else None
        v, have = C.c_float(), C.c_int32()
        self.ctx.check(self.ctx.lib.mcb_static_step_run_pipelined(self.h, hx.ctypes.data if hx is not None else None,
                                                                  hy.ctypes.data if hy is not None else None, C.byref(v), C.byref(have)))
        self._prev, self._last = getattr(self, "_last", None), (hx, hy)
        return v.value if have.value else None

    def drain(self):
        v, have = C.c_float(), C.c_int32()
        self.ctx.check(self.ctx.lib.mcb_static_step_drain(self.h, C.byref(v), C.byref(have)))
        return v.value if have.value else None

    @property
    def kernels_per_step(self):
        v = C.c_int64()
        self.ctx.check(self.ctx.lib.mcb_static_step_launches(self.h, C.byref(v)))
        return v.value

    def close(self):
        if self.h and self.ctx.h:  # a closed context has already freed everything the step owned
            self.ctx.lib.mcb_static_step_release(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
