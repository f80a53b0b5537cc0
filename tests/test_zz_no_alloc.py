"""The allocation-free LayerNorm backward entry point against the regular one.

Who needs it: a caller that owns the GPU's memory plan and forbids device allocation inside the
library -- it passes a stream plus input and output buffers and expects nothing else to be
created.  The regular mcb_layer_norm_backward cannot serve that caller, because it keeps the
per-block partial sums of dgamma / dbeta in scratch memory that the context allocates on demand.
mcb_layer_norm_backward_noalloc keeps them in a fixed array inside the library image instead.

The test calls the new entry point through the C ABI twice in a row, with different sizes, so the
second call runs over whatever the first one left in the shared array, and compares each result
with the regular entry point on the same inputs and, as a second and independent comparand, with the
CPU oracle (2e-5 relative per tensor, the tolerance the other LayerNorm tests use; the paths sum the
partials in a different order), so a defect shared by both device entry points cannot hide.  The file
is named so pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def close(a, b, tol=2e-5):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape
    err = np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)
    assert err <= tol, f"relative error {err:.3e} > {tol}"


def run_pair(mc, ctx, rng, rows, dim, g_dt, use_stats, oracle):
    lib = ctx.lib
    x = (rng.standard_normal((rows, dim)) * 2 + 0.5).astype(np.float32)
    g = rng.standard_normal((rows, dim)).astype(np.float32)
    gamma = (rng.standard_normal(dim) * 0.2 + 1).astype(np.float32)
    beta = np.zeros(dim, np.float32)
    dxv, dgam, dg = ctx.array(x), ctx.array(gamma), ctx.array(g, g_dt)
    mean = rstd = None
    if use_stats:
        y, mean, rstd = ctx.empty((rows, dim)), ctx.empty((rows,)), ctx.empty((rows,))
        dbeta_in = ctx.array(beta)
        ctx.check(lib.mcb_layer_norm(ctx.h, dxv.ptr, dgam.ptr, dbeta_in.ptr, 1e-5, y.ptr, mc.F32, mean.ptr, rstd.ptr, rows, dim))
    mp, rp = (mean.ptr if mean else None), (rstd.ptr if rstd else None)
    ref = [ctx.empty((rows, dim)), ctx.empty((dim,)), ctx.empty((dim,))]
    ctx.check(lib.mcb_layer_norm_backward(ctx.h, dxv.ptr, dgam.ptr, dg.ptr, g_dt, 1e-5, mp, rp, ref[0].ptr, ref[1].ptr, ref[2].ptr, rows, dim))
    out = [ctx.empty((rows, dim)), ctx.empty((dim,)), ctx.empty((dim,))]
    stream = C.c_void_p(lib.mcb_stream(ctx.h))
    st = lib.mcb_layer_norm_backward_noalloc(stream, dxv.ptr, dgam.ptr, dg.ptr, g_dt, 1e-5, mp, rp, out[0].ptr, out[1].ptr, out[2].ptr, rows, dim)
    assert st == 0, lib.mcb_noalloc_last_error()
    for a, b in zip(out, ref):
        close(a.numpy(), b.numpy())
    g_seen = oracle.round_bf16(g) if g_dt == mc.BF16 else g  # the gradient values the device read
    for a, b in zip(out, oracle.layer_norm_backward(x, gamma, g_seen, 1e-5)):
        close(a.numpy(), b)


def test_noalloc_layer_norm_backward_matches_regular_entry_point(oracle):
    import modernchainer_b200 as mc
    ctx = mc.Context(0)
    try:
        lib = ctx.lib
        rng = np.random.default_rng(77)
        # two calls in a row; the second is smaller and narrower, so stale partial sums of the first
        # stay in the shared array next to the ones it writes
        run_pair(mc, ctx, rng, 1000, 768, mc.F32, True, oracle)
        run_pair(mc, ctx, rng, 37, 130, mc.BF16, False, oracle)
        run_pair(mc, ctx, rng, 1, 4096, mc.F32, False, oracle)
        # sizes beyond the built-in array are refused with a message and nothing is enqueued
        stream = C.c_void_p(lib.mcb_stream(ctx.h))
        st = lib.mcb_layer_norm_backward_noalloc(stream, None, None, None, mc.F32, 1e-5, None, None, None, None, None, 4, 4097)
        assert st == 5
        assert b"4096" in lib.mcb_noalloc_last_error()
        ctx.sync()
    finally:
        ctx.close()
