"""Run-twice determinism and canary-band checks.

Determinism: with the MCB_DETERMINISTIC knob a training step gives the same bits from run to run -- the embedding
gradient is added in position order (which is also the order of the reference's CPU loop,
crates/modern-chainer-cpu/src/kernels.rs:1783-1815, so it equals the oracle bit for bit), tensor-core GEMMs run
without split reductions, and max-pool gradients of overlapping windows are gathered per input element.

Canary bands: every array the op front end makes is surrounded by 256 bytes of a fixed pattern, once at its natural
alignment and once moved 4 bytes off it (which sends kernels down their unaligned paths); after a sweep of ops at odd
sizes no band may have changed.  This stands in for a memory checker on the kernels' ragged edges.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(2024)


def randn(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


@pytest.fixture(scope="module")
def mc():
    import modernchainer_b200 as m
    return m


@pytest.fixture()
def ctx(mc):
    c = mc.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("g_dt", ["f32", "bf16"])
def test_ordered_embedding_backward_equals_the_oracle_bit_for_bit(mc, ctx, oracle, g_dt):
    ops = mc.ops(ctx)
    n, vocab, dim = 3000, 50, 70  # sixty tokens per id on average: long chains of additions per row
    ids = RNG.integers(0, vocab, n).astype(np.int64)
    ids[:5] = ids[-1]
    g = randn(n, dim)
    dt = mc.BF16 if g_dt == "bf16" else mc.F32
    if g_dt == "bf16":
        g = oracle.round_bf16(g)
    want = oracle.embedding_backward(ids, (vocab, dim), g)
    with ctx.knob("MCB_DETERMINISTIC"):
        got = ops.embedding_backward(ids, (vocab, dim), g, g_dt=dt)
        again = ops.embedding_backward(ids, (vocab, dim), g, g_dt=dt)
    assert np.array_equal(got, want)
    assert np.array_equal(got, again)
    # the default (float atomics) agrees to rounding
    assert np.abs(ops.embedding_backward(ids, (vocab, dim), g, g_dt=dt) - want).max() <= 1e-5 * np.abs(want).max()
    # a bad id is still reported
    ids[7] = vocab
    with ctx.knob("MCB_DETERMINISTIC"):
        with pytest.raises(mc.McbError):
            ops.embedding_backward(ids, (vocab, dim), g, g_dt=dt)


@pytest.mark.parametrize("kernel,stride,pad,hw", [(3, 1, 1, 9), (3, 2, 0, 11), (2, 1, 0, 6), (5, 3, 2, 13)])
def test_gathered_max_pool_backward_equals_the_oracle_bit_for_bit(mc, ctx, oracle, kernel, stride, pad, hw):
    ops = mc.ops(ctx)
    x = np.round(randn(2, 3, hw, hw) * 2)  # many ties inside a window: the reference's tie rule decides
    oh = (hw + 2 * pad - kernel) // stride + 1
    g = randn(2, 3, oh, oh)
    want = oracle.max_pool2d_backward(x, g, kernel, stride, pad)
    with ctx.knob("MCB_DETERMINISTIC"):
        got = ops.max_pool2d_backward(x, g, kernel, stride, pad)
    assert np.array_equal(got, want)
    assert np.abs(ops.max_pool2d_backward(x, g, kernel, stride, pad) - want).max() <= 1e-6 * max(np.abs(want).max(), 1.0)


def step_bits(mc, ctx, kind, cfg, x, y, amp, steps=2):
    """Loss and gradient bits of `steps` training steps from a fresh model (same seeded initialisation every time)."""
    m = mc.Model(ctx, kind, cfg)
    ps = m.parameters()
    keep = mc.Arena(ctx, ps)
    opt = mc.Adam(ctx, 1e-3)
    out = []
    for _ in range(steps):
        mc.zero_grad(ps)
        if amp:
            with mc.autocast(mc.BF16):
                loss = m.loss(mc.Variable.constant(ctx, x), mc.Variable.constant(ctx, y))
        else:
            loss = m.loss(mc.Variable.constant(ctx, x), mc.Variable.constant(ctx, y))
        loss.backward()
        out.append(loss.data.copy().view(np.uint32))
        out += [p.grad.copy().view(np.uint32) for p in ps]
        opt.update(ps)
    out += [p.data.copy().view(np.uint32) for p in ps]
    del keep
    return out


@pytest.mark.parametrize("amp", [False, True])
def test_decoder_step_is_reproducible_run_to_run(mc, ctx, amp):
    vocab, d, heads, ff, layers, s, b = 512, 256, 4, 1024, 2, 256, 8  # 2048 tokens over 512 ids: every id repeats
    ids = RNG.integers(0, vocab, (b, s)).astype(np.int64)
    tgt = np.concatenate([ids[:, 1:], RNG.integers(0, vocab, (b, 1))], 1).astype(np.int64)
    ctx.set_knob("MCB_DETERMINISTIC", 1)
    runs = [step_bits(mc, ctx, "decoder", [vocab, d, heads, ff, layers, 0], ids, tgt, amp) for _ in range(3)]
    for other in runs[1:]:
        assert len(other) == len(runs[0])
        for i, (a, b_) in enumerate(zip(runs[0], other)):
            assert np.array_equal(a, b_), f"tensor {i} differs between two runs"


def test_cnn_step_is_reproducible_run_to_run(mc, ctx):
    cin, c1, c2, hw, classes, b = 3, 16, 32, 16, 10, 32
    x = randn(b, cin, hw, hw)
    y = RNG.integers(0, classes, b).astype(np.int64)
    ctx.set_knob("MCB_DETERMINISTIC", 1)
    runs = [step_bits(mc, ctx, "cnn", [cin, c1, c2, hw, classes], x, y, False) for _ in range(3)]
    for other in runs[1:]:
        for i, (a, b_) in enumerate(zip(runs[0], other)):
            assert np.array_equal(a, b_), f"tensor {i} differs between two runs"


@pytest.mark.parametrize("shift", [0, 4])
def test_no_kernel_writes_outside_its_arrays(mc, ctx, shift):
    """Odd sizes on both sides of each kernel's vector width and tile, outputs between canary bands."""
    ctx.guard(256, shift)
    ops = mc.ops(ctx)
    checked = 0
    for n in (1, 3, 255, 1001, 4099):
        x, g = randn(n), randn(n)
        ops.binary(0, x, g), ops.unary(0, x), ops.scale(x, 0.5), ops.relu(x), ops.gelu(x), ops.relu_backward(x, g), ops.gelu_backward(x, g)
        ops.cast(x, mc.F32, mc.BF16), ops.cast(x, mc.F32, mc.F16), ops.sum_all(x)
        m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
        ops.adam_update(x, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 1)
        ops.adam_flat(x, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 1)
        ops.check_finite(g)
        checked = ctx.check_guards()
    for rows, cols in ((1, 1), (3, 5), (7, 129), (9, 1023), (5, 1025), (3, 4100), (2, 13001), (130, 7)):
        x, g = randn(rows, cols), randn(rows, cols)
        y = ops.softmax(x)
        ops.softmax_backward(x, g), ops.softmax_backward_from_output(y, g)
        gam, bet = randn(cols), randn(cols)
        ops.layer_norm(x, gam, bet, 1e-5), ops.layer_norm(x, gam, bet, 1e-5, out_dt=mc.BF16), ops.layer_norm_backward(x, gam, g, 1e-5)
        ops.col_sum(x), ops.sum_to(x, (1, cols)), ops.sum_to(x, (rows, 1)), ops.transpose2d(x)
        lab = RNG.integers(0, cols, rows).astype(np.int64)
        ops.softmax_cross_entropy(x, lab), ops.softmax_cross_entropy_backward(x, lab), ops.softmax_ce_fused(x, lab)
        ids = RNG.integers(0, 11, rows).astype(np.int64)
        ops.embedding(ids, randn(11, cols)), ops.embedding_backward(ids, (11, cols), g)
        with ctx.knob("MCB_DETERMINISTIC"):
            ops.embedding_backward(ids, (11, cols), g)
        checked = ctx.check_guards()
    for m_, n_, k_ in ((1, 1, 1), (5, 7, 3), (129, 65, 33), (200, 130, 1000), (3, 10, 4097)):
        a, b = randn(m_, k_), randn(k_, n_)
        ops.matmul(a, b)
        w, bias = randn(n_, k_), randn(n_)
        ops.linear(a, w, bias), ops.linear(a, w, bias, act=1), ops.linear_backward(randn(m_, n_), a, w)
        checked = ctx.check_guards()
    # the tensor-core GEMM and the 16-bit attention kernels take 16-byte aligned operands only (TMA); off alignment they
    # must refuse with a status, not run
    for m_, n_, k_ in ((128, 8, 64), (136, 24, 72), (1000, 200, 136), (264, 776, 4104)):  # n, k multiples of 8
        a, b = randn(m_, k_), randn(n_, k_)
        if shift:
            with pytest.raises(mc.McbError):
                ops.gemm_bf16(a, False, b, False, m_, n_, k_, out_dt=mc.F32)
            continue
        for out_dt in (mc.F32, mc.BF16):
            ops.gemm_bf16(a, False, b, False, m_, n_, k_, out_dt=out_dt, bias=randn(n_))
        ops.gemm_bf16(a, False, b, False, m_, n_, k_, out_dt=mc.F32, accumulate=True, split_k=3, init=randn(m_, n_))
        checked = ctx.check_guards()
    for nb, heads, s, d in ((1, 2, 5, 16), (2, 3, 129, 24), (1, 4, 300, 256)):
        q, k, v, g = (randn(nb, s, d) for _ in range(4))
        for causal in (False, True):
            ops.attention(q, k, v, heads, causal), ops.attention_backward(q, k, v, g, heads, causal)
            if shift and d == 256:
                with pytest.raises(mc.McbError):
                    ops.attention(q, k, v, heads, causal, dt=mc.BF16)
            elif not shift:
                ops.attention(q, k, v, heads, causal, dt=mc.BF16), ops.attention_backward(q, k, v, g, heads, causal, dt=mc.BF16)
        checked = ctx.check_guards()
    for nb, c, hw, o, k, stride, pad in ((1, 1, 5, 1, 3, 1, 1), (2, 3, 9, 5, 3, 2, 0), (3, 4, 13, 8, 5, 1, 2), (64, 3, 32, 32, 3, 1, 1)):
        x, w, bias = randn(nb, c, hw, hw), randn(o, c, k, k), randn(o)
        out = ops.conv2d(x, w, bias, stride, pad)
        ops.conv2d_backward(x, w, randn(*out.shape), stride, pad)
        p = ops.max_pool2d(x, 2, 2, 0)
        ops.max_pool2d_backward(x, randn(*p.shape), 2, 2, 0)
        with ctx.knob("MCB_DETERMINISTIC"):
            p = ops.max_pool2d(x, 3, 1, 1)
            ops.max_pool2d_backward(x, randn(*p.shape), 3, 1, 1)
        checked = ctx.check_guards()
    assert checked > 0


def test_knobs_are_per_context_and_unknown_names_are_refused(mc, ctx):
    """The environment is read once, when a context is created; afterwards a knob changes only through mcb_set_knob,
    for that context alone."""
    import os
    with pytest.raises(mc.McbError):
        ctx.set_knob("MCB_NO_SUCH_KNOB", 1)
    ops = mc.ops(ctx)
    x = randn(64, 8, 16, 16)  # 38 M multiply-adds: large enough for the tensor-core convolution
    w, b = randn(32, 8, 3, 3) * 0.2, randn(32)
    tc = ops.conv2d(x, w, b, 1, 1)
    os.environ["MCB_CONV_DIRECT"] = "1"  # too late for this context: it keeps the tensor-core path
    try:
        assert np.array_equal(ops.conv2d(x, w, b, 1, 1), tc)
        other = mc.Context(0)  # a context created now reads it
        try:
            direct = mc.ops(other).conv2d(x, w, b, 1, 1)
        finally:
            other.close()
    finally:
        os.environ.pop("MCB_CONV_DIRECT", None)
    ctx.set_knob("MCB_CONV_DIRECT", 1)
    assert np.array_equal(ops.conv2d(x, w, b, 1, 1), direct)  # the same kernels as the other context ran
    ctx.set_knob("MCB_CONV_DIRECT", None)
    assert np.array_equal(ops.conv2d(x, w, b, 1, 1), tc)
    assert not np.array_equal(direct, tc) and np.abs(direct - tc).max() <= 2e-6 * np.abs(tc).max()  # two different kernels
