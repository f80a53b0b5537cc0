"""IEEE f16 as the second low-precision type of the path (the reference's ComputeType::F16 and
autocast(DType::F16), crates/modern-chainer-cuda/src/backend.rs:109-136, src/ops.rs:419-597,724,776,808,
crates/modern-chainer-core/src/autocast.rs:6-44): casts, the tcgen05 GEMM and attention with f16 operands,
16-bit storage kernels, and the reference's own mixed-precision tests restated call for call
(crates/modern-chainer-cuda/tests/cuda.rs:611-681 compute types against f32, 764-803 the AMP training loop
under autocast(F16) with GradScaler(1024, growth interval 10)).

Tolerances: f16 has 11 significant bits, so a value stored in f16 is within 2^-11 relative of the f32
value it was rounded from (2^-10 is asserted); GEMMs with f16 operands and f32 output are exact products
summed in f32 (2e-5 against the f64 product of the rounded operands)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

F32, F16, BF16 = 0, 4, 5


@pytest.fixture(scope="module")
def mc():
    import modernchainer_b200 as m
    return m


@pytest.fixture(scope="module")
def ctx(mc):
    c = mc.Context(0)
    yield c
    c.close()


@pytest.fixture(scope="module")
def ops(mc, ctx):
    return mc.ops(ctx)


RNG = np.random.default_rng(4321)


def randn(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


def close(a, b, tol):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape
    err = np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)
    assert err <= tol, f"relative error {err:.3e} > {tol}"


def f16_close(a, ref, ulps=1.0):
    a, ref = np.asarray(a, np.float64), np.asarray(ref, np.float64)
    assert np.all(np.abs(a - ref) <= np.abs(ref) * 2.0 ** -10 * ulps + np.abs(ref).max() * 2.0 ** -10 * 1e-2 + 1e-30)


def test_f16_cast_matches_the_reference_conversion(ops, oracle):
    """f32 -> f16 -> f32 against the oracle's restatement of core/src/dtype.rs:75-134, bit for bit, over the
    normal range, overflow, infinities and values that round to zero.  Results in the f16 SUBNORMAL range are
    excluded from the bit comparison: the reference's subnormal branch adds a rounding bias that is only
    round-half-even for one shift amount, so it truncates there, while the device instruction (and this
    library) rounds to nearest even as IEEE 754 prescribes; both stay within one subnormal step (2^-24)."""
    x = np.concatenate([randn(20001) * 50, randn(5000) * 1e-3, np.array([65504.0, 65519.9, 65520.0, 1e6, -1e6, np.inf, -np.inf, 0.0, -0.0, 1e-9,
                                                                          1.0009765625, 1.00048828125, 1.00146484375, 6.103515625e-05], np.float32)])
    got = ops.cast(x, F32, F16).numpy()
    ref = oracle.round_f16(x)
    normal = (np.abs(x) >= 2.0 ** -14) | (np.abs(x) < 2.0 ** -25)
    assert np.array_equal(got[normal], ref[normal])
    xs = randn(4000) * 2.0 ** -17  # mostly subnormal in f16
    gs, rs = ops.cast(xs, F32, F16).numpy(), oracle.round_f16(xs)
    assert np.abs(gs - rs).max() <= 2.0 ** -24
    assert np.abs(gs.astype(np.float64) - xs).max() <= 2.0 ** -25  # round to nearest: at most half a step away
    # widening is exact both ways
    h = ops.cast(x, F32, F16)
    back = ops.ctx.empty(h.shape, F32)
    ops.ctx.check(ops.lib.mcb_cast(ops.ctx.h, h.ptr, F16, back.ptr, F32, h.size))
    assert np.array_equal(back.numpy(), got)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (8, 8, 8), (136, 72, 200), (1000, 776, 328), (2048, 768, 768), (8192, 768, 1024)])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
def test_tc_gemm_f16_operands(ops, oracle, m, n, k, a_mn, b_mn):
    a = randn(k, m) if a_mn else randn(m, k)
    b = randn(k, n) if b_mn else randn(n, k)
    A = oracle.round_f16(a).astype(np.float64)
    B = oracle.round_f16(b).astype(np.float64)
    ref = (A.T if a_mn else A) @ (B if b_mn else B.T)
    bias = randn(n)
    close(ops.gemm_lowp(F16, a, a_mn, b, b_mn, m, n, k, out_dt=F32, bias=bias), ref + bias, 2e-5)
    out16 = ops.gemm_lowp(F16, a, a_mn, b, b_mn, m, n, k, out_dt=F16, bias=bias)
    assert np.abs(out16 - (ref + bias)).max() <= np.abs(ref).max() * 2.0 ** -10
    init = randn(m, n)
    close(ops.gemm_lowp(F16, a, a_mn, b, b_mn, m, n, k, out_dt=F32, accumulate=True, split_k=1, init=init), ref + init, 2e-5)


def test_tc_gemm_rejects_mixed_16_bit_types(mc, ops):
    with pytest.raises(mc.McbError) as e:
        ops.gemm_lowp(F16, randn(16, 16), 0, randn(16, 16), 0, 16, 16, 16, out_dt=BF16)
    assert e.value.status == 4


def test_f16_storage_kernels(ops, oracle):
    x, g = oracle.round_f16(randn(4099) * 2), oracle.round_f16(randn(4099))
    f16_close(ops.gelu(x, dt=F16), oracle.gelu(x))
    f16_close(ops.gelu_backward(x, g, dt=F16), oracle.gelu_backward(x, g), 2.0)  # hardware tanh approximation, 2^-11
    assert np.array_equal(ops.relu(x, dt=F16), oracle.relu(x))
    assert np.array_equal(ops.relu_backward(x, g, dt=F16), oracle.relu_backward(x, g))
    a, b = oracle.round_f16(randn(10007)), oracle.round_f16(randn(10007))
    assert np.array_equal(ops.add_inplace(a, b, dt=F16), oracle.round_f16(a + b))
    m = oracle.round_f16(randn(300, 776))
    close(ops.col_sum(m, dt=F16), m.astype(np.float64).sum(0), 1e-5)
    # LayerNorm with f16 output / f16 upstream gradient: generic kernel (64 rows) and the bulk pipeline (2048 rows)
    for rows in (64, 2048):
        xx, gg = randn(rows, 768), oracle.round_f16(randn(rows, 768))
        gam, bet = (randn(768) * 0.2 + 1).astype(np.float32), randn(768) * 0.1
        f16_close(ops.layer_norm(xx, gam, bet, 1e-5, out_dt=F16), oracle.layer_norm(xx, gam, bet, 1e-5))
        for got, want in zip(ops.layer_norm_backward(xx, gam, gg, 1e-5, g_dt=F16), oracle.layer_norm_backward(xx, gam, gg, 1e-5)):
            close(got, want, 2e-5)
    # loss head over f16 logits: loss in f32, gradient rounded to f16
    lg = oracle.round_f16(randn(32, 4096) * 2)
    lab = RNG.integers(0, 4096, 32).astype(np.int64)
    loss, grad = ops.softmax_ce_fused(lg, lab, dt=F16, upstream=512.0)
    close(float(loss), float(oracle.softmax_cross_entropy(lg, lab)), 1e-6)
    ref = oracle.scale(oracle.softmax_cross_entropy_backward(lg, lab), 512.0)
    assert np.abs(grad - ref).max() <= np.abs(ref).max() * 2.0 ** -10
    # embedding scatter of an f16 gradient, and the inf/nan scan on f16 bits
    ids = RNG.integers(0, 50, 200).astype(np.int64)
    ge = oracle.round_f16(randn(200, 64))
    close(ops.embedding_backward(ids, (50, 64), ge, g_dt=F16), oracle.embedding_backward(ids, (50, 64), ge), 1e-5)
    bits = np.asarray(ge.reshape(-1), np.float16)
    assert ops.check_finite(bits.view(np.uint16), g_dt=F16) == 0
    bits[777] = np.inf
    assert ops.check_finite(bits.view(np.uint16), g_dt=F16) == 1
    bits[777] = 1.0
    bits[12000] = np.nan
    assert ops.check_finite(bits.view(np.uint16), g_dt=F16) == 1


@pytest.mark.parametrize("n,s,h,causal", [(1, 64, 1, True), (2, 256, 3, True), (2, 256, 3, False), (1, 100, 2, True), (1, 1024, 2, True)])
def test_fused_attention_f16_head_dim_64(ops, oracle, n, s, h, causal):
    d = 64 * h
    q, k, v, g = (oracle.round_f16(randn(n, s, d)) for _ in range(4))
    out, lse = ops.attention(q, k, v, h, causal, dt=F16)
    ref = oracle.attention(q, k, v, h, causal)
    # probabilities are rounded to f16 (2^-11) before the P V product and exp2 is the hardware approximation
    assert np.abs(out - ref).max() <= max(np.abs(ref).max(), 1e-3) * 2.0 ** -9
    for a, r in zip(ops.attention_backward(q, k, v, g, h, causal, dt=F16), oracle.attention_backward(q, k, v, g, h, causal)):
        assert np.abs(a - r).max() <= max(np.abs(r).max(), 1e-3) * 2.0 ** -8, np.abs(a - r).max() / np.abs(r).max()


def test_reference_compute_types_match_f32(mc, ctx):
    """crates/modern-chainer-cuda/tests/cuda.rs:611-681 as written: linear + GELU of sin / cos data under
    ComputeType F16 (|d| < 0.08) and Bf16 (< 0.15) against F32, then matmul under F16 (< 0.1)."""
    F = mc.F
    batch, inp, out = 16, 32, 8
    x = np.sin(np.arange(batch * inp, dtype=np.float32) * np.float32(0.017)).reshape(batch, inp)
    w = (np.cos(np.arange(out * inp, dtype=np.float32) * np.float32(0.013)) * np.float32(0.2)).reshape(out, inp)
    bias = (np.arange(out, dtype=np.float32) * np.float32(0.01))
    gx, gw, gb = mc.Variable.constant(ctx, x), mc.Variable.constant(ctx, w), mc.Variable.constant(ctx, bias)
    try:
        ctx.set_compute_type(0)
        ref = F.linear_activation(gx, gw, gb, "gelu").data
        for compute, tol in ((2, 0.08), (1, 0.15)):
            ctx.set_compute_type(compute)
            mixed = F.linear_activation(gx, gw, gb, "gelu")
            assert mixed.dtype == (mc.F16 if compute == 2 else mc.BF16)  # the op really ran in that type
            assert np.abs(mixed.data - ref).max() < tol
            assert np.abs(mixed.data - ref).max() > 0.0
        b = np.sin(np.arange(inp * out, dtype=np.float32) * np.float32(0.007)).reshape(inp, out)
        ga, gbm = mc.Variable.constant(ctx, x), mc.Variable.constant(ctx, b)
        ctx.set_compute_type(0)
        ref = F.matmul(ga, gbm).data
        ctx.set_compute_type(2)
        assert np.abs(F.matmul(ga, gbm).data - ref).max() < 0.1
    finally:
        ctx.set_compute_type(0)


def test_reference_amp_training_loop_under_f16_autocast(mc, ctx, oracle):
    """crates/modern-chainer-cuda/tests/cuda.rs:764-803 as written: Linear(2 -> 1) from the given parts, MSE on four
    samples, 40 steps of Adam(0.01) under autocast(F16) with GradScaler(1024, growth interval 10); every step is
    applied and the loss goes down.  The same loop on the f16 oracle gives the loss curve to compare with."""
    F = mc.F
    w, b = mc.Variable(ctx, np.array([[0.2, -0.4]], np.float32)), mc.Variable(ctx, np.array([0.1], np.float32))
    x = mc.Variable(ctx, np.array([[1.0, 2.0], [2.0, 1.0], [3.0, 1.0], [4.0, 2.0]], np.float32))
    t = mc.Variable.constant(ctx, np.array([[3.0], [4.0], [5.0], [6.0]], np.float32))
    opt, sc = mc.Adam(ctx, 0.01), mc.GradScaler(ctx, 1024.0, growth_interval=10)
    ow, ob = oracle.Variable(np.array([[0.2, -0.4]], np.float32)), oracle.Variable(np.array([0.1], np.float32))
    ox = oracle.Variable(np.array([[1.0, 2.0], [2.0, 1.0], [3.0, 1.0], [4.0, 2.0]], np.float32))
    ot = oracle.Variable.constant(np.array([[3.0], [4.0], [5.0], [6.0]], np.float32))
    oopt, osc = oracle.Adam(0.01), oracle.GradScaler(1024.0, growth_interval=10)
    first = last = None
    for step in range(40):
        mc.zero_grad([w, b])
        with mc.autocast(mc.F16):
            d = F.sub(F.linear(x, w, b), t)
            loss = F.mean(F.mul(d, d))
        last = float(loss.data)
        first = last if first is None else first
        sc.scale_loss(loss).backward()
        assert sc.step(opt, [w, b]) is True
        oracle.zero_grad([ow, ob])
        with oracle.amp(oracle.F16):
            od = oracle.F.sub(oracle.F.linear(ox, ow, ob), ot)
            oloss = oracle.F.mean(oracle.F.mul(od, od))
        osc.scale_loss(oloss).backward()
        assert osc.step(oopt, [ow, ob]) is True
        assert abs(last - float(oloss.data)) <= 2e-3 * abs(float(oloss.data)) + 1e-6, (step, last, float(oloss.data))
    assert last < first
    assert sc.scale == osc.scale == 1024.0 * 2 ** 4 and sc.growth_tracker == osc.growth_tracker


def test_f16_overflow_makes_the_scaler_back_off(mc, ctx):
    """What f16 autocast needs the GradScaler for: with a loss scale of 2^24 the scaled gradients of a Linear
    exceed 65504 in f16, the inf/nan scan finds them, the step is skipped (parameters bit-identical), the scale
    is halved, and once it is small enough the steps are applied again."""
    rng = np.random.default_rng(5)
    m = mc.Model(ctx, "mlp", [64, 32, 8])
    ps = m.parameters()
    keep = mc.Arena(ctx, ps)
    x = mc.Variable.constant(ctx, rng.standard_normal((16, 64)).astype(np.float32))
    y = mc.Variable.constant(ctx, rng.integers(0, 8, 16).astype(np.int64))
    opt, sc = mc.Adam(ctx, 1e-3), mc.GradScaler(ctx, 2.0 ** 24)
    before = [p.data.copy() for p in ps]
    applied = []
    for _ in range(14):
        mc.zero_grad(ps)
        with mc.autocast(mc.F16):
            loss = m.loss(x, y)
        sc.scale_loss(loss).backward()
        applied.append(sc.step(opt, ps))
        if not any(applied):  # nothing applied so far: every parameter still has its initial bits
            assert all(np.array_equal(a, p.data) for a, p in zip(before, ps))
    assert applied[0] is False and applied[-1] is True
    assert sc.scale == 2.0 ** 24 / 2 ** applied.count(False)  # one halving per skipped step, no growth yet
    del keep
