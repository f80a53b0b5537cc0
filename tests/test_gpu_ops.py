"""GPU parity of every op-level entry point of the C ABI against the CPU oracle, on seeded
inputs, including the literal cases of the reference's own CUDA-vs-CPU tests
(crates/modern-chainer-cuda/tests/cuda.rs:24-108, 563-584, 1314-1390) and ragged / odd sizes.

Tolerances: f32 kernels within 1e-5 relative, norm-wise per tensor (max |d| / max |ref|), the bar
the north star states; Adam and the inf/nan scan bit-exact; bf16-storage kernels within bf16
rounding of the f32 result (2^-8 relative per element)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


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


def close(a, b, tol=1e-5):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.size == 0:
        return
    scale = max(np.abs(b).max(), 1e-30)
    err = np.abs(a - b).max() / scale
    assert err <= tol, f"relative error {err:.3e} > {tol}"


def bf16_close(a, ref):
    a, ref = np.asarray(a, np.float64), np.asarray(ref, np.float64)
    assert np.all(np.abs(a - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-30 + 2.0 ** -7 * np.abs(ref).max() * 1e-2)


RNG = np.random.default_rng(1234)


def randn(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("shapes", [((2, 3), (2, 3)), ((2, 3), (3,)), ((5, 1, 4), (3, 1)), ((7,), ()), ((), (4, 5)),
                                    ((1031, 517), (1031, 517)), ((64, 768), (768,)), ((3, 1, 5), (1, 4, 1))])
@pytest.mark.parametrize("op", [0, 1, 2, 3])
def test_binary_broadcast(ops, oracle, shapes, op):
    a, b = randn(*shapes[0]), randn(*shapes[1]) + (3.0 if op == 3 else 0.0)
    assert np.array_equal(ops.binary(op, a, b), oracle.binary(op, a, b))


def test_binary_rejects_bad_broadcast(mc, ops):
    with pytest.raises(mc.McbError) as e:
        ops.binary(0, randn(2, 3), randn(4))
    assert e.value.status == 2


def test_reference_core_literals(ops, oracle):
    a = np.array([0.5, -1.0, 2.0, 3.0, -0.5, 0.25], np.float32).reshape(2, 3)
    b = np.array([1.5, 0.5, -2.0, 0.25, 4.0, -1.0], np.float32).reshape(2, 3)
    assert np.array_equal(ops.binary(0, a, b), oracle.add(a, b))
    assert np.array_equal(ops.binary(2, a, b), oracle.mul(a, b))
    assert np.array_equal(ops.relu(a), oracle.relu(a))
    assert np.array_equal(ops.scale(a, -2.5), oracle.scale(a, -2.5))
    m = (np.arange(35, dtype=np.float32) * np.float32(0.1) - np.float32(1.0)).reshape(5, 7)
    n = (np.float32(1.0) - np.arange(21, dtype=np.float32) * np.float32(0.07)).reshape(7, 3)
    close(ops.matmul(m, n), oracle.matmul(m, n))
    x = np.arange(1, 9, dtype=np.float32).reshape(4, 2)
    w = np.sin(np.arange(6, dtype=np.float32) * np.float32(0.13)).reshape(3, 2)
    bias = np.array([0.1, -0.2, 0.3], np.float32)
    close(ops.linear(x, w, bias), oracle.linear(x, w, bias))
    assert abs(float(ops.sum_all(x)) - 36.0) < 1e-4
    assert np.array_equal(ops.sum_to(x, (2,)), oracle.sum_to(x, (2,)))
    logits = (np.arange(12, dtype=np.float32) * np.float32(0.1) - np.float32(0.5)).reshape(4, 3)
    lab = np.array([0, 1, 2, 1], np.int64)
    assert abs(float(ops.softmax_cross_entropy(logits, lab)) - float(oracle.softmax_cross_entropy(logits, lab))) < 1e-6


@pytest.mark.parametrize("n", [1, 3, 4, 1000, 32768 + 5, 1 << 20])
def test_activations_f32(ops, oracle, n):
    x, g = randn(n) * 2, randn(n)
    x[: min(n, 3)] = [0.0, -0.0, np.nan][: min(n, 3)]
    assert np.array_equal(ops.relu(x), oracle.relu(x))
    assert np.array_equal(ops.relu_backward(x, g), oracle.relu_backward(x, g))
    x = np.nan_to_num(x)
    close(ops.gelu(x), oracle.gelu(x), 1e-6)
    close(ops.gelu_backward(x, g), oracle.gelu_backward(x, g), 1e-5)


def test_gelu_backward_stays_finite_where_reference_overflows(ops, oracle):
    # the reference composes tanh from exp(-2c): NaN below x ~ -10.05; the fused kernel is finite there
    x = np.array([-12.0, -10.5, 10.5], np.float32)
    assert np.isnan(oracle.gelu_backward(x, np.ones(3, np.float32))[:2]).all()
    out = ops.gelu_backward(x, np.ones(3, np.float32))
    assert np.isfinite(out).all() and abs(out[2] - 1.0) < 1e-6 and abs(out[0]) < 1e-6


def test_activations_bf16_storage(ops, oracle):
    x, g = oracle.round_bf16(randn(4099) * 2), oracle.round_bf16(randn(4099))
    bf16_close(ops.gelu(x, dt=5), oracle.gelu(x))
    bf16_close(ops.gelu_backward(x, g, dt=5), oracle.gelu_backward(x, g))
    assert np.array_equal(ops.relu_backward(x, g, dt=5), oracle.relu_backward(x, g))


def test_unary_and_scale(ops, oracle):
    x = np.abs(randn(1001)) + 0.1
    for op in range(7):
        close(ops.unary(op, x), oracle.unary(op, x), 1e-6)
    assert np.array_equal(ops.scale(x, 1.0 / 3.0), oracle.scale(x, 1.0 / 3.0))


def test_cast_is_round_to_nearest_even(mc, ops, oracle):
    x = np.concatenate([randn(5001) * 100, np.array([1.00390625, 1.005859375, 65504.0, 1e-40, np.inf, -np.inf], np.float32)])
    assert np.array_equal(ops.cast(x, 0, 5).numpy(), oracle.round_bf16(x))
    import torch
    assert np.array_equal(ops.cast(x, 0, 4).numpy(), torch.from_numpy(x).half().numpy())


def test_add_inplace(ops, oracle):
    a, b = randn(10007), randn(10007)
    assert np.array_equal(ops.add_inplace(a, b), a + b)


# ------------------------------------------------------------------ reductions
@pytest.mark.parametrize("n", [1, 7, 4096, 1 << 20, (1 << 21) + 3])
def test_sum_all(ops, oracle, n):
    x = randn(n)
    close(float(ops.sum_all(x)), float(oracle.sum_all(x)), 1e-6 + 1e-6 * np.sqrt(n) * 1e-2)


@pytest.mark.parametrize("src,dst", [((4, 2), (2,)), ((8192, 768), (768,)), ((3, 4, 5), (4, 5)), ((3, 4, 5), (1, 5)), ((3, 4, 5), (5,)),
                                     ((6, 7), (6, 1)), ((2, 3), (2, 3)), ((9, 5), (1,)), ((2, 3, 4), (1, 1, 1))])
def test_sum_to(ops, oracle, src, dst):
    a = randn(*src)
    close(ops.sum_to(a, dst), oracle.sum_to(a, dst), 1e-5)


def test_col_sum_bf16(ops, oracle):
    a = oracle.round_bf16(randn(1000, 96))
    close(ops.col_sum(a, dt=5), a.astype(np.float64).sum(0), 1e-5)


# widths on both sides of each kernel choice: a warp per row up to 1024 columns, a block per row while the row fits
# shared memory, three sweeps beyond; multiples of four (128-bit loads) and not; a last block with idle warps
@pytest.mark.parametrize("rows,cols", [(2, 3), (1, 1), (7, 129), (64, 1000), (13, 1023), (9, 1024), (3, 1025), (5, 5000), (4, 6144),
                                       (3, 6145), (2, 12288), (2, 13001), (4099, 64)])
def test_softmax_and_backward(ops, oracle, rows, cols):
    x, g = randn(rows, cols) * 3, randn(rows, cols)
    y = ops.softmax(x)
    close(y, oracle.softmax(x))
    close(ops.softmax_backward(x, g), oracle.softmax_backward(x, g))
    close(ops.softmax_backward_from_output(y, g), oracle.softmax_backward(x, g))


def test_reference_backward_literals(ops, oracle):
    x = np.array([0.2, -0.4, 0.7, 0.1, 0.3, -0.2], np.float32).reshape(2, 3)
    gam = np.array([1.0, 0.9, 1.1], np.float32)
    g = np.array([0.3, -0.2, 0.4, 0.1, 0.5, -0.1], np.float32).reshape(2, 3)
    for a, b in zip(ops.layer_norm_backward(x, gam, g, 1e-5), oracle.layer_norm_backward(x, gam, g, 1e-5)):
        assert np.abs(a - b).max() < 1e-5  # the reference's own bar (cuda.rs:1342-1389)
    assert np.abs(ops.softmax_backward(x, g) - oracle.softmax_backward(x, g)).max() < 1e-5
    ids = np.array([0, 2, 0], np.int64)
    eg = np.array([0.2, 0.1, -0.4, 0.3, 0.5, -0.2], np.float32).reshape(3, 2)
    assert np.abs(ops.embedding_backward(ids, (3, 2), eg) - oracle.embedding_backward(ids, (3, 2), eg)).max() < 1e-5


@pytest.mark.parametrize("rows,dim", [(2, 3), (1, 1), (33, 768), (257, 512), (5, 1023), (3, 4100)])
def test_layer_norm_forward_backward(ops, oracle, rows, dim):
    x, g = randn(rows, dim) * 2 + 0.5, randn(rows, dim)
    gam, bet = randn(dim) * 0.2 + 1, randn(dim) * 0.1
    y, mean, rstd = ops.layer_norm(x, gam, bet, 1e-5, with_stats=True)
    close(y, oracle.layer_norm(x, gam, bet, 1e-5))
    ref = oracle.layer_norm_backward(x, gam, g, 1e-5)
    for a, b in zip(ops.layer_norm_backward(x, gam, g, 1e-5), ref):
        close(a, b, 2e-5)
    for a, b in zip(ops.layer_norm_backward(x, gam, g, 1e-5, stats=(mean, rstd)), ref):
        close(a, b, 2e-5)


@pytest.mark.parametrize("rows,dim", [(1500, 128), (1189, 768), (2051, 1000), (1300, 1024)])
def test_layer_norm_pipeline_kernels(ops, oracle, rows, dim):
    """From 8 x 148 rows on (dim % 8 == 0, dim <= 1024) LayerNorm is a persistent bulk-copy pipeline:
    ragged last row block, f32 and bf16 in/out, statistics given or recomputed."""
    x, g = randn(rows, dim) * 2 + 0.5, randn(rows, dim)
    gam, bet = randn(dim) * 0.2 + 1, randn(dim) * 0.1
    y, mean, rstd = ops.layer_norm(x, gam, bet, 1e-5, with_stats=True)
    want = oracle.layer_norm(x, gam, bet, 1e-5)
    close(y, want)
    bf16_close(ops.layer_norm(x, gam, bet, 1e-5, out_dt=5), want)
    ref = oracle.layer_norm_backward(x, gam, g, 1e-5)
    for a, b in zip(ops.layer_norm_backward(x, gam, g, 1e-5), ref):
        close(a, b, 2e-5)
    for a, b in zip(ops.layer_norm_backward(x, gam, g, 1e-5, stats=(mean, rstd)), ref):
        close(a, b, 2e-5)
    gb = oracle.round_bf16(g)
    for a, b in zip(ops.layer_norm_backward(x, gam, gb, 1e-5, g_dt=5, stats=(mean, rstd)), oracle.layer_norm_backward(x, gam, gb, 1e-5)):
        close(a, b, 2e-5)


def test_layer_norm_bf16_io(ops, oracle):
    x, g = randn(64, 768), oracle.round_bf16(randn(64, 768))
    gam, bet = np.ones(768, np.float32), np.zeros(768, np.float32)
    bf16_close(ops.layer_norm(x, gam, bet, 1e-5, out_dt=5), oracle.layer_norm(x, gam, bet, 1e-5))
    for a, b in zip(ops.layer_norm_backward(x, gam, g, 1e-5, g_dt=5), oracle.layer_norm_backward(x, gam, g, 1e-5)):
        close(a, b, 2e-5)


@pytest.mark.parametrize("n,c", [(4, 3), (1, 1), (128, 10), (37, 1000), (16, 32000)])
@pytest.mark.parametrize("ldt", [np.int64, np.int32, np.uint8])
def test_softmax_cross_entropy(ops, oracle, n, c, ldt):
    x = randn(n, c) * 2
    lab = RNG.integers(0, min(c, 200), n).astype(ldt)
    close(float(ops.softmax_cross_entropy(x, lab)), float(oracle.softmax_cross_entropy(x, lab)), 1e-6)
    ref = oracle.softmax_cross_entropy_backward(x, lab)
    close(ops.softmax_cross_entropy_backward(x, lab), ref)
    loss, grad = ops.softmax_ce_fused(x, lab, upstream=1024.0)
    close(float(loss), float(oracle.softmax_cross_entropy(x, lab)), 1e-6)
    close(grad, oracle.scale(ref, 1024.0))


def test_softmax_cross_entropy_bf16_logits(ops, oracle):
    x = oracle.round_bf16(randn(32, 4096) * 2)
    lab = RNG.integers(0, 4096, 32).astype(np.int64)
    loss, grad = ops.softmax_ce_fused(x, lab, dt=5)
    close(float(loss), float(oracle.softmax_cross_entropy(x, lab)), 1e-6)
    ref = oracle.softmax_cross_entropy_backward(x, lab)
    assert np.abs(grad - ref).max() <= np.abs(ref).max() * 2.0 ** -8


@pytest.mark.parametrize("bad", [np.array([0, 3], np.int64), np.array([-1, 0], np.int64), np.array([0, -5], np.int32)])
def test_label_range_errors_match_cpu_rules(mc, ctx, ops, oracle, bad):
    x = np.zeros((2, 3), np.float32)
    with pytest.raises(oracle.OracleError) as eo:
        oracle.softmax_cross_entropy_backward(x, bad)
    for fn in (ops.softmax_cross_entropy_backward, ops.softmax_cross_entropy, lambda a, b: ops.softmax_ce_fused(a, b)):
        with pytest.raises(mc.McbError) as e:
            fn(x, bad)
        assert e.value.status == eo.value.status == 5
    # the context stays usable and the error word is cleared
    assert np.array_equal(ops.relu(np.array([1.0, -1.0], np.float32)), [1.0, 0.0])
    with pytest.raises(mc.McbError) as e:
        ops.softmax_cross_entropy(x, np.array([0.0, 1.0], np.float32))
    assert e.value.status == 4  # UnsupportedDType, like target_indices


def test_empty_batch(ops):
    assert float(ops.softmax_cross_entropy(np.zeros((0, 3), np.float32), np.zeros(0, np.int64))) == 0.0


@pytest.mark.parametrize("idt", [np.int64, np.int32, np.uint8])
def test_embedding(mc, ops, oracle, idt):
    w = randn(200, 96)
    ids = RNG.integers(0, 200, (4, 37)).astype(idt)
    assert np.array_equal(ops.embedding(ids, w), oracle.embedding(ids, w))
    g = randn(4 * 37, 96)
    close(ops.embedding_backward(ids.reshape(-1), (200, 96), g), oracle.embedding_backward(ids.reshape(-1), (200, 96), g))
    w2 = randn(7, 5)  # dim not a multiple of 4: scalar path
    ids2 = np.array([6, 0, 6, 6], idt)
    assert np.array_equal(ops.embedding(ids2, w2), oracle.embedding(ids2, w2))
    if idt != np.uint8:
        with pytest.raises(mc.McbError) as e:
            ops.embedding(np.array([0, 7], idt), w2)
        assert e.value.status == 5
        with pytest.raises(mc.McbError):
            ops.embedding_backward(np.array([-1], idt), (7, 5), randn(1, 5))


# ------------------------------------------------------------------ GEMM family (exact f32 path)
@pytest.mark.parametrize("m,k,n", [(5, 7, 3), (1, 1, 1), (128, 784, 100), (128, 100, 10), (65, 130, 67), (256, 4096, 10)])
def test_linear_family_f32(ops, oracle, m, k, n):
    x, w, b, g = randn(m, k), randn(n, k) * 0.1, randn(n), randn(m, n)
    close(ops.linear(x, w, b), oracle.linear(x, w, b))
    close(ops.linear(x, w, None), oracle.linear(x, w, None))
    close(ops.matmul(x, np.ascontiguousarray(w.T)), oracle.matmul(x, np.ascontiguousarray(w.T)))
    for a, r in zip(ops.linear_backward(g, x, w), oracle.linear_backward(g, x, w)):
        close(a, r)


def test_linear_activation_f32(ops, oracle):
    x, w, b = randn(33, 20), randn(12, 20), randn(12)
    close(ops.linear(x, w, b, act=1), oracle.relu(oracle.linear(x, w, b)))
    close(ops.linear(x, w, b, act=2), oracle.gelu(oracle.linear(x, w, b)), 2e-5)


# ------------------------------------------------------------------ tensor-core GEMM
def gemm_ref(oracle, a, a_mn, b, b_mn):
    A = oracle.round_bf16(a).astype(np.float64)
    B = oracle.round_bf16(b).astype(np.float64)
    A = A.T if a_mn else A          # -> [M, K]
    B = B if b_mn else B.T          # -> [K, N]
    return A @ B


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 128), (256, 512, 512), (8, 8, 8), (136, 72, 200), (1000, 776, 328),
                                   (2048, 768, 768), (512, 2304, 768)])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
def test_tc_gemm_layouts(ops, oracle, m, n, k, a_mn, b_mn):
    a = randn(k, m) if a_mn else randn(m, k)
    b = randn(k, n) if b_mn else randn(n, k)
    ref = gemm_ref(oracle, a, a_mn, b, b_mn)
    out = ops.gemm_bf16(a, a_mn, b, b_mn, m, n, k, out_dt=0)
    close(out, ref, 2e-5)  # exact bf16 products, f32 accumulation in TMEM
    out16 = ops.gemm_bf16(a, a_mn, b, b_mn, m, n, k, out_dt=5)
    assert np.abs(out16 - ref).max() <= np.abs(ref).max() * 2.0 ** -8


@pytest.mark.parametrize("m,n,k,a_mn,b_mn", [(8192, 768, 1024, 0, 0), (8100, 760, 1000, 0, 1), (8192, 768, 640, 1, 1)])
def test_tc_gemm_split_tail(ops, oracle, m, n, k, a_mn, b_mn):
    """96 tiles of 256 x 256 on 74 CTA pairs: the 22 tiles of the second wave are cut into K slices whose
    f32 partial sums meet in a workspace, and a finishing kernel adds the bias and writes the output
    (MCB_TC_SPLIT_TAIL=1 forces that form, =0 forbids it).  Both forms against the f64 product."""
    import os
    a = randn(k, m) if a_mn else randn(m, k)
    b = randn(k, n) if b_mn else randn(n, k)
    bias = randn(n)
    ref = gemm_ref(oracle, a, a_mn, b, b_mn) + bias
    outs = {}
    try:
        for knob in ("1", "0"):
            ops.ctx.set_knob("MCB_TC_SPLIT_TAIL", int(knob))
            out = ops.gemm_bf16(a, a_mn, b, b_mn, m, n, k, out_dt=0, bias=bias)
            close(out, ref, 2e-5)
            out16 = ops.gemm_bf16(a, a_mn, b, b_mn, m, n, k, out_dt=5, bias=bias)
            assert np.abs(out16 - ref).max() <= np.abs(ref).max() * 2.0 ** -8
            outs[knob] = (out, out16)
            # accumulating f32 output (weight-gradient form): the slices add straight into it
            init = randn(m, n)
            close(ops.gemm_bf16(a, a_mn, b, b_mn, m, n, k, out_dt=0, accumulate=True, split_k=1, init=init), ref - bias + init, 2e-5)
    finally:
        ops.ctx.set_knob("MCB_TC_SPLIT_TAIL", None)
    close(outs["1"][0], outs["0"][0], 2e-6)  # same products, another grouping of the f32 sums


def test_tc_gemm_bias_accumulate_splitk(ops, oracle):
    m, n, k = 768, 768, 4096
    a, b, bias = randn(k, m), randn(k, n), randn(n)  # weight-gradient shape: both operands MN-major
    ref = gemm_ref(oracle, a, 1, b, 1)
    close(ops.gemm_bf16(a, 1, b, 1, m, n, k, out_dt=0, bias=bias), ref + bias, 2e-5)
    init = randn(m, n)
    close(ops.gemm_bf16(a, 1, b, 1, m, n, k, out_dt=0, accumulate=True, split_k=8, init=init), ref + init, 2e-5)
    close(ops.gemm_bf16(a, 1, b, 1, m, n, k, out_dt=0, accumulate=True, split_k=1, init=init), ref + init, 2e-5)


def test_tc_gemm_rejects_unaligned(mc, ops):
    with pytest.raises(mc.McbError) as e:
        ops.gemm_bf16(randn(16, 12), 0, randn(16, 12), 0, 16, 16, 12)
    assert e.value.status == 5


# ------------------------------------------------------------------ attention / conv
@pytest.mark.parametrize("n,s,d,h,causal", [(1, 2, 2, 1, True), (2, 17, 24, 3, False), (2, 64, 128, 2, True), (1, 130, 64, 1, True)])
def test_attention_f32(ops, oracle, n, s, d, h, causal):
    q, k, v, g = randn(n, s, d), randn(n, s, d), randn(n, s, d), randn(n, s, d)
    out, _ = ops.attention(q, k, v, h, causal)
    close(out, oracle.attention(q, k, v, h, causal))
    for a, r in zip(ops.attention_backward(q, k, v, g, h, causal), oracle.attention_backward(q, k, v, g, h, causal)):
        close(a, r, 2e-5)


def test_attention_bf16_storage(ops, oracle):
    q, k, v, g = (oracle.round_bf16(randn(2, 128, 128)) for _ in range(4))
    out, _ = ops.attention(q, k, v, 2, True, dt=5)
    ref = oracle.attention(q, k, v, 2, True)
    assert np.abs(out - ref).max() <= np.abs(ref).max() * 2.0 ** -7
    for a, r in zip(ops.attention_backward(q, k, v, g, 2, True, dt=5), oracle.attention_backward(q, k, v, g, 2, True)):
        assert np.abs(a - r).max() <= np.abs(r).max() * 2.0 ** -6


@pytest.mark.parametrize("n,s,h,causal", [(1, 64, 1, True), (2, 256, 3, True), (2, 256, 3, False), (1, 100, 2, True), (3, 130, 1, False),
                                          (1, 1, 1, True), (1, 1024, 2, True)])
def test_fused_attention_bf16_head_dim_64(ops, oracle, n, s, h, causal):
    d = 64 * h
    q, k, v, g = (oracle.round_bf16(randn(n, s, d)) for _ in range(4))
    out, lse = ops.attention(q, k, v, h, causal, dt=5)
    ref = oracle.attention(q, k, v, h, causal)
    assert np.abs(out - ref).max() <= max(np.abs(ref).max(), 1e-3) * 2.0 ** -7
    # log-sum-exp of the scaled scores, per (sample, head, query)
    sc = np.einsum("nqhd,nkhd->nhqk", q.reshape(n, s, h, 64).astype(np.float64), k.reshape(n, s, h, 64).astype(np.float64)) / 8.0
    if causal:
        sc = np.where(np.tril(np.ones((s, s), bool)), sc, -np.inf)
    ref_lse = np.log(np.exp(sc - sc.max(-1, keepdims=True)).sum(-1)) + sc.max(-1)
    assert np.abs(lse - ref_lse).max() <= 2e-3
    for a, r in zip(ops.attention_backward(q, k, v, g, h, causal, dt=5), oracle.attention_backward(q, k, v, g, h, causal)):
        assert np.abs(a - r).max() <= max(np.abs(r).max(), 1e-3) * 2.0 ** -6, np.abs(a - r).max() / np.abs(r).max()


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("n,s,h,causal", [(1, 64, 1, True), (2, 256, 3, True), (2, 256, 3, False), (1, 100, 2, True), (3, 130, 1, False),
                                          (1, 1024, 2, True), (2, 700, 2, True), (4, 1024, 5, True), (5, 640, 6, False)])
def test_fused_attention_dq_from_stored_ds_equals_recomputed(ops, oracle, n, s, h, causal, dt):
    """dQ is taken from the dS tiles the dK/dV kernel leaves (one bulk copy of its shared-memory tile per pair of
    tiles); MCB_FLASH_DQ_RECOMPUTE keeps the kernel that evaluates S, dP and dS a second time.  Both multiply the same
    rounded dS by the same K in the same order: identical bits; dK and dV must not notice the copies either.  The last
    two cases have more jobs (tiles x samples x heads: 160 and 150) than the GPU has SMs, so the persistent CTAs of both
    tile-pair kernels walk several jobs each; MCB_FLASH_BWD_ONE_JOB (one CTA per job) must give the same bits again."""
    import modernchainer_b200 as mc
    d = 64 * h
    code = mc.BF16 if dt == "bf16" else mc.F16
    rnd = oracle.round_bf16 if dt == "bf16" else oracle.round_f16
    q, k, v, g = (rnd(randn(n, s, d)) for _ in range(4))
    got = ops.attention_backward(q, k, v, g, h, causal, dt=code)
    with ops.ctx.knob("MCB_FLASH_DQ_RECOMPUTE"):
        ref = ops.attention_backward(q, k, v, g, h, causal, dt=code)
        with ops.ctx.knob("MCB_FLASH_BWD_ONE_JOB"):
            one = ops.attention_backward(q, k, v, g, h, causal, dt=code)
    for a, r, o in zip(got, ref, one):
        assert np.array_equal(a, r) and np.array_equal(a, o)


@pytest.mark.parametrize("shape,wshape,stride,pad", [((1, 2, 3, 3), (2, 2, 2, 2), 1, 0), ((4, 3, 32, 32), (8, 3, 3, 3), 1, 1),
                                                     ((2, 5, 9, 7), (4, 5, 3, 3), 2, 1)])
def test_conv2d(ops, oracle, shape, wshape, stride, pad):
    x, w, b = randn(*shape), randn(*wshape) * 0.3, randn(wshape[0])
    y = oracle.conv2d(x, w, b, stride, pad)
    close(ops.conv2d(x, w, b, stride, pad), y)
    g = randn(*y.shape)
    for a, r in zip(ops.conv2d_backward(x, w, g, stride, pad), oracle.conv2d_backward(x, w, g, stride, pad)):
        close(a, r, 2e-5)


@pytest.mark.parametrize("shape,wshape,stride,pad", [((32, 16, 16, 16), (32, 16, 3, 3), 1, 1), ((64, 8, 33, 31), (16, 8, 3, 3), 2, 1),
                                                     ((16, 4, 24, 24), (24, 4, 5, 5), 1, 2)])
def test_conv2d_tensor_core_path(ops, oracle, shape, wshape, stride, pad):
    """From about 2^24 multiply-adds on, convolution runs as a column matrix and tensor-core GEMMs over f16 hi / lo
    pieces of the f32 operands (three GEMMs per product: exact f16 products, f32 accumulation, the dropped lo x lo
    term is 2^-22 of the result).  Against the oracle at the f32 bar, and against the direct f32 kernels
    (MCB_CONV_DIRECT) much closer than that; strides, paddings, a 5x5 kernel whose column count (100) is padded to 104."""
    import os
    x, w, b = randn(*shape), randn(*wshape) * 0.2, randn(wshape[0])
    out = ops.conv2d(x, w, b, stride, pad)
    g = randn(*out.shape)
    with oracle.threaded():
        close(out, oracle.conv2d(x, w, b, stride, pad), 1e-5)
        ref = oracle.conv2d_backward(x, w, g, stride, pad)
    got = ops.conv2d_backward(x, w, g, stride, pad)
    for a, r in zip(got, ref):
        close(a, r, 1e-5)
    ops.ctx.set_knob("MCB_CONV_DIRECT", 1)
    try:
        close(out, ops.conv2d(x, w, b, stride, pad), 2e-6)
        for a, r in zip(got, ops.conv2d_backward(x, w, g, stride, pad)):
            close(a, r, 2e-6)
    finally:
        ops.ctx.set_knob("MCB_CONV_DIRECT", None)


def test_max_pool_tie_rule(ops, oracle):
    x = randn(3, 4, 8, 8)
    x[0, 0, 0:2, 0:2] = 1.5   # four equal maxima: first of each window row gets the gradient
    x[1, 1, 2, 2] = x[1, 1, 3, 3] = 9.0
    y = oracle.max_pool2d(x, 2, 2, 0)
    assert np.array_equal(ops.max_pool2d(x, 2, 2, 0), y)
    g = randn(*y.shape)
    assert np.array_equal(ops.max_pool2d_backward(x, g, 2, 2, 0), oracle.max_pool2d_backward(x, g, 2, 2, 0))
    y3 = oracle.max_pool2d(x, 3, 1, 1)
    assert np.array_equal(ops.max_pool2d(x, 3, 1, 1), y3)
    close(ops.max_pool2d_backward(x, randn(*y3.shape) * 0 + 1, 3, 1, 1), oracle.max_pool2d_backward(x, np.ones_like(y3), 3, 1, 1))


# ------------------------------------------------------------------ optimizer
def test_adam_bit_exact(ops, oracle):
    n = 100003
    p, g, m, v = randn(n) * 0.02, randn(n) * 1e-3, randn(n) * 1e-4, np.abs(randn(n)) * 1e-6
    for step in (1, 2, 7, 1000):
        ref = oracle.adam_update(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, step)
        for a, r in zip(ops.adam_update(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, step), ref):
            assert np.array_equal(a, r)
        fp, fm, fv, _ = ops.adam_flat(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, step)
        assert np.array_equal(fp, ref[0]) and np.array_equal(fm, ref[1]) and np.array_equal(fv, ref[2])
    lit = oracle.adam_update(np.full(1024, 0.1, np.float32), np.full(1024, 0.01, np.float32), np.zeros(1024), np.zeros(1024), 0.001, 0.9, 0.999, 1e-8, 1)
    got = ops.adam_update(np.full(1024, 0.1, np.float32), np.full(1024, 0.01, np.float32), np.zeros(1024), np.zeros(1024), 0.001, 0.9, 0.999, 1e-8, 1)
    assert all(np.array_equal(a, b) for a, b in zip(got, lit))


def test_adam_flat_unscale_shadow_skip(mc, ops, oracle):
    n = 65536 + 17
    p, m, v = randn(n) * 0.02, np.zeros(n, np.float32), np.zeros(n, np.float32)
    g = randn(n) * 1e-3
    scale = 65536.0
    gs = oracle.f32_to_bf16_bits(g * np.float32(scale))            # bf16 grads stored pre-multiplied by the loss scale
    unscaled = oracle.scale(oracle.bf16_bits_to_f32(gs), 1.0 / scale)
    ref = oracle.adam_update(p, unscaled, m, v, 1e-3, 0.9, 0.999, 1e-8, 1)
    fp, fm, fv, sh = ops.adam_flat(p, gs, m, v, 1e-3, 0.9, 0.999, 1e-8, 1, inv_scale=1.0 / scale, g_dt=5, shadow=True)
    assert np.array_equal(fp, ref[0]) and np.array_equal(fm, ref[1]) and np.array_equal(fv, ref[2])
    assert np.array_equal(sh, oracle.round_bf16(ref[0]))
    sp, sm, sv, _ = ops.adam_flat(p, gs, m, v, 1e-3, 0.9, 0.999, 1e-8, 1, inv_scale=1.0 / scale, g_dt=5, skip=1)
    assert np.array_equal(sp, p) and np.array_equal(sm, m) and np.array_equal(sv, v)  # skipped step: bit-exact no-op


@pytest.mark.parametrize("n", [1, 5, 4096, 1000003])
def test_check_finite_bit_exact(ops, oracle, n):
    g = randn(n)
    assert ops.check_finite(g) == 0 == (oracle.count_non_finite(g) > 0)
    for val in (np.inf, -np.inf, np.nan):
        for pos in {0, n - 1, n // 2}:
            h = g.copy()
            h[pos] = val
            assert ops.check_finite(h) == 1
            hb = oracle.f32_to_bf16_bits(h)
            hb[pos] = {np.inf: 0x7F80, -np.inf: 0xFF80}.get(val, 0x7FC0)
            assert ops.check_finite(hb, g_dt=5) == 1
    assert ops.check_finite(oracle.f32_to_bf16_bits(g), g_dt=5) == 0
    assert ops.check_finite(np.array([3.3e38, -3.3e38, 1e-45], np.float32)) == 0
