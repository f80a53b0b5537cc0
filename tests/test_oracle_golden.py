"""Pins the CPU oracle against every literal the reference's own tests hold for the
training-step path, and re-runs the reference's central-difference gradcheck
(same inputs, eps 1e-3, rtol 1e-3, atol 1e-4) on the oracle's backward formulas.

Sources of the literals (paths relative to the reference project root):
  crates/modern-chainer-cpu/tests/linear.rs:4-13
  crates/modern-chainer-cpu/tests/paged_attention.rs:121-136
  crates/modern-chainer-cuda/tests/cuda.rs:24-108, 563-584, 1314-1390
  crates/modern-chainer-autograd/tests/gradcheck.rs (all cases on the path)
  crates/modern-chainer-optim/tests/amp.rs:14-66, optimizer.rs:8-56
  crates/modern-chainer-core/src/rng.rs:69-87, init.rs:16-29
"""
import math

import numpy as np
import pytest


def gradcheck(ref, f, inputs, eps=1e-3, rtol=1e-3, atol=1e-4):
    """crates/modern-chainer-autograd/src/gradcheck.rs:10-98."""
    for v in inputs:
        v.cleargrad()
    f(inputs).backward()
    for idx, v in enumerate(inputs):
        if not v.requires_grad:
            continue
        analytic = np.zeros(v.data.size, np.float32) if v.grad is None else v.grad.reshape(-1)
        base = v.data.reshape(-1)
        for e in range(base.size):
            def ev(delta):
                d = base.copy()
                d[e] = np.float32(d[e] + np.float32(delta))
                args = list(inputs)
                args[idx] = ref.Variable(d.reshape(v.data.shape))
                with ref.no_grad():
                    return float(f(args).data.reshape(-1)[0])
            numeric = (ev(eps) - ev(-eps)) / (2.0 * np.float32(eps))
            exp = float(analytic[e])
            sc = max(abs(exp), abs(numeric), 1.0)
            assert abs(exp - numeric) <= atol + rtol * sc, (idx, e, exp, numeric)


def V(ref, data, shape):
    return ref.Variable(np.array(data, np.float32).reshape(shape))


def test_linear_known_value(oracle):
    y = oracle.linear(np.array([[1.0, 2.0]]), np.array([[-1.2074714, 0.9428667]]), np.array([0.0]))
    assert abs(float(y[0, 0]) - 0.678262) < 1e-4


def test_gelu_matches_formula(oracle):
    x = np.array([-1.0, 0.0, 0.5, 2.0], np.float32)
    y = oracle.gelu(x)
    for a, b in zip(x, y):
        exp = 0.5 * a * (1.0 + math.tanh(math.sqrt(2.0 / math.pi) * (a + 0.044715 * a ** 3)))
        assert abs(float(b) - exp) < 1e-5


def test_core_ops_literals(oracle):
    a = np.array([0.5, -1.0, 2.0, 3.0, -0.5, 0.25], np.float32).reshape(2, 3)
    b = np.array([1.5, 0.5, -2.0, 0.25, 4.0, -1.0], np.float32).reshape(2, 3)
    assert np.array_equal(oracle.add(a, b), a + b)
    assert np.array_equal(oracle.mul(a, b), a * b)
    assert np.array_equal(oracle.relu(a), np.maximum(a, 0))
    assert np.array_equal(oracle.scale(a, -2.5), a * np.float32(-2.5))
    m = (np.arange(35, dtype=np.float32) * np.float32(0.1) - np.float32(1.0)).reshape(5, 7)
    n = (np.float32(1.0) - np.arange(21, dtype=np.float32) * np.float32(0.07)).reshape(7, 3)
    assert np.allclose(oracle.matmul(m, n), m.astype(np.float64) @ n.astype(np.float64), atol=1e-5)
    x = np.arange(1, 9, dtype=np.float32).reshape(4, 2)
    assert abs(float(oracle.sum_all(x)) - 36.0) < 1e-4
    assert np.array_equal(oracle.sum_to(x, (2,)), np.array([16.0, 20.0], np.float32))
    logits = (np.arange(12, dtype=np.float32) * np.float32(0.1) - np.float32(0.5)).reshape(4, 3)
    lab = np.array([0, 1, 2, 1], np.int64)
    lse = np.log(np.exp(logits.astype(np.float64)).sum(1))
    exp = float(np.mean(lse - logits[np.arange(4), lab]))
    assert abs(float(oracle.softmax_cross_entropy(logits, lab)) - exp) < 1e-6


def test_adam_literal_step(oracle):
    n = 1024
    p, m, v = oracle.adam_update(np.full(n, 0.1, np.float32), np.full(n, 0.01, np.float32), np.zeros(n), np.zeros(n),
                                 0.001, 0.9, 0.999, 1e-8, 1)
    # first step with zero moments: m = 0.1*g, v = 0.001*g*g, update = lr * sign(g) (up to eps)
    assert np.allclose(m, 0.001, rtol=1e-6) and np.allclose(v, 1e-7, rtol=1e-4)
    assert np.allclose(p, 0.1 - 0.001, atol=1e-6)


def test_backward_literals_vs_closed_form(oracle):
    ids = np.array([0, 2, 0], np.int64)
    g = np.array([0.2, 0.1, -0.4, 0.3, 0.5, -0.2], np.float32).reshape(3, 2)
    dw = oracle.embedding_backward(ids, (3, 2), g)
    assert np.allclose(dw, [[0.7, -0.1], [0, 0], [-0.4, 0.3]], atol=1e-6)
    x = np.array([0.2, -0.4, 0.7, 0.1, 0.3, -0.2], np.float32).reshape(2, 3)
    gam = np.array([1.0, 0.9, 1.1], np.float32)
    gr = np.array([0.3, -0.2, 0.4, 0.1, 0.5, -0.1], np.float32).reshape(2, 3)
    dx, dg, db = oracle.layer_norm_backward(x, gam, gr, 1e-5)
    x64 = x.astype(np.float64)
    mu = x64.mean(1, keepdims=True)
    inv = 1 / np.sqrt(x64.var(1, keepdims=True) + 1e-5)
    xh = (x64 - mu) * inv
    dy = gr * gam
    ref_dx = (dy - dy.mean(1, keepdims=True) - xh * (dy * xh).mean(1, keepdims=True)) * inv
    assert np.allclose(dx, ref_dx, atol=1e-5)
    assert np.allclose(dg, (gr * xh).sum(0), atol=1e-5) and np.allclose(db, gr.sum(0), atol=1e-6)
    p = np.exp(x64) / np.exp(x64).sum(1, keepdims=True)
    assert np.allclose(oracle.softmax_backward(x, gr), p * (gr - (p * gr).sum(1, keepdims=True)), atol=1e-6)


def test_python_api_formulas(oracle):
    # python/tests/test_nn_ops.py:17-45: softmax and layer_norm against NumPy, default_rng(0)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 7)).astype(np.float32)
    e = np.exp(x - x.max(1, keepdims=True))
    assert np.allclose(oracle.softmax(x), e / e.sum(1, keepdims=True), rtol=1e-4)
    g, b = np.ones(7, np.float32), np.zeros(7, np.float32)
    mu, var = x.mean(1, keepdims=True), x.var(1, keepdims=True)
    assert np.allclose(oracle.layer_norm(x, g, b, 1e-5), (x - mu) / np.sqrt(var + 1e-5), rtol=1e-4, atol=1e-5)


def test_rng_and_he_normal(oracle):
    a, b = oracle.Rng(7), oracle.Rng(7)
    assert [a.next_u64() for _ in range(8)] == [b.next_u64() for _ in range(8)]
    assert oracle.Rng(1).next_u64() != oracle.Rng(2).next_u64()
    v = oracle.Rng(42).normal_vec(20000, 0.0, 1.0)
    assert abs(float(v.mean())) < 0.05 and abs(float(v.var()) - 1.0) < 0.05
    w = oracle.he_normal((256, 128), 128, 0)
    assert abs(float(w.std()) - math.sqrt(2.0 / 128)) < 0.01
    assert np.array_equal(w, oracle.he_normal((256, 128), 128, 0))


def test_bf16_rne(oracle):
    x = np.array([1.0, 1.00390625, 1.005859375, 3.14159, -2.5e-3, 65504.0, np.inf], np.float32)
    bits = oracle.f32_to_bf16_bits(x)
    assert bits[0] == 0x3F80 and bits[1] == 0x3F80 and bits[2] == 0x3F81 and bits[-1] == 0x7F80
    import torch
    assert np.array_equal(oracle.round_bf16(x), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_gradients_accumulate_and_tape_semantics(oracle):
    F = oracle.F
    a = V(oracle, [1.0, 2.0], (2,))
    F.sum(a).backward()
    F.sum(F.mul(a, a)).backward()
    assert abs(a.grad[0] - 3.0) < 1e-6 and abs(a.grad[1] - 5.0) < 1e-6
    a.cleargrad()
    assert a.grad is None
    with oracle.no_grad():
        y = F.relu(V(oracle, [1.0, -1.0], (2,)))
    assert y.is_leaf()
    a = V(oracle, [1.0, 2.0], (2,))
    b = F.mul(a, a)
    b.unchain_backward()
    b.backward()
    assert a.grad is None


CASES = {
    "add_broadcast": (lambda F, xs: F.sum(F.add(xs[0], xs[1])),
                      [([0.2, -0.4, 0.1, 0.3, 0.5, -0.2], (2, 3)), ([0.1, 0.2, -0.3], (3,))]),
    "mul": (lambda F, xs: F.sum(F.mul(xs[0], xs[1])), [([0.5, 1.2, -0.7, 0.3], (2, 2)), ([0.4, -0.9, 0.8, 1.1], (2, 2))]),
    "div": (lambda F, xs: F.sum(F.div(xs[0], xs[1])), [([0.5, 1.2, -0.7, 0.3], (2, 2)), ([0.4, -0.9, 0.8, 1.1], (2, 2))]),
    "matmul": (lambda F, xs: F.sum(F.matmul(xs[0], xs[1])),
               [([0.2, -0.1, 0.4, 0.3, 0.2, -0.5], (2, 3)), ([0.1, 0.2, -0.3, 0.4, 0.5, -0.2], (3, 2))]),
    "relu": (lambda F, xs: F.sum(F.relu(xs[0])), [([-0.5, 0.2, 0.7, -1.2], (2, 2))]),
    "sqrt": (lambda F, xs: F.sum(F.sqrt(xs[0])), [([0.25, 0.5, 1.0, 2.0], (4,))]),
    "matmul_relu_chain": (lambda F, xs: F.sum(F.relu(F.add(F.matmul(xs[0], xs[1]), xs[2]))),
                          [([0.2, -0.3, 0.5, 0.1, 0.7, -0.2], (2, 3)), ([0.1, -0.2, 0.3, 0.4, 0.5, -0.6], (3, 2)),
                           ([0.1, -0.1], (2,))]),
    "fused_linear": (lambda F, xs: F.sum(F.linear(xs[0], xs[1], xs[2])),
                     [([0.2, -0.3, 0.5, 0.1, 0.7, -0.2], (2, 3)), ([0.1, -0.2, 0.3, 0.4, 0.5, -0.6], (2, 3)),
                      ([0.1, -0.1], (2,))]),
    "softmax": (lambda F, xs: F.sum(F.softmax(xs[0])), [([0.2, -0.4, 0.7, 0.1, 0.3, -0.2], (2, 3))]),
    "layer_norm": (lambda F, xs: (lambda y: F.sum(F.mul(y, y)))(F.layer_norm(xs[0], xs[1], xs[2], 1e-5)),
                   [([0.2, -0.4, 0.7, 0.1, 0.3, -0.2], (2, 3)), ([1.0, 0.9, 1.1], (3,)), ([0.1, -0.1, 0.0], (3,))]),
    "exp": (lambda F, xs: F.sum(F.exp(xs[0])), [([0.2, -0.1, 0.4, 0.3], (2, 2))]),
    "log": (lambda F, xs: F.sum(F.log(xs[0])), [([0.5, 1.2, 0.7, 2.0], (2, 2))]),
    "sigmoid": (lambda F, xs: F.sum(F.sigmoid(xs[0])), [([0.2, -0.1, 0.4, 0.3], (2, 2))]),
    "gelu": (lambda F, xs: F.sum(F.gelu(xs[0])), [([0.2, -0.3, 0.5, 0.1], (2, 2))]),
    "max_pool": (lambda F, xs: F.sum(F.max_pool2d(xs[0], 2, 2, 0)),
                 [([0.1, 0.2, -0.3, 0.4, 0.5, -0.6, 0.7, 0.8, -0.9, 0.2, -0.1, 0.3, -0.4, 0.5, 0.6, -0.7, 0.8, -0.9],
                   (1, 2, 3, 3))]),
    "conv2d": (lambda F, xs: F.sum(F.conv2d(xs[0], xs[1], xs[2], 1, 0)),
               [([0.1, 0.2, -0.3, 0.4, 0.5, -0.6, 0.7, 0.8, -0.9, 0.2, -0.1, 0.3, -0.4, 0.5, 0.6, -0.7, 0.8, -0.9],
                 (1, 2, 3, 3)),
                ([0.2, -0.1, 0.3, 0.4, -0.2, 0.1, 0.5, -0.3, 0.15, -0.25, 0.35, -0.45, 0.55, -0.65, 0.75, -0.85],
                 (2, 2, 2, 2)), ([0.1, -0.2], (2,))]),
    "reshape": (lambda F, xs: F.sum(F.reshape(xs[0], (3, 2))), [([0.2, -0.1, 0.3, 0.4, -0.5, 0.6], (2, 3))]),
    "attention": (lambda F, xs: (lambda y: F.sum(F.mul(y, y)))(F.multi_head_attention(xs[0], xs[1], xs[2], 1, True)),
                  [([0.2, -0.1, 0.4, 0.3], (1, 2, 2)), ([0.1, 0.2, -0.3, 0.4], (1, 2, 2)),
                   ([0.5, -0.2, 0.3, 0.1], (1, 2, 2))]),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_gradcheck_cases(oracle, name):
    f, ins = CASES[name]
    gradcheck(oracle, lambda xs: f(oracle.F, xs), [V(oracle, d, s) for d, s in ins])


def test_gradcheck_sce_and_embedding(oracle):
    F = oracle.F
    logits = V(oracle, [0.2, 1.3, -0.4, 0.5, -1.0, 0.8], (2, 3))
    target = oracle.Variable.constant(np.array([1, 2], np.int64))
    gradcheck(oracle, lambda xs: F.softmax_cross_entropy(xs[0], xs[1]), [logits, target])
    w = V(oracle, [0.1, 0.2, -0.3, 0.4, 0.5, -0.6], (3, 2))
    ids = oracle.Variable.constant(np.array([0, 2, 0], np.int64))
    gradcheck(oracle, lambda xs: F.sum(F.embedding(xs[0], xs[1])), [ids, w])


def test_grad_scaler_literals(oracle):
    p = V(oracle, [1.0], (1,))
    p.grad = np.array([2048.0], np.float32)
    sc = oracle.GradScaler(1024.0)
    assert sc.step(oracle.SGD(1.0), [p]) is True
    assert abs(float(p.data[0]) + 1.0) < 1e-5 and sc.growth_tracker == 1
    p = V(oracle, [1.0], (1,))
    p.grad = np.array([np.inf], np.float32)
    sc = oracle.GradScaler(1024.0)
    assert sc.step(oracle.SGD(1.0), [p]) is False
    assert sc.scale == 512.0 and p.grad is None and float(p.data[0]) == 1.0
    p = V(oracle, [1.0], (1,))
    p.grad = np.array([0.0], np.float32)
    sc = oracle.GradScaler(1024.0, growth_interval=1)
    assert sc.step(oracle.SGD(1.0), [p]) is True and sc.scale == 2048.0


def test_label_rules(oracle):
    x = np.zeros((2, 3), np.float32)
    for dt in (np.int64, np.int32, np.uint8):
        oracle.softmax_cross_entropy_backward(x, np.array([0, 2], dt))
    for bad in (np.array([0, 3], np.int64), np.array([-1, 0], np.int64)):
        with pytest.raises(oracle.OracleError) as e:
            oracle.softmax_cross_entropy_backward(x, bad)
        assert e.value.status == 5
    with pytest.raises(oracle.OracleError):
        oracle.embedding(np.array([5], np.int64), np.zeros((3, 2), np.float32))
    assert float(oracle.softmax_cross_entropy(np.zeros((0, 3), np.float32), np.zeros(0, np.int64))) == 0.0


def test_adam_fits_linear_regression(oracle):
    F = oracle.F
    model = oracle.Linear(1, 1, 0)
    opt = oracle.Adam(0.05)
    x = oracle.Variable(np.array([[1.0], [2.0], [3.0], [4.0]], np.float32))
    t = oracle.Variable.constant(np.array([[2.0], [4.0], [6.0], [8.0]], np.float32))
    loss = None
    for _ in range(1200):
        d = F.sub(model(x), t)
        loss = F.mean(F.mul(d, d))
        oracle.zero_grad(model.parameters())
        loss.backward()
        opt.update(model.parameters())
        if float(loss.data.reshape(-1)[0]) < 1e-4:
            break
    assert float(loss.data.reshape(-1)[0]) < 1e-2


def test_oracle_transpose_and_permute_follow_the_reference_index_rule():
    """permute_data (autograd/src/host_ops.rs:703-735) restated as a scalar loop on a small tensor:
    the value at source coordinates c lands at output coordinates (c[axes[0]], c[axes[1]], ...);
    the oracle's numpy form must place every element identically, forward and backward."""
    import itertools
    from oracle import ref as oracle
    dims = (2, 3, 4)
    x = np.arange(24, dtype=np.float32).reshape(dims)
    for axes in itertools.permutations(range(3)):
        out_dims = [dims[a] for a in axes]
        want = np.zeros(out_dims, np.float32)
        for c in itertools.product(*[range(d) for d in dims]):
            want[tuple(c[a] for a in axes)] = x[c]
        v = oracle.Variable(x)
        y = oracle.F.permute(v, axes)
        assert np.array_equal(y.data, want)
        up = np.arange(24, dtype=np.float32).reshape(out_dims) * 0.5
        oracle.F.sum(oracle.F.mul(y, oracle.Variable.constant(up))).backward()
        back = np.zeros(dims, np.float32)
        for c in itertools.product(*[range(d) for d in dims]):
            back[c] = up[tuple(c[a] for a in axes)]
        assert np.array_equal(v.grad, back)
    m = oracle.Variable(np.arange(6, dtype=np.float32).reshape(2, 3))
    t = oracle.F.transpose(m)
    assert np.array_equal(t.data, m.data.T) and t.data.flags["C_CONTIGUOUS"]
    with pytest.raises(ValueError):
        oracle.F.transpose(oracle.Variable(x))
    with pytest.raises(ValueError):
        oracle.F.permute(oracle.Variable(x), (0, 1))
    with pytest.raises(ValueError):
        oracle.F.permute(oracle.Variable(x), (0, 0, 1))


def test_oracle_mcn_container_roundtrip_and_byte_layout(tmp_path):
    """crates/modern-chainer-serial/tests/roundtrip.rs with the same two tensors, plus the byte layout
    of serial/src/lib.rs:14-33 spelled out for the first entry."""
    import struct
    from oracle import ref as oracle
    w = np.array([0.1, 0.2, 0.3, 0.4, 0.5, 0.6], np.float32).reshape(2, 3)
    b = np.array([1.0, 2.0], np.float32)
    path = str(tmp_path / "t.mcn")
    oracle.mcn_save(path, [("W", w), ("b", b)])
    loaded = oracle.mcn_load(path)
    assert len(loaded) == 2 and loaded[0][0] == "W" and loaded[0][1].shape == (2, 3) and loaded[0][1].dtype == np.float32
    assert np.array_equal(loaded[0][1], w) and np.array_equal(loaded[1][1], b)
    raw = open(path, "rb").read()
    want = b"MCHN0001" + struct.pack("<I", 2) + struct.pack("<I", 1) + b"W" + bytes([0]) + struct.pack("<I", 2) + \
        struct.pack("<QQ", 2, 3) + struct.pack("<Q", 24) + w.tobytes()
    assert raw[:len(want)] == want
    open(path, "wb").write(b"NOTMCHN1" + raw[8:])
    with pytest.raises(ValueError):
        oracle.mcn_load(path)


def test_threaded_oracle_is_bit_identical(oracle):
    """The "threaded" oracle mode (full-size parity cases) spreads independent loop iterations over host
    cores; every value is produced by the same operations in the same order as in the one-thread checker:
    a decoder step, a >= 1M-MAC GEMM family, attention and the convolution pair, bit for bit."""
    rng = np.random.default_rng(3)

    def run():
        out = []
        m = oracle.Decoder(160, 64, 2, 128, 1, 0)
        ids = np.random.default_rng(1).integers(0, 160, (2, 48)).astype(np.int64)
        loss = m.loss(oracle.Variable.constant(ids), oracle.Variable.constant(ids))
        loss.backward()
        out += [loss.data] + [p.grad for p in m.parameters()]
        x, w, g = (np.random.default_rng(s).standard_normal(sh).astype(np.float32) for s, sh in ((4, (130, 200)), (5, (70, 200)), (6, (130, 70))))
        out += [oracle.linear(x, w), oracle.matmul(x, np.ascontiguousarray(w.T))] + [t for t in oracle.linear_backward(g, x, w) if t is not None]
        xi = np.random.default_rng(7).random((3, 4, 9, 9)).astype(np.float32)
        wc = np.random.default_rng(8).standard_normal((5, 4, 3, 3)).astype(np.float32)
        gc = np.random.default_rng(9).standard_normal((3, 5, 9, 9)).astype(np.float32)
        out += [oracle.conv2d(xi, wc, None, 1, 1)] + list(oracle.conv2d_backward(xi, wc, gc, 1, 1))
        return out

    a = run()
    with oracle.threaded():
        b = run()
    assert len(a) == len(b) and all(np.array_equal(p, q) for p, q in zip(a, b))


def test_f16_conversion_follows_the_reference_rule(oracle):
    """core/src/dtype.rs:75-134.  In the normal range of f16, for overflow, infinities and NaN the reference rule
    is IEEE round-to-nearest-even, so numpy's float16 gives the expected bits; in the subnormal range the
    reference's own bias arithmetic is restated as written (it is close to truncation there), pinned by hand-worked cases."""
    rng = np.random.default_rng(12)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 30, np.array([65504.0, 65519.99, 65520.0, 1e9, -1e9, np.inf, -np.inf, 0.0, -0.0, 1.0009765625,
                                                                                      1.00048828125, 1.00146484375, 6.103515625e-05, 1e-10], np.float32)])
    normal = (np.abs(x) >= 2.0 ** -14) | (x == 0) | (np.abs(x) < 2.0 ** -25)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = oracle.f32_to_f16_bits(x)
    assert np.array_equal(got[normal], want[normal])
    assert np.array_equal(oracle.f16_bits_to_f32(want), want.view(np.float16).astype(np.float32))  # widening is exact
    nan_bits = int(oracle.f32_to_f16_bits(np.array([np.nan], np.float32))[0])
    assert (nan_bits & 0x7c00) == 0x7c00 and (nan_bits & 0x200)  # quiet NaN
    # subnormal results, worked through the reference's arithmetic: m = frac | 0x800000, shift = 14 - h_exp,
    # h = (m + ((m >> (shift - 1)) & 1) + 0xfff) >> shift
    #   2^-15            exp 112, h_exp 0, shift 14, m = 0x800000: bit 13 of m is 0 -> (0x800000 + 0xfff) >> 14 = 0x200
    #   1.5 * 2^-24      exp 103, h_exp -9, shift 23, m = 0xC00000: bit 22 is 1 -> (0xC00000 + 0x1000) >> 23 = 1
    #   1.999 * 2^-24    truncates to 1 as well (IEEE would round it to 2)
    sub = np.array([2.0 ** -15, 1.5 * 2.0 ** -24, 1.999 * 2.0 ** -24], np.float32)
    assert oracle.f32_to_f16_bits(sub).tolist() == [0x200, 1, 1]
    assert float(oracle.round_f16(np.array([2.0 ** -26], np.float32))[0]) == 0.0  # below 2^-25: signed zero


def test_low_precision_oracle_rounds_where_a_16_bit_step_stores(oracle):
    """oracle.amp(): every Linear output is a 16-bit value, GEMM operands are 16-bit values, the result differs
    from the f32 oracle by format error only, and f16 (11 bits) lands about 8 times closer than bf16 (8 bits)."""
    rng = np.random.default_rng(21)
    x = oracle.Variable.constant(rng.standard_normal((2, 16, 32)).astype(np.float32))
    t = oracle.Variable.constant(rng.standard_normal((2, 16, 32)).astype(np.float32))

    def grads(mode):
        m = oracle.EncoderBlock(32, 2, 64)
        if mode is None:
            m.loss(x, t).backward()
        else:
            with oracle.amp(mode):
                y = oracle.F.linear(oracle.Variable.constant(x.data.reshape(32, 32)), m.w1.W, m.w1.b)
                rounded = oracle.round_bf16(y.data) if mode == oracle.BF16 else oracle.round_f16(y.data)
                assert np.array_equal(y.data, rounded)
                oracle.GradScaler(1024.0).scale_loss(m.loss(x, t)).backward()
            for p in m.parameters():
                p.grad = p.grad / np.float32(1024.0)
        return [p.grad for p in m.parameters()]

    f32, b16, h16 = grads(None), grads(oracle.BF16), grads(oracle.F16)
    eb = max(np.abs(a - r).max() / np.abs(r).max() for a, r in zip(b16, f32) if np.abs(r).max() > 1e-6)
    eh = max(np.abs(a - r).max() / np.abs(r).max() for a, r in zip(h16, f32) if np.abs(r).max() > 1e-6)
    assert 1e-4 < eb < 5e-2 and eh < eb / 3


def test_oracle_reproduces_the_committed_step_vectors(oracle):
    """tests/golden/step_vectors.npz was written by the single-threaded oracle (tests/golden/make_step_vectors.py); a
    restatement that drifts shows up here before it moves the target of the GPU tests."""
    import importlib.util
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_step_vectors", os.path.join(here, "golden", "make_step_vectors.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    try:
        vec = mod.run(oracle)
    finally:
        oracle.set_mode("checker")
    old = np.load(mod.OUT)
    assert sorted(old.files) == sorted(vec)
    for k in vec:
        assert np.array_equal(old[k], vec[k]), k
