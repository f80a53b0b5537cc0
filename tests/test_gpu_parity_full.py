"""Parity of whole training steps against the CPU oracle AT THE WIDTHS OF THE BENCHMARK CONFIGURATIONS,
so that the code paths that only engage at scale are compared with the oracle and not with another
GPU path: 256-wide pair tiles and the split tail of the tcgen05 GEMM, the bulk-copy LayerNorm
pipeline (from 8 x 148 rows), the streaming loss gradient over a 32000-wide vocabulary, causal
attention over eight 128-query tiles, the direct convolution at 32x32 images.

The oracle runs in its "threaded" mode: the checker's arithmetic, operation for operation, with
independent loop iterations on several host cores (bit-identical to the one-thread checker, see
tests/test_oracle_golden.py::test_threaded_oracle_is_bit_identical).

Tolerances (norm-wise per tensor, max |d| / max |ref|):
  f32 steps      1e-5, the bar stated for f32.  Where the oracle itself is the limit (it follows the
                 reference's sequential f32 accumulation over 10^4..10^5 terms, whose own rounding error is
                 a few 1e-6 of the result), the test also computes the same sum in f64 and requires the GPU
                 value to be at least as close to the f64 value as the oracle's is, plus 1e-5.
  bf16/f16 AMP   against the low-precision oracle (oracle.amp: same formulas, the tensors a 16-bit path stores in
                 16 bits rounded to nearest even at the same points, same loss scale), per tensor:
                 ||g - o||_2 / ||o||_2 <= 2^-7 AND max |g - o| / max |o| <= 2^-6 for bf16, 2^-9 and 2^-8 for f16 (three
                 more mantissa bits; measured errors are eight times smaller) (the single worst of up to 24.6M
                 elements may be off by one bf16 step of the tensor's peak: on-chip roundings the oracle does not
                 model - attention probabilities and dS in 16 bits, hardware exp2 / tanh - and the order of the
                 f32 sums).  The loss within 2e-3.
  exact-zero gradients (the key-projection bias: softmax is shift invariant) hold only rounding noise on
                 both sides and are compared in absolute terms against the largest gradient of the model.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
AMP_TOL = 2.0 ** -7


@pytest.fixture(scope="module")
def mc():
    import modernchainer_b200 as m
    return m


@pytest.fixture(scope="module")
def ctx(mc):
    c = mc.Context(0)
    yield c
    c.close()


def per_tensor_errors(ggrads, ograds, zero_grad_idx=(), l2=False):
    """max |g - o| / max |o| per tensor (l2: ||g - o||_2 / ||o||_2); the tensors in zero_grad_idx against the
    model's largest gradient (largest l2 norm per element count)."""
    top = max(float(np.abs(o).max()) for o in ograds)
    top_rms = max(float(np.sqrt(np.mean(o.astype(np.float64) ** 2))) for o in ograds)
    errs = []
    for i, (g, o) in enumerate(zip(ggrads, ograds)):
        assert g is not None and g.shape == o.shape, i
        d = g.astype(np.float64) - o
        if l2:
            den = top_rms if i in zero_grad_idx else max(float(np.sqrt(np.mean(o.astype(np.float64) ** 2))), 1e-30)
            errs.append(float(np.sqrt(np.mean(d ** 2))) / den)
        else:
            den = top if i in zero_grad_idx else max(float(np.abs(o).max()), 1e-30)
            errs.append(float(np.abs(d).max()) / den)
    return errs


def check_amp(gg, og, zero_idx, what):
    tol = AMP_TOL if "bf16" in what else AMP_TOL / 4
    report(per_tensor_errors(gg, og, zero_idx, l2=True), tol, what + " (l2)")
    report(per_tensor_errors(gg, og, zero_idx), 2 * tol, what + " (max)")


def gpu_grads(mc, ctx, kind, cfg, x, y, autocast=None, scale=None):
    gm = mc.Model(ctx, kind, cfg)
    ps = gm.parameters()
    keep = mc.Arena(ctx, ps)
    gx, gy = mc.Variable.constant(ctx, x), mc.Variable.constant(ctx, y)
    if autocast is None:
        loss = gm.loss(gx, gy)
        loss.backward()
        grads = [p.grad for p in ps]
    else:
        sc = mc.GradScaler(ctx, scale)
        with mc.autocast(autocast):
            loss = gm.loss(gx, gy)
        sc.scale_loss(loss).backward()
        grads = [p.grad / np.float32(scale) for p in ps]
    out = float(loss.data.reshape(-1)[0]), grads, [p.data.copy() for p in ps]
    del keep
    return out


def oracle_grads(oracle, omodel, x, y, amp=None, scale=None):
    """amp: the 16-bit type of the low-precision oracle; the loss is scaled like the GPU step scales it (f16 gradients
    of an unscaled loss underflow: that is what the GradScaler is for) and the gradients are unscaled afterwards."""
    ox, oy = oracle.Variable.constant(x), oracle.Variable.constant(y)
    with oracle.threaded():
        if amp is None:
            loss = omodel.loss(ox, oy)
            loss.backward()
            grads = [p.grad for p in omodel.parameters()]
        else:
            with oracle.amp(amp):
                loss = omodel.loss(ox, oy)
                oracle.GradScaler(scale).scale_loss(loss).backward()
            grads = [p.grad / np.float32(scale) for p in omodel.parameters()]
    return float(loss.data.reshape(-1)[0]), grads


def decoder_batch(rng, vocab, b, s):
    ids = rng.integers(0, vocab, (b, s)).astype(np.int64)
    tgt = np.concatenate([ids[:, 1:], rng.integers(0, vocab, (b, 1))], 1).astype(np.int64)
    return ids, tgt


def decoder_key_bias(layers):
    # parameter order: tok_emb, then 16 tensors per layer (ln1 g/b, wq bq wk bk wv bv wo bo, ln2 g/b, w1 b1 w2 b2)
    return {1 + 16 * l + 5 for l in range(layers)}


def report(errs, tol, what):
    worst = int(np.argmax(errs))
    print("%s: worst tensor %d %.3e (limit %.3e); all: %s" % (what, worst, errs[worst], tol, ["%.1e" % e for e in errs]))
    assert errs[worst] <= tol, "%s: tensor %d off by %.3e > %.3e; all: %s" % (what, worst, errs[worst], tol, ["%.1e" % e for e in errs])


# ------------------------------------------------------------------ C4: decoder layer + head at d=768 / vocab 32000 / seq 1024
C4 = dict(vocab=32000, d=768, heads=12, ff=3072, seq=1024)


def test_c4_layer_and_head_f32_at_full_width(mc, ctx, oracle):
    """One decoder layer, final LayerNorm and the 32000-wide head with one full 1024-token sequence on
    the exact-f32 kernels: loss and all 20 gradient tensors against the f32 oracle at 1e-5."""
    rng = np.random.default_rng(1240)
    c = C4
    ids, tgt = decoder_batch(rng, c["vocab"], 1, c["seq"])
    cfg = [c["vocab"], c["d"], c["heads"], c["ff"], 1, 0]
    lg, gg, _ = gpu_grads(mc, ctx, "decoder", cfg, ids, tgt)
    lo, og = oracle_grads(oracle, oracle.Decoder(*cfg), ids, tgt)
    assert abs(lg - lo) <= F32_TOL * abs(lo), (lg, lo)
    report(per_tensor_errors(gg, og, decoder_key_bias(1)), F32_TOL, "c4 f32")


@pytest.mark.parametrize("lowp", ["bf16", "f16"])
def test_c4_layer_and_head_amp_at_full_width(mc, ctx, oracle, lowp):
    """The same model under autocast with two sequences (2048 rows: pair-tile GEMMs with the split tail,
    bulk-copy LayerNorm forward and backward with their by-products, packed q/k/v attention over eight
    query tiles, streaming loss gradient) against the low-precision oracle."""
    rng = np.random.default_rng(1241)
    c = C4
    dt = mc.BF16 if lowp == "bf16" else mc.F16
    odt = oracle.BF16 if lowp == "bf16" else oracle.F16
    ids, tgt = decoder_batch(rng, c["vocab"], 2, c["seq"])
    cfg = [c["vocab"], c["d"], c["heads"], c["ff"], 1, 0]
    lg, gg, _ = gpu_grads(mc, ctx, "decoder", cfg, ids, tgt, autocast=dt, scale=65536.0)
    lo, og = oracle_grads(oracle, oracle.Decoder(*cfg), ids, tgt, amp=odt, scale=65536.0)
    assert abs(lg - lo) <= 2e-3 * abs(lo), (lg, lo)
    check_amp(gg, og, decoder_key_bias(1), "c4 " + lowp)


# ------------------------------------------------------------------ C2: encoder block d=512 / 8 heads / ff 2048 / seq 256
def encoder_batch(rng, b, s, d):
    return rng.standard_normal((b, s, d)).astype(np.float32), rng.standard_normal((b, s, d)).astype(np.float32)


ENC_KEY_BIAS = {5}  # ln1 g/b, wq bq wk bk ...


def test_c2_block_f32_at_full_width(mc, ctx, oracle):
    rng = np.random.default_rng(1242)
    x, t = encoder_batch(rng, 8, 256, 512)
    cfg = [512, 8, 2048, 0]
    lg, gg, _ = gpu_grads(mc, ctx, "encoder", cfg, x, t)
    lo, og = oracle_grads(oracle, oracle.EncoderBlock(512, 8, 2048), x, t)
    assert abs(lg - lo) <= F32_TOL * abs(lo), (lg, lo)
    report(per_tensor_errors(gg, og, ENC_KEY_BIAS), F32_TOL, "c2 f32")


@pytest.mark.parametrize("lowp", ["bf16", "f16"])
def test_c2_block_amp_at_full_size(mc, ctx, oracle, lowp):
    """Configuration 2 as stated: batch 32 x seq 256 (8192 rows), GradScaler 2^16 (with it no gradient of this
    step leaves the normal range of f16 either: the largest scaled gradient is of order 1, the smallest that
    matters of order 1e-4)."""
    rng = np.random.default_rng(1243)
    dt = mc.BF16 if lowp == "bf16" else mc.F16
    odt = oracle.BF16 if lowp == "bf16" else oracle.F16
    x, t = encoder_batch(rng, 32, 256, 512)
    cfg = [512, 8, 2048, 0]
    lg, gg, _ = gpu_grads(mc, ctx, "encoder", cfg, x, t, autocast=dt, scale=65536.0)
    lo, og = oracle_grads(oracle, oracle.EncoderBlock(512, 8, 2048), x, t, amp=odt, scale=65536.0)
    assert abs(lg - lo) <= 2e-3 * abs(lo), (lg, lo)
    check_amp(gg, og, ENC_KEY_BIAS, "c2 " + lowp)


# ------------------------------------------------------------------ C3: the CNN at 32x32x3, channels 32/64, batch 256
def test_c3_cnn_f32_at_full_size(mc, ctx, oracle):
    """Configuration 3 as stated, with the convolutions on their tensor-core path (column matrix + f16 hi/lo GEMMs).

    ReLU and max-pooling make the gradient a discontinuous function of the forward values: where a pre-activation is
    within rounding distance of zero, or the two largest entries of a pooling window within rounding distance of each
    other, two correct f32 implementations route the gradient differently and a single such flip moves a weight
    gradient by about 1 / sqrt(#terms) of its size.  The test therefore separates the two questions:
      (1) gating: the GPU's ReLU masks and pooling choices agree with the oracle's except for at most 1e-5 of the
          decisions, and the loss agrees to 1e-5;
      (2) arithmetic: with the GPU's own gating decisions imposed, every parameter gradient is within 1e-5 (norm-wise)
          of the same backward pass carried out in f64.
    When no decision differs at all, the gradients are also compared with the oracle directly at 1e-5 (or, where the
    oracle's sequential f32 sums of 262144 terms are themselves further from f64 than that, the GPU must be at least
    as close to f64 as the oracle is, plus 1e-5)."""
    rng = np.random.default_rng(1244)
    x = rng.random((256, 3, 32, 32)).astype(np.float32)
    y = rng.integers(0, 10, 256).astype(np.int64)
    F = mc.F
    gm = mc.Model(ctx, "cnn", [3, 32, 64, 32, 10])   # the model's seeded parameters; the tape below is the model's own op sequence
    w1, b1, w2, b2, wf, bf = gm.parameters()
    keep = mc.Arena(ctx, gm.parameters())
    gx, gy = mc.Variable.constant(ctx, x), mc.Variable.constant(ctx, y)
    z1 = F.conv2d(gx, w1, b1, 1, 1)
    a1 = F.relu(z1)
    p1 = F.max_pool2d(a1, 2, 2, 0)
    z2 = F.conv2d(p1, w2, b2, 1, 1)
    a2 = F.relu(z2)
    p2 = F.max_pool2d(a2, 2, 2, 0)
    loss = F.softmax_cross_entropy(F.linear(F.reshape(p2, (256, 4096)), wf, bf), gy)
    model_loss = gm.loss(gx, gy)
    assert float(loss.data) == float(model_loss.data)  # same ops as the model's own forward
    loss.backward()
    gg = [p.grad for p in (w1, b1, w2, b2, wf, bf)]
    gating = [(z1.data > 0), pool_choice(a1.data), (z2.data > 0), pool_choice(a2.data)]

    om = oracle.CNN(3, 32, 64, 32, 10)
    ox, oy = oracle.Variable.constant(x), oracle.Variable.constant(y)
    with oracle.threaded():
        oz1 = oracle.F.conv2d(ox, om.c1.W, om.c1.b, 1, 1)
        oa1 = oracle.F.relu(oz1)
        op1 = oracle.F.max_pool2d(oa1, 2, 2, 0)
        oz2 = oracle.F.conv2d(op1, om.c2.W, om.c2.b, 1, 1)
        oa2 = oracle.F.relu(oz2)
        op2 = oracle.F.max_pool2d(oa2, 2, 2, 0)
        ol = oracle.F.softmax_cross_entropy(oracle.F.linear(oracle.F.reshape(op2, (256, 4096)), om.fc.W, om.fc.b), oy)
        ol.backward()
    og = [p.grad for p in om.parameters()]
    lg, lo = float(loss.data), float(ol.data)
    assert abs(lg - lo) <= F32_TOL * abs(lo), (lg, lo)
    ogating = [(oz1.data > 0), pool_choice(oa1.data), (oz2.data > 0), pool_choice(oa2.data)]
    flips = [int((a != b).sum()) for a, b in zip(gating, ogating)]
    sizes = [a.size for a in gating]
    print("c3 gating decisions that differ from the oracle's:", flips, "of", sizes)
    assert all(f <= 1e-5 * n for f, n in zip(flips, sizes)), (flips, sizes)

    exact = cnn_grads_f64(om, x, y, gating)
    errs = per_tensor_errors(gg, exact)
    report(errs, F32_TOL, "c3 f32 vs f64 under the GPU's gating")
    if not any(flips):
        exact_o = cnn_grads_f64(om, x, y, ogating)
        for i, e in enumerate(per_tensor_errors(gg, og)):
            if e > F32_TOL:
                den = max(float(np.abs(exact_o[i]).max()), 1e-30)
                e_orc = float(np.abs(og[i] - exact_o[i]).max()) / den
                assert errs[i] <= e_orc + F32_TOL, (i, e, errs[i], e_orc)
    del keep


def pool_choice(a):
    """Index (0..3, row-major in the 2x2 window) of the first maximum of every pooling window of a [n, c, h, w] array."""
    n, c, h, w = a.shape
    win = a.reshape(n, c, h // 2, 2, w // 2, 2).transpose(0, 1, 2, 4, 3, 5).reshape(n, c, h // 2, w // 2, 4)
    return win.argmax(-1).astype(np.int8)


def cnn_grads_f64(om, x, y, gating):
    """The CNN's parameter gradients in f64 with numpy (im2col products), with the ReLU masks and pooling choices given
    (gating = [relu1 mask, pool1 choice, relu2 mask, pool2 choice]): the backward pass as a smooth function of its inputs."""
    def im2col(a):  # [n, c, h, w] -> [n, h, w, c*9] for a 3x3 kernel with padding 1
        n, c, h, w = a.shape
        p = np.pad(a, ((0, 0), (0, 0), (1, 1), (1, 1)))
        cols = np.empty((n, h, w, c, 3, 3), a.dtype)
        for ky in range(3):
            for kx in range(3):
                cols[:, :, :, :, ky, kx] = p[:, :, ky:ky + h, kx:kx + w].transpose(0, 2, 3, 1)
        return cols.reshape(n, h, w, c * 9)

    def conv(a, wt, b):
        o = wt.shape[0]
        return (im2col(a) @ wt.reshape(o, -1).T + b).transpose(0, 3, 1, 2)

    def pool(a, choice):
        n, c, h, w = a.shape
        win = a.reshape(n, c, h // 2, 2, w // 2, 2).transpose(0, 1, 2, 4, 3, 5).reshape(n, c, h // 2, w // 2, 4)
        return np.take_along_axis(win, choice[..., None].astype(np.int64), -1)[..., 0]

    def pool_back(g, choice, shape):
        n, c, h, w = shape
        out = np.zeros((n, c, h // 2, w // 2, 4), g.dtype)
        np.put_along_axis(out, choice[..., None].astype(np.int64), g[..., None], -1)
        return out.reshape(n, c, h // 2, w // 2, 2, 2).transpose(0, 1, 2, 4, 3, 5).reshape(n, c, h, w)

    def conv_back(a, wt, g):
        o = wt.shape[0]
        gm = g.transpose(0, 2, 3, 1).reshape(-1, o)
        cols = im2col(a).reshape(gm.shape[0], -1)
        dw = (gm.T @ cols).reshape(wt.shape)
        db = gm.sum(0)
        dcols = (gm @ wt.reshape(o, -1)).reshape(a.shape[0], a.shape[2], a.shape[3], a.shape[1], 3, 3)
        dp = np.zeros((a.shape[0], a.shape[1], a.shape[2] + 2, a.shape[3] + 2), a.dtype)
        for ky in range(3):
            for kx in range(3):
                dp[:, :, ky:ky + a.shape[2], kx:kx + a.shape[3]] += dcols[:, :, :, :, ky, kx].transpose(0, 3, 1, 2)
        return dp[:, :, 1:-1, 1:-1], dw, db

    f = np.float64
    relu1, choice1, relu2, choice2 = gating
    w1, b1, w2, b2, wf, bf = (p.data.astype(f) for p in om.parameters())
    a0 = x.astype(f)
    z1 = conv(a0, w1, b1)
    p1 = pool(z1 * relu1, choice1)
    z2 = conv(p1, w2, b2)
    p2 = pool(z2 * relu2, choice2)
    flat = p2.reshape(p2.shape[0], -1)
    logits = flat @ wf.T + bf
    e = np.exp(logits - logits.max(1, keepdims=True))
    prob = e / e.sum(1, keepdims=True)
    prob[np.arange(len(y)), y] -= 1.0
    gl = prob / len(y)
    dwf, dbf = gl.T @ flat, gl.sum(0)
    g = (gl @ wf).reshape(p2.shape)
    g = pool_back(g, choice2, z2.shape) * relu2
    g, dw2, db2 = conv_back(p1, w2, g)
    g = pool_back(g, choice1, z1.shape) * relu1
    _, dw1, db1 = conv_back(a0, w1, g)
    return [dw1, db1, dw2, db2, dwf, dbf]
