"""The `chainer` facade (modernchainer_b200/chainer) on the GPU: the behaviours the reference's Python
tests exercise (python/tests/test_basic.py, test_nn_ops.py, test_devices.py) and its example training
loop (python/examples/train_mlp.py), written against the same public names.  Values are checked
against numpy / the oracle where the reference's tests only check shapes."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def chainer():
    # as a user of the reference would import it: a top-level package called `chainer`
    sys.path.insert(0, os.path.join(ROOT, "modernchainer_b200"))
    try:
        import chainer as ch
        import chainer.functions  # noqa: F401
        import chainer.links  # noqa: F401
        import chainer.optimizers  # noqa: F401
        yield ch
    finally:
        sys.path.remove(os.path.join(ROOT, "modernchainer_b200"))


def test_version_and_devices(chainer):
    assert chainer.__version__
    assert chainer.cuda_available() is True
    assert chainer.vulkan_available() is False and chainer.vulkan_devices() == []
    chainer.synchronize("cuda")


def test_linear_forward_backward_and_initialiser(chainer, oracle):
    F, L = chainer.functions, chainer.links
    layer = L.Linear(2, 1, seed=1)
    assert np.array_equal(layer.W.array, oracle.he_normal((1, 2), 2, 1))  # same seeded values as nn::Linear
    x = chainer.Variable(chainer.Tensor.from_list([1.0, 2.0, 3.0, 4.0], [2, 2]))
    y = layer(x)
    assert y.shape == [2, 1] and y.grad_fn is not None and x.grad_fn is None
    F.sum(y).backward()
    assert layer.W.grad.tolist() == [4.0, 6.0] and layer.b.grad.tolist() == [2.0]
    assert np.allclose(x.grad.numpy(), np.repeat(layer.W.array, 2, 0))


def test_optimizers_follow_setup_update_zero_grad(chainer):
    F, L, O = chainer.functions, chainer.links, chainer.optimizers
    for make in (lambda: O.SGD(0.1), lambda: O.MomentumSGD(0.05, 0.9), lambda: O.Adam(0.05), lambda: O.AdamW(0.05, 0.01)):
        layer = L.Linear(1, 1, seed=3)
        x = chainer.Variable(chainer.Tensor.from_list([1.0, 2.0], [2, 1]))
        target = chainer.Variable.constant(chainer.Tensor.from_list([2.0, 4.0], [2, 1]))
        opt = make()
        opt.setup(layer.parameters())
        before = layer.W.data.tolist()
        first = None
        for _ in range(30):
            diff = F.sub(layer(x), target)
            loss = F.mean(F.mul(diff, diff))
            opt.zero_grad()
            loss.backward()
            opt.update()
            first = first if first is not None else loss.data.tolist()[0]
        assert layer.W.data.tolist() != before
        assert loss.data.tolist()[0] < first


def test_chain_container_and_numpy_interop(chainer):
    F, L = chainer.functions, chainer.links

    class MLP(chainer.Chain):
        def __init__(self):
            super().__init__()
            with self.init_scope():
                self.l1 = L.Linear(2, 3, seed=0)
                self.l2 = L.Linear(3, 1, seed=0)

        def forward(self, x):
            return self.l2(F.relu(self.l1(x)))

    model = MLP()
    assert len(model.parameters()) == 4 and set(model.children()) == {"l1", "l2"}
    out = model(chainer.Variable(chainer.Tensor.from_list([0.1, 0.2], [1, 2])))
    assert out.shape == [1, 1]
    model.cleargrads()
    t = chainer.Tensor.from_numpy(np.arange(6, dtype=np.float32).reshape(2, 3))
    assert t.shape == [2, 3] and t.dtype == "f32" and t.ndim == 2 and t.numel() == 6
    assert t.numpy().tolist() == [[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]]
    assert t.to("cuda").device == "cuda" and chainer.Tensor.zeros([2, 2]).tolist() == [0.0] * 4


def test_elementwise_and_layout_functions(chainer):
    F = chainer.functions
    a = chainer.Variable(chainer.Tensor.from_list([4.0, 9.0], [2]))
    b = chainer.Variable(chainer.Tensor.from_list([2.0, 3.0], [2]))
    assert F.sqrt(a).data.tolist() == [2.0, 3.0]
    assert F.div(a, b).data.tolist() == [2.0, 3.0]
    assert F.neg(a).data.tolist() == [-4.0, -9.0] and F.abs(F.neg(a)).data.tolist() == [4.0, 9.0]
    assert F.scale(a, 0.5).data.tolist() == [2.0, 4.5]
    m = chainer.Variable(chainer.Tensor.from_list([1.0, 2.0, 3.0, 4.0], [2, 2]))
    assert F.transpose(m).data.tolist() == [1.0, 3.0, 2.0, 4.0]
    x = chainer.Variable(chainer.Tensor.from_numpy(np.arange(6, dtype=np.float32).reshape(2, 3)))
    assert F.reshape(x, [3, 2]).shape == [3, 2] and F.permute(x, [1, 0]).shape == [3, 2]
    assert np.allclose(F.silu(x).array, x.array / (1.0 + np.exp(-x.array)), rtol=1e-6)
    for name in ("dropout", "clamp", "rms_norm", "average_pool2d", "conv_transpose2d"):
        with pytest.raises(NotImplementedError):
            getattr(F, name)(x)


@pytest.mark.parametrize("device", ["cpu", "cuda"])
def test_softmax_layer_norm_values_and_gradients(chainer, device):
    F = chainer.functions
    values = np.random.default_rng(0).standard_normal((2, 3), dtype=np.float32)
    x = chainer.Variable(chainer.Tensor.from_numpy(values, device=device))
    assert x.device == device
    probs = F.softmax(x)
    expected = np.exp(values - values.max(axis=1, keepdims=True))
    expected /= expected.sum(axis=1, keepdims=True)
    np.testing.assert_allclose(probs.array, expected, rtol=1e-4, atol=1e-5)
    F.sum(probs).backward()
    assert x.grad is not None
    x = chainer.Variable(chainer.Tensor.from_numpy(values, device=device))
    gamma = chainer.Variable(chainer.Tensor.from_numpy(np.ones(3, np.float32), device=device))
    beta = chainer.Variable(chainer.Tensor.from_numpy(np.zeros(3, np.float32), device=device))
    norm = F.layer_norm(x, gamma, beta)
    np.testing.assert_allclose(norm.array, (values - values.mean(-1, keepdims=True)) / np.sqrt(values.var(-1, keepdims=True) + 1e-5),
                               rtol=1e-4, atol=1e-4)
    F.sum(norm).backward()
    assert x.grad is not None and gamma.grad is not None and beta.grad is not None


def test_conv_pool_embedding_attention(chainer):
    F = chainer.functions
    image = np.arange(9, dtype=np.float32).reshape(1, 1, 3, 3) / 10.0
    x = chainer.Variable(chainer.Tensor.from_numpy(image))
    w = chainer.Variable(chainer.Tensor.from_numpy(np.ones((1, 1, 2, 2), np.float32)))
    conv = F.conv2d(x, w, None, 1, 0)
    want = np.array([[image[0, 0, i:i + 2, j:j + 2].sum() for j in range(2)] for i in range(2)], np.float32)
    np.testing.assert_allclose(conv.array.reshape(2, 2), want, rtol=1e-5, atol=1e-5)
    assert F.max_pool2d(x, 2, 1, 0).shape == [1, 1, 2, 2]
    ids = chainer.Variable(chainer.Tensor.from_numpy(np.array([0, 2, 0], np.int64)))
    weight = chainer.Variable(chainer.Tensor.from_numpy(np.arange(6, dtype=np.float32).reshape(3, 2) / 10.0))
    out = F.embedding(ids, weight)
    assert out.shape == [3, 2]
    F.sum(out).backward()
    assert weight.grad.tolist() == [2.0, 2.0, 0.0, 0.0, 1.0, 1.0]
    q = chainer.Variable(chainer.Tensor.from_numpy(np.array([[[0.2, -0.1], [0.4, 0.3]]], np.float32)))
    k = chainer.Variable(chainer.Tensor.from_numpy(np.array([[[0.1, 0.2], [-0.3, 0.4]]], np.float32)))
    v = chainer.Variable(chainer.Tensor.from_numpy(np.array([[[0.5, -0.2], [0.3, 0.1]]], np.float32)))
    attn = F.multi_head_attention(q, k, v, 1, True)
    assert attn.shape == [1, 2, 2]
    assert np.allclose(attn.array[0, 0], [0.5, -0.2])  # causal: the first query sees only the first key
    F.sum(attn).backward()
    assert q.grad is not None


def test_links_shapes_and_seeds(chainer, oracle):
    F, L = chainer.functions, chainer.links
    conv = L.Conv2d(1, 2, 3, stride=1, padding=1)
    assert np.array_equal(conv.W.array, oracle.he_normal((2, 1, 3, 3), 9, 0))
    y = conv(chainer.Variable(chainer.Tensor.from_numpy(np.ones((1, 1, 4, 4), np.float32))))
    assert y.shape == [1, 2, 4, 4]
    assert L.LayerNorm(4)(F.reshape(y, [8, 4])).shape == [8, 4]
    emb = L.Embedding(8, 4)
    assert emb(chainer.Variable(chainer.Tensor.from_numpy(np.array([0, 2, 4], np.int64)))).shape == [3, 4]
    attn = L.MultiHeadAttention(4, 2)
    assert len(attn.parameters()) == 8 and np.array_equal(attn.wk.W.array, oracle.he_normal((4, 4), 4, 2))
    assert attn(chainer.Variable(chainer.Tensor.from_numpy(np.ones((2, 3, 4), np.float32)))).shape == [2, 3, 4]
    assert L.BatchNorm(2)(y).shape == y.shape and len(L.BatchNorm(2).parameters()) == 2
    for name in ("RMSNorm", "ConvTranspose2d"):
        with pytest.raises(NotImplementedError):
            getattr(L, name)(2)


def test_batch_norm_values_and_gradients(chainer):
    """F.batch_norm (a host op of the reference, host_ops.rs:478-600) composed from ops of the path: values against the
    closed form in f64, gradients against the closed-form batch-norm backward."""
    import chainer.functions as F
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 3, 5, 2)).astype(np.float32) * 2 + 1
    gamma, beta = rng.standard_normal(3).astype(np.float32), rng.standard_normal(3).astype(np.float32)
    up = rng.standard_normal(x.shape).astype(np.float32)
    xv, gv, bv = (chainer.Variable(chainer.Tensor.from_numpy(a)) for a in (x, gamma, beta))
    y = F.batch_norm(xv, gv, bv)
    x64 = x.astype(np.float64)
    mean, var = x64.mean((0, 2, 3), keepdims=True), x64.var((0, 2, 3), keepdims=True)
    xhat = (x64 - mean) / np.sqrt(var + 1e-5)
    want = xhat * gamma.reshape(1, 3, 1, 1) + beta.reshape(1, 3, 1, 1)
    assert np.abs(y.array - want).max() <= 1e-5 * np.abs(want).max()
    F.sum(F.mul(y, chainer.Variable.constant(chainer.Tensor.from_numpy(up)))).backward()
    g = up.astype(np.float64)
    dxhat = g * gamma.reshape(1, 3, 1, 1)
    dx = (dxhat - dxhat.mean((0, 2, 3), keepdims=True) - xhat * (dxhat * xhat).mean((0, 2, 3), keepdims=True)) / np.sqrt(var + 1e-5)
    for got, ref in ((xv.grad.numpy(), dx), (gv.grad.numpy(), (g * xhat).sum((0, 2, 3))), (bv.grad.numpy(), g.sum((0, 2, 3)))):
        assert np.abs(got - ref).max() <= 2e-5 * max(np.abs(ref).max(), 1e-30)


def test_mlp_training_loop_learns(chainer):
    """The shape of python/examples/train_mlp.py: Chain of two Linear links, softmax cross-entropy, Adam."""
    F, L, O = chainer.functions, chainer.links, chainer.optimizers
    rng = np.random.default_rng(0)
    xs = rng.standard_normal((256, 16)).astype(np.float32)
    ys = (xs[:, 0] + xs[:, 1] > 0).astype(np.int64)

    class Net(chainer.Chain):
        def __init__(self):
            super().__init__()
            with self.init_scope():
                self.l1 = L.Linear(16, 32, seed=0)
                self.l2 = L.Linear(32, 2, seed=1)

        def forward(self, x):
            return self.l2(F.relu(self.l1(x)))

    net = Net()
    opt = O.Adam(0.01)
    opt.setup(net.parameters())
    x, t = chainer.Variable.constant(chainer.Tensor.from_numpy(xs)), chainer.Variable.constant(chainer.Tensor.from_numpy(ys))
    losses = []
    for _ in range(60):
        loss = F.softmax_cross_entropy(net(x), t)
        opt.zero_grad()
        loss.backward()
        opt.update()
        losses.append(loss.data.tolist()[0])
    assert losses[-1] < 0.5 * losses[0]
    acc = (net(x).array.argmax(1) == ys).mean()
    assert acc > 0.9
