#!/usr/bin/env python
"""Writes tests/golden/step_vectors.npz: losses, gradients and Adam-updated parameters of two training steps of four
small models, computed by the single-threaded CPU oracle (oracle/ref.py over oracle/mc_oracle.c) from seeded inputs.

    python tests/golden/make_step_vectors.py            # rewrite the fixture
    python tests/golden/make_step_vectors.py --check    # exit 1 if the oracle no longer reproduces it bit for bit

The reference itself (Rust, no toolchain here) cannot produce vectors, and its tests hold no gradient arrays; what pins
the oracle to the reference are the literals and gradient checks of tests/test_oracle_golden.py.  This fixture pins the
oracle to ITSELF over time (a changed restatement shows up as a changed fixture) and gives the GPU tests a committed
target that needs no oracle run: tests/test_gpu_tape.py compares the CUDA path with it at 1e-5.
Models and inputs are those of the small-size step tests: the four model families at toy widths, same seeds."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "step_vectors.npz")
STEPS, LR = 2, 1e-3


def cases(ref):
    """name -> (kind, cfg for the library's Model, oracle model, x, y, indices of gradients that are exactly zero in
    exact arithmetic: the key-projection biases)"""
    out = {}
    rng = np.random.default_rng(4242)
    out["mlp"] = ("mlp", [20, 16, 5], ref.MLP([20, 16, 5]), rng.standard_normal((12, 20)).astype(np.float32),
                  rng.integers(0, 5, 12).astype(np.int64), ())
    d, heads, ff = 32, 2, 64
    x = rng.standard_normal((2, 12, d)).astype(np.float32)
    out["encoder"] = ("encoder", [d, heads, ff, 0], ref.EncoderBlock(d, heads, ff), x, (x * 0.5).astype(np.float32), (5,))
    out["cnn"] = ("cnn", [3, 4, 8, 8, 5], ref.CNN(3, 4, 8, 8, 5), rng.standard_normal((4, 3, 8, 8)).astype(np.float32),
                  rng.integers(0, 5, 4).astype(np.int64), ())
    vocab, layers = 40, 2
    ids = rng.integers(0, vocab, (2, 12)).astype(np.int64)
    tgt = np.concatenate([ids[:, 1:], rng.integers(0, vocab, (2, 1))], 1).astype(np.int64)
    out["decoder"] = ("decoder", [vocab, d, heads, ff, layers, 0], ref.Decoder(vocab, d, heads, ff, layers, 0), ids, tgt,
                      tuple(1 + 16 * l + 5 for l in range(layers)))
    return out


def run(ref):
    ref.set_mode("checker")
    vec = {}
    for name, (kind, cfg, model, x, y, zero) in cases(ref).items():
        params, opt = model.parameters(), ref.Adam(LR)
        vec[f"{name}/cfg"] = np.asarray(cfg, np.int64)
        vec[f"{name}/x"], vec[f"{name}/y"] = x, y
        vec[f"{name}/zero_idx"] = np.asarray(zero, np.int64)  # gradients that are exactly zero in exact arithmetic
        for step in range(STEPS):
            ref.zero_grad(params)
            loss = model.loss(ref.Variable.constant(x), ref.Variable.constant(y))
            loss.backward()
            vec[f"{name}/loss{step}"] = np.asarray(loss.data, np.float32).reshape(1)
            for i, p in enumerate(params):
                vec[f"{name}/grad{step}/{i}"] = np.asarray(p.grad, np.float32)
            opt.update(params)
        for i, p in enumerate(params):
            vec[f"{name}/param/{i}"] = np.asarray(p.data, np.float32)
    return vec


def main():
    sys.path.insert(0, ROOT)
    from oracle import ref
    ref.build()
    vec = run(ref)
    if "--check" in sys.argv:
        old = np.load(OUT)
        bad = [k for k in vec if k not in old.files or not np.array_equal(old[k], vec[k])] + [k for k in old.files if k not in vec]
        if bad:
            sys.stderr.write("the oracle no longer reproduces tests/golden/step_vectors.npz: %s\n" % ", ".join(bad[:8]))
            sys.exit(1)
        return
    np.savez_compressed(OUT, **vec)
    print("wrote", OUT, os.path.getsize(OUT), "bytes,", len(vec), "arrays")


if __name__ == "__main__":
    main()
