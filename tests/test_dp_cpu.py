"""Host-side logic of the data-parallel path on CPU, two gloo ranks.

What the GPU path does per step: every rank runs backward on its own shard, gradient buckets of the
flat arena are summed over ranks (NCCL on the GPU, gloo here), the 1/world factor is folded into the
optimizer's unscale factor, and the inf/nan scan runs on the reduced gradients so all ranks take the
same skip decision.  These tests check, with the CPU oracle as the engine:
  * N ranks at batch B == one rank at batch N*B (losses are batch means), to f32 tolerance;
  * bucket plans from the library's host-only planner are identical on every rank and cover every
    parameter exactly once, in contiguous arena ranges walked from the last parameter back;
  * a non-finite gradient on ONE rank makes EVERY rank skip the step (flag taken after the reduction).
"""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import ctypes as C, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    import torch, torch.distributed as td
    from oracle import ref
    from modernchainer_b200 import _lib
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    td.init_process_group("gloo", rank=rank, world_size=world)
    lib = _lib.load()
    rng = np.random.default_rng(7)
    B = 16
    x = rng.standard_normal((B * world, 20)).astype(np.float32)
    y = rng.integers(0, 5, B * world).astype(np.int64)
    inject = os.environ.get("INJECT_NAN") == "1"

    def grads(xs, ys):
        m = ref.MLP((20, 12, 5))
        loss = m.loss(ref.Variable.constant(xs), ref.Variable.constant(ys))
        loss.backward()
        return m, [p.grad.copy() for p in m.parameters()]

    # local shard
    m, g_local = grads(x[rank * B:(rank + 1) * B], y[rank * B:(rank + 1) * B])
    if inject and rank == 1:
        g_local[0][3, 4] = np.nan
    sizes = np.array([g.size for g in g_local], np.int64)
    # flat arena with 64-element slots, as the library lays it out
    slots = (sizes + 63) // 64 * 64
    off = np.concatenate([[0], np.cumsum(slots)[:-1]])
    flat = np.zeros(int(slots.sum()), np.float32)
    for g, o in zip(g_local, off):
        flat[o:o + g.size] = g.reshape(-1)
    bucket_of = np.zeros(len(sizes), np.int32)
    nb = C.c_int32()
    assert lib.mcb_dp_plan_buckets(slots.ctypes.data_as(C.c_void_p), len(sizes), 256, bucket_of.ctypes.data_as(C.c_void_p), C.byref(nb)) == 0
    plans = [None] * world
    td.all_gather_object(plans, bucket_of.tolist())
    assert all(p == plans[0] for p in plans), plans
    # every bucket is one contiguous arena range; buckets are numbered from the arena's end
    covered = np.zeros(flat.size, bool)
    for b in range(nb.value):
        idx = [i for i in range(len(sizes)) if bucket_of[i] == b]
        assert idx == list(range(idx[0], idx[-1] + 1))
        lo, hi = int(off[idx[0]]), int(off[idx[-1]] + slots[idx[-1]])
        assert not covered[lo:hi].any()
        covered[lo:hi] = True
        t = torch.from_numpy(flat[lo:hi])
        td.all_reduce(t)  # sum, bucket by bucket, last parameters first
    assert covered.all() and bucket_of[-1] == 0 and bucket_of[0] == nb.value - 1
    found = int(ref.count_non_finite(flat) > 0)  # scan AFTER the reduction: identical on all ranks
    flags = [None] * world
    td.all_gather_object(flags, found)
    assert len(set(flags)) == 1, flags
    if inject:
        assert found == 1
    else:
        # mean over ranks == gradient of the full batch on one rank
        _, g_full = grads(x, y)
        inv = np.float32(1.0 / world)
        for g, o, s in zip(g_full, off, sizes):
            got = flat[o:o + s] * inv
            err = np.abs(got - g.reshape(-1)).max() / max(np.abs(g).max(), 1e-30)
            assert err < 2e-6, err
        # and one Adam step from the averaged gradients leaves every rank with the same parameters
        opt = ref.Adam(1e-3)
        for p, o, s in zip(m.parameters(), off, sizes):
            p.grad = (flat[o:o + s] * inv).reshape(p.data.shape)
        opt.update(m.parameters())
        digest = float(sum(np.abs(p.data).sum() for p in m.parameters()))
        ds = [None] * world
        td.all_gather_object(ds, digest)
        assert len(set(ds)) == 1, ds
    td.destroy_process_group()
    print("rank", rank, "ok")
""")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(world, extra_env):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), **extra_env)
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER.format(root=ROOT)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append((p.returncode, out.decode()))
    for rc, out in outs:
        assert rc == 0, out


def test_two_ranks_equal_one_rank_at_twice_the_batch(oracle):
    _run(2, {})


def test_non_finite_gradient_on_one_rank_skips_everywhere(oracle):
    _run(2, {"INJECT_NAN": "1"})
