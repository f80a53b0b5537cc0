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


# ------------------------------------------------------------------ the product's round logic over a recording transport
# mcb_dp_sim_* runs the same host code as the GPU path (bucket readiness, the one-backward-per-step rule, error and
# timeout handling); only the transport is replaced by one that records and can be told to fail.  No device is touched:
# failures are injected on the host, never provoked on a GPU.
import ctypes as C

import pytest


class Sim:
    def __init__(self, sizes, bucket_elems, world=2):
        from modernchainer_b200 import _lib
        self.lib = _lib.load()
        self.n = len(sizes)
        arr = np.asarray(sizes, np.int64)
        self.h = C.c_void_p()
        assert self.lib.mcb_dp_sim_create(arr.ctypes.data, self.n, bucket_elems, world, C.byref(self.h)) == 0

    def close(self):
        self.lib.mcb_dp_sim_release(self.h)

    def log(self):
        buf = (C.c_int32 * 64)()
        n = self.lib.mcb_dp_sim_log(self.h, buf, 64)
        return list(buf[:n])

    def err(self):
        return (self.lib.mcb_dp_sim_last_error(self.h) or b"").decode()

    def __getattr__(self, name):
        fn = getattr(self.lib, "mcb_dp_sim_" + name)
        return lambda *a: fn(self.h, *a)


SLOTS = [1024, 64, 2048, 64, 512, 64]  # parameter slots in arena order; 2200-element buckets -> {3,4,5}, {1,2}, {0}


def test_dp_round_buckets_start_as_their_last_gradient_arrives_and_every_bucket_takes_part():
    s = Sim(SLOTS, 2200)
    try:
        assert s.buckets() == 3 and [s.bucket_of(i) for i in range(6)] == [2, 1, 1, 0, 0, 0]
        assert s.backward_begin() == 0
        for p in (5, 3):
            assert s.grad_ready(p) == 0
        assert s.log() == []            # bucket 0 still misses parameter 4
        assert s.grad_ready(4) == 0
        assert s.log() == [0]           # complete: its all-reduce is enqueued while backward goes on
        assert s.grad_ready(2) == 0 and s.log() == [0]
        # parameter 1 and 0 never receive a gradient (unused branch): the optimizer still sends every bucket,
        # in bucket order, so the ranks' collectives pair up, then joins the streams once
        assert s.finish() == 0
        assert s.log() == [0, 1, 2] and s.joins() == 1
        # next step: counters were reset
        assert s.backward_begin() == 0
        for p in reversed(range(6)):
            assert s.grad_ready(p) == 0
        assert s.log() == [0, 1, 2, 0, 1, 2]
        assert s.finish() == 0 and s.joins() == 2 and s.aborted() == 0
    finally:
        s.close()


def test_dp_second_backward_before_the_optimizer_is_refused_and_zero_grad_reopens():
    s = Sim(SLOTS, 2200)
    try:
        assert s.backward_begin() == 0
        for p in reversed(range(6)):
            assert s.grad_ready(p) == 0
        assert s.backward_begin() == 7 and "one backward pass per optimizer step" in s.err()  # Unsupported, nothing enqueued
        assert s.log() == [0, 1, 2]
        assert s.zero_grad() == 0        # gradients dropped: waits for their all-reduces (join) and starts over
        assert s.joins() == 1
        assert s.backward_begin() == 0
    finally:
        s.close()


@pytest.mark.parametrize("what", ["enqueue", "async", "timeout"])
def test_dp_failures_abort_the_communicator_and_stay_failed(what):
    s = Sim(SLOTS, 2200)
    try:
        assert s.backward_begin() == 0
        if what == "enqueue":      # this rank fails before it can take part in bucket 1
            s.inject(0, 1)
            for p in (5, 4, 3):
                assert s.grad_ready(p) == 0
            assert s.grad_ready(2) == 0
            assert s.grad_ready(1) == 8 and "enqueue of bucket 1 failed" in s.err()
        elif what == "async":      # a peer (or the network) fails: the transport's error word is seen at the next enqueue
            for p in (5, 4, 3):
                assert s.grad_ready(p) == 0
            s.inject(1, 0)
            assert s.grad_ready(2) == 0
            assert s.grad_ready(1) == 8 and "asynchronous error: simulated remote error" in s.err()
        else:                      # a peer never joins: the bounded host wait runs out instead of blocking for ever
            for p in reversed(range(6)):
                assert s.grad_ready(p) == 0
            assert s.finish() == 0
            s.inject(2, 1)
            import time
            t0 = time.time()
            assert s.host_wait(150) == 8 and "timed out" in s.err()
            assert 0.1 < time.time() - t0 < 5.0
        assert s.aborted() == 1
        # sticky: every later call reports the dead communicator, nothing more is enqueued, no second abort
        n = len(s.log())
        assert s.grad_ready(0) == 8 and s.finish() == 8 and s.backward_begin() == 8 and s.host_wait(10) == 8
        assert len(s.log()) == n and s.aborted() == 1
    finally:
        s.close()


def test_dp_healthy_host_wait_returns_at_once():
    s = Sim(SLOTS, 2200)
    try:
        assert s.host_wait(1000) == 0 and s.aborted() == 0
    finally:
        s.close()


PLAN_WORKER = textwrap.dedent("""
    import ctypes as C, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    import torch.distributed as td
    from modernchainer_b200 import _lib
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    td.init_process_group("gloo", rank=rank, world_size=world)
    lib = _lib.load()
    sizes = np.array([1024, 64, 2048, 64, 512, 64], np.int64)
    # MISMATCH=1: rank 1 was started with another bucket size, so its plan differs
    bucket = 2200 if not (os.environ.get("MISMATCH") == "1" and rank == 1) else 1100
    h = C.c_void_p()
    assert lib.mcb_dp_sim_create(sizes.ctypes.data, 6, bucket, world, C.byref(h)) == 0
    mine = int(lib.mcb_dp_sim_plan_checksum(h))
    allc = [None] * world
    td.all_gather_object(allc, mine)
    arr = (C.c_uint64 * world)(*allc)
    st = lib.mcb_dp_check_plan_checksums(arr, world)
    assert st == (5 if os.environ.get("MISMATCH") == "1" else 0), (st, allc)   # every rank reaches the same verdict
    td.destroy_process_group()
    print("rank", rank, "ok")
""")


def _run_worker(src, world, extra_env):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), **extra_env)
        procs.append(subprocess.Popen([sys.executable, "-c", src.format(root=ROOT)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        assert p.returncode == 0, out.decode()


@pytest.mark.parametrize("mismatch", ["0", "1"])
def test_bucket_plan_checksum_exchange_between_two_ranks(mismatch):
    _run_worker(PLAN_WORKER, 2, {"MISMATCH": mismatch})


CLIP_WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    import torch, torch.distributed as td
    from oracle import ref
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    td.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(11)
    B = 16
    x = rng.standard_normal((B * world, 20)).astype(np.float32)
    y = rng.integers(0, 5, B * world).astype(np.int64)

    def grads(xs, ys):
        m = ref.MLP((20, 12, 5))
        m.loss(ref.Variable.constant(xs), ref.Variable.constant(ys)).backward()
        return m

    m = grads(x[rank * B:(rank + 1) * B], y[rank * B:(rank + 1) * B])
    for p in m.parameters():          # what the buckets hold after the exchange: the SUM over ranks
        t = torch.from_numpy(p.grad)
        td.all_reduce(t)
    # the library's rule for a data-parallel arena: the norm is that of the mean (sum * 1/world), the factor
    # max_norm / norm is applied to the sum, and the optimizer's 1/world turns the clipped sum into the clipped mean
    max_norm = 0.05
    total = sum(float(ref.sum_all(ref.mul(p.grad, p.grad))) for p in m.parameters())
    norm = float(np.sqrt(total)) / world
    f = max_norm / norm if norm > max_norm else 1.0
    clipped_mean = [ref.scale(ref.scale(p.grad, f), 1.0 / world) for p in m.parameters()]
    # one rank at world * B
    full = grads(x, y)
    n_full = ref.clip_grad_norm(full.parameters(), max_norm)
    assert abs(norm - n_full) <= 2e-6 * n_full, (norm, n_full)
    assert n_full > max_norm
    for a, p in zip(clipped_mean, full.parameters()):
        assert np.abs(a - p.grad).max() <= 2e-6 * max(np.abs(p.grad).max(), 1e-30)
    td.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_clipping_on_two_ranks_equals_one_rank_at_twice_the_batch(oracle):
    _run_worker(CLIP_WORKER, 2, {})
