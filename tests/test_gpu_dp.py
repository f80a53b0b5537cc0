"""The product's data-parallel path on two GPUs: one process per GPU, gradients exchanged by NCCL inside
the library (mcb_dp_init / mcb_dp_attach), through the tape step and through the captured (CUDA Graph) step.

Asserted on every rank:
  * replicas are bit-identical after every step (same reduced gradients, same update);
  * two ranks at batch B give the gradients of one rank at batch 2B on the concatenated shards within f32
    tolerance (1e-5 norm-wise per tensor; the sum over ranks is taken in another order);
  * a second backward pass before the optimizer is refused (MCB_UNSUPPORTED) and changes nothing;
  * mcb_clip_grad_norm reports the norm of the MEAN gradient (the single-rank value at batch 2B).
Skipped where fewer than two devices are visible.  NVLS is switched off for the child processes
(plain NVLink peer traffic), the conservative setting for tests in which ranks come and go."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import ctypes as C, os, sys
    import numpy as np
    sys.path.insert(0, {root!r})
    import torch.distributed as td
    import modernchainer_b200 as mc
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    td.init_process_group("gloo", rank=rank, world_size=world)
    ctx = mc.Context(rank)
    lib = ctx.lib
    uid = (C.c_char * 128)()
    if rank == 0:
        ctx.check(lib.mcb_dp_unique_id(uid))
    obj = [bytes(uid)]
    td.broadcast_object_list(obj, src=0)
    ctx.check(lib.mcb_dp_init(ctx.h, rank, world, obj[0]))

    def gather(arrs):
        out = [None] * world
        td.all_gather_object(out, [a.tobytes() for a in arrs])
        return out

    rng = np.random.default_rng(5)
    B, S, V = 2, 64, 512
    cfg = [V, 128, 2, 256, 2, 0]
    ids = rng.integers(0, V, (B * world, S)).astype(np.int64)
    tgt = rng.integers(0, V, (B * world, S)).astype(np.int64)
    mine = slice(rank * B, (rank + 1) * B)

    # ---- f32 tape step: two ranks at batch B against one (local, unattached) model at batch 2B
    m = mc.Model(ctx, "decoder", cfg)
    ps = m.parameters()
    arena = mc.Arena(ctx, ps)
    ctx.check(lib.mcb_dp_attach(ctx.h, arena.h, 256 << 10))
    full = mc.Model(ctx, "decoder", cfg)
    fps = full.parameters()
    keep = mc.Arena(ctx, fps)
    full.loss(mc.Variable.constant(ctx, ids), mc.Variable.constant(ctx, tgt)).backward()
    want = [p.grad for p in fps]

    loss = m.loss(mc.Variable.constant(ctx, ids[mine]), mc.Variable.constant(ctx, tgt[mine]))
    loss.backward()
    # a second backward pass before the optimizer: refused, nothing enqueued
    again = m.loss(mc.Variable.constant(ctx, ids[mine]), mc.Variable.constant(ctx, tgt[mine]))
    try:
        again.backward()
        raise SystemExit("second backward pass was not refused")
    except mc.McbError as e:
        assert e.status == 7, e
    norm = mc.clip_grad_norm(ps, 1e9)   # closes the round (waits for the buckets); limit far away: gradients untouched
    got = [p.grad / np.float32(world) for p in ps]   # buckets hold the sum; the optimizer folds in 1 / world
    top = max(float(np.abs(w).max()) for w in want)
    for i, (g, w) in enumerate(zip(got, want)):
        den = top if i in (6, 22) else max(float(np.abs(w).max()), 1e-30)   # key-projection biases: exact zero gradients
        err = float(np.abs(g - w).max()) / den
        assert err <= 1e-5, (i, err)
    want_norm = float(np.sqrt(sum(float((w.astype(np.float64) ** 2).sum()) for w in want)))
    assert abs(norm - want_norm) <= 1e-5 * want_norm, (norm, want_norm)
    opt = mc.Adam(ctx, 1e-3)
    opt.update(ps)
    reps = gather([p.data for p in ps])
    assert all(r == reps[0] for r in reps), "replicas differ after the tape step"

    # ---- bf16 captured step with a GradScaler, five replays: replicas stay bit-identical, the loss falls
    sc = mc.GradScaler(ctx, 65536.0)
    mc.zero_grad(ps)
    with mc.autocast(mc.BF16):      # one eager step first: NCCL sets up its connections outside the capture
        l0 = m.loss(mc.Variable.constant(ctx, ids[mine]), mc.Variable.constant(ctx, tgt[mine]))
    sc.scale_loss(l0).backward()
    sc.step_async(opt, ps)
    step = mc.StaticStep(m, opt, ids[mine], tgt[mine], scaler=sc, autocast_dtype=mc.BF16)
    losses = []
    for _ in range(5):
        step.run(ids[mine], tgt[mine])
        losses.append(step.loss())
    assert losses[-1] < losses[0], losses
    reps = gather([p.data for p in ps])
    assert all(r == reps[0] for r in reps), "replicas differ after the captured steps"
    step.close()
    ctx.check(lib.mcb_dp_shutdown(ctx.h))
    td.destroy_process_group()
    print("rank", rank, "ok", losses)
""")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_gpu_replicas_stay_identical_and_match_one_rank_at_twice_the_batch():
    import modernchainer_b200 as mc
    if mc.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                   MCB_DP_TIMEOUT_MS="120000")
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER.format(root=ROOT)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    for p in procs:
        try:
            out, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        assert p.returncode == 0, out.decode()[-4000:]
