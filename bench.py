#!/usr/bin/env python
"""Benchmark of the training step: train samples/sec (fwd + bwd + GradScaler + Adam, device
timed, max over ranks).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c2|c3|c1|c5] [--impl ours|reference]

Workloads (synthetic inputs from fixed seeds, random-init weights of the named architecture):
  c4  12-layer decoder d=768 h=12 ff=3072 vocab=32000 seq=1024 batch 8 per GPU, bf16 autocast  (default; the
      configuration the metric is quoted on)
  c2  one pre-LN encoder block d=512 h=8 ff=2048 seq=256 batch 32, bf16 autocast, MSE loss
  c3  CNN conv3x3(3->32)-ReLU-pool-conv3x3(32->64)-ReLU-pool-Linear(4096->10) on 32x32x3 images, f32, batch 256
  c1  MLP 784-100-10, f32, batch 128
  c5  optimizer stress: flat 125M f32 parameters, bf16 gradients stored pre-multiplied by the loss scale
      2^16, inf/nan injected on odd steps; metric = HBM GB/s of the fused check + unscale + Adam pass

One JSON line is printed by rank 0.  `value` is timed with inputs resident on the device; `e2e` repeats
the same steps with the per-step host->device copy of the inputs (pinned memory) and a device->host read
of the loss inside the timed region.  For N > 1 the script is launched by torchrun (one rank per GPU);
ranks exchange gradients through NCCL inside the library and the step time is the max over ranks.
`--impl reference` times the CPU restatement of the reference's CPU backend (oracle/) on the host cores.
"""
import argparse
import ctypes as C
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c4": dict(kind="decoder", vocab=32000, d=768, heads=12, ff=3072, layers=12, seq=1024, batch=8, amp=True),
    "c2": dict(kind="encoder", d=512, heads=8, ff=2048, seq=256, batch=32, amp=True),
    "c1": dict(kind="mlp", sizes=(784, 100, 10), batch=128, amp=False),
    "c3": dict(kind="cnn", cin=3, c1=32, c2=64, hw=32, classes=10, batch=256, amp=False),
    "c5": dict(kind="optimizer", n=125_000_000),
    "gemm": dict(kind="gemm"),
}
PROF_CLASSES = ["gemm_tc", "gemm_f32", "attention", "optimizer", "norm", "loss", "elementwise", "reduce", "embedding", "conv"]


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tf_burst=p["bf16_tflops"], tf_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, src="fallback")


# DRAM bytes of the c4 step's GEMM launches, measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum of every tc_gemm launch
# of one tape step of the 2-layer model:
#   ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --clock-control none -k regex:tc_gemm_kernel -s 81 -c 27 --csv \
#       python bench.py --workload c4 --layers 2 --steps 1 --warmup 3 --no-cpu-baseline --no-graph
# ): the three lm_head launches together, and the twelve launches of one layer together.  Traffic
# grows in proportion to the layer count (every layer launches the same twelve shapes).  The figure belongs to the GEMM source it was
# measured with: `kernel_sha256` is the SHA-256 of modernchainer_b200/csrc/gemm_tc.cu at capture time, and a build whose source differs
# reports traffic null (with the reason) instead of a stale number.
GEMM_TRAFFIC = {"lm_head_bytes": 1937.8e6, "per_layer_bytes": 529.0e6,
                "kernel_sha256": "6e5ee17be7035caf1b498eb35888caa66ca361f7d11f5ac3834d653d9ab78f11"}


def gemm_traffic(layers):
    import hashlib
    src = os.path.join(ROOT, "modernchainer_b200", "csrc", "gemm_tc.cu")
    try:
        sha = hashlib.sha256(open(src, "rb").read()).hexdigest()
    except OSError:
        return None, "GEMM source not found beside the library: the ncu capture cannot be matched to this build"
    if sha != GEMM_TRAFFIC["kernel_sha256"]:
        return None, "the GEMM kernel source has changed since the ncu capture of its DRAM traffic was taken"
    per_launch = (GEMM_TRAFFIC["lm_head_bytes"] + GEMM_TRAFFIC["per_layer_bytes"] * layers) / (3 + 12 * layers)
    return per_launch, ("ncu dram__bytes_read.sum + dram__bytes_write.sum of every GEMM launch of a 2-layer step of this kernel source, "
                        "scaled by the layer count; bytes per launch, mean over the step's GEMMs")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc = index, None
        self.path = tempfile.mktemp(suffix=".csv")

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def count(self):
        try:
            return sum(1 for _ in open(self.path))
        except OSError:
            return 0

    def cover(self, work, sync, want=3, limit_s=3.0):
        """A timed region shorter than nvidia-smi's sampling period leaves no sample: repeat the same work, untimed, until
        `want` samples exist (or `limit_s` has passed).  Returns the number of extra repetitions."""
        if not self.proc:
            return 0
        extra, t0 = 0, time.perf_counter()
        while self.count() < want and time.perf_counter() - t0 < limit_s:
            work()
            extra += 1
            if extra % 16 == 0:
                sync()
        sync()
        return extra

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ synthetic data
def make_inputs(name, cfg, rank):
    rng = np.random.default_rng(1234 + list(WORKLOADS).index(name) + 1000 * rank)
    if cfg["kind"] == "decoder":
        ids = rng.integers(0, cfg["vocab"], (cfg["batch"], cfg["seq"])).astype(np.int64)
        tgt = np.concatenate([ids[:, 1:], rng.integers(0, cfg["vocab"], (cfg["batch"], 1))], 1).astype(np.int64)
        return ids, tgt
    if cfg["kind"] == "encoder":
        shape = (cfg["batch"], cfg["seq"], cfg["d"])
        return rng.standard_normal(shape).astype(np.float32), rng.standard_normal(shape).astype(np.float32)
    if cfg["kind"] == "mlp":
        return rng.standard_normal((cfg["batch"], cfg["sizes"][0])).astype(np.float32), rng.integers(0, cfg["sizes"][-1], cfg["batch"]).astype(np.int64)
    if cfg["kind"] == "cnn":
        return (rng.random((cfg["batch"], cfg["cin"], cfg["hw"], cfg["hw"])).astype(np.float32),
                rng.integers(0, cfg["classes"], cfg["batch"]).astype(np.int64))
    raise ValueError(name)


def model_cfg(cfg):
    if cfg["kind"] == "decoder":
        return [cfg["vocab"], cfg["d"], cfg["heads"], cfg["ff"], cfg["layers"], 0]
    if cfg["kind"] == "encoder":
        return [cfg["d"], cfg["heads"], cfg["ff"], 0]
    if cfg["kind"] == "cnn":
        return [cfg["cin"], cfg["c1"], cfg["c2"], cfg["hw"], cfg["classes"]]
    return list(cfg["sizes"])


def step_flops(cfg):
    """Algorithmic GEMM + attention flops of one fwd+bwd step (per GPU)."""
    if cfg["kind"] == "decoder":
        t = cfg["batch"] * cfg["seq"]
        lin = cfg["layers"] * (4 * cfg["d"] ** 2 + 2 * cfg["d"] * cfg["ff"]) + cfg["vocab"] * cfg["d"]
        attn = cfg["layers"] * 14 * cfg["batch"] * cfg["heads"] * cfg["seq"] ** 2 * (cfg["d"] // cfg["heads"]) * 0.5
        return 6.0 * lin * t + attn
    if cfg["kind"] == "encoder":
        t = cfg["batch"] * cfg["seq"]
        return 6.0 * (4 * cfg["d"] ** 2 + 2 * cfg["d"] * cfg["ff"]) * t + 14 * cfg["batch"] * cfg["heads"] * cfg["seq"] ** 2 * (cfg["d"] // cfg["heads"])
    if cfg["kind"] == "cnn":
        hw, c0, c1, c2 = cfg["hw"], cfg["cin"], cfg["c1"], cfg["c2"]
        conv1 = 2.0 * hw * hw * c1 * c0 * 9            # per image: output positions x output channels x (C K K) MACs x 2
        conv2 = 2.0 * (hw // 2) ** 2 * c2 * c1 * 9
        fc = 2.0 * c2 * (hw // 4) ** 2 * cfg["classes"]
        return 3.0 * cfg["batch"] * (conv1 + conv2 + fc)  # forward + data gradient + weight gradient
    s = cfg["sizes"]
    return 6.0 * cfg["batch"] * (s[0] * s[1] + s[1] * s[2])


# ------------------------------------------------------------------ distributed plumbing
class Dist:
    def __init__(self, gpus):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.td = None
        if self.world > 1:
            import torch.distributed as td  # host-side rendezvous only; gradients travel through NCCL inside libmcb
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            td.init_process_group("gloo", rank=self.rank, world_size=self.world)
            self.td = td

    def barrier(self):
        if self.td:
            self.td.barrier()

    def bcast_bytes(self, b):
        if not self.td:
            return b
        obj = [b]
        self.td.broadcast_object_list(obj, src=0)
        return obj[0]

    def max(self, v):
        if not self.td:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        self.td.all_reduce(t, op=self.td.ReduceOp.MAX)
        return float(t[0])

    def close(self):
        if self.td:
            self.td.destroy_process_group()


# ------------------------------------------------------------------ our arm
def run_ours(args, dist):
    import modernchainer_b200 as mc
    name, cfg = args.workload, dict(WORKLOADS[args.workload])
    if args.layers and "layers" in cfg:
        cfg["layers"] = args.layers  # reduced depth for profiler captures; not a benchmark configuration
    ctx = mc.Context(dist.local)
    lib = ctx.lib
    pk = peaks()
    if cfg["kind"] == "optimizer":
        return run_c5(args, dist, mc, ctx, pk)
    if cfg["kind"] == "gemm":
        return run_gemm(args, dist, mc, ctx, pk)
    if dist.world > 1:
        uid = (C.c_char * 128)()
        if dist.rank == 0:
            ctx.check(lib.mcb_dp_unique_id(uid))
        raw = dist.bcast_bytes(bytes(uid))
        ctx.check(lib.mcb_dp_init(ctx.h, dist.rank, dist.world, raw))
    model = mc.Model(ctx, cfg["kind"], model_cfg(cfg))
    params = model.parameters()
    arena = mc.Arena(ctx, params)
    if dist.world > 1:
        ctx.check(lib.mcb_dp_attach(ctx.h, arena.h, args.bucket_mb << 20))
    opt = mc.Adam(ctx, 1e-3)
    scaler = mc.GradScaler(ctx, 65536.0) if cfg["amp"] else None
    x_np, y_np = make_inputs(name, cfg, dist.rank)
    x, y = mc.Variable.constant(ctx, x_np), mc.Variable.constant(ctx, y_np)

    # pinned staging buffers for the end-to-end loop
    def pinned(a):
        p = C.c_void_p()
        ctx.check(lib.mcb_host_alloc(a.nbytes, C.byref(p)))
        C.memmove(p, a.ctypes.data_as(C.c_void_p), a.nbytes)
        return p
    hx, hy = pinned(x_np), pinned(y_np)
    hloss = C.c_void_p()
    ctx.check(lib.mcb_host_alloc(8, C.byref(hloss)))
    xin, yin = ctx.empty(x_np.shape, mc.api._DT_OF[x_np.dtype]), ctx.empty(y_np.shape, mc.api._DT_OF[y_np.dtype])
    ctx.check(lib.mcb_memcpy_h2d(ctx.h, xin.ptr, hx, x_np.nbytes))
    ctx.check(lib.mcb_memcpy_h2d(ctx.h, yin.ptr, hy, y_np.nbytes))

    def var_of(dev, host):
        # variable whose storage is refreshed from pinned host memory every step
        return mc.Variable.constant(ctx, host)

    def one_step(xv, yv):
        mc.zero_grad(params)
        if cfg["amp"]:
            with mc.autocast(mc.BF16):
                loss = model.loss(xv, yv)
            scaler.scale_loss(loss).backward()
            scaler.step_async(opt, params)
        else:
            loss = model.loss(xv, yv)
            loss.backward()
            opt.update(params)
        return loss

    def e2e_step():
        # host -> device copy of this step's inputs from pinned memory, then the step, then the loss read-back
        ctx.check(lib.mcb_var_set_data(x.h, hx))
        ctx.check(lib.mcb_var_set_data(y.h, hy))
        loss = one_step(x, y)
        out = np.empty((), np.float32)
        ctx.check(lib.mcb_var_data(loss.h, out.ctypes.data_as(C.c_void_p)))
        return float(out)

    first_loss = last_loss = None
    sampler = ClockSampler(dist.local)
    if dist.rank == 0:
        sampler.start()  # nvidia-smi needs a moment before its first sample: start it ahead of the warm-up
    for i in range(args.warmup):
        l = one_step(x, y)
        if i == 0:
            first_loss = float(l.data)
    ctx.sync()
    dist.barrier()
    launches0 = ctx.launch_count()
    e0, e1 = ctx.event(), ctx.event()
    ctx.sync()
    dist.barrier()
    ctx.record(e0)
    for _ in range(args.steps):
        l = one_step(x, y)
    ctx.record(e1)
    ms_resident = ctx.elapsed_ms(e0, e1)
    ctx.sync()
    dist.barrier()
    launches = ctx.launch_count() - launches0
    last_loss = float(l.data)

    # end-to-end: inputs from pinned host memory every step, loss read back every step
    dist.barrier()
    ctx.sync()
    t0 = time.perf_counter()
    ctx.record(e0)
    for _ in range(args.steps):
        last_e2e = e2e_step()
    ctx.record(e1)
    ms_e2e_dev = ctx.elapsed_ms(e0, e1)
    ctx.sync()
    wall_e2e = (time.perf_counter() - t0) * 1e3
    dist.barrier()
    clocks = None
    if dist.world == 1:
        extra = sampler.cover(lambda: one_step(x, y), ctx.sync)
        clocks = sampler.stop()
        if extra:
            clocks["extra_untimed_steps"] = extra  # the timed steps alone were shorter than one sampling period
    elif dist.rank == 0:
        clocks = sampler.stop()

    # per-kernel-class device time over the same steps (event pairs around each launch group)
    ctx.check(lib.mcb_prof_enable(ctx.h, 1))
    for _ in range(min(args.steps, 3)):
        one_step(x, y)
    prof = {}
    for k, cname in enumerate(PROF_CLASSES):
        n, ms, fl, by = C.c_int64(), C.c_double(), C.c_double(), C.c_double()
        ctx.check(lib.mcb_prof_read(ctx.h, k, C.byref(n), C.byref(ms), C.byref(fl), C.byref(by)))
        if n.value:
            prof[cname] = dict(launches=n.value, ms=ms.value, flops=fl.value, bytes=by.value)
    ctx.check(lib.mcb_prof_enable(ctx.h, 0))

    # the same step captured as one CUDA Graph and replayed (single GPU): resident and end-to-end timings
    graph = None
    graph_error = None
    step = None
    if args.graph:
        try:
            step = mc.StaticStep(model, opt, x_np, y_np, scaler=scaler, autocast_dtype=mc.BF16 if cfg["amp"] else None)
        except mc.McbError as exc:  # stay on the tape path and say so
            graph_error = str(exc)
    if dist.max(0.0 if step is not None else 1.0) > 0.0 and step is not None:  # all ranks or none
        step.close()
        step = None
    if step is not None:
        for _ in range(args.warmup):
            ctx.check(lib.mcb_static_step_run(step.h, None, None))
        ctx.sync()
        dist.barrier()
        ctx.record(e0)
        for _ in range(args.steps):
            ctx.check(lib.mcb_static_step_run(step.h, None, None))
        ctx.record(e1)
        g_res = dist.max(ctx.elapsed_ms(e0, e1) / args.steps)
        ctx.sync()
        dist.barrier()
        # end to end: pinned host inputs copied every step and every step's loss read back, one step behind (the
        # public pipelined call: step i + 1 is queued on the device while the host waits for the loss of step i); the
        # last loss is drained inside the timed region
        prev, have = C.c_float(), C.c_int32()
        losses_read = 0
        t0 = time.perf_counter()
        for _ in range(args.steps):
            ctx.check(lib.mcb_static_step_run_pipelined(step.h, hx, hy, C.byref(prev), C.byref(have)))
            losses_read += have.value
        ctx.check(lib.mcb_static_step_drain(step.h, C.byref(prev), C.byref(have)))
        losses_read += have.value
        g_loss = prev.value
        g_e2e = dist.max((time.perf_counter() - t0) * 1e3 / args.steps)
        assert losses_read == args.steps, losses_read
        gb = cfg["batch"] * dist.world
        # the same replays once more beside the device-side clock sampler (a one-thread kernel reading %globaltimer and
        # clock64): the SM clock the step really runs at, which nvidia-smi's 200 ms samples cannot resolve
        sm_trace = None
        if dist.world == 1:  # with several ranks the replay holds collectives: no rank may run it alone
            dur_us = int(g_res * 1e3 * args.steps * 1.2) + 300
            ctx.check(lib.mcb_clock_trace_start(ctx.h, dur_us, max(10, dur_us // 200)))
            for _ in range(args.steps):
                ctx.check(lib.mcb_static_step_run(step.h, None, None))
            ctx.sync()
            mhz = (C.c_double * 256)()
            cnt = C.c_int32(0)
            ctx.check(lib.mcb_clock_trace_read(ctx.h, mhz, 256, C.byref(cnt)))
            tr = sorted(mhz[i] for i in range(cnt.value))
            if tr:
                sm_trace = {"median": tr[len(tr) // 2], "min": tr[0], "max": tr[-1], "samples": len(tr)}
        graph = {"ms_per_step": g_res, "samples_per_s": gb / (g_res / 1e3), "e2e_ms_per_step": g_e2e,
                 "e2e_samples_per_s": gb / (g_e2e / 1e3), "kernels_per_step": step.kernels_per_step, "loss_last": g_loss,
                 "sm_mhz_trace": sm_trace}
        step.close()

    ms_step = dist.max(ms_resident / args.steps)
    ms_step_e2e = dist.max(max(ms_e2e_dev, wall_e2e) / args.steps)
    global_batch = cfg["batch"] * dist.world
    # replicas must stay bit-identical: same init, same reduced gradients, same update on every rank
    in_sync = None
    if dist.world > 1:
        digest = [float(np.abs(params[i].data.astype(np.float64)).sum()) for i in (1, 3, len(params) - 1)]
        in_sync = dist.max(max(digest)) == max(digest) and -dist.max(-min(digest)) == min(digest) and \
            dist.max(digest[1]) == digest[1] and -dist.max(-digest[1]) == digest[1]
        in_sync = dist.max(0.0 if in_sync else 1.0) == 0.0
    result = None
    if dist.rank == 0:
        psteps = min(args.steps, 3)
        kernels = {}
        for cname, r in prof.items():
            sec = r["ms"] / 1e3
            kernels[cname] = dict(launches_per_step=r["launches"] / psteps, ms_per_step=r["ms"] / psteps,
                                  tflops=(r["flops"] / sec / 1e12) if r["flops"] and sec > 0 else None,
                                  gbs=(r["bytes"] / sec / 1e9) if r["bytes"] and sec > 0 else None)
        dom = max(prof, key=lambda c: prof[c]["ms"])
        r = prof[dom]
        if dom in ("gemm_tc", "gemm_f32", "attention", "conv"):
            achieved = r["flops"] / (r["ms"] / 1e3) / 1e12
            traffic = traffic_src = None
            if dom == "gemm_tc" and cfg["kind"] == "decoder" and (cfg["vocab"], cfg["d"], cfg["ff"], cfg["seq"], cfg["batch"]) == (32000, 768, 3072, 1024, 8):
                traffic, traffic_src = gemm_traffic(cfg["layers"])
            roof = dict(bound="tensor", kernel=dom, achieved=achieved, peak=pk["tf_sustained"], unit="TFLOP/s", frac=achieved / pk["tf_sustained"],
                        traffic=traffic, traffic_source=traffic_src, peak_source=pk["src"] + " (sustained cuBLAS bf16)",
                        avg_launch_ms=r["ms"] / r["launches"])
        else:
            achieved = r["bytes"] / (r["ms"] / 1e3) / 1e9
            roof = dict(bound="hbm", kernel=dom, achieved=achieved, peak=pk["hbm"], unit="GB/s", frac=achieved / pk["hbm"], traffic=None,
                        peak_source=pk["src"], avg_launch_ms=r["ms"] / r["launches"])
        tape = {"ms_per_step": ms_step, "e2e_ms_per_step": ms_step_e2e, "gpu_launches": int(launches)}
        path = "tape (one launch per kernel)" + (f"; graph capture failed: {graph_error}" if graph_error else "")
        if graph:  # the headline is the step as a user would run it in a loop: captured once, replayed
            ms_step, ms_step_e2e = graph["ms_per_step"], graph["e2e_ms_per_step"]
            launches = graph["kernels_per_step"] * args.steps
            path = "cuda graph replay of the recorded tape step (StaticStep)"
        result = {
            "metric": "train samples/sec (fwd+bwd+Adam, device-timed, max over ranks)", "value": global_batch / (ms_step / 1e3),
            "unit": "samples/s", "n_gpus": dist.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "step_path": path, "tape_step": tape,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if cfg["amp"] else "f32", "data": "synthetic",
            "config": {"workload": workload_string(name, cfg), "global_batch": global_batch,
                       "parallelism": f"dp{dist.world}", "l2": "per-step working set (activations + 3.8 GB optimizer state) exceeds the 126 MB L2",
                       "grad_bucket_mb": args.bucket_mb},
            "e2e": {"value": global_batch / (ms_step_e2e / 1e3), "unit": "samples/s", "h2d_bytes_per_step": int(x_np.nbytes + y_np.nbytes),
                    "d2h_bytes_per_step": 4, "ms_per_step": ms_step_e2e,
                    "note": "every step copies its inputs from pinned host memory and every step's loss is read on the host; on the graph path the loss "
                            "of step i is read while step i + 1 runs (mcb_static_step_run_pipelined), the last one before the clock stops"},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "kernels": kernels,
            "model_tflops": step_flops(cfg) / (ms_step / 1e3) / 1e12, "loss_first": first_loss, "loss_last": last_loss,
            "replicas_in_sync": in_sync, "cuda_graph_step": graph,
        }
        if "optimizer" in kernels and kernels["optimizer"]["gbs"]:
            # the GradScaler scan + unscale + Adam pass of THIS step (28 bytes per parameter with f32 gradients, 26 with 16-bit ones),
            # against the measured HBM copy peak: the c5 workload's figure at this model's parameter count
            result["fused_update_hbm"] = {"achieved": kernels["optimizer"]["gbs"], "peak": pk["hbm"], "unit": "GB/s",
                                          "frac": kernels["optimizer"]["gbs"] / pk["hbm"], "peak_source": pk["src"]}
    if dist.world > 1:
        ctx.check(lib.mcb_dp_shutdown(ctx.h))
    return result


def run_gemm(args, dist, mc, ctx, pk):
    """Single tcgen05 GEMM shape, timed alone (used for per-shape roofline numbers and ncu captures).
    --gemm m,n,k[,a_mn,b_mn]: D[m,n] = A B with bf16 operands, bf16 output."""
    lib = ctx.lib
    f = [int(v) for v in args.gemm.split(",")]
    m, n, k = f[:3]
    a_mn, b_mn = (f[3], f[4]) if len(f) >= 5 else (0, 0)
    rng = np.random.default_rng(0)
    a = ctx.array(rng.standard_normal(m * k).astype(np.float32), mc.BF16)
    b = ctx.array(rng.standard_normal(n * k).astype(np.float32), mc.BF16)
    d = ctx.zeros((m * n,), mc.BF16)

    def run():
        ctx.check(lib.mcb_gemm_bf16(ctx.h, a.ptr, a_mn, b.ptr, b_mn, d.ptr, mc.BF16, None, m, n, k, 0, 1))
    for _ in range(args.warmup):
        run()
    e0, e1 = ctx.event(), ctx.event()
    ctx.record(e0)
    for _ in range(args.steps):
        run()
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1) / args.steps
    tf = 2.0 * m * n * k / (ms / 1e3) / 1e12
    # the same loop once more beside the device-side clock sampler: the SM clock these launches really ran at
    import ctypes as C
    dur_us = int(ms * 1e3 * args.steps * 1.2) + 300
    ctx.check(lib.mcb_clock_trace_start(ctx.h, dur_us, max(10, dur_us // 100)))
    for _ in range(args.steps):
        run()
    mhz = (C.c_double * 256)()
    cnt = C.c_int32(0)
    ctx.check(lib.mcb_clock_trace_read(ctx.h, mhz, 256, C.byref(cnt)))
    tr = sorted(mhz[i] for i in range(cnt.value))
    trace = {"median": tr[len(tr) // 2], "min": tr[0], "max": tr[-1], "samples": len(tr)} if tr else None
    return {"metric": "bf16 GEMM TFLOP/s", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "sm_mhz_trace": trace,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"gemm m={m} n={n} k={k} a_mn={a_mn} b_mn={b_mn}"}, "gpu_launches": args.steps,
            "roofline": {"bound": "tensor", "kernel": "tc_gemm_kernel", "achieved": tf, "peak": pk["tf_burst"], "unit": "TFLOP/s",
                         "frac": tf / pk["tf_burst"], "traffic": None, "peak_source": pk["src"] + " (burst cuBLAS bf16)"}}


def run_c5(args, dist, mc, ctx, pk):
    """Optimizer-path stress test: fused inf/nan check + unscale + Adam over a flat buffer."""
    lib = ctx.lib
    n = args.n_params or WORKLOADS["c5"]["n"]
    rng = np.random.default_rng(1238)
    scale = 65536.0
    p = ctx.array(rng.standard_normal(n, dtype=np.float32) * np.float32(0.02))
    m, v, shadow = ctx.zeros((n,)), ctx.zeros((n,)), ctx.empty((n,), mc.BF16)
    g_clean = mc.f32_to_bf16_bits(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-3 * scale))
    g_bad = g_clean.copy()
    pos = rng.choice(n, 12500, replace=False)
    g_bad[pos[:6250:2]] = 0x7F80
    g_bad[pos[1:6250:2]] = 0xFF80
    g_bad[pos[6250:]] = 0x7FC0
    dg = [ctx.array(g_clean, mc.BF16), ctx.array(g_bad, mc.BF16)]
    flag = ctx.zeros((1,), mc.I32)
    hflag = np.zeros(1, np.int32)

    def step(i, e2e=False):
        g = dg[i & 1]  # inf/nan present on odd steps
        ctx.check(lib.mcb_memset(ctx.h, flag.ptr, 0, 4))
        ctx.check(lib.mcb_check_finite(ctx.h, g.ptr, mc.BF16, n, flag.ptr))
        ctx.check(lib.mcb_adam_flat(ctx.h, p.ptr, g.ptr, mc.BF16, m.ptr, v.ptr, shadow.ptr, n, 1e-3, 0.9, 0.999, 1e-8, i // 2 + 1, 1.0 / scale, flag.ptr))
        if e2e:
            ctx.check(lib.mcb_memcpy_d2h(ctx.h, hflag.ctypes.data_as(C.c_void_p), flag.ptr, 4))

    for i in range(args.warmup):
        step(i)
    ctx.sync()
    sampler = ClockSampler(dist.local)
    sampler.start()
    l0 = ctx.launch_count()
    e0, e1 = ctx.event(), ctx.event()
    ctx.record(e0)
    for i in range(args.steps):
        step(i)
    ctx.record(e1)
    ms = ctx.elapsed_ms(e0, e1)
    launches = ctx.launch_count() - l0
    ctx.record(e0)
    for i in range(args.steps):
        step(i, e2e=True)
    ctx.record(e1)
    ms_e2e = ctx.elapsed_ms(e0, e1)
    nxt = [args.steps]

    def again():
        step(nxt[0])
        nxt[0] += 1
    extra = sampler.cover(again, ctx.sync)
    clocks = sampler.stop()
    if extra:
        clocks["extra_untimed_steps"] = extra
    applied = (args.steps + 1) // 2
    skipped = args.steps - applied
    # algorithmic bytes: applied step 26 B/param (+2 for the bf16 shadow this library also writes), skipped step 2 B/param
    alg = applied * 28.0 * n + skipped * 2.0 * n
    gbs = alg / (ms / 1e3) / 1e9
    # isolated timing of the applied pass for the roofline entry
    ctx.check(lib.mcb_prof_enable(ctx.h, 1))
    for i in range(0, 8, 2):
        step(i)
    cnt, pms, fl, by = C.c_int64(), C.c_double(), C.c_double(), C.c_double()
    ctx.check(lib.mcb_prof_read(ctx.h, 3, C.byref(cnt), C.byref(pms), C.byref(fl), C.byref(by)))
    ctx.check(lib.mcb_prof_enable(ctx.h, 0))
    ach = by.value / (pms.value / 1e3) / 1e9
    return {
        "metric": "fused GradScaler check + unscale + Adam, HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": workload_string("c5", WORKLOADS["c5"]),
                                        "l2": "3.5 GB working set exceeds the 126 MB L2"},
        "e2e": {"value": alg / (ms_e2e / 1e3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "check_finite + adam_flat (applied steps)", "achieved": ach, "peak": pk["hbm"], "unit": "GB/s",
                     "frac": ach / pk["hbm"], "traffic": None, "peak_source": pk["src"]},
    }


# ------------------------------------------------------------------ CPU arm
def cpu_sample(name, threads_note=True):
    """Times a bounded sample of the workload on the CPU oracle (threaded build) and returns
    (samples_per_sec, cores, description)."""
    from oracle import ref
    ref.build()
    ref.use_fast(True)
    cores = ref.lib(True).mco_num_threads()
    cfg = WORKLOADS[name]
    rng = np.random.default_rng(99)
    t0 = time.perf_counter()
    if cfg["kind"] == "decoder":
        # one full-length sequence through one decoder layer, and one through embedding + final norm + lm_head + loss;
        # a sample of the workload costs layers * t_layer + t_head (declared: the 12-layer step at batch 8 takes minutes).
        # Each is run three times (about 10-20 s of CPU work in all) and the fastest run counts.
        seq, d = cfg["seq"], cfg["d"]
        ids = rng.integers(0, cfg["vocab"], (1, seq)).astype(np.int64)
        m1 = ref.Decoder(cfg["vocab"], d, cfg["heads"], cfg["ff"], 1, 0)
        m0 = ref.Decoder(cfg["vocab"], d, cfg["heads"], cfg["ff"], 0, 0)
        opt = ref.Adam(1e-3)

        def run(m):
            best = None
            for _ in range(3):
                t = time.perf_counter()
                ref.zero_grad(m.parameters())
                loss = m.loss(ref.Variable.constant(ids), ref.Variable.constant(ids))
                loss.backward()
                opt.update(m.parameters())
                dt = time.perf_counter() - t
                best = dt if best is None else min(best, dt)
            return best
        t_head = run(m0)
        t_both = run(m1)
        t_layer = max(t_both - t_head, 1e-9)
        per_sample = cfg["layers"] * t_layer + t_head
        desc = (f"oracle (C restatement of the reference CPU backend, {cores} OpenMP threads), batch 1 of {cfg['batch']}: fwd+bwd+Adam of 1 sequence of {seq} tokens through "
                f"1 layer ({t_layer:.2f} s) and through embedding+head+loss ({t_head:.2f} s), best of 3 each; samples/s = 1 / ({cfg['layers']}*layer + head)")
        return 1.0 / per_sample, cores, desc
    if cfg["kind"] == "encoder":
        b = 2
        x = rng.standard_normal((b, cfg["seq"], cfg["d"])).astype(np.float32)
        m = ref.EncoderBlock(cfg["d"], cfg["heads"], cfg["ff"])
        opt = ref.Adam(1e-3)
        t = time.perf_counter()
        loss = m.loss(ref.Variable.constant(x), ref.Variable.constant(x))
        loss.backward()
        opt.update(m.parameters())
        dt = time.perf_counter() - t
        return b / dt, cores, f"oracle, {cores} threads: one fwd+bwd+Adam step at batch {b} of {cfg['batch']}"
    if cfg["kind"] == "cnn":
        x, y = make_inputs(name, cfg, 0)
        m, opt = ref.CNN(cfg["cin"], cfg["c1"], cfg["c2"], cfg["hw"], cfg["classes"]), ref.Adam(1e-3)
        reps = 3
        t = time.perf_counter()
        for _ in range(reps):
            ref.zero_grad(m.parameters())
            loss = m.loss(ref.Variable.constant(x), ref.Variable.constant(y))
            loss.backward()
            opt.update(m.parameters())
        dt = (time.perf_counter() - t) / reps
        return cfg["batch"] / dt, cores, (f"oracle, {cores} threads over samples / output channels (the reference runs its conv and pool host ops on one thread): "
                                          f"mean of {reps} full steps at batch {cfg['batch']}")
    if cfg["kind"] == "mlp":
        x, y = make_inputs(name, cfg, 0)
        m, opt = ref.MLP(cfg["sizes"]), ref.Adam(1e-3)
        reps = 20
        t = time.perf_counter()
        for _ in range(reps):
            ref.zero_grad(m.parameters())
            loss = m.loss(ref.Variable.constant(x), ref.Variable.constant(y))
            loss.backward()
            opt.update(m.parameters())
        dt = (time.perf_counter() - t) / reps
        return cfg["batch"] / dt, cores, f"oracle, {cores} threads: mean of {reps} full steps"
    n = 8_000_000
    p, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    t = time.perf_counter()
    ref.count_non_finite(g)
    ref.adam_update(p, ref.scale(g, 1.0 / 65536.0), m, v, 1e-3, 0.9, 0.999, 1e-8, 1)
    dt = time.perf_counter() - t
    return 28.0 * n / dt / 1e9, cores, f"oracle, {cores} threads: scan + unscale + Adam over {n} parameters"


def workload_string(name, cfg):
    """The `config.workload` of a line: the same for this library's arm and for the reference arm."""
    if name == "c5":
        return "c5: flat 125M f32 params, bf16 grads pre-multiplied by 2^16, inf/nan on odd steps"
    return f"{name}: " + json.dumps({k: v for k, v in cfg.items()})


def run_reference(args, dist):
    if dist.rank != 0:
        return None
    vals = []
    for _ in range(max(1, min(args.steps, 3))):
        v, cores, desc = cpu_sample(args.workload)
        vals.append(v)
    v = float(np.median(vals))
    unit = "GB/s" if args.workload == "c5" else "samples/s"
    return {"impl": "reference", "metric": "train samples/sec (fwd+bwd+Adam, device-timed, max over ranks)" if unit != "GB/s" else "fused GradScaler check + unscale + Adam, HBM GB/s",
            "value": v, "unit": unit, "n_gpus": dist.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_string(args.workload, WORKLOADS[args.workload]),
                       "note": "the reference is Rust and cannot be built here; this arm times the C restatement of its CPU backend on the host cores, "
                               "on a bounded sample of the same workload (cpu_baseline.sample)"},
            "cpu_baseline": {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c4", choices=list(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bucket-mb", type=int, default=64, help="gradient all-reduce bucket (measured at N=8: 64 MB 11.5 ms, 32 MB 11.8 ms per step)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--n-params", type=int, default=0, help="c5 only: number of parameters (default 125M)")
    ap.add_argument("--gemm", default="8192,3072,768", help="gemm workload: m,n,k[,a_mn,b_mn]")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="time only the tape step (one launch per kernel), not its CUDA Graph replay")
    ap.add_argument("--layers", type=int, default=0, help="c4 only: override the layer count (small cases for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    # stdout carries exactly one JSON line: whatever libraries print on file descriptor 1 while the run lasts
    # (NCCL's version banner, for one) goes to stderr instead
    sys.stdout.flush()
    out_fd = os.dup(1)
    os.dup2(2, 1)
    dist = Dist(args.gpus)
    if args.impl == "reference":
        res = run_reference(args, dist)
    else:
        res = run_ours(args, dist)
        if res is not None and dist.world == 1 and not args.no_cpu_baseline and args.workload in ("c1", "c2", "c3", "c4", "c5"):
            v, cores, desc = cpu_sample(args.workload)
            res["cpu_baseline"] = {"value": v, "unit": res["unit"], "cores": cores, "kind": "port", "sample": desc}
    dist.close()
    sys.stdout.flush()
    os.dup2(out_fd, 1)
    os.close(out_fd)
    if dist.rank == 0 and res is not None:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
