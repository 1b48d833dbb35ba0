#!/usr/bin/env python
"""Headline benchmark: training samples/s (forward + backward + AdamW) of the
CIFAR-shaped VGG-style CNN, global batch 1024 sharded over N GPUs, f32 with
3xTF32 contractions, synthetic data, He-initialised weights.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload vgg_cifar|vgg_cifar_bn|small_cnn|wide_mlp|transformer_lm] [--math 3xtf32|tf32|fp32]

For N > 1 launch under torchrun (one rank per GPU); run without torchrun the
script re-launches itself through `python -m torch.distributed.run`.
Rank 0 prints ONE JSON line.

* value        whole-job samples/s with the step's inputs already resident in HBM
* e2e          the same through the host-buffer entry points (nrs_trainer_stage_next +
               nrs_trainer_step_staged): pinned host inputs copied in (the copy of batch i+1
               overlapping step i), loss copied out, every step; `unpipelined_value` is the
               plain nrs_trainer_step (copy, step, read-back in sequence)
* roofline     the dominant contraction family, timed with CUDA events bracketed around
               its launches inside the timed region (nrs_profile_*; every fourth timed step)
* cpu_baseline the CPU restatement of the reference's training loop (oracle/), timed on
               this host on a bounded batch
* --impl reference  times that CPU restatement alone (the reference is a Rust crate and
               no Rust toolchain exists in the image, so its own binary cannot be built)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "train samples/s (fwd+bwd+AdamW)"
WORKLOADS = {"vgg_cifar": ("VGG_CIFAR", 1024, 3), "small_cnn": ("SMALL_CNN", 64, 1), "wide_mlp": ("WIDE_MLP", 16384, 5),
             "vgg_cifar_bn": ("VGG_CIFAR_BN", 1024, 7)}
CPU_SAMPLE_BATCH = {"vgg_cifar": 16, "small_cnn": 64, "wide_mlp": 32, "vgg_cifar_bn": 16}
MATH = {"3xtf32": 0, "tf32": 1, "fp32": 2}
PROF_NAMES = ["conv_fwd", "conv_dgrad", "conv_wgrad", "gemm", "adamw", "batchnorm"]


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="vgg_cifar", choices=list(WORKLOADS) + ["transformer_lm"])
    ap.add_argument("--math", default="3xtf32", choices=list(MATH))
    ap.add_argument("--global-batch", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fuse", action="store_true")
    return ap.parse_args()


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_burst=float(d["bf16_tflops"]),
                    bf16_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


def model_flops_per_sample(layers, in_shape):
    """Algorithmic FLOP of one forward pass per sample, and of forward+backward (the first
    layer's data gradient is not computed: its input does not require a gradient)."""
    shp = list(in_shape)
    fwd = 0.0
    total = 0.0
    first = True
    for l in layers:
        if l[0] == "conv":
            _, ci, co, k, s, p = l
            oh, ow = (shp[1] + 2 * p - k) // s + 1, (shp[2] + 2 * p - k) // s + 1
            f = 2.0 * co * oh * ow * ci * k * k
            fwd += f
            total += f * (2 if first else 3)
            shp = [co, oh, ow]
            first = False
        elif l[0] == "linear":
            f = 2.0 * l[1] * l[2]
            fwd += f
            total += f * (2 if first else 3)
            shp = [l[2]]
            first = False
        elif l[0] == "maxpool":
            shp = [shp[0], (shp[1] - l[1]) // l[2] + 1, (shp[2] - l[1]) // l[2] + 1]
        elif l[0] == "flatten":
            n = 1
            for d in shp:
                n *= d
            shp = [n]
    return fwd, total


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._proc, self._t0 = index, [], None, 0.0

    def __enter__(self):
        # one long-running sampler (50 ms period): a fresh nvidia-smi per sample takes longer than a short timed region
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu=timestamp,{self.Q}",
                                           "--format=csv,noheader,nounits", "-lms", "50"],
                                          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.3)          # let it come up; samples from before this point are dropped
        except Exception:
            self._proc = None
        self._t0 = time.time()
        return self

    def __exit__(self, *a):
        if not self._proc:
            return
        t1 = time.time()
        self._proc.terminate()
        try:
            out, _ = self._proc.communicate(timeout=5)
        except Exception:
            self._proc.kill()
            out = ""
        import datetime
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
            except ValueError:
                continue
            if self._t0 - 0.02 <= ts <= t1 + 0.02:
                self.rows.append(parts[1:])

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def cpu_reference_run(workload: str, steps: int, warmup: int, min_seconds: float = 0.0):
    """Times the CPU restatement of the reference's training loop on a bounded batch."""
    from oracle import models
    from oracle.nrs_oracle import Oracle
    cfg = getattr(models, WORKLOADS[workload][0])
    seed = 1234 + WORKLOADS[workload][2]
    batch = CPU_SAMPLE_BATCH[workload]
    o = Oracle("f32")
    params = models.he_init(cfg["layers"], seed)
    hp = models.ADAMW_HP
    opt = models.OracleAdamW(o, hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["wd"])
    x, t = models.synthetic_batch(cfg, batch, seed + 1, uniform01=(workload == "small_cnn"))
    extra = dict(buffers=models.bn_buffers(cfg["layers"]), rng={"seed": seed, "offset": 0})
    for _ in range(max(0, warmup)):
        models.train_step(o, cfg["layers"], params, opt, x, t, **extra)
    done = 0
    t0 = time.perf_counter()
    while done < steps or (time.perf_counter() - t0) < min_seconds:
        models.train_step(o, cfg["layers"], params, opt, x, t, **extra)
        done += 1
        if done >= steps and min_seconds <= 0:
            break
        if time.perf_counter() - t0 > 120:
            break
    dt = time.perf_counter() - t0
    cores = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    return dict(value=batch * done / dt, ms_per_step=1e3 * dt / done, steps=done, batch=batch, cores=cores,
                sample=f"{done} training steps of {cfg['name']} at batch {batch} "
                       f"(conv/matmul loops OpenMP-parallel as the reference's Rayon loops are)")


def conv_microbench(ctx, stream, iters=10):
    """The conv microbenchmark configuration: Conv2d [256,64,32,32] -> 128, 3x3 s1 p1; forward, data gradient and weight
    gradient timed separately through the raw C ABI (staging included), algorithmic TFLOP/s each."""
    import ctypes as C
    import torch
    from neuralrs_b200 import _lib
    l = _lib.lib()
    n, ci, h, w, co = 256, 64, 32, 32, 128
    g = torch.Generator(device="cuda").manual_seed(1236)
    x = torch.randn(n, ci, h, w, device="cuda", generator=g)
    wt = torch.randn(co, ci, 3, 3, device="cuda", generator=g) * (2.0 / (ci * 9)) ** 0.5
    b = torch.zeros(co, device="cuda")
    dy = torch.randn(n, co, h, w, device="cuda", generator=g)
    y, dx, dw = torch.empty_like(dy), torch.empty_like(x), torch.empty_like(wt)
    P = lambda t: C.c_void_p(t.data_ptr())
    dims = (n, ci, h, w, co, 3, 3, 1, 1)
    calls = {
        "fwd": lambda: l.nrs_conv2d_fwd(ctx.h, P(x), P(wt), P(b), P(y), *dims, 0),
        "dgrad": lambda: l.nrs_conv2d_bwd(ctx.h, P(x), P(wt), P(dy), P(dx), None, None, *dims, 0),
        "wgrad": lambda: l.nrs_conv2d_bwd(ctx.h, P(x), P(wt), P(dy), None, P(dw), None, *dims, 0),
    }
    flop = 2.0 * n * co * h * w * ci * 9
    out = {"shape": "x[256,64,32,32] w[128,64,3,3] s1 p1", "gflop_per_pass": flop / 1e9}
    for name, fn in calls.items():
        for _ in range(3):
            _lib.check(ctx.h, fn())
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            _lib.check(ctx.h, fn())
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        out[name] = {"ms": ms, "tflops": flop / (ms / 1e3) / 1e12}
    return out


def batchnorm_microbench(ctx, stream, hbm_peak_gbs, iters=10):
    """BatchNorm2d (training mode) and Dropout on the conv microbenchmark's activation shape [256,64,32,32]
    through the raw C ABI.  HBM-bound: the algorithmic bytes are one read of every input tensor and one write
    of every output tensor (forward x -> y, xhat: 3 tensors; backward g, xhat -> dx: 3 tensors; dropout
    a, mask -> out: 3 tensors); the kernels read their inputs twice (statistics, then the elementwise pass),
    which the fraction shows."""
    import ctypes as C
    import torch
    from neuralrs_b200 import _lib
    l = _lib.lib()
    n, c, h, w = 256, 64, 32, 32
    g = torch.Generator(device="cuda").manual_seed(1240)
    x = torch.randn(n, c, h, w, device="cuda", generator=g) * 2 + 1
    dy = torch.randn(n, c, h, w, device="cuda", generator=g)
    gamma, beta = torch.ones(c, device="cuda"), torch.zeros(c, device="cuda")
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    y, xhat, dx, mask = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    istd, dg, db = torch.empty(c, device="cuda"), torch.empty(c, device="cuda"), torch.empty(c, device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())
    F = C.c_float
    tensor_bytes = x.numel() * 4
    calls = {
        "bn_fwd": (3, lambda: l.nrs_batchnorm_fwd(ctx.h, P(x), P(gamma), P(beta), P(rm), P(rv), P(y), P(xhat), P(istd),
                                                  n, c, h * w, F(1e-5), F(0.9), 1)),
        "bn_bwd": (3, lambda: l.nrs_batchnorm_bwd(ctx.h, P(dy), P(xhat), P(istd), P(gamma), P(dx), P(dg), P(db),
                                                  n, c, h * w, 1, 0, 0)),
        "dropout_mask": (1, lambda: l.nrs_dropout_mask(ctx.h, P(mask), x.numel(), F(0.3))),
        "mask_mul": (3, lambda: l.nrs_mask_mul(ctx.h, P(x), P(mask), P(y), x.numel(), 1, 0)),
    }
    out = {"shape": "x[256,64,32,32]", "tensor_mb": tensor_bytes / 1e6, "hbm_peak_gbs": hbm_peak_gbs}
    for name, (tensors, fn) in calls.items():
        for _ in range(3):
            _lib.check(ctx.h, fn())
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            _lib.check(ctx.h, fn())
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        gbs = tensors * tensor_bytes / (ms / 1e3) / 1e9
        out[name] = {"ms": ms, "algorithmic_gbs": gbs, "frac": gbs / hbm_peak_gbs}
    return out


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel of a family from
# the `ncu --set full` captures summarised under profiles/: (bytes, per-GPU batch of the capture,
# kernel).  Traffic of these kernels is proportional to the pixel count, so it is scaled to the
# per-GPU batch of this run.
NCU_TRAFFIC = {
    ("vgg_cifar", "3xtf32", "conv_wgrad"): (270.87e6 + 3.69e6, 256, "tc_wgrad_rows_kernel<2,4> (64->64 ch, 32x32)"),
    ("vgg_cifar", "3xtf32", "conv_fwd"): (68.37e6 + 5.44e6, 256, "tc_kernel<128,2,ConvPolicy> (128->128 ch, 16x16)"),
    ("vgg_cifar", "3xtf32", "conv_dgrad"): (68.37e6 + 5.44e6, 256, "tc_kernel<128,2,ConvPolicy> (128->128 ch, 16x16)"),
}


def ncu_traffic(workload, math, family, per_gpu_batch):
    hit = NCU_TRAFFIC.get((workload, math, family))
    if not hit:
        return {"traffic": None}
    nbytes, cap_batch, kernel = hit
    return {"traffic": nbytes * per_gpu_batch / cap_batch, "traffic_unit": "bytes per launch", "traffic_kernel": kernel,
            "traffic_source": f"ncu --set full capture at per-GPU batch {cap_batch} (profiles/), scaled by the pixel count"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    global_batch = args.global_batch or WORKLOADS[args.workload][1]
    r = cpu_reference_run(args.workload, args.steps, min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "samples/s", "n_gpus": args.gpus,
        "steps": r["steps"], "warmup": min(args.warmup, 1), "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "global_batch": global_batch, "cpu_sample_batch": r["batch"],
                   "note": "CPU restatement of the reference's own training loop (oracle/); the Rust crate cannot "
                           "be built here (no cargo/rustc in the image)"},
        "cpu_baseline": {"value": r["value"], "unit": "samples/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from neuralrs_b200 import _lib, cuda
    from oracle import models   # model tables + synthetic data only; never on the timed path

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cfg = getattr(models, WORKLOADS[args.workload][0])
    seed = 1234 + WORKLOADS[args.workload][2]
    global_batch = args.global_batch or WORKLOADS[args.workload][1]
    b0, b1 = cuda.dp_shard_range(global_batch, rank, world)
    batch = b1 - b0

    ctx = cuda.Context(local_rank)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    ctx.set_math_mode(MATH[args.math])
    hp = models.ADAMW_HP
    tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                      hp["wd"], fuse=not args.no_fuse, ctx=ctx)
    tr.set_params(models.he_init(cfg["layers"], seed))       # identical bytes on every rank
    if world > 1:
        box = [cuda.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        tr.enable_dp(rank, world, box[0], global_batch)

    # Synthetic batches: a few distinct ones, rotated, pinned on the host and resident on the device.
    n_sets = 4
    xs_pin, ts_pin, xs_dev, ts_dev = [], [], [], []
    for i in range(n_sets):
        x, t = models.synthetic_batch(cfg, global_batch, seed + 10 + i, uniform01=(args.workload == "small_cnn"))
        xp = torch.from_numpy(np.ascontiguousarray(x[b0:b1])).pin_memory()
        tp = torch.from_numpy(np.ascontiguousarray(t[b0:b1])).pin_memory()
        xs_pin.append(xp); ts_pin.append(tp)
        xs_dev.append(xp.cuda(non_blocking=True)); ts_dev.append(tp.cuda(non_blocking=True))
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        barrier()
        if world > 1:
            tms = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            ms = float(tms.item())
        return ms

    dev_step = lambda i: tr.step_device(xs_dev[i % n_sets].data_ptr(), ts_dev[i % n_sets].data_ptr(), batch, False)
    host_step = lambda i: tr.step_ptr(xs_pin[i % n_sets].data_ptr(), ts_pin[i % n_sets].data_ptr(), batch, True)

    def staged_loop(total):
        """End-to-end steps with the input copy double-buffered: batch i+1 is staged (asynchronous copy from
        pinned memory on the copy stream) before step i is issued; every step still reads its loss back."""
        def fn(i):
            if i == 0:
                tr.stage_next_ptr(xs_pin[0].data_ptr(), ts_pin[0].data_ptr(), batch)
            if i + 1 < total:
                j = (i + 1) % n_sets
                tr.stage_next_ptr(xs_pin[j].data_ptr(), ts_pin[j].data_ptr(), batch)
            tr.step_staged(True)
        return fn

    for i in range(max(3, args.warmup)):
        dev_step(i)
    l = _lib.lib()
    _lib.check(ctx.h, l.nrs_profile_reset(ctx.h))
    # The per-family CUDA-event brackets sit between kernels, where they defeat the chaining of
    # consecutive launches; they are switched on for every fourth timed step only (the first
    # included), and the family figures are scaled to the bracketed steps.
    bracket_every = 4
    bracketed = len(range(0, args.steps, bracket_every))

    def dev_step_bracketed(i):
        l.nrs_profile_enable(ctx.h, 1 if i % bracket_every == 0 else 0)
        dev_step(i)
    launches0 = ctx.launch_count()
    with ClockSampler(local_rank) as clk:
        ms = timed(dev_step_bracketed, args.steps)
    launches = ctx.launch_count() - launches0
    import ctypes as C
    prof = {}
    for kind, name in enumerate(PROF_NAMES):
        pms, work, calls = C.c_double(), C.c_double(), C.c_uint64()
        _lib.check(ctx.h, l.nrs_profile_get(ctx.h, kind, C.byref(pms), C.byref(work), C.byref(calls)))
        prof[name] = dict(ms=pms.value, work=work.value, calls=int(calls.value))
    _lib.check(ctx.h, l.nrs_profile_enable(ctx.h, 0))
    _lib.check(ctx.h, l.nrs_profile_reset(ctx.h))
    loss = tr.last_loss()

    for i in range(2):
        host_step(i)
    ms_e2e_plain = timed(host_step, args.steps)
    warm = staged_loop(2)
    for i in range(2):
        warm(i)
    ms_e2e = timed(staged_loop(args.steps), args.steps)

    if rank == 0:
        peaks = measured_peaks()
        value = global_batch * args.steps / (ms / 1e3)
        e2e_value = global_batch * args.steps / (ms_e2e / 1e3)
        fwd_flop, step_flop = model_flops_per_sample(cfg["layers"], cfg["in_shape"])
        # dominant contraction family by device time
        fam = max(("conv_fwd", "conv_dgrad", "conv_wgrad", "gemm"), key=lambda k: prof[k]["ms"])
        f = prof[fam]
        achieved = (f["work"] / (f["ms"] / 1e3) / 1e12) if f["ms"] > 0 else 0.0
        tf32_peak = peaks["bf16_sustained"] / 2.0
        contraction_ms = sum(prof[k]["ms"] for k in ("conv_fwd", "conv_dgrad", "conv_wgrad", "gemm"))
        contraction_work = sum(prof[k]["work"] for k in ("conv_fwd", "conv_dgrad", "conv_wgrad", "gemm"))
        adam = prof["adamw"]
        x_bytes = sum(int(np.prod((global_batch,) + tuple(cfg["in_shape"]))) * 4 for _ in range(1))
        t_bytes = global_batch * cfg["classes"] * 4
        line = {
            "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "global_batch": global_batch, "per_gpu_batch": batch,
                       "parallelism": f"dp{world}", "math": args.math, "fused_epilogues": not args.no_fuse,
                       "init": "He N(0,sqrt(2/fan_in)), seed %d" % seed,
                       "l2": "per-step working set (activations + gradients) is several times the 126 MB L2; "
                             "4 input batches rotated",
                       "algorithmic_gflop_per_step": step_flop * global_batch / 1e9,
                       "tensor_core_path": bool(l.nrs_has_tensor_core_path())},
            "loss": loss,
            "e2e": {"value": e2e_value, "unit": "samples/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": x_bytes + t_bytes, "d2h_bytes_per_step": 4 * world,
                    "api": "nrs_trainer_stage_next + nrs_trainer_step_staged: the copy of batch i+1 overlaps step i",
                    "unpipelined_value": global_batch * args.steps / (ms_e2e_plain / 1e3),
                    "unpipelined_api": "nrs_trainer_step: copy, step and loss read-back in sequence"},
            "gpu_launches": launches * world,
            "clocks": clk.summary(),
            "roofline": {"bound": "tensor", "kernel": fam, "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                         "frac": achieved / tf32_peak if tf32_peak else None,
                         **ncu_traffic(args.workload, args.math, fam, batch),
                         "peak_source": f"{peaks['source']}: sustained bf16 cuBLAS / 2 (dense TF32 runs at half the bf16 "
                                        f"rate); 3xTF32 issues 3x the algorithmic FLOP counted in `achieved`",
                         "launch_ms_avg": f["ms"] / f["calls"] if f["calls"] else None, "calls": f["calls"],
                         "all_contractions_tflops": (contraction_work / (contraction_ms / 1e3) / 1e12) if contraction_ms else None,
                         "families_ms_per_step": {k: prof[k]["ms"] / bracketed for k in prof},
                         "bracketed_steps": bracketed,
                         "adamw_gbs": (adam["work"] / (adam["ms"] / 1e3) / 1e9) if adam["ms"] > 0 else None,
                         "batchnorm_gbs": (prof["batchnorm"]["work"] / (prof["batchnorm"]["ms"] / 1e3) / 1e9)
                         if prof["batchnorm"]["ms"] > 0 else None,
                         "hbm_peak_gbs": peaks["hbm_gbs"]},
        }
        if world == 1 and args.workload == "vgg_cifar":
            line["conv_microbench"] = conv_microbench(ctx, stream)
            line["batchnorm_microbench"] = batchnorm_microbench(ctx, stream, peaks["hbm_gbs"])
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_reference_run(args.workload, 1, 1, min_seconds=10.0)
            line["cpu_baseline"] = {"value": r["value"], "unit": "samples/s", "cores": r["cores"], "kind": "port",
                                    "sample": r["sample"]}
        print(json.dumps(line), flush=True)
    tr.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_transformer_lm(args):
    """The transformer language-model configuration (a parity configuration, not the headline): token embedding + positional
    encoding + 2 post-LN transformer blocks (GELU feed-forward, causal attention) + vocabulary head +
    cross-entropy + AdamW at batch 32, sequence 128, vocabulary 1000, d_model 256, 8 heads, d_ff 1024,
    driven op by op through the node-level C ABI the way the reference's examples drive its API."""
    import numpy as np
    import torch
    from neuralrs_b200 import _lib, cuda
    from neuralrs_b200.cuda import Node, backward_graph, graph, loss, nn, optim
    from neuralrs_b200.cuda import runtime as gpu
    B, S, V, D, H, FF, NB = 32, 128, 1000, 256, 8, 1024, 2
    ctx = cuda.default_context()
    ctx.set_math_mode(MATH[args.math])
    rng = np.random.default_rng(1238)

    def on_gpu(a):
        n = Node.new(np.ascontiguousarray(a, np.float32), list(np.shape(a)))
        gpu.to_cuda(n)
        return n
    mk = lambda *sh: rng.standard_normal(sh).astype(np.float32) / np.sqrt(sh[0])
    emb = on_gpu(rng.standard_normal((V, D)).astype(np.float32) * 0.5)
    blocks = []
    for _ in range(NB):
        w = {k: on_gpu(mk(D, D)) for k in ("q", "k", "v", "o")}
        mha = nn.MultiHeadAttention(w["q"], w["k"], w["v"], w["o"], D, H, True)
        blocks.append(nn.TransformerBlock(mha, nn.LayerNorm(on_gpu(np.ones(D)), on_gpu(np.zeros(D)), 1e-5),
                                          nn.LayerNorm(on_gpu(np.ones(D)), on_gpu(np.zeros(D)), 1e-5),
                                          nn.Linear(on_gpu(mk(D, FF)), on_gpu(np.zeros(FF))),
                                          nn.Linear(on_gpu(mk(FF, D)), on_gpu(np.zeros(D))), D, FF, _lib.ACT_GELU))
    head_w, head_b = on_gpu(mk(D, V)), on_gpu(np.zeros(V))
    params = [emb] + [q for blk in blocks for q in blk.parameters()] + [head_w, head_b]
    embedding, pe = nn.Embedding(emb, V, D), nn.PositionalEncoding(D, S)
    opt = optim.AdamW(1e-3, 0.9, 0.999, 1e-8, 1e-4)
    batches = []
    for _ in range(4):
        ids = rng.integers(0, V, (B, S))
        onehot = np.zeros((B * S, V), np.float32)
        onehot[np.arange(B * S), np.roll(ids, -1, axis=1).ravel()] = 1
        batches.append((ids, on_gpu(onehot)))

    def step(i):
        ids, target = batches[i % len(batches)]
        gpu.zero_grad(params)
        h = pe.forward(embedding.forward_batch(ids))
        for blk in blocks:
            h = blk.forward(h)
        logits = graph.add(graph.matmul(graph.reshape(h, [B * S, D]), head_w), head_b)
        value = loss.cross_entropy(logits, target)     # reads the loss back, as the reference's API does
        loss.cross_entropy_backward(logits, target)
        backward_graph(logits)
        opt.step(params)
        return value

    l = _lib.lib()
    for i in range(max(3, args.warmup)):
        step(i)
    l.nrs_sync(ctx.h)
    launches0 = l.nrs_launch_count(ctx.h)
    clk = ClockSampler(0)
    with clk:                      # entering and leaving the sampler takes time of its own: keep it outside dt
        t0 = time.perf_counter()
        for i in range(args.steps):
            last = step(i)
        l.nrs_sync(ctx.h)
        dt = time.perf_counter() - t0
    launches = l.nrs_launch_count(ctx.h) - launches0
    # forward FLOP per token: QKV/O projections 4*2*D*D, scores and mixing 2*2*S*D, feed-forward 2*2*D*FF per block; head 2*D*V
    fwd = NB * (8.0 * D * D + 4.0 * S * D + 4.0 * D * FF) + 2.0 * D * V
    line = {"metric": METRIC, "value": B * args.steps / dt, "unit": "samples/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "transformer_lm", "global_batch": B, "seq_len": S, "vocab": V, "d_model": D, "heads": H,
                       "d_ff": FF, "blocks": NB, "math": args.math, "tokens_per_s": B * S * args.steps / dt,
                       "algorithmic_gflop_per_step": 3.0 * fwd * B * S / 1e9,
                       "timing": "host wall clock around K steps with a device sync on both sides: every step is "
                                 "driven op by op from Python and reads its loss back, so this IS the end-to-end number",
                       "l2": "4 token batches rotated; the working set of a step (activations of 2 blocks) exceeds no cache "
                             "claim: this configuration is launch-bound"},
            "loss": float(last),
            "e2e": {"value": B * args.steps / dt, "unit": "samples/s", "h2d_bytes_per_step": B * S * 4, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches), "clocks": clk.summary(),
            "roofline": None, "cpu_baseline": None}
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 500), __file__] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.workload == "transformer_lm":
        if args.impl == "reference" or args.gpus > 1:
            print(json.dumps({"impl": args.impl, "unavailable": "transformer_lm is a single-GPU parity configuration; "
                                                               "the reference arm and N > 1 run the default workload"}))
            return
        run_transformer_lm(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
