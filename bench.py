#!/usr/bin/env python
"""Headline benchmark: training samples/s (forward + backward + AdamW) of the
CIFAR-shaped VGG-style CNN, global batch 1024 sharded over N GPUs, f32 with
3xTF32 contractions, synthetic data, He-initialised weights.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload vgg_cifar|vgg_cifar_bn|small_cnn|wide_mlp|transformer_lm] [--math 3xtf32|tf32|fp32]

For N > 1 launch under torchrun (one rank per GPU); run without torchrun the
script re-launches itself through `python -m torch.distributed.run`.
Rank 0 prints ONE JSON line.

* value        whole-job samples/s with the step's inputs already resident in HBM: the MEDIAN of
               `windows.n` back-to-back windows of K steps each (min / max beside it)
* e2e          the same through the host-buffer entry points (nrs_trainer_stage_next[_tokens] +
               nrs_trainer_step_staged): pinned host inputs copied in (the copy of batch i+1
               overlapping step i), loss copied out, every step; `unpipelined_value` is the
               plain nrs_trainer_step[_tokens] (copy, step, read-back in sequence)
* roofline     the dominant contraction family, timed with CUDA events bracketed around
               its launches inside the timed region (nrs_profile_*; every fourth timed step)
* cpu_baseline the CPU restatement of the reference's training loop (oracle/), timed on
               this host's cores on a bounded batch; `fast` = the reference's fast forward kernels
* dp_check     (N > 1) one step on a fixed 64-sample batch before timing: replicas bit-identical,
               and the relative difference to rank 0 doing the same step alone on the whole batch
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
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "train samples/s (fwd+bwd+AdamW)"
# workload -> (table in neuralrs_b200.workloads, global batch, seed offset, CPU sample batch)
WORKLOADS = {"vgg_cifar": ("VGG_CIFAR", 1024, 3, 32), "small_cnn": ("SMALL_CNN", 64, 1, 64),
             "wide_mlp": ("WIDE_MLP", 16384, 5, 64), "vgg_cifar_bn": ("VGG_CIFAR_BN", 1024, 7, 32),
             "transformer_lm": ("TRANSFORMER_LM", 32, 4, 2)}
# Configurations that state a batch without sharding it ("Batch 32 ... data-parallel at 1/2/4/8 GPUs"): every
# GPU takes that batch (weak scaling).  The others state a GLOBAL batch "sharded over 1/2/4/8" (strong).
PER_GPU_BATCH = {"transformer_lm"}
MATH = {"3xtf32": 0, "tf32": 1, "fp32": 2}
PROF_NAMES = ["conv_fwd", "conv_dgrad", "conv_wgrad", "gemm", "adamw", "batchnorm"]
N_WINDOWS = 5


def batch_plan(args, world):
    """(global batch, "weak" | "strong") of this run."""
    base = args.global_batch or WORKLOADS[args.workload][1]
    if args.workload in PER_GPU_BATCH and not args.global_batch:
        return base * world, "weak"
    return base, "strong"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="vgg_cifar", choices=list(WORKLOADS) + ["conv_layer"],
                    help="a model configuration, or conv_layer: the single-convolution configuration "
                         "(x[256,64,32,32] -> 128 channels, 3x3) with its batch sharded over the GPUs")
    ap.add_argument("--math", default="3xtf32", choices=list(MATH))
    ap.add_argument("--global-batch", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-microbench", action="store_true")
    ap.add_argument("--only-microbench", action="store_true",
                    help="N=1: skip the training loops and print only the micro-benchmarks (the command the ncu captures of "
                         "the HBM-bound and attention kernels under profiles/ run)")
    ap.add_argument("--no-fuse", action="store_true")
    ap.add_argument("--per-rank-batchnorm", action="store_true",
                    help="at N > 1, normalise with each rank's own shard statistics instead of the global batch's")
    return ap.parse_args()


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_burst=float(d["bf16_tflops"]),
                    bf16_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


def model_flops_per_sample(layers, in_shape):
    """Algorithmic FLOP of one forward pass per sample, and of forward+backward (the first contraction's
    data gradient is not computed: its input does not require a gradient).  A token model's sample is one
    sequence; attention scores and mixing are counted in full (the causal half included)."""
    shp = list(in_shape)
    fwd = total = 0.0
    first, tokens = True, 1
    for l in layers:
        f = None
        if l[0] == "conv":
            _, ci, co, k, s, p = l
            oh, ow = (shp[1] + 2 * p - k) // s + 1, (shp[2] + 2 * p - k) // s + 1
            f = 2.0 * co * oh * ow * ci * k * k
            shp = [co, oh, ow]
        elif l[0] == "linear":
            f = 2.0 * l[1] * l[2] * tokens
            shp = shp[:-1] + [l[2]]
        elif l[0] == "embedding":
            tokens = shp[0]
            shp = [shp[0], l[2]]
        elif l[0] == "transformer_block":
            d, ff = l[1], l[3]
            f = tokens * (8.0 * d * d + 4.0 * tokens * d + 4.0 * d * ff)
        elif l[0] == "maxpool":
            shp = [shp[0], (shp[1] - l[1]) // l[2] + 1, (shp[2] - l[1]) // l[2] + 1]
        elif l[0] == "flatten":
            n = 1
            for d in shp:
                n *= d
            shp = [n]
        if f is not None:
            fwd += f
            total += f * (2 if first else 3)
            first = False
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


# ----------------------------------------------------------------------------- CPU baseline (oracle/)

def cpu_reference_run(workload: str, steps: int, warmup: int, min_seconds: float = 0.0, max_seconds: float = 150.0):
    """Times the CPU restatement of the reference's training loop on a bounded batch, on every host core
    (the launcher's OMP_NUM_THREADS=1 is overridden: the reference's Rayon pools use all cores)."""
    from oracle import models, nrs_oracle
    from oracle.nrs_oracle import Oracle
    cores = nrs_oracle.host_cores()
    nrs_oracle.set_threads(cores)
    cfg = getattr(models, WORKLOADS[workload][0])
    seed = 1234 + WORKLOADS[workload][2]
    batch = WORKLOADS[workload][3]
    o = Oracle("f32")
    params = models.he_init(cfg["layers"], seed)
    hp = models.ADAMW_HP
    opt = models.OracleAdamW(o, hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["wd"])
    if cfg.get("token_model"):
        ids, labels = models.synthetic_tokens(cfg, batch, seed + 1)

        def step():
            loss, grads, _ = models.lm_forward_backward(o, cfg["layers"], params, ids, labels)
            opt.step(params, grads)
            return loss
    else:
        x, t = models.synthetic_batch(cfg, batch, seed + 1, uniform01=(workload == "small_cnn"))
        extra = dict(buffers=models.bn_buffers(cfg["layers"]), rng={"seed": seed, "offset": 0})

        def step():
            return models.train_step(o, cfg["layers"], params, opt, x, t, **extra)
    t_w = time.perf_counter()
    done_w = 0
    for _ in range(max(0, warmup)):
        step()
        done_w += 1
        if time.perf_counter() - t_w > max_seconds / 3:      # bounded: a slow host must not stall the run
            break
    done = 0
    t0 = time.perf_counter()
    while done < steps or (time.perf_counter() - t0) < min_seconds:
        step()
        done += 1
        if done >= steps and min_seconds <= 0:
            break
        if time.perf_counter() - t0 > max_seconds:
            break
    dt = time.perf_counter() - t0
    return dict(value=batch * done / dt, ms_per_step=1e3 * dt / done, steps=done, warmup=done_w, batch=batch,
                cores=nrs_oracle.get_threads(),
                sample=f"{done} training steps of {cfg['name']} at batch {batch} on {cores} host cores "
                       f"(conv/matmul loops OpenMP-parallel as the reference's Rayon loops are)")


def cpu_fast_forward(workload: str, seconds: float = 4.0):
    """Upper bound of the reference's CPU path: the FORWARD pass of the model with the reference's fast kernels
    restated (conv2d_im2col over matmul_simd, src/ops/im2col.rs:59-98, src/ops/simd.rs:42-77: AVX2 + all cores);
    the reference has no fast backward kernels, so the naive forward is timed beside it for the ratio."""
    from oracle import models, nrs_oracle
    from oracle.nrs_oracle import Oracle
    cfg = getattr(models, WORKLOADS[workload][0])
    if cfg.get("token_model") or any(l[0] in ("batchnorm", "dropout", "dropout2d") for l in cfg["layers"]):
        return None
    nrs_oracle.set_threads(nrs_oracle.host_cores())
    o = Oracle("f32")
    seed = 1234 + WORKLOADS[workload][2]
    batch = WORKLOADS[workload][3]
    params = models.he_init(cfg["layers"], seed)
    x, _ = models.synthetic_batch(cfg, batch, seed + 1, uniform01=(workload == "small_cnn"))

    def forward(fast):
        a, pi = x, 0
        for l in cfg["layers"]:
            if l[0] == "conv":
                a = (nrs_oracle.conv2d_im2col if fast else o.conv2d_fwd)(a, params[pi], params[pi + 1], l[4], l[5])
                pi += 2
            elif l[0] == "linear":
                a = o.bias_add_fwd(nrs_oracle.matmul_simd(a, params[pi]) if fast else o.matmul_fwd(a, params[pi]), params[pi + 1])
                pi += 2
            elif l[0] == "relu":
                a = o.relu_fwd(a)
            elif l[0] == "gelu":
                a = o.gelu_fwd(a)
            elif l[0] == "maxpool":
                a, _ = o.maxpool_fwd(a, l[1], l[2])
            elif l[0] == "flatten":
                a = a.reshape(a.shape[0], -1)
        return a
    out = {}
    for name, fast in (("fast", True), ("naive", False)):
        forward(fast)
        n, t0 = 0, time.perf_counter()
        while n < 2 or time.perf_counter() - t0 < seconds:
            forward(fast)
            n += 1
        out[name] = batch * n / (time.perf_counter() - t0)
    return {"fwd_samples_per_s": out["fast"], "naive_fwd_samples_per_s": out["naive"], "batch": batch,
            "kernels": "conv2d_im2col + matmul_simd (AVX2 FMA, all cores), forward pass only: the reference has no fast "
                       "backward kernels; activations / pooling from the naive port"}


# ----------------------------------------------------------------------------- micro-benchmarks (N = 1)

def _time_calls(ctx, stream, fn, iters):
    import torch
    from neuralrs_b200 import _lib
    for _ in range(3):
        _lib.check(ctx.h, fn())
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        _lib.check(ctx.h, fn())
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


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
        "dgrad+wgrad": lambda: l.nrs_conv2d_bwd(ctx.h, P(x), P(wt), P(dy), P(dx), P(dw), None, *dims, 0),
    }
    flop = 2.0 * n * co * h * w * ci * 9
    out = {"shape": "x[256,64,32,32] w[128,64,3,3] s1 p1", "gflop_per_pass": flop / 1e9}
    for name, fn in calls.items():
        ms = _time_calls(ctx, stream, fn, iters)
        passes = 2 if "+" in name else 1
        out[name] = {"ms": ms, "tflops": passes * flop / (ms / 1e3) / 1e12}
    # The same calls with the activations' TF32 planes made once (nrs_planes_cache), which is how a training step
    # runs them: x is staged once for the forward pass and the weight gradient, dy once for both gradients.
    _lib.check(ctx.h, l.nrs_planes_cache(ctx.h, P(x), n, ci, h, w))
    _lib.check(ctx.h, l.nrs_planes_cache(ctx.h, P(dy), n, co, h, w))
    cached = {}
    for name, fn in calls.items():
        ms = _time_calls(ctx, stream, fn, iters)
        passes = 2 if "+" in name else 1
        cached[name] = {"ms": ms, "tflops": passes * flop / (ms / 1e3) / 1e12}
    _lib.check(ctx.h, l.nrs_planes_drop(ctx.h, P(x)))
    _lib.check(ctx.h, l.nrs_planes_drop(ctx.h, P(dy)))
    out["operands_cached"] = cached
    return out


def batchnorm_microbench(ctx, stream, hbm_peak_gbs, iters=10):
    """BatchNorm2d (training mode) and Dropout on the conv microbenchmark's activation shape [256,64,32,32]
    through the raw C ABI.  HBM-bound: the algorithmic bytes are one read of every input tensor and one write
    of every output tensor."""
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
        ms = _time_calls(ctx, stream, fn, iters)
        gbs = tensors * tensor_bytes / (ms / 1e3) / 1e9
        out[name] = {"ms": ms, "algorithmic_gbs": gbs, "frac": gbs / hbm_peak_gbs}
    return out


def hbm_microbench(ctx, stream, hbm_peak_gbs, iters=10):
    """The HBM-bound kernels at bandwidth-bound sizes (every tensor >= 64 MB, well beyond L2 when summed) through the
    raw C ABI: algorithmic bytes = one read of every input tensor and one write of every output tensor, over the
    CUDA-event time of `iters` back-to-back calls; frac is against the measured copy bandwidth."""
    import ctypes as C
    import torch
    from neuralrs_b200 import _lib
    l = _lib.lib()
    P = lambda t: C.c_void_p(t.data_ptr())
    F = C.c_float
    g = torch.Generator(device="cuda").manual_seed(1241)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    out = {"hbm_peak_gbs": hbm_peak_gbs, "iters": iters}

    def entry(name, nbytes, fn, shape):
        ms = _time_calls(ctx, stream, fn, iters)
        gbs = nbytes / (ms / 1e3) / 1e9
        out[name] = {"shape": shape, "ms": ms, "algorithmic_mb": nbytes / 1e6, "algorithmic_gbs": gbs, "frac": gbs / hbm_peak_gbs}
    # LayerNorm over rows of 256 features (the language model's d_model)
    rows, f = 65536, 256
    x, gy = rn(rows, f), rn(rows, f)
    gamma, beta = torch.rand(f, device="cuda") + 0.5, rn(f)
    y, xhat, dx = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    istd, dgm, dbt = torch.empty(rows, device="cuda"), torch.empty(f, device="cuda"), torch.empty(f, device="cuda")
    tb = x.numel() * 4
    entry("layernorm_fwd", 3 * tb + rows * 4, lambda: l.nrs_layernorm_fwd(ctx.h, P(x), P(gamma), P(beta), P(y), P(xhat), P(istd), rows, f, F(1e-5)),
          "x[65536,256] -> y, xhat, istd")
    entry("layernorm_bwd_dx", 3 * tb + rows * 4, lambda: l.nrs_layernorm_bwd(ctx.h, P(gy), P(xhat), P(istd), P(gamma), P(dx), None, None, rows, f, 0, 0),
          "g, xhat, istd -> dx [65536,256]")
    entry("layernorm_bwd", 3 * tb + rows * 4, lambda: l.nrs_layernorm_bwd(ctx.h, P(gy), P(xhat), P(istd), P(gamma), P(dx), P(dgm), P(dbt), rows, f, 0, 0),
          "g, xhat, istd -> dx, dgamma, dbeta in one launch (+ the partial-sum fold): what the graph operator issues")
    entry("layernorm_bwd_params", 2 * tb, lambda: l.nrs_layernorm_bwd(ctx.h, P(gy), P(xhat), P(istd), P(gamma), None, P(dgm), P(dbt), rows, f, 0, 0),
          "g, xhat -> dgamma, dbeta [256]")
    del x, gy, y, xhat, dx
    # softmax over rows of 128 (the attention score width)
    rows, wd = 131072, 128
    x, gy = rn(rows, wd), rn(rows, wd)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    tb = x.numel() * 4
    entry("softmax_fwd", 2 * tb, lambda: l.nrs_softmax_fwd(ctx.h, P(x), P(y), rows, wd), "x[131072,128] -> y")
    entry("softmax_bwd", 3 * tb, lambda: l.nrs_softmax_bwd(ctx.h, P(y), P(gy), P(dx), rows, wd, 0), "y, g -> dx [131072,128]")
    del x, gy, y, dx
    # cross-entropy forward + backward over the wide MLP's logits
    rows, cl = 16384, 1000
    logits = rn(rows, cl)
    target = torch.zeros(rows, cl, device="cuda")
    target[torch.arange(rows, device="cuda"), torch.randint(0, cl, (rows,), device="cuda", generator=g)] = 1.0
    grad, loss_dev = torch.empty_like(logits), torch.zeros(1, device="cuda")
    tb = logits.numel() * 4
    entry("cross_entropy_fwd_bwd", 3 * tb, lambda: l.nrs_ce_fwd_bwd(ctx.h, P(logits), P(target), P(loss_dev), P(grad), rows, cl, rows),
          "logits, one-hot [16384,1000] -> loss, grad")
    del logits, target, grad
    # AdamW over the wide MLP's 71.2 M parameters: 28 B per parameter
    n = 71222248
    p, gr, m, v = rn(n), rn(n), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    entry("adamw", 28 * n, lambda: l.nrs_adamw_step(ctx.h, P(p), P(gr), P(m), P(v), C.c_size_t(n), F(1e-3), F(0.9), F(0.999), F(1e-8),
                                                    F(1e-4), F(0.1), F(0.001), F(1.0)), "71.2 M parameters")
    del p, gr, m, v
    # max-pool 2x2 forward / backward on the conv microbenchmark's activation
    nb, c, h, w = 256, 64, 32, 32
    x = rn(nb, c, h, w)
    y = torch.empty(nb, c, h // 2, w // 2, device="cuda")
    am = torch.empty(nb, c, h // 2, w // 2, device="cuda", dtype=torch.int32)
    gy, dx = torch.randn_like(y), torch.empty_like(x)
    entry("maxpool_fwd", x.numel() * 4 + 2 * y.numel() * 4, lambda: l.nrs_maxpool_fwd(ctx.h, P(x), P(y), P(am), nb, c, h, w, 2, 2),
          "x[256,64,32,32] -> y, argmax")
    entry("maxpool_bwd", x.numel() * 4 + 2 * y.numel() * 4, lambda: l.nrs_maxpool_bwd(ctx.h, P(gy), P(am), P(dx), nb, c, h, w, 2, 2, 0),
          "g, argmax -> dx[256,64,32,32]")
    return out


def attention_microbench(ctx, stream, iters=20):
    """The fused attention core at the language-model configuration's shape (batch 32, sequence 128, 8 heads of 32,
    causal) through the raw C ABI: forward (scores, softmax, mixing) and backward (five products), tensor cores in
    the TF32 modes.  Algorithmic FLOP: 4 S^2 d_head per (batch, head) forward, 10 S^2 d_head backward."""
    import ctypes as C
    import torch
    from neuralrs_b200 import _lib
    l = _lib.lib()
    B, S, H, dh = 32, 128, 8, 32
    g = torch.Generator(device="cuda").manual_seed(1242)
    q, k, v, do = (torch.randn(B, S, H * dh, device="cuda", generator=g) for _ in range(4))
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    probs = torch.empty(B * H, S, S, device="cuda")
    P = lambda t: C.c_void_p(t.data_ptr())
    fwd = _time_calls(ctx, stream, lambda: l.nrs_attention_fwd(ctx.h, P(q), P(k), P(v), P(out), P(probs), B, S, H, dh, 1), iters)
    bwd = _time_calls(ctx, stream, lambda: l.nrs_attention_bwd(ctx.h, P(q), P(k), P(v), P(probs), P(do), P(dq), P(dk), P(dv),
                                                               B, S, H, dh, 0, 0, 0), iters)
    flop = 4.0 * S * S * dh * B * H
    return {"shape": "batch 32, seq 128, 8 heads x 32, causal", "fwd_us": fwd * 1e3, "bwd_us": bwd * 1e3,
            "fwd_tflops": flop / (fwd / 1e3) / 1e12, "bwd_tflops": 2.5 * flop / (bwd / 1e3) / 1e12}


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


def cpu_baseline_entry(r):
    return {"value": r["value"], "unit": "samples/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    global_batch, scaling = batch_plan(args, args.gpus)
    r = cpu_reference_run(args.workload, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "samples/s", "n_gpus": args.gpus,
        "steps": r["steps"], "warmup": r["warmup"], "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "global_batch": global_batch, "cpu_sample_batch": r["batch"],
                   "note": "CPU restatement of the reference's own training loop (oracle/) on every host core; the Rust "
                           "crate cannot be built here (no cargo/rustc in the image); each step is a bounded sample "
                           "(cpu_sample_batch samples) of the workload"},
        "cpu_baseline": cpu_baseline_entry(r),
        "e2e": {"value": r["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import ctypes as C
    import numpy as np
    import torch
    import torch.distributed as dist

    from neuralrs_b200 import _lib, cuda, workloads

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cfg = getattr(workloads, WORKLOADS[args.workload][0])
    tokens = bool(cfg.get("token_model"))
    seed = 1234 + WORKLOADS[args.workload][2]
    global_batch, scaling = batch_plan(args, world)
    b0, b1 = cuda.dp_shard_range(global_batch, rank, world)
    batch = b1 - b0
    rows_per_sample = cfg["in_shape"][0] if tokens else 1

    ctx = cuda.Context(local_rank)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    ctx.set_math_mode(MATH[args.math])
    hp = workloads.ADAMW_HP
    l = _lib.lib()
    init = workloads.he_init(cfg["layers"], seed)       # identical bytes on every rank

    def make_trainer(dp_batch=None):
        tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                          hp["wd"], fuse=not args.no_fuse, ctx=ctx)
        tr.set_params(init)
        if world > 1 and dp_batch:
            box = [cuda.dp_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            tr.enable_dp(rank, world, box[0], dp_batch)
            if not args.per_rank_batchnorm:
                tr.set_sync_batchnorm(True)     # only BatchNorm layers look at it
        return tr

    def make_batch(n, s):
        """(inputs, targets) as contiguous numpy arrays: float samples + one-hot rows, or token ids + next-token labels."""
        if tokens:
            ids, labels = workloads.synthetic_tokens(cfg, n, s)
            return ids, labels.reshape(n, rows_per_sample)
        return workloads.synthetic_batch(cfg, n, s, uniform01=(args.workload == "small_cnn"))

    def device_step(tr, x_ptr, t_ptr, n, want_loss=False):
        return (tr.step_tokens_device if tokens else tr.step_device)(x_ptr, t_ptr, n, want_loss)

    # ---- data-parallel check before timing: one step on a fixed 64-sample batch
    dp_check = None
    if world > 1:
        chk_n = 64
        cx, ct = make_batch(chk_n, seed + 99)
        c0, c1 = cuda.dp_shard_range(chk_n, rank, world)
        _lib.check(ctx.h, l.nrs_rng_seed(ctx.h, C.c_uint64(seed)))     # both runs draw from the start of the same stream
        tr_dp = make_trainer(chk_n)
        xs = torch.from_numpy(np.ascontiguousarray(cx[c0:c1])).cuda()
        ts = torch.from_numpy(np.ascontiguousarray(ct[c0:c1])).cuda()
        share = device_step(tr_dp, xs.data_ptr(), ts.data_ptr(), c1 - c0, True)
        flat = np.concatenate([tr_dp.get_param(i) for i in range(tr_dp.n_params)])
        tr_dp.close()
        mine = torch.from_numpy(flat).cuda()
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        identical = bool(torch.equal(lo, hi))            # every rank holds the same bits
        loss_sum = torch.tensor([share], device="cuda", dtype=torch.float64)
        dist.all_reduce(loss_sum)
        if rank == 0:
            _lib.check(ctx.h, l.nrs_rng_seed(ctx.h, C.c_uint64(seed)))
            tr_one = make_trainer()
            xf, tf = torch.from_numpy(np.ascontiguousarray(cx)).cuda(), torch.from_numpy(np.ascontiguousarray(ct)).cuda()
            full_loss = device_step(tr_one, xf.data_ptr(), tf.data_ptr(), chk_n, True)
            ref = np.concatenate([tr_one.get_param(i) for i in range(tr_one.n_params)])
            tr_one.close()
            start = np.concatenate([p.ravel() for p in init])
            upd, upd_ref = flat.astype(np.float64) - start, ref.astype(np.float64) - start
            dp_check = {"batch": chk_n, "replicas_bit_identical": identical,
                        "rel_err_vs_rank0_full_batch_step": float(np.linalg.norm(flat - ref) / np.linalg.norm(ref)),
                        "rel_err_of_the_update": float(np.linalg.norm(upd - upd_ref) / max(np.linalg.norm(upd_ref), 1e-30)),
                        "loss_sum_of_shares": float(loss_sum.item()), "loss_rank0_full_batch": full_loss}
        dist.barrier()

    tr = make_trainer(global_batch)

    # Synthetic batches: a few distinct ones, rotated, pinned on the host and resident on the device.
    n_sets = 4
    xs_pin, ts_pin, xs_dev, ts_dev = [], [], [], []
    for i in range(n_sets):
        x, t = make_batch(global_batch, seed + 10 + i)
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

    dev_step = lambda i: device_step(tr, xs_dev[i % n_sets].data_ptr(), ts_dev[i % n_sets].data_ptr(), batch)
    host_fn = l.nrs_trainer_step_tokens if tokens else l.nrs_trainer_step
    stage_fn = l.nrs_trainer_stage_next_tokens if tokens else l.nrs_trainer_stage_next
    loss_box = C.c_float()

    def host_step(i):
        _lib.check(ctx.h, host_fn(tr.h, C.c_void_p(xs_pin[i % n_sets].data_ptr()), C.c_void_p(ts_pin[i % n_sets].data_ptr()),
                                  batch, C.byref(loss_box)))

    def stage(j):
        _lib.check(ctx.h, stage_fn(tr.h, C.c_void_p(xs_pin[j].data_ptr()), C.c_void_p(ts_pin[j].data_ptr()), batch))

    def staged_loop(total):
        """End-to-end steps with the input copy double-buffered: batch i+1 is staged (asynchronous copy from
        pinned memory on the copy stream) before step i is issued; every step still reads its loss back."""
        def fn(i):
            if i == 0:
                stage(0)
            if i + 1 < total:
                stage((i + 1) % n_sets)
            tr.step_staged(True)
        return fn

    for i in range(max(3, args.warmup)):
        dev_step(i)
    _lib.check(ctx.h, l.nrs_profile_reset(ctx.h))
    # The per-family CUDA-event brackets sit between kernels, where they defeat the chaining of
    # consecutive launches; they are switched on for every fourth timed step only (the first
    # included), and the family figures are scaled to the bracketed steps.
    bracket_every = 4
    bracketed = len(range(0, args.steps, bracket_every)) * N_WINDOWS

    def dev_step_bracketed(i):
        l.nrs_profile_enable(ctx.h, 1 if i % bracket_every == 0 else 0)
        dev_step(i)
    launches0 = ctx.launch_count()
    windows = []
    with ClockSampler(local_rank) as clk:
        for _ in range(N_WINDOWS):
            windows.append(timed(dev_step_bracketed, args.steps))
    launches = (ctx.launch_count() - launches0) // N_WINDOWS
    ms = statistics.median(windows)
    prof = {}
    for kind, name in enumerate(PROF_NAMES):
        pms, work, calls = C.c_double(), C.c_double(), C.c_uint64()
        _lib.check(ctx.h, l.nrs_profile_get(ctx.h, kind, C.byref(pms), C.byref(work), C.byref(calls)))
        prof[name] = dict(ms=pms.value, work=work.value, calls=int(calls.value))
    _lib.check(ctx.h, l.nrs_profile_enable(ctx.h, 0))
    _lib.check(ctx.h, l.nrs_profile_reset(ctx.h))
    loss = tr.last_loss()
    if world > 1:     # every rank holds its share of the global-mean loss
        lt = torch.tensor([loss], device="cuda", dtype=torch.float64)
        dist.all_reduce(lt)
        loss = float(lt.item())

    def lagged_loop(total):
        """The same with every step's loss read one step behind (nrs_trainer_step_staged_lagged): step i is issued,
        then the host waits for the loss of step i-1 only; the last step's loss is read (synchronously) inside the
        timed region too, so K steps read K losses."""
        def fn(i):
            if i == 0:
                stage(0)
            if i + 1 < total:
                stage((i + 1) % n_sets)
            tr.step_staged_lagged()
            if i + 1 == total:
                tr.last_loss()
        return fn

    # the headline end-to-end form first, right after the device-resident windows; its two comparison forms after it
    warm = lagged_loop(2)
    for i in range(2):
        warm(i)
    e2e_windows = [timed(lagged_loop(args.steps), args.steps) for _ in range(3)]
    ms_e2e = statistics.median(e2e_windows)
    warm = staged_loop(2)
    for i in range(2):
        warm(i)
    sync_windows = [timed(staged_loop(args.steps), args.steps) for _ in range(3)]
    ms_e2e_sync = statistics.median(sync_windows)
    for i in range(2):
        host_step(i)
    ms_e2e_plain = timed(host_step, args.steps)

    if rank == 0:
        peaks = measured_peaks()
        per_s = lambda w_ms: global_batch * args.steps / (w_ms / 1e3)
        fwd_flop, step_flop = model_flops_per_sample(cfg["layers"], cfg["in_shape"])
        contractions = ("conv_fwd", "conv_dgrad", "conv_wgrad", "gemm")
        fam = max(contractions, key=lambda k: prof[k]["ms"])      # dominant contraction family by device time
        f = prof[fam]
        achieved = (f["work"] / (f["ms"] / 1e3) / 1e12) if f["ms"] > 0 else 0.0
        tf32_peak = peaks["bf16_sustained"] / 2.0
        umma = C.c_double()
        _lib.check(ctx.h, l.nrs_measure_tf32_umma_peak(ctx.h, C.byref(umma)))
        contraction_ms = sum(prof[k]["ms"] for k in contractions)
        contraction_work = sum(prof[k]["work"] for k in contractions)
        adam = prof["adamw"]
        x_bytes = int(np.prod((global_batch,) + tuple(cfg["in_shape"]))) * 4
        t_bytes = global_batch * rows_per_sample * (4 if tokens else cfg["classes"] * 4)
        issue = 3.0 if args.math == "3xtf32" else 1.0
        line = {
            "metric": METRIC, "value": per_s(ms), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "windows": {"n": N_WINDOWS, "steps_each": args.steps, "statistic": "median",
                        "ms_per_step_min": min(windows) / args.steps, "ms_per_step_max": max(windows) / args.steps,
                        "ms_per_step_in_order": [w / args.steps for w in windows],
                        "value_min": per_s(max(windows)), "value_max": per_s(min(windows))},
            "config": {"workload": args.workload, "global_batch": global_batch, "per_gpu_batch": batch,
                       "parallelism": f"dp{world}", "math": args.math, "fused_epilogues": not args.no_fuse,
                       "init": "He N(0,sqrt(2/fan_in)), seed %d" % seed,
                       "l2": "per-step working set (activations + gradients) is several times the 126 MB L2; "
                             "4 input batches rotated",
                       "algorithmic_gflop_per_step": step_flop * global_batch / 1e9,
                       "tensor_core_path": bool(l.nrs_has_tensor_core_path())},
            "loss": loss,
            "e2e": {"value": per_s(ms_e2e), "unit": "samples/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": x_bytes + t_bytes, "d2h_bytes_per_step": 4 * world,
                    "windows": {"n": len(e2e_windows), "statistic": "median", "value_min": per_s(max(e2e_windows)),
                                "value_max": per_s(min(e2e_windows)),
                                "ms_per_step_in_order": [w / args.steps for w in e2e_windows]},
                    "api": "nrs_trainer_stage_next%s + nrs_trainer_step_staged_lagged: the copy of batch i+1 overlaps step i and "
                           "the loss of step i is read after step i+1 has been issued (every step's loss is read inside the "
                           "timed region, the last one synchronously)" % ("_tokens" if tokens else ""),
                    "synchronous_loss_value": per_s(ms_e2e_sync),
                    "synchronous_loss_api": "nrs_trainer_step_staged: the loss of step i is read before step i+1 is issued",
                    "unpipelined_value": per_s(ms_e2e_plain),
                    "unpipelined_api": "nrs_trainer_step%s: copy, step and loss read-back in sequence" % ("_tokens" if tokens else "")},
            "gpu_launches": launches * world,
            "clocks": clk.summary(),
            "roofline": {"bound": "tensor", "kernel": fam, "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                         "frac": achieved / tf32_peak if tf32_peak else None,
                         **ncu_traffic(args.workload, args.math, fam, batch),
                         "peak_source": f"{peaks['source']}: sustained bf16 cuBLAS / 2 (dense TF32 runs at half the bf16 "
                                        f"rate); {args.math} issues {issue:.0f}x the algorithmic FLOP counted in `achieved`",
                         "issued_tflops": achieved * issue,
                         "frac_issued_of_peak": achieved * issue / tf32_peak if tf32_peak else None,
                         "tf32_umma_peak_tflops": umma.value,
                         "frac_issued_of_umma_peak": achieved * issue / umma.value if umma.value else None,
                         "tf32_umma_peak_source": "measured in this run: back-to-back tcgen05.mma.kind::tf32 128x256x8 from "
                                                  "shared memory on every SM (nrs_measure_tf32_umma_peak)",
                         "launch_ms_avg": f["ms"] / f["calls"] if f["calls"] else None, "calls": f["calls"],
                         "all_contractions_tflops": (contraction_work / (contraction_ms / 1e3) / 1e12) if contraction_ms else None,
                         "families_ms_per_step": {k: prof[k]["ms"] / bracketed for k in prof},
                         "bracketed_steps": bracketed,
                         "adamw_gbs": (adam["work"] / (adam["ms"] / 1e3) / 1e9) if adam["ms"] > 0 else None,
                         "batchnorm_gbs": (prof["batchnorm"]["work"] / (prof["batchnorm"]["ms"] / 1e3) / 1e9)
                         if prof["batchnorm"]["ms"] > 0 else None,
                         "hbm_peak_gbs": peaks["hbm_gbs"]},
        }
        if dp_check:
            line["dp_check"] = dp_check
        if world == 1 and args.workload == "transformer_lm" and not args.no_microbench:
            line["attention_microbench"] = attention_microbench(ctx, stream)
        if world == 1 and args.workload == "vgg_cifar" and not args.no_microbench:
            line["conv_microbench"] = conv_microbench(ctx, stream)
            line["batchnorm_microbench"] = batchnorm_microbench(ctx, stream, peaks["hbm_gbs"])
            line["hbm_microbench"] = hbm_microbench(ctx, stream, peaks["hbm_gbs"])
            line["attention_microbench"] = attention_microbench(ctx, stream)
            line["other_configs"] = other_configs(ctx, stream, args.math)
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_reference_run(args.workload, 1, 1, min_seconds=10.0)
            line["cpu_baseline"] = cpu_baseline_entry(r)
            line["cpu_baseline"]["fast"] = cpu_fast_forward(args.workload)
        print(json.dumps(line), flush=True)
    tr.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def other_configs(ctx, stream, math, steps=10):
    """The other configurations through the same native trainer, resident inputs, one GPU: a short device-timed
    run each (3 warm-up steps, `steps` timed), so that the default line carries a figure for every configuration."""
    import numpy as np
    import torch
    from neuralrs_b200 import cuda, workloads
    hp = workloads.ADAMW_HP
    out = {}
    for name in ("small_cnn", "transformer_lm", "wide_mlp"):
        table, batch, seed_off, _ = WORKLOADS[name]
        cfg = getattr(workloads, table)
        tokens = bool(cfg.get("token_model"))
        tr = cuda.Trainer(cfg["layers"], cfg["in_shape"], cfg["classes"], hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                          hp["wd"], fuse=True, ctx=ctx)
        tr.set_params(workloads.he_init(cfg["layers"], 1234 + seed_off))
        if tokens:
            x, t = workloads.synthetic_tokens(cfg, batch, 1234 + seed_off + 10)
            t = t.reshape(batch, cfg["in_shape"][0])
        else:
            x, t = workloads.synthetic_batch(cfg, batch, 1234 + seed_off + 10, uniform01=(name == "small_cnn"))
        xd, td = torch.from_numpy(np.ascontiguousarray(x)).cuda(), torch.from_numpy(np.ascontiguousarray(t)).cuda()
        step = tr.step_tokens_device if tokens else tr.step_device
        for _ in range(3):
            step(xd.data_ptr(), td.data_ptr(), batch, False)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step(xd.data_ptr(), td.data_ptr(), batch, False)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        _, step_flop = model_flops_per_sample(cfg["layers"], cfg["in_shape"])
        out[name] = {"batch": batch, "ms_per_step": ms, "samples_per_s": batch / (ms / 1e3),
                     "algorithmic_tflops": step_flop * batch / (ms / 1e3) / 1e12, "math": math, "steps": steps}
        tr.close()
        del xd, td
    return out


def run_conv_layer(args):
    """The single-convolution configuration at N GPUs: Conv2d x[256,64,32,32] -> 128, 3x3 s1 p1, batch sharded
    contiguously over the ranks.  Forward and data gradient need no exchange; the weight gradient is summed over
    the ranks (one 295 KB all-reduce on the library's communicator).  Each pass is timed on its own with CUDA events
    (max over ranks), activations' operand planes made once as in a training step."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from neuralrs_b200 import _lib, cuda
    rank, local_rank = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = cuda.Context(local_rank)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    ctx.set_math_mode(MATH[args.math])
    l = _lib.lib()
    global_n, ci, h, w, co = args.global_batch or 256, 64, 32, 32, 128
    b0, b1 = cuda.dp_shard_range(global_n, rank, world)
    n = b1 - b0
    dp = None
    if world > 1:
        box = [cuda.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        dp = cuda.DataParallel(rank, world, box[0], global_n, timeout_ms=300000.0, ctx=ctx)
    g = torch.Generator(device="cuda").manual_seed(1236)          # every rank draws the full tensors, keeps its shard
    x = torch.randn(global_n, ci, h, w, device="cuda", generator=g)[b0:b1].contiguous()
    wt = torch.randn(co, ci, 3, 3, device="cuda", generator=g) * (2.0 / (ci * 9)) ** 0.5
    dy = torch.randn(global_n, co, h, w, device="cuda", generator=g)[b0:b1].contiguous()
    bias = torch.zeros(co, device="cuda")
    y, dx, dw = torch.empty_like(dy), torch.empty_like(x), torch.empty_like(wt)
    P = lambda t: C.c_void_p(t.data_ptr())
    dims = (n, ci, h, w, co, 3, 3, 1, 1)

    def wgrad():
        st = l.nrs_conv2d_bwd(ctx.h, P(x), P(wt), P(dy), None, P(dw), None, *dims, 0)
        if st == 0 and dp:
            dp.all_reduce_sum(dw.data_ptr(), dw.numel())
        return st
    calls = {"fwd": lambda: l.nrs_conv2d_fwd(ctx.h, P(x), P(wt), P(bias), P(y), *dims, 0),
             "dgrad": lambda: l.nrs_conv2d_bwd(ctx.h, P(x), P(wt), P(dy), P(dx), None, None, *dims, 0),
             "wgrad": wgrad}
    _lib.check(ctx.h, l.nrs_planes_cache(ctx.h, P(x), n, ci, h, w))
    _lib.check(ctx.h, l.nrs_planes_cache(ctx.h, P(dy), n, co, h, w))
    iters, flop = max(args.steps, 1), 2.0 * global_n * co * h * w * ci * 9
    passes, launches0 = {}, ctx.launch_count()
    with ClockSampler(local_rank) as clk:
        for name, fn in calls.items():
            for _ in range(max(3, args.warmup)):
                _lib.check(ctx.h, fn())
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(iters):
                _lib.check(ctx.h, fn())
            e1.record(stream)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            if world > 1:
                t = torch.tensor([ms], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            passes[name] = {"ms": ms, "tflops": flop / (ms / 1e3) / 1e12}
    launches = ctx.launch_count() - launches0
    # the summed weight gradient is the same on every rank
    check = None
    if world > 1:
        lo, hi = dw.clone(), dw.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        check = {"weight_gradient_identical_on_all_ranks": bool(torch.equal(lo, hi))}
    if rank == 0:
        total_ms = sum(p["ms"] for p in passes.values())
        peaks = measured_peaks()
        line = {"metric": "conv forward + data gradient + weight gradient, algorithmic TFLOP/s", "value": 3 * flop / (total_ms / 1e3) / 1e12,
                "unit": "TFLOP/s", "n_gpus": world, "steps": iters, "warmup": max(3, args.warmup), "ms_per_step": total_ms,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "conv_layer", "shape": f"x[{global_n},64,32,32] w[128,64,3,3] s1 p1", "per_gpu_batch": n,
                           "parallelism": f"dp{world}", "math": args.math,
                           "operands": "TF32 planes of x and dy made once (nrs_planes_cache), as in a training step",
                           "l2": "x + dy and their planes are 600 MB per rank at N=1 (75 MB at N=8: below L2 there)"},
                "passes": passes, "gpu_launches": launches * world, "clocks": clk.summary(),
                "roofline": {"bound": "tensor", "kernel": "conv (three passes)", "achieved": 3 * flop / (total_ms / 1e3) / 1e12 / world,
                             "peak": peaks["bf16_sustained"] / 2.0, "unit": "TFLOP/s per GPU",
                             "frac": 3 * flop / (total_ms / 1e3) / 1e12 / world / (peaks["bf16_sustained"] / 2.0), "traffic": None,
                             "note": "algorithmic; 3xtf32 issues three times as much"},
                "e2e": None, "cpu_baseline": None}
        if check:
            line["dp_check"] = check
        print(json.dumps(line), flush=True)
    _lib.check(ctx.h, l.nrs_planes_drop(ctx.h, P(x)))
    _lib.check(ctx.h, l.nrs_planes_drop(ctx.h, P(dy)))
    if dp:
        dp.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_only_microbench(args):
    import torch
    from neuralrs_b200 import cuda
    torch.cuda.set_device(0)
    ctx = cuda.Context(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    ctx.set_math_mode(MATH[args.math])
    peaks = measured_peaks()
    line = {"microbench_only": True, "math": args.math,
            "hbm_microbench": hbm_microbench(ctx, stream, peaks["hbm_gbs"], iters=max(1, min(args.steps, 10))),
            "batchnorm_microbench": batchnorm_microbench(ctx, stream, peaks["hbm_gbs"], iters=max(1, min(args.steps, 10))),
            "attention_microbench": attention_microbench(ctx, stream, iters=max(1, min(args.steps, 20))),
            "conv_microbench": conv_microbench(ctx, stream, iters=max(1, min(args.steps, 10)))}
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    if args.only_microbench:
        return run_only_microbench(args)
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 500), __file__] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.workload == "conv_layer":
        if args.impl == "reference":
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the reference arm times whole training steps; "
                                  "run it with a model workload"}), flush=True)
            return
        return run_conv_layer(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
