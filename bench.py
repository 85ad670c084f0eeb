#!/usr/bin/env python
"""Throughput of the convolution / matrix-multiply inference path on B200, through the backend's C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c0|c1|c2|c3|c4] [--impl ours|reference]

One "step" is one forward pass over one batch of synthetic inputs.  Default workload: benchmark configuration 3 -- 20x20 board,
32 input planes (Bernoulli p = 0.3), stem 3x3 32 -> 256, 20 residual blocks of two 3x3 256 -> 256 convolutions with bias and
ReLU, 1x1 policy head, global-average-pool + dense value head, fp16, batch 1024 per GPU, He-normal random weights.  With N > 1
(launched by torch.distributed.run) every rank runs the same per-GPU batch on its own GPU: weak scaling, no collective on
the forward path.

The JSON line printed by rank 0 carries:
  value         positions/s with the input already resident in HBM (device time, CUDA events, max over ranks)
  e2e           positions/s through the C ABI with HOST buffers: pinned host -> device copy of the input, forward, device ->
                host copy of the outputs, inside the timed region (wall clock).  Two contexts take the steps in turn so that
                one step's copies overlap the other's arithmetic (--no-overlap: one context); with small configurations their
                kernels also overlap, so e2e can exceed the single-stream `value`
  roofline      the dominant kernel of the configuration's 3x3 layer, timed alone with CUDA events on the context's stream
  cpu_baseline  minml's own CPU backend (oracle/_ref, else the C port) on the host cores, on a bounded sample
  other_configs (N = 1, default configuration only) the same measurements, with fewer steps, for configurations 0, 1, 2 and 4
  dropin_host   (N = 1, trunk configurations, when oracle/_ref/trunk_dropin was built) positions/s of the same trunk through
                minml's own unmodified C++ host code (Graph::predict) with this library as its CUDA backend
  ranks         (N > 1) per-rank ms_per_step and median SM clock: min / median / max over ranks and the slowest rank's index
`--impl reference` times only the CPU implementation and prints the same line shape with "impl": "reference".
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from minml_b200 import synthetic  # noqa: E402  (numpy only: does not load the CUDA library)

CONFIGS = {
    # name: batch per GPU, height, width, input planes, channels, blocks
    "c0": dict(kind="layer_fp32", batch=64, height=15, width=15, planes=128, channels=128, blocks=0,
               label="config0: one 3x3 convolution layer, NHWC fp32, batch 64, 15x15, 128->128, stride 1, same padding, y = ReLU(conv + bias), "
                     "issued as minml's Conv2D issues it (Winograd call triple)"),
    "c1": dict(batch=256, height=15, width=15, planes=32, channels=128, blocks=10,
               label="config1: 15x15 board, 32 planes, stem 3x3 32->128, 10 residual blocks x 2 conv3x3 128->128, policy 1x1 + value GAP/dense, fp16"),
    "c2": dict(kind="int8_trunk", batch=512, height=20, width=20, planes=32, channels=128, blocks=10,
               label="config2: int8 trunk, 20x20 board, 32 planes, 128 channels, 10 residual blocks, per-channel int8 weights, per-tensor int8 "
                     "activations calibrated on 64 seeded batches, int32 accumulate, fp32 requantisation, fp16 heads"),
    "c3": dict(batch=1024, height=20, width=20, planes=32, channels=256, blocks=20,
               label="config3: 20x20 board, 32 planes, stem 3x3 32->256, 20 residual blocks x 2 conv3x3 256->256, policy 1x1 + value GAP/dense, fp16"),
    "c4": dict(kind="hybrid", batch=256, height=15, width=15, planes=256, channels=256, blocks=1, heads=8, ffn=1024,
               label="config4: 15x15 board as 225 tokens, embed 256: 3x3 residual block, pre-LN attention (8 heads of 32, relative-position bias), "
                     "FFN 256->1024->256 ReLU, fp16"),
}
SEED = 1237
METRIC = {"trunk": "positions/sec for ResNet trunk", "int8_trunk": "positions/sec for ResNet trunk", "hybrid": "positions/sec for conv+attention block",
          "layer_fp32": "positions/sec for one 3x3 convolution layer"}
DTYPE = {"trunk": "f16", "int8_trunk": "i8", "hybrid": "f16", "layer_fp32": "f32"}


def flops_per_position(cfg):
    """Algorithmic (direct-convolution) FLOPs per batch item."""
    hw = cfg["height"] * cfg["width"]
    c = cfg["channels"]
    kind = cfg.get("kind", "trunk")
    if kind == "hybrid":
        return 2 * 2 * hw * 9 * c * c + 2 * hw * c * (3 * c + c + 2 * cfg["ffn"]) + 4 * hw * hw * c
    if kind == "layer_fp32":
        return 2 * hw * 9 * cfg["planes"] * c
    return 2 * hw * 9 * cfg["planes"] * c + cfg["blocks"] * 2 * (2 * hw * 9 * c * c) + 2 * hw * c + 2 * c * 3


def config0_arrays(cfg, batch, seed):
    """x ~ U[-1, 1], w ~ N(0, sqrt(2 / (9 * cin))), bias ~ N(0, 0.01), as configuration 0 states."""
    r = np.random.default_rng(seed)
    cin, cout = cfg["planes"], cfg["channels"]
    x = r.uniform(-1, 1, (batch, cfg["height"], cfg["width"], cin)).astype(np.float32)
    w = (r.standard_normal((cout, 3, 3, cin)) * np.sqrt(2.0 / (9 * cin))).astype(np.float32)
    bias = (r.standard_normal(cout) * 0.01).astype(np.float32)
    return x, w, bias


# ---------------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs (reading only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------- CPU arm
def cpu_reference_arm(cfg, steps, warmup, threads=None, per_thread=8, budget_s=90.0):
    """minml's CPU backend (fp32, its own F(5x5,3x3) choice for inference, src/layers/Conv2D.cpp:463-467) on a bounded
    sample: every host thread runs the whole network on its own shard of `per_thread` positions (the forward path of the CPU
    backend is single-threaded per context, so independent shards are how it uses all cores).  `steps` timed steps after
    `warmup` untimed ones, cut short when the timed region would pass `budget_s` seconds.  Loads only oracle/ code."""
    from tests import checkers
    threads = threads or os.cpu_count() or 1
    kind_of = cfg.get("kind", "trunk")
    hybrid = kind_of == "hybrid"
    ref_lib = None if hybrid else checkers.load_reference_cpu()
    kind = "reference" if ref_lib is not None else "port"
    if hybrid:  # the conv + attention block runs on the oracle (fp32, scalar C), one shard per host thread
        per_thread = min(per_thread, 2)
        weights = synthetic.make_hybrid_weights(SEED, cfg["channels"], cfg["heads"], cfg["ffn"], max(cfg["height"], cfg["width"]))
        x = np.random.default_rng(SEED + 1).standard_normal((threads * per_thread, cfg["height"], cfg["width"], cfg["channels"])).astype(np.float32)
        oracle = checkers.load_oracle()
        from tests.util_cpu import oracle_hybrid

        def run(i):
            oracle_hybrid(oracle, weights, x[i * per_thread:(i + 1) * per_thread], cfg["heads"])
    elif kind_of == "layer_fp32":
        x, w, bias = config0_arrays(cfg, threads * per_thread, SEED + 1)
        if ref_lib is not None:
            workers = [checkers.load_reference_cpu() if i else ref_lib for i in range(threads)]  # one backend context per thread
            cache = ref_lib.winograd_weight_transform(w, 5)

            def run(i):
                workers[i].conv3x3_winograd(x[i * per_thread:(i + 1) * per_thread], w, bias, None, "relu", 5, cache)
        else:
            oracle = checkers.load_oracle()

            def run(i):
                oracle.conv2d(x[i * per_thread:(i + 1) * per_thread], w, bias, None, "relu")
    else:
        weights = synthetic.make_trunk_weights(SEED, cfg["planes"], cfg["channels"], cfg["blocks"])
        x, _ = synthetic.bernoulli_planes((threads * per_thread, cfg["height"], cfg["width"], cfg["planes"]), SEED + 1)
        if ref_lib is not None:
            workers = [checkers.load_reference_cpu() if i else ref_lib for i in range(threads)]
            # transformed weights are computed once per layer and cached, as Conv2D does (src/layers/Conv2D.cpp:356-363)
            names = ["stem_w"] + ["b%d_w%d" % (blk, j) for blk in range(cfg["blocks"]) for j in (1, 2)]
            cache = {n: ref_lib.winograd_weight_transform(weights[n], 5) for n in names}

            def conv(r, xs, wn, bn, ext):
                return r.conv3x3_winograd(xs, weights[wn], weights[bn], ext, "relu", 5, cache[wn])

            def run(i):
                r = workers[i]
                a = conv(r, x[i * per_thread:(i + 1) * per_thread], "stem_w", "stem_b", None)
                for blk in range(cfg["blocks"]):
                    t = conv(r, a, "b%d_w1" % blk, "b%d_b1" % blk, None)
                    a = conv(r, t, "b%d_w2" % blk, "b%d_b2" % blk, a)
                rows = a.reshape(-1, cfg["channels"])
                r.gemm_ex(rows, weights["policy_w"].reshape(1, -1), weights["policy_b"], "linear")
                r.gemm_ex(r.global_average_pooling(a), weights["value_w"], weights["value_b"], "linear")
        else:
            oracle = checkers.load_oracle()
            from tests.util_cpu import oracle_trunk

            def run(i):
                oracle_trunk(oracle, weights, x[i * per_thread:(i + 1) * per_thread], cfg["blocks"])

    def step():
        ts = [threading.Thread(target=run, args=(i,)) for i in range(threads)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()

    for _ in range(warmup):
        step()
    done = 0
    t0 = time.perf_counter()
    while done < steps:
        step()
        done += 1
        if (time.perf_counter() - t0) * (done + 1) / done > budget_s:
            break  # the next step would pass the time budget
    dt = time.perf_counter() - t0
    positions = threads * per_thread * done
    what = {"hybrid": "block", "layer_fp32": "layer", "int8_trunk": "trunk (fp32 arithmetic also for the int8 configuration)"}.get(kind_of, "trunk")
    return {"value": positions / dt, "unit": "positions/s", "cores": threads, "kind": kind,
            "sample": "%d positions per step (%d per host thread, %d threads, one backend context each), %d timed steps after %d warm-up, fp32, whole %s" % (
                threads * per_thread, per_thread, threads, done, warmup, what),
            "seconds": dt, "ms_per_step": dt / done * 1e3, "steps": done, "warmup": warmup}


# ---------------------------------------------------------------------------------------------------- rooflines
def timed_launches(B, ctx, fn, reps=10):
    """Device seconds per call of `fn` (launches queued behind a short busy-wait so that they run back to back; CUDA events on
    the context's stream)."""
    for _ in range(3):
        fn()
    ctx.synchronize()
    ctx.hold_stream(0.12 * reps + 0.2)
    e0 = B.lib.cuda_create_event(ctx.handle)
    for _ in range(reps):
        fn()
    e1 = B.lib.cuda_create_event(ctx.handle)
    ctx.synchronize()
    sec = B.lib.cuda_get_time_between_events(e0, e1) / reps
    B.lib.cuda_destroy_event(e0)
    B.lib.cuda_destroy_event(e1)
    return sec


def recorded_traffic(key):
    """DRAM bytes per launch from the committed ncu summary of that kernel and size (profiles/traffic.json), else None."""
    traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(traffic_file):
        return json.load(open(traffic_file)).get(key)
    return None


def layer_roofline(B, L, ctx, cfg, peaks, torch, fused=True):
    """Times the three kernels of one channels -> channels fp16 3x3 layer alone and the fused kernel that replaces them, and
    returns the roofline record of the dominant kernel."""
    b, h, w, c = cfg["batch"], cfg["height"], cfg["width"], cfg["channels"]
    tiles = b * ((h + 3) // 4) * ((w + 3) // 4)
    rng = np.random.default_rng(3)
    wt = (rng.standard_normal((c, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
    conv = L.Conv2D(ctx, wt, np.zeros(c, np.float32), "relu", torch.float16)
    x = torch.randn((b, h, w, c), device=ctx.device, dtype=torch.float16)
    res = torch.randn((b, h, w, c), device=ctx.device, dtype=torch.float16)
    y = torch.empty_like(x)
    ws = L.Workspace(ctx)
    ws.reserve(conv.workspace_bytes(x.shape))
    ctx.set_fusion(False)
    conv.forward([x, res], y, ws)  # builds the transformed weights
    v = ws.view((36, tiles, c), torch.float16)
    m = ws.view((36, tiles, c), torch.float16, 36 * tiles * c * 2)
    act_bytes = b * h * w * c * 2
    mat_bytes = 36 * tiles * c * 2
    stages = {
        "winograd_input_transform": (lambda: B.winogradInputTransform(ctx, wt.shape, x, v, 4), act_bytes + mat_bytes),
        "gemm_tc (36 batched products)": (lambda: B.gemmBatched(ctx, "n", v, "t", conv.transformed, m), 2 * mat_bytes + 36 * c * c * 2),
        "winograd_output_transform": (lambda: B.winogradOutputTransform(ctx, wt.shape, m, y, conv.bias, res, "relu", 4), mat_bytes + 2 * act_bytes),
    }
    out = {name: dict(seconds=timed_launches(B, ctx, fn), bytes=nbytes) for name, (fn, nbytes) in stages.items()}
    ctx.set_fusion(True)
    eager = {"ms": {k: s["seconds"] * 1e3 for k, s in out.items()}, "gbs": {k: s["bytes"] / s["seconds"] / 1e9 for k, s in out.items()},
             "note": "the three-kernel path (fusion off): GB/s = algorithmic bytes of each kernel / its time"}
    if not fused:
        total = sum(s["seconds"] for s in out.values())
        name, top = max(out.items(), key=lambda kv: kv[1]["seconds"])
        hbm = top["bytes"] / top["seconds"] / 1e9
        return {"kernel": name, "bound": "hbm", "achieved": hbm, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": hbm / peaks["hbm_gbs"],
                "traffic": None, "peak_source": peaks["source"], "launch_ms": top["seconds"] * 1e3, "share_of_layer": top["seconds"] / total,
                "algorithmic_bytes": top["bytes"], "eager_layer": eager}
    # the whole layer is ONE kernel: the tcgen05 implicit-GEMM convolution (launched by the recognised call triple)
    sec = timed_launches(B, ctx, lambda: conv.forward([x, res], y, ws))
    flops = 2.0 * b * h * w * 9 * c * c
    tf = flops / sec / 1e12
    nbytes = 3 * act_bytes + 9 * c * c * 2
    return {"kernel": "kernel_conv3x3_igemm (fp16, %d -> %d, fused bias + residual + ReLU)" % (c, c), "bound": "tensor", "achieved": tf,
            "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"],
            "traffic": recorded_traffic("kernel_conv3x3_igemm") if (c, b) == (256, 1024) else recorded_traffic("kernel_conv3x3_igemm_fp16_c%d_b%d" % (c, b)),
            "peak_source": peaks["source"] + ", burst figure (kernel timed alone)", "launch_ms": sec * 1e3,
            "algorithmic_flops": flops, "algorithmic_bytes": nbytes, "hbm_gbs_at_algorithmic_bytes": nbytes / sec / 1e9,
            "eager_layer": eager}


def int8_layer_roofline(B, L, ctx, cfg, peaks, torch):
    """One channels -> channels int8 3x3 layer (im2row -> int8 GEMM -> requantise, recognised and run as one tcgen05 kernel).
    There is no measured int8 peak: the record uses twice the measured bf16 figure, the ratio of the nominal dense peaks."""
    b, h, w, c = cfg["batch"], cfg["height"], cfg["width"], cfg["channels"]
    rows = b * h * w
    rng = np.random.default_rng(3)
    qw = rng.integers(-127, 128, (c, 3, 3, c), dtype=np.int8)
    conv = L.QuantizedConv2D(ctx, qw, np.full(c, 1e-4, np.float32), np.zeros(c, np.float32), (0.02, 0.0), (0.05, 0.0), "relu", torch.int8)
    x = torch.randint(-128, 128, (b, h, w, c), device=ctx.device, dtype=torch.int8)
    res = torch.randint(-128, 128, (b, h, w, c), device=ctx.device, dtype=torch.int8)
    y = torch.empty_like(x)
    ws = L.Workspace(ctx)
    ws.reserve(conv.workspace_bytes(x.shape))
    sec = timed_launches(B, ctx, lambda: conv.forward([x, res], y, ws, (0.03, 0.0)))
    ops = 2.0 * rows * 9 * c * c
    tops = ops / sec / 1e12
    nbytes = 3 * rows * c + 9 * c * c
    peak = 2.0 * peaks["bf16_tflops"]
    return {"kernel": "kernel_conv3x3_igemm (int8, %d -> %d, fused requantise + residual + ReLU)" % (c, c), "bound": "tensor", "achieved": tops,
            "peak": peak, "unit": "TFLOP/s", "frac": tops / peak, "traffic": recorded_traffic("kernel_conv3x3_igemm_int8_c%d_b%d" % (c, b)),
            "peak_source": "2 x the bf16 figure of " + peaks["source"] + " (int8 dense peak is nominally twice bf16; no int8 figure is measured)",
            "launch_ms": sec * 1e3, "algorithmic_flops": ops, "algorithmic_bytes": nbytes, "hbm_gbs_at_algorithmic_bytes": nbytes / sec / 1e9}


def fp32_layer_roofline(B, L, ctx, cfg, peaks, torch):
    """Configuration 0's layer itself (fp32, bias + ReLU), timed as the host issues it.  fp32 products run on the tensor cores
    as three TF32 products of split operands (full fp32 accuracy), so the record's peak is a third of the TF32 rate, itself
    taken as half the measured bf16 figure (the ratio of the nominal dense peaks; no TF32 figure is measured)."""
    b, h, w, cin, c = cfg["batch"], cfg["height"], cfg["width"], cfg["planes"], cfg["channels"]
    x_np, wt, bias = config0_arrays(cfg, b, 3)
    conv = L.Conv2D(ctx, wt, bias, "relu", torch.float32)
    x = torch.from_numpy(x_np).to(ctx.device)
    y = torch.empty((b, h, w, c), device=ctx.device, dtype=torch.float32)
    ws = L.Workspace(ctx)
    ws.reserve(conv.workspace_bytes(x.shape))
    conv.forward([x], y, ws)  # the first call also transforms the weights
    before = B.launch_count()
    conv.forward([x], y, ws)
    ctx.synchronize()
    launches = B.launch_count() - before
    sec = timed_launches(B, ctx, lambda: conv.forward([x], y, ws))
    flops = 2.0 * b * h * w * 9 * cin * c
    tf = flops / sec / 1e12
    nbytes = (b * h * w * (cin + c) + 9 * cin * c) * 4
    peak = peaks["bf16_tflops"] / 2.0 / 3.0
    return {"kernel": "3x3 convolution layer fp32 %d -> %d (%d kernel launch%s per layer)" % (cin, c, launches, "" if launches == 1 else "es"),
            "bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
            "peak_source": "one sixth of the bf16 figure of " + peaks["source"] + ": TF32 is nominally half of bf16, and an fp32-accurate product is "
                           "three TF32 products",
            "launch_ms": sec * 1e3, "launches_per_layer": launches, "algorithmic_flops": flops, "algorithmic_bytes": nbytes,
            "hbm_gbs_at_algorithmic_bytes": nbytes / sec / 1e9,
            "note": "4.2 GFLOP and 15 MB per layer: at this size the launch is latency-sized (a few microseconds), far from either roofline"}


def l2_note(activation_mb):
    if activation_mb > 126.0:
        return "activations of every layer (%.0f MB) exceed the 126 MB L2, no flush needed" % activation_mb
    return ("activations of a layer are %.0f MB and stay in the 126 MB L2 from one layer to the next, which is how this workload runs in "
            "production; no flush between steps, every step rewrites all of them" % activation_mb)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------------- GPU arm
class Pipe:
    """One backend context with its own copy of the network, staging buffer, pinned host buffers and (unless --no-graph) the
    CUDA graph of one step recorded on the context's stream.  One step = the whole network on one batch: the calls of a step
    are recorded once and replayed, because the small configurations would otherwise be paced by the Python host (about 50 us
    per layer of ctypes calls against 25 us of kernel), which minml's C++ host is not."""

    def __init__(self, args, cfg, local, seed, torch, B, L):
        self.torch, self.B = torch, B
        self.ctx = B.Context(local)
        self.ctx.set_fusion(not args.eager)
        ctx = self.ctx
        kind = cfg.get("kind", "trunk")
        batch = cfg["batch"]
        if kind == "hybrid":
            weights = synthetic.make_hybrid_weights(SEED, cfg["channels"], cfg["heads"], cfg["ffn"], max(cfg["height"], cfg["width"]))
            net = L.HybridBlock(ctx, weights, batch, cfg["height"], cfg["width"], cfg["channels"], cfg["heads"], cfg["ffn"])
            tokens = np.random.default_rng(seed).standard_normal((batch, cfg["height"], cfg["width"], cfg["channels"])).astype(np.float16)
            self.in_host = torch.from_numpy(tokens).pin_memory()
            self.out_hosts = [torch.empty(tokens.shape, dtype=torch.float16).pin_memory()]
            self.predict = lambda x: (net.predict(x),)
        elif kind == "layer_fp32":
            x, w, bias = config0_arrays(cfg, batch, seed)
            net = L.Conv2D(ctx, w, bias, "relu", torch.float32)
            ws = L.Workspace(ctx)
            ws.reserve(net.workspace_bytes(x.shape))
            y = torch.empty((batch, cfg["height"], cfg["width"], cfg["channels"]), dtype=torch.float32, device=ctx.device)
            self.in_host = torch.from_numpy(x).pin_memory()
            self.out_hosts = [torch.empty(y.shape, dtype=torch.float32).pin_memory()]

            def predict(xd):
                net.forward([xd], y, ws)
                return (y,)
            self.predict = predict
        else:
            weights = synthetic.make_trunk_weights(SEED, cfg["planes"], cfg["channels"], cfg["blocks"])
            shape = (batch, cfg["height"], cfg["width"], cfg["planes"], cfg["channels"], cfg["blocks"])
            if kind == "int8_trunk":
                from minml_b200 import networks as N
                net = N.QuantizedTrunk(ctx, weights, *shape, calibration_batches=64, calibrator=args.calibrator)
            else:
                net = L.ResNetTrunk(ctx, weights, *shape)
            _, packed = synthetic.bernoulli_planes((batch, cfg["height"], cfg["width"], cfg["planes"]), seed)
            self.in_host = torch.from_numpy(packed).pin_memory()
            self.out_hosts = [torch.empty((batch, cfg["height"], cfg["width"], 1), dtype=torch.float16).pin_memory(),
                              torch.empty((batch, 3), dtype=torch.float16).pin_memory()]
            self.predict = net.predict
        self.net = net
        self.in_stage = self.in_host.to(ctx.device)
        self.h2d = self.in_host.numel() * self.in_host.element_size()
        self.d2h = sum(t.numel() * t.element_size() for t in self.out_hosts)
        self.graph, self.outs, self.launches_per_step, self.note = None, None, 0, "calls issued one by one"
        torch.cuda.synchronize(ctx.device)
        for _ in range(max(args.warmup, 3)):
            self.step()
        ctx.synchronize()
        if not args.no_graph:
            try:
                self.stream = ctx.torch_stream()
                g = torch.cuda.CUDAGraph()
                before = B.launch_count()
                with torch.cuda.graph(g, stream=self.stream):
                    self.outs = self.predict(self.in_stage)
                self.launches_per_step = B.launch_count() - before
                self.graph = g
                self.note = "CUDA graph of one step (%d kernels) replayed on the context's stream" % self.launches_per_step
                for _ in range(3):
                    self.step()
                ctx.synchronize()
            except Exception as exc:  # capture is an optimisation of the launch path only
                self.graph = None
                self.note = "calls issued one by one (graph capture failed: %s)" % str(exc)[:120]

    def step(self):
        """The network on what the staging buffer holds (device resident)."""
        if self.graph is not None:
            with self.torch.cuda.stream(self.stream):
                self.graph.replay()
            return self.outs
        return self.predict(self.in_stage)

    def step_from_host(self):
        """Pinned host input -> device, the network, results -> pinned host; all queued on the context's stream, nothing waited for."""
        lib = self.B.lib
        lib.cuda_memcpy_from_host(self.ctx.handle, ctypes.c_void_p(self.in_stage.data_ptr()), 0, ctypes.c_void_p(self.in_host.data_ptr()), self.h2d)
        outs = self.step()
        for dst, src in zip(self.out_hosts, outs):
            lib.cuda_memcpy_to_host(self.ctx.handle, ctypes.c_void_p(dst.data_ptr()), ctypes.c_void_p(src.data_ptr()), 0, src.numel() * src.element_size())


def measure(args, cfg, replicas, steps, sample_clocks=True):
    """value / e2e / roofline of one configuration on this rank's GPU (max over ranks for the times); rank 0 returns the record."""
    import torch
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    local = replicas.local_rank
    world, rank = replicas.world, replicas.rank
    barrier = replicas.barrier
    batch = cfg["batch"]
    kind = cfg.get("kind", "trunk")
    pipe = Pipe(args, cfg, local, replicas.input_seed(SEED), torch, B, L)
    ctx = pipe.ctx

    sampler = ClockSampler(local)
    if sample_clocks:
        sampler.start()
    launches0 = B.launch_count()
    barrier()
    e0 = B.lib.cuda_create_event(ctx.handle)
    for _ in range(steps):
        pipe.step()
    e1 = B.lib.cuda_create_event(ctx.handle)
    ctx.synchronize()
    local_dev_s = B.lib.cuda_get_time_between_events(e0, e1)
    B.lib.cuda_destroy_event(e0)
    B.lib.cuda_destroy_event(e1)
    barrier()
    dev_s = replicas.max_over_ranks([local_dev_s])[0]
    launches = (B.launch_count() - launches0) if pipe.graph is None else pipe.launches_per_step * steps
    resident = [t.detach().cpu().clone() for t in pipe.step()]

    # End to end through the C ABI with host buffers.  Two contexts (two streams, two copies of the network) take the steps in
    # turn, so that the copies of one step overlap the arithmetic of the other; the caller collects the result of step i when it
    # comes back to that context for step i + 2 (or + 3), i.e. every step's result is waited for inside the timed region.
    # (a step that moves tens of megabytes each way over PCIe -- the token tensors of the conv + attention block -- gets a third
    # context, so that one step's copy-in, another's arithmetic and a third's copy-out run at the same time: the link is full duplex)
    n_pipes = 1 if args.no_overlap else (3 if pipe.h2d + pipe.d2h > (8 << 20) else 2)
    pipes = [pipe] + [Pipe(args, cfg, local, replicas.input_seed(SEED), torch, B, L) for _ in range(n_pipes - 1)]
    for p in pipes:
        p.step_from_host()
        p.ctx.synchronize()
    barrier()
    t0 = time.perf_counter()
    for i in range(steps):
        p = pipes[i % len(pipes)]
        p.ctx.synchronize()  # the result of this context's previous step is in host memory now
        p.step_from_host()
    for p in pipes:
        p.ctx.synchronize()
    e2e_wall = time.perf_counter() - t0
    barrier()
    e2e_s = replicas.max_over_ranks([e2e_wall])[0]
    clocks = sampler.stop() if sample_clocks else None

    # sanity: the host-fed runs computed what the resident run computed, and nothing overflowed
    outputs_ok = all(bool(torch.isfinite(h.float()).all()) and torch.equal(h, r) for p in pipes for h, r in zip(p.out_hosts, resident))
    per_rank = None
    if world > 1:  # who is the slowest rank, and at what clock
        ms = replicas.gather_floats(local_dev_s / steps * 1e3)
        mhz = replicas.gather_floats((clocks or {}).get("sm_mhz") or 0.0)
        per_rank = {"ms_per_step": {"min": min(ms), "median": float(np.median(ms)), "max": max(ms), "all": ms}, "slowest_rank": int(np.argmax(ms)),
                    "sm_mhz_median_per_rank": mhz, "note": "weak scaling without a collective: the step time of the job is the slowest rank's"}
    result = None
    if rank == 0:
        peaks = load_peaks()
        if kind == "int8_trunk":
            roof = int8_layer_roofline(B, L, ctx, cfg, peaks, torch)
        elif kind == "layer_fp32":
            roof = fp32_layer_roofline(B, L, ctx, cfg, peaks, torch)
        else:
            roof = layer_roofline(B, L, ctx, cfg, peaks, torch, fused=not args.eager)
        total_positions = replicas.global_units(batch) * steps
        value = total_positions / dev_s
        fpp = flops_per_position(cfg)
        elem = {"int8_trunk": 1, "layer_fp32": 4}.get(kind, 2)
        result = {
            "metric": METRIC[kind], "value": value, "unit": "positions/s", "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": dev_s / steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": DTYPE[kind], "data": "synthetic", "outputs_finite_and_equal": outputs_ok,
            "config": {"workload": cfg["label"], "batch_per_gpu": batch, "global_batch": batch * world, "parallelism": "dp%d replicas" % world,
                       "conv3x3": "three kernels per layer (fusion off)" if args.eager else "fused (one kernel per layer where the fused kernel takes the shape)",
                       "launch": pipe.note,
                       "e2e_overlap": "%d contexts take the steps in turn (copies of one overlap the arithmetic of the others)" % len(pipes) if len(pipes) > 1 else "none",
                       "l2": l2_note(batch * cfg["height"] * cfg["width"] * cfg["channels"] * elem / 1e6)},
            "algorithmic_tflops": value * fpp / 1e12,
            "frac_of_nominal_dense_peak": value * fpp / world / {"int8_trunk": 4.5e15, "layer_fp32": 1.125e15 / 3}.get(kind, 2.25e15),
            "e2e": {"value": total_positions / e2e_s, "unit": "positions/s", "h2d_bytes_per_step": pipe.h2d, "d2h_bytes_per_step": pipe.d2h,
                    "ms_per_step": e2e_s / steps * 1e3},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
        }
        if per_rank is not None:
            result["ranks"] = per_rank
    for p in pipes:
        p.ctx.close()
    del pipes, pipe
    torch.cuda.empty_cache()
    return result


def dropin_host(cfg, repeats):
    """The same trunk through minml's own unmodified host code: oracle/_ref/trunk_dropin (the reference's Graph / layers / core
    sources linked with this library as THE CUDA backend) times `repeats` calls of Graph::predict after three warm-up calls."""
    binary = os.path.join(ROOT, "oracle", "_ref", "trunk_dropin")
    if cfg.get("kind", "trunk") != "trunk":
        return None
    if not os.path.exists(binary):
        return {"unavailable": "oracle/_ref/trunk_dropin not built (it needs the reference checkout at build time)"}
    argv = [binary] + [str(cfg[k]) for k in ("batch", "height", "width", "planes", "channels", "blocks")] + ["fp16", str(repeats)]
    try:
        out = subprocess.run(argv, capture_output=True, text=True, timeout=300, env=dict(os.environ, DROPIN_TIMING_ONLY="1"))
        rec = json.loads(out.stdout.strip().splitlines()[-1])
        return {"value": rec["positions_per_s"], "unit": "positions/s", "repeats": repeats, "nodes": rec["nodes"],
                "how": "minml's unmodified Graph::predict (one stream, no CUDA graph, input resident) over libminml_b200.so, wall clock around the loop"}
    except Exception as exc:
        return {"unavailable": "trunk_dropin failed: %s" % str(exc)[:160]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the short measurements of the other configurations (N = 1 default run)")
    ap.add_argument("--no-graph", action="store_true", help="issue every backend call from the host each step instead of replaying a CUDA graph")
    ap.add_argument("--no-overlap", action="store_true", help="end-to-end steps on one context, one after the other")
    ap.add_argument("--calibrator", default="max_abs", choices=["max_abs", "histogram"],
                    help="int8 configuration: activation transforms by the max-abs rule the configuration states, or by minml's histogram calibrator")
    ap.add_argument("--eager", action="store_true", help="three kernels per 3x3 layer (fusion off) instead of the fused convolution")
    ap.add_argument("--layer", action="store_true", help="time only one channels -> channels 3x3 layer (the roofline record); used for ncu captures")
    ap.add_argument("--layer-batch", type=int, default=0, help="batch size for --layer (default: the config's)")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    kind = cfg.get("kind", "trunk")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank != 0:
            return
        base = cpu_reference_arm(cfg, max(args.steps, 1), max(args.warmup, 0), budget_s=120.0)
        line = {"impl": "reference", "metric": METRIC[kind], "value": base["value"], "unit": "positions/s", "n_gpus": args.gpus,
                "steps": base["steps"], "warmup": base["warmup"], "steps_requested": args.steps, "ms_per_step": base["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": cfg["label"],
                           "note": "host CPU implementation; each step is a bounded sample of the workload (the timed steps stop early only if they "
                                   "would pass 120 s)"},
                "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": base["value"], "unit": "positions/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the backend has no CPU fallback")
    if args.layer:
        from minml_b200 import backend as B
        from minml_b200 import layers as L
        cfg = dict(cfg, batch=args.layer_batch or cfg["batch"])
        ctx = B.Context(0)
        if kind == "int8_trunk":
            rec = int8_layer_roofline(B, L, ctx, cfg, load_peaks(), torch)
        elif kind == "layer_fp32":
            rec = fp32_layer_roofline(B, L, ctx, cfg, load_peaks(), torch)
        else:
            rec = layer_roofline(B, L, ctx, cfg, load_peaks(), torch, fused=not args.eager)
        print(json.dumps(rec))
        ctx.close()
        return

    from minml_b200.replicas import Replicas
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    replicas = Replicas("nccl")
    result = measure(args, cfg, replicas, args.steps)
    if rank == 0:
        if world == 1 and args.config == "c3" and not args.no_other_configs:
            others = []
            for name in ("c0", "c1", "c2", "c4"):
                try:
                    rec = measure(args, CONFIGS[name], replicas, min(args.steps, 10), sample_clocks=False)
                    rec = {k: rec[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "dtype", "outputs_finite_and_equal", "algorithmic_tflops",
                                               "e2e", "gpu_launches", "roofline")}
                    rec["roofline"].pop("eager_layer", None)
                    rec["config"] = name
                    rec["workload"] = CONFIGS[name]["label"]
                    hosted = dropin_host(CONFIGS[name], 50)
                    if hosted is not None:
                        rec["dropin_host"] = hosted
                    others.append(rec)
                except Exception as exc:  # the headline line must not depend on a side measurement
                    others.append({"config": name, "error": str(exc)[:200]})
            result["other_configs"] = others
        if world == 1:
            hosted = dropin_host(cfg, 20)
            if hosted is not None:
                result["dropin_host"] = hosted
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_reference_arm(cfg, 2, 1, budget_s=25.0)
            result["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        else:
            result["cpu_baseline"] = None
        print(json.dumps(result))
    replicas.close()


if __name__ == "__main__":
    main()
