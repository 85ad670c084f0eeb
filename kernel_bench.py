"""Per-kernel timing of every hot entry point of the backend at the sizes of the benchmark configurations.

    python kernel_bench.py [--config c3|c1|c2|c4] [--reps N] [--only substring]

Each entry point is timed alone with CUDA events on the context's stream (3 warm-up calls, N timed calls).  For every kernel
the line gives the time, the algorithmic bytes (each input read once, each output written once) and FLOPs of one call, and
the achieved GB/s and TFLOP/s as fractions of the measured peaks (MEASURED_PEAKS.json at the repository root, else the
fallback figures 6650 GB/s and 1590 TFLOP/s).  Working sets are the real activation sizes of the configuration, which for
c3 exceed the L2 cache; smaller configurations are noted as L2-resident in the output.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from minml_b200 import backend as B  # noqa: E402
from minml_b200 import layers as L  # noqa: E402

SIZES = {
    "c3": dict(batch=1024, h=20, w=20, c=256, planes=32),
    "c1": dict(batch=256, h=15, w=15, c=128, planes=32),
    "c2": dict(batch=512, h=20, w=20, c=128, planes=32),
    "c4": dict(batch=256, h=15, w=15, c=256, planes=32),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timed(ctx, fn, reps):
    for _ in range(3):
        fn()
    ctx.synchronize()
    ctx.hold_stream(0.12 * reps + 0.2)  # the launches below queue up behind this wait and then run back to back
    e0 = B.lib.cuda_create_event(ctx.handle)
    for _ in range(reps):
        fn()
    e1 = B.lib.cuda_create_event(ctx.handle)
    ctx.synchronize()
    sec = B.lib.cuda_get_time_between_events(e0, e1) / reps
    B.lib.cuda_destroy_event(e0)
    B.lib.cuda_destroy_event(e1)
    return sec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c3", choices=sorted(SIZES))
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    s = SIZES[args.config]
    b, h, w, c, planes = s["batch"], s["h"], s["w"], s["c"], s["planes"]
    hbm, tflops, source = peaks()
    ctx = B.Context(0)
    rng = np.random.default_rng(0)
    f16 = torch.float16
    act_bytes = b * h * w * c * 2
    tiles = b * ((h + 3) // 4) * ((w + 3) // 4)

    def rand(*shape, dtype=f16):
        return (torch.randn(shape, device="cuda") * 0.5).to(dtype)

    x, res, y = rand(b, h, w, c), rand(b, h, w, c), torch.empty((b, h, w, c), device="cuda", dtype=f16)
    wt = (rng.standard_normal((c, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
    conv = L.Conv2D(ctx, wt, np.zeros(c, np.float32), "relu", f16)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(x.shape))
    v = ws.view((36, tiles, c), f16)
    m = ws.view((36, tiles, c), f16, 36 * tiles * c * 2)
    mat_bytes = 36 * tiles * c * 2
    bias = rand(c)
    rows = b * h * w
    results = []

    def add(name, fn, nbytes, flops=0.0, note=""):
        if args.only and args.only not in name:
            return
        sec = timed(ctx, fn, args.reps)
        rec = {"kernel": name, "config": args.config, "ms": sec * 1e3, "algorithmic_MB": nbytes / 1e6, "GB/s": nbytes / sec / 1e9,
               "hbm_frac": nbytes / sec / 1e9 / hbm, "peaks": source}
        if flops:
            rec["TFLOP/s"] = flops / sec / 1e12
            rec["tensor_frac"] = flops / sec / 1e12 / tflops
        if note:
            rec["note"] = note
        results.append(rec)
        print(json.dumps(rec), flush=True)

    # ---- the fused 3x3 layer (one kernel for the recognised call triple) and its three-kernel equivalent
    ctx.set_fusion(True)
    add("conv3x3 fused (fp16, bias+residual+relu)", lambda: conv.forward([x, res], y, ws), 3 * act_bytes + 9 * c * c * 2,
        2.0 * rows * 9 * c * c)
    ctx.set_fusion(False)
    conv.forward([x, res], y, ws)
    add("winograd_input_transform", lambda: B.winogradInputTransform(ctx, wt.shape, x, v, 4), act_bytes + mat_bytes)
    add("gemm_batched 36 x [tiles,c] x [c,c]^T", lambda: B.gemmBatched(ctx, "n", v, "t", conv.transformed, m), 2 * mat_bytes + 36 * c * c * 2,
        2.0 * 36 * tiles * c * c)
    # the two products of the backward pass, whose operands the tensor core reads MN-major: dV = dM x U ('n','n'), dU = dM^T x V ('t','n')
    du = torch.empty((36, c, c), device="cuda", dtype=f16)
    add("gemm_batched 36 x [tiles,c] x [c,c] ('n','n', backward)", lambda: B.gemmBatched(ctx, "n", m, "n", conv.transformed, v),
        2 * mat_bytes + 36 * c * c * 2, 2.0 * 36 * tiles * c * c)
    add("gemm_batched 36 x [tiles,c]^T x [tiles,c] ('t','n', weight update)", lambda: B.gemmBatched(ctx, "t", m, "n", v, du),
        2 * mat_bytes + 36 * c * c * 2, 2.0 * 36 * tiles * c * c)
    add("winograd_output_transform (+bias+residual+relu)", lambda: B.winogradOutputTransform(ctx, wt.shape, m, y, conv.bias, res, "relu", 4),
        mat_bytes + 2 * act_bytes)
    add("winograd_weight_transform", lambda: B.winogradWeightTransform(ctx, conv.weights, conv.transformed, False, 4), (9 + 36) * c * c * 2)
    ctx.set_fusion(True)

    # ---- heads: 1x1 policy convolution (N = 1), global average pooling, dense value head (N = 3)
    wp, bp, bv = rand(1, c), rand(1), rand(3)
    pol = torch.empty((rows, 1), device="cuda", dtype=f16)
    add("gemm_ex 1x1 policy head [rows,c] x [1,c]^T", lambda: B.gemm_ex(ctx, pol, 1.0, "n", x.view(rows, c), "t", wp, 0.0, None, bp, "linear"),
        act_bytes + rows * 2, 2.0 * rows * c)
    pooled = torch.empty((b, c), device="cuda", dtype=f16)
    add("global_average_pooling", lambda: B.globalAveragePoolingForward(ctx, x, pooled), act_bytes + b * c * 2)
    wv = rand(3, c)
    val = torch.empty((b, 3), device="cuda", dtype=f16)
    add("gemm_ex dense value head [b,c] x [3,c]^T", lambda: B.gemm_ex(ctx, val, 1.0, "n", pooled, "t", wv, 0.0, None, bv, "linear"),
        b * c * 2 + b * 6, 2.0 * b * c * 3, note="launch-latency bound at this size")

    # ---- 1x1 convolutions / dense layers of the attention block: gemm_ex with fused bias (+ residual, + ReLU)
    for n_out, k_in, label in ((3 * c, c, "qkv projection"), (c, c, "output projection + residual"), (4 * c, c, "FFN up + relu"),
                               (c, 4 * c, "FFN down + residual")):
        a_in = rand(rows, k_in)
        w_in, b_in = rand(n_out, k_in), rand(n_out)
        out = torch.empty((rows, n_out), device="cuda", dtype=f16)
        ext = rand(rows, n_out) if "residual" in label else None
        act = "relu" if "relu" in label else "linear"
        add("gemm_ex [rows,%d] x [%d,%d]^T %s" % (k_in, n_out, k_in, label),
            lambda a_in=a_in, w_in=w_in, b_in=b_in, out=out, ext=ext, act=act: B.gemm_ex(ctx, out, 1.0, "n", a_in, "t", w_in, 1.0 if ext is not None else 0.0,
                                                                                          ext, b_in, act),
            rows * (k_in + n_out * (2 if ext is not None else 1)) * 2 + n_out * k_in * 2, 2.0 * rows * n_out * k_in)
        del a_in, w_in, out, ext

    # ---- fp32 operands: three TF32 products of split operands by default, one TF32 product once the host allows TF32
    rows32 = rows // 2
    a32, w32 = torch.randn((rows32, c), device="cuda"), torch.randn((c, c), device="cuda")
    d32 = torch.empty((rows32, c), device="cuda")
    add("gemm fp32 [rows/2,c] x [c,c]^T split operands", lambda: B.gemm(ctx, "n", a32, "t", w32, d32), 2 * rows32 * c * 4 + c * c * 4,
        2.0 * rows32 * c * c, note="tensor_frac is against the bf16 peak; TF32 runs at half of it and this path needs 3 products")
    ctx.enable_tf32(True)
    add("gemm fp32 [rows/2,c] x [c,c]^T as TF32", lambda: B.gemm(ctx, "n", a32, "t", w32, d32), 2 * rows32 * c * 4 + c * c * 4,
        2.0 * rows32 * c * c, note="tensor_frac is against the bf16 peak; TF32 runs at half of it")
    ctx.enable_tf32(False)
    del a32, d32

    # ---- elementwise / layout
    packed = torch.randint(0, 2 ** 31 - 1, (b, h, w, 1), device="cuda", dtype=torch.int32)
    x0 = torch.empty((b, h, w, planes), device="cuda", dtype=f16)
    add("unpack_input (32 planes)", lambda: B.unpackInput(ctx, packed, x0), rows * 4 + rows * planes * 2)
    add("add_bias_act (relu)", lambda: B.addBiasAct(ctx, x, bias, y, "relu"), 2 * act_bytes)
    add("activation_forward (relu)", lambda: B.activationForward(ctx, x, y, "relu"), 2 * act_bytes)
    add("add_tensors (y = x1 + x2)", lambda: B.addTensors(ctx, y, 1.0, x, 1.0, res), 3 * act_bytes)
    xf = torch.empty((b, h, w, c), device="cuda", dtype=torch.float32)
    add("convert_type fp16 -> fp32", lambda: B.convertType(ctx, xf, x), act_bytes * 3)
    gamma, beta = rand(c), rand(c)
    add("layernorm_forward", lambda: B.layernormForward(ctx, x, y, gamma, beta), 2 * act_bytes)
    add("softmax_forward (rows of c)", lambda: B.softmaxForward(ctx, x.view(rows, c), y.view(rows, c)), 2 * act_bytes)

    # ---- int8: fused convolution and the eager steps
    xq = torch.randint(-128, 128, (b, h, w, c), device="cuda", dtype=torch.int8)
    extq = torch.randint(-128, 128, (b, h, w, c), device="cuda", dtype=torch.int8)
    yq = torch.empty((b, h, w, c), device="cuda", dtype=torch.int8)
    qw = rng.integers(-127, 128, (c, 3, 3, c), dtype=np.int8)
    qconv = L.QuantizedConv2D(ctx, qw, np.full(c, 1e-4, np.float32), np.zeros(c, np.float32), (0.02, 0.0), (0.05, 0.0), "relu", torch.int8)
    qws = L.Workspace()
    qws.reserve(qconv.workspace_bytes(xq.shape))
    add("conv3x3 fused (int8, requantise+relu, no residual)", lambda: qconv.forward([xq], yq, qws), 2 * rows * c + 9 * c * c,
        2.0 * rows * 9 * c * c)
    add("conv3x3 fused (int8, requantise+residual+relu)", lambda: qconv.forward([xq, extq], yq, qws, (0.03, 0.0)), 3 * rows * c + 9 * c * c,
        2.0 * rows * 9 * c * c, note="tensor_frac is against the bf16 peak; the int8 peak is twice that")
    ctx.set_fusion(False)
    acc = qws.view((rows, c), torch.int32)
    rows_i8 = qws.view((rows, 9 * c), torch.int8, rows * c * 4)
    add("im2row int8 3x3", lambda: B.im2row(ctx, xq, rows_i8, 3, False, np.int8(0)), rows * c + rows * 9 * c)
    add("gemm int8 [rows,9c] x [c,9c]^T -> int32", lambda: B.gemm(ctx, "n", rows_i8, "t", qconv.weights.view(c, 9 * c), acc),
        rows * 9 * c + rows * c * 4 + 9 * c * c, 2.0 * rows * 9 * c * c)
    add("quantized_scale_shift_act -> int8", lambda: B.quantized_scale_shift_act(ctx, yq, (0.05, 0.0), acc, qconv.channel_scales, qconv.bias, "relu",
                                                                                 extq, (0.03, 0.0)), rows * c * 4 + 2 * rows * c)
    ctx.set_fusion(True)

    # ---- attention (config 4 geometry: 8 heads of c / 8)
    heads = 8
    qkv = rand(b, h, w, 3 * c)
    n = 2 * max(h, w) - 1
    table = rand(heads, n, (n + 3) // 4 * 4)
    att = torch.empty((b, h, w, c), device="cuda", dtype=f16)
    t = h * w
    add("multi_head_attention_forward (8 heads, rel-pos bias)", lambda: B.multiHeadAttentionForward(ctx, qkv, att, table, heads), 4 * act_bytes,
        4.0 * b * heads * t * t * (c // heads))
    if c // heads == 32 and t <= 462:  # the kernels the default chooses between, each forced
        for kernel, name in ((1, "tcgen05 wherever possible"), (2, "tcgen05 with one CTA per (head, item)"), (3, "warp-level mma.sync kernel")):
            B.set_attention_kernel(kernel)
            add("multi_head_attention_forward, %s (8 heads, rel-pos bias)" % name, lambda: B.multiHeadAttentionForward(ctx, qkv, att, table, heads),
                4 * act_bytes, 4.0 * b * heads * t * t * (c // heads))
        B.set_attention_kernel(0)

    # ---- what one tensor-core instruction costs by N (one SM, 2 000 instructions back to back): the basis of the tile-shape notes
    if not args.only or "tcgen05.mma" in args.only:
        cycles = {str(nn): [round(B.lib.mb200_probe_mma_cycles(ctx.handle, nn, a), 1) for a in (0, 1)] for nn in (16, 32, 64, 128, 256)}
        ctx.check()
        print(json.dumps({"probe": "tcgen05.mma cycles (kind::f16, M = 128, K = 16) by N: [A in shared memory, A in tensor memory]", "cycles": cycles}), flush=True)

    # ---- layers next to the convolution path: batch norm at inference, depthwise 7x7 (fp16 and int8), channel scaling
    avg_var = torch.cat([torch.randn(1, c, device="cuda"), torch.rand(1, c, device="cuda") + 0.5]).contiguous()
    add("batchnorm_inference (+relu)", lambda: B.batchnormInference(ctx, x, y, gamma, beta, avg_var, "relu"), 2 * act_bytes)
    wdw = rand(7, 7, c)
    add("depthwise_conv_forward 7x7 fp16", lambda: B.depthwiseConvForward(ctx, x, wdw, y, bias), 2 * act_bytes + 49 * c * 2)
    wdq = torch.randint(-127, 128, (7, 7, c), device="cuda", dtype=torch.int8)
    dscale, dbias = torch.full((c,), 1e-4, device="cuda"), torch.zeros(c, device="cuda")
    add("quantized_depthwise_conv_forward 7x7 int8", lambda: B.quantized_depthwise_conv_forward(ctx, xq, wdq, dscale, dbias, yq, (0.05, 0.0), 0),
        2 * rows * c + 49 * c)
    add("rmsnorm_forward", lambda: B.rmsnormForward(ctx, x, y, gamma), 2 * act_bytes)
    deep = torch.empty((b, (h + 1) // 2, (w + 1) // 2, 4 * c), device="cuda", dtype=f16)
    add("space_to_depth 2x2", lambda: B.spaceToDepth(ctx, x, deep), act_bytes + deep.numel() * 2)
    add("depth_to_space 2x2", lambda: B.depthToSpace(ctx, deep, y), act_bytes + deep.numel() * 2)
    del deep
    gate = rand(b, c)
    add("channel_scaling_forward", lambda: B.channelScalingForward(ctx, x, gate, y), 2 * act_bytes + b * c * 2)
    ctx.close()


if __name__ == "__main__":
    main()
