"""Bandwidth-bound entry points on the GPU against the oracle: bias/activation, tensor sums, pooling, unpacking,
conversion, transposition, softmax, layer norm, attention, and the eager int8 steps."""
import os

import numpy as np
import pytest
import torch

from tests.util import FP16_REL, FP32_TOL, INT8_REL, dev, host, init_for_test, max_rel_err, mean_abs_diff

pytestmark = pytest.mark.gpu


def close(dtype, got, want, what=""):
    if dtype == torch.float16:
        assert max_rel_err(got, want) <= FP16_REL, what
    else:
        assert mean_abs_diff(got, want) <= FP32_TOL, what


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(23, 35), (4, 15, 15, 128), (1, 7), (3, 1000)])
def test_add_bias_act_and_activation(ctx, oracle, dtype, shape):
    from minml_b200 import backend as B
    x = init_for_test(shape)
    bias = init_for_test((shape[-1],), 1.0)
    if dtype == torch.float16:
        x, bias = x.astype(np.float16).astype(np.float32), bias.astype(np.float16).astype(np.float32)
    for act in ("linear", "sigmoid", "tanh", "relu", "leaky_relu"):
        y = torch.full(shape, float("nan"), device="cuda", dtype=dtype)
        B.addBiasAct(ctx, dev(x, dtype), dev(bias, dtype), y, act)
        ctx.synchronize()
        close(dtype, host(y), oracle.add_bias_act(x, bias, act), act)
        y2 = torch.full(shape, float("nan"), device="cuda", dtype=dtype)
        B.activationForward(ctx, dev(x, dtype), y2, act)
        ctx.synchronize()
        close(dtype, host(y2), oracle.add_bias_act(x, None, act), act)
    # alpha / beta:  y = act(x + b) * alpha + beta * y
    y = dev(init_for_test(shape, 2.0), dtype)
    y0 = host(y).copy()
    B.addBiasAct(ctx, dev(x, dtype), dev(bias, dtype), y, "relu", alpha=0.5, beta=2.0)
    ctx.synchronize()
    close(dtype, host(y), oracle.add_bias_act(x, bias, "relu") * 0.5 + 2.0 * y0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("n", [1, 37, 4096, 100003])
def test_add_tensors(ctx, dtype, n):
    from minml_b200 import backend as B
    x1, x2, x3, y = [init_for_test((n,), s) for s in (0.0, 1.0, 2.0, 3.0)]
    if dtype == torch.float16:
        x1, x2, x3, y = [t.astype(np.float16).astype(np.float32) for t in (x1, x2, x3, y)]
    yd = dev(y, dtype)
    B.addTensors(ctx, yd, 1.0, dev(x1, dtype), 0.5, dev(x2, dtype), -2.0, dev(x3, dtype), 0.25)
    ctx.synchronize()
    close(dtype, host(yd), x1 + 0.5 * x2 - 2.0 * x3 + 0.25 * y)
    yd = dev(y, dtype)
    B.addTensors(ctx, yd, 1.0, dev(x1, dtype), 1.0, dev(x2, dtype))  # residual add: y = x1 + x2
    ctx.synchronize()
    close(dtype, host(yd), x1 + x2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(3, 5, 7, 36), (4, 15, 15, 128), (2, 20, 20, 256), (2, 3, 3, 5)])
def test_global_average_pooling(ctx, oracle, dtype, shape):
    from minml_b200 import backend as B
    x = init_for_test(shape)
    if dtype == torch.float16:
        x = x.astype(np.float16).astype(np.float32)
    y = torch.full((shape[0], shape[3]), float("nan"), device="cuda", dtype=dtype)
    B.globalAveragePoolingForward(ctx, dev(x, dtype), y)
    ctx.synchronize()
    close(dtype, host(y), oracle.global_average_pooling(x))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int8])
@pytest.mark.parametrize("channels", [32, 35, 64, 5])
def test_unpack_input_is_exact(ctx, oracle, dtype, channels):
    from minml_b200 import backend as B
    rows = 7 * 9
    words = (channels + 31) // 32
    packed = np.random.default_rng(channels).integers(0, 2 ** 32, size=rows * words, dtype=np.uint64).astype(np.uint32)
    dst = torch.full((7, 9, channels), 3, device="cuda", dtype=dtype)
    B.unpackInput(ctx, dev(packed.view(np.int32)), dst)
    ctx.synchronize()
    assert np.array_equal(host(dst).astype(np.float32), oracle.unpack_input(packed, (7, 9, channels)))


def test_convert_and_transpose(ctx):
    from minml_b200 import backend as B
    x = init_for_test((1237,), 0.0, 50.0)
    for src_t, dst_t in ((torch.float32, torch.float16), (torch.float16, torch.float32), (torch.float32, torch.int8), (torch.int8, torch.float32),
                         (torch.int32, torch.float16)):
        src = dev(x).to(src_t)
        dst = torch.zeros(1237, device="cuda", dtype=dst_t)
        B.convertType(ctx, dst, src)
        ctx.synchronize()
        if dst_t == torch.int8:  # the backend converts by truncation through fp32, like static_cast in the reference
            assert torch.equal(dst, src.float().trunc().to(torch.int8))
        else:
            assert torch.equal(dst, src.float().to(dst_t))
    for dtype in (torch.float32, torch.float16, torch.int8):
        t = (dev(init_for_test((3, 37, 45))) * 100).to(dtype).contiguous()
        out = torch.zeros(3, 45, 37, device="cuda", dtype=dtype)
        B.transpose_021(ctx, t, out)
        ctx.synchronize()
        assert torch.equal(out, t.transpose(1, 2).contiguous())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_softmax(ctx, oracle, dtype):
    from minml_b200 import backend as B
    for shape in ((50, 3), (7, 225), (3, 1000)):
        x = init_for_test(shape, 0.0, 3.0)
        if dtype == torch.float16:
            x = x.astype(np.float16).astype(np.float32)
        y = torch.zeros(shape, device="cuda", dtype=dtype)
        B.softmaxForward(ctx, dev(x, dtype), y)
        ctx.synchronize()
        close(dtype, host(y), oracle.softmax(x))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(3, 5, 7, 36), (2, 15, 15, 256), (11, 33), (37, 512), (5, 3, 1024)])
def test_layernorm(ctx, oracle, dtype, shape):
    from minml_b200 import backend as B
    r = np.random.default_rng(1)
    x = r.standard_normal(shape).astype(np.float32)
    ext = r.standard_normal(shape).astype(np.float32)
    gamma = r.standard_normal(shape[-1]).astype(np.float32)
    beta = r.standard_normal(shape[-1]).astype(np.float32)
    if dtype == torch.float16:
        x, ext, gamma, beta = [t.astype(np.float16).astype(np.float32) for t in (x, ext, gamma, beta)]
    for e in (None, ext):
        y = torch.zeros(shape, device="cuda", dtype=dtype)
        B.layernormForward(ctx, dev(x, dtype), y, dev(gamma, dtype), dev(beta, dtype), None if e is None else dev(e, dtype))
        ctx.synchronize()
        close(dtype, host(y), oracle.layernorm(x, gamma, beta, e))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("cfg", [(2, 5, 6, 2, 8, False), (2, 15, 15, 8, 32, False), (1, 4, 4, 3, 16, True), (1, 9, 7, 4, 20, False)])
def test_multi_head_attention(ctx, oracle, dtype, cfg):
    # reference: test/backend/test_attention.cpp:273-300,441-503
    from minml_b200 import backend as B
    b, h, w, heads, d, symmetric = cfg
    r = np.random.default_rng(h * w)
    parts = 2 if symmetric else 3
    x = r.standard_normal((b, h, w, parts * heads * d)).astype(np.float32)
    n = 2 * max(h, w) - 1
    table = (r.standard_normal((heads, n, (n + 3) // 4 * 4)) * 0.5).astype(np.float32)
    if dtype == torch.float16:
        x, table = x.astype(np.float16).astype(np.float32), table.astype(np.float16).astype(np.float32)
    for t in (None, table):
        y = torch.zeros((b, h, w, heads * d), device="cuda", dtype=dtype)
        B.multiHeadAttentionForward(ctx, dev(x, dtype), y, None if t is None else dev(t, dtype), heads, symmetric)
        ctx.synchronize()
        close(dtype, host(y), oracle.mha_forward(x, heads, t, symmetric))
    assert B.multiHeadAttentionGetWorkspaceSize((b, h, w, parts * heads * d), table.shape, heads) == b * heads * (h * w) ** 2


# ---------------------------------------------------------------------------------------------------- eager int8 steps
@pytest.mark.parametrize("dtype", [torch.int8, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 6, 7, 12, 3), (3, 20, 20, 32, 3), (2, 5, 5, 7, 3), (2, 4, 4, 16, 1), (1, 9, 9, 8, 5)])
def test_im2row_is_exact(ctx, oracle, dtype, shape):
    # reference: test/backend/test_gemm_conv.cpp:68-178 (exact equality)
    from minml_b200 import backend as B
    b, h, w, c, k = shape
    x = (init_for_test((b, h, w, c)) * 100).astype({torch.int8: np.int8, torch.float16: np.float16, torch.float32: np.float32}[dtype])
    for invert in (False, True):
        for pad in (None, 3):
            out = torch.zeros((b * h * w, k * k * c), device="cuda", dtype=dtype)
            B.im2row(ctx, dev(x), out, k, invert, pad)
            ctx.synchronize()
            want = oracle.im2row(x, k, invert, pad)
            assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("shape", [(11 * 12 * 13, 44), (300, 128), (7, 5)])
def test_scale_shift_act(ctx, oracle, shape):
    # reference: test/backend/test_quantization.cpp:173-240 (int8 and fp32 outputs, with and without ext)
    from minml_b200 import backend as B
    r = np.random.default_rng(shape[1])
    acc = r.integers(-30000, 30000, shape, dtype=np.int32)
    scales = r.uniform(1e-4, 1e-3, shape[1]).astype(np.float32)
    bias = r.standard_normal(shape[1]).astype(np.float32)
    ext = r.integers(-128, 128, shape, dtype=np.int8)
    out_qd, ext_qd = (0.06, 0.2), (0.03, -0.1)
    for act in ("linear", "relu", "sigmoid", "tanh"):
        for e in (None, ext):
            want8, wantf = oracle.scale_shift_act(acc, scales, bias, out_qd, act, e, ext_qd)
            y8 = torch.zeros(shape, device="cuda", dtype=torch.int8)
            B.quantized_scale_shift_act(ctx, y8, out_qd, dev(acc), dev(scales), dev(bias), act, None if e is None else dev(e), ext_qd)
            yf = torch.zeros(shape, device="cuda", dtype=torch.float32)
            B.quantized_scale_shift_act(ctx, yf, out_qd, dev(acc), dev(scales), dev(bias), act, None if e is None else dev(e), ext_qd)
            ctx.synchronize()
            assert max_rel_err(host(yf), wantf) <= 1e-5
            assert np.max(np.abs(host(y8).astype(np.int32) - want8.astype(np.int32))) <= 1  # fused multiply-add may move a tie
            assert np.mean(host(y8) != want8) <= 1e-3


def test_dequantize(ctx):
    from minml_b200 import backend as B
    q = dev(np.arange(-128, 128, dtype=np.int8))
    out = torch.zeros(256, device="cuda")
    B.dequantize(ctx, q, out, 0.05, -0.3)
    ctx.synchronize()
    assert torch.allclose(out, q.float() * 0.05 - 0.3, atol=1e-6)


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(ctx, oracle):
    """The failure path of the tensor-core kernels, driven without any of them misbehaving: a small kernel waits (bounded) on a
    barrier nothing completes, gives up and writes the context's status word; synchronize reports the sticky error; after that the
    same context computes a correct convolution."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    ctx.synchronize()
    B.lib.mb200_selftest_bounded_wait(ctx.handle, 2000)
    with pytest.raises(B.BackendError, match="gave up on a bounded wait"):
        ctx.synchronize()
    ctx.synchronize()  # the error was reported once and cleared
    r = np.random.default_rng(0)
    x = r.uniform(-1, 1, (2, 9, 9, 64)).astype(np.float16).astype(np.float32)
    wt = (r.standard_normal((64, 3, 3, 64)) * 0.05).astype(np.float16).astype(np.float32)
    conv = L.Conv2D(ctx, wt, None, "relu", torch.float16)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(x.shape))
    y = torch.empty((2, 9, 9, 64), device="cuda", dtype=torch.float16)
    conv.forward([dev(x, torch.float16)], y, ws)
    ctx.synchronize()
    assert max_rel_err(host(y), oracle.conv2d(x, wt, None, None, "relu")) <= 1e-2


def test_empty_tensors_launch_nothing_and_record_no_error(ctx):
    """Zero-sized batches, as the reference's layers may see them for an empty request: every entry point returns without a launch."""
    from minml_b200 import backend as B
    f16 = torch.float16
    before = B.launch_count()
    x = torch.empty((0, 15, 15, 128), device="cuda", dtype=f16)
    y = torch.empty((0, 15, 15, 128), device="cuda", dtype=f16)
    w = torch.zeros((128, 3, 3, 128), device="cuda", dtype=f16)
    bias = torch.zeros(128, device="cuda", dtype=f16)
    B.convolutionImplicitGemmForward(ctx, x, w, y, bias, None, "relu")
    B.addBiasAct(ctx, x, bias, y, "relu")
    B.activationForward(ctx, x, y, "relu")
    B.addTensors(ctx, y, 1.0, x, 1.0, x)
    B.layernormForward(ctx, x, y, bias, bias)
    B.globalAveragePoolingForward(ctx, x, torch.empty((0, 128), device="cuda", dtype=f16))
    B.gemm(ctx, "n", torch.empty((0, 64), device="cuda", dtype=f16), "t", torch.zeros((32, 64), device="cuda", dtype=f16),
           torch.empty((0, 32), device="cuda", dtype=f16))
    B.softmaxForward(ctx, torch.empty((0, 10), device="cuda", dtype=f16), torch.empty((0, 10), device="cuda", dtype=f16))
    B.depthwiseConvForward(ctx, x, torch.zeros((7, 7, 128), device="cuda", dtype=f16), y, bias)
    B.batchnormInference(ctx, x, y, bias, bias, torch.zeros((2, 128), device="cuda"), "relu")
    ctx.synchronize()
    assert B.launch_count() == before


def test_mma_cost_probe(ctx):
    """The probe behind the tile-shape notes: an N = 256 instruction takes the 128 cycles the peak rate implies, and N = 32 is far from
    a quarter of N = 128 (there is a floor), whichever memory A comes from."""
    from minml_b200 import backend as B
    c256 = B.lib.mb200_probe_mma_cycles(ctx.handle, 256, 0)
    c128 = B.lib.mb200_probe_mma_cycles(ctx.handle, 128, 1)
    c32 = B.lib.mb200_probe_mma_cycles(ctx.handle, 32, 1)
    ctx.check()
    assert 115.0 <= c256 <= 145.0 and 57.0 <= c128 <= 75.0 and 30.0 <= c32 <= 64.0, (c256, c128, c32)
    assert B.lib.mb200_probe_mma_cycles(ctx.handle, 48, 0) < 0  # only the five sizes it was built for
    with pytest.raises(B.BackendError):
        ctx.check()  # (reported on the context, and cleared by the report)


def test_kernel_bench_tool_runs_and_reports_every_kernel():
    """The per-kernel timing tool (python kernel_bench.py) at the smallest configuration: one JSON line per kernel,
    finite positive times, fractions of the peaks in range."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "kernel_bench.py"), "--config", "c1", "--reps", "2"], cwd=root, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    probes = [r for r in lines if "probe" in r]  # (the tcgen05.mma cost table: one line, no kernel of the path)
    assert len(probes) == 1 and set(probes[0]["cycles"]) == {"16", "32", "64", "128", "256"}
    records = [r for r in lines if "kernel" in r]
    assert len(records) + len(probes) == len(lines)
    names = [r["kernel"] for r in records]
    assert len(records) >= 30 and len(set(names)) == len(names)
    for needle in ("conv3x3 fused (fp16", "conv3x3 fused (int8", "gemm_batched", "multi_head_attention", "depthwise_conv_forward", "rmsnorm"):
        assert any(needle in n for n in names), needle
    for r in records:
        assert 0.0 < r["ms"] < 100.0 and 0.0 < r["hbm_frac"] < 1.5, r


@pytest.mark.parametrize("cfg", [
    (2, 15, 15, 8, False, None),   # config 4's shape: 225 tokens, one box of 240 keys, two CTAs per SM
    (2, 20, 20, 4, False, None),   # 400 tokens: two boxes of 200 keys, 512 columns of tensor memory, four query tiles
    (3, 5, 6, 2, True, None),      # q = k, 30 tokens: 32 keys, 32 columns
    (1, 16, 16, 3, False, None),   # exactly 256 tokens
    (2, 17, 17, 2, False, None),   # 289 tokens: two boxes of 160
    (2, 9, 7, 4, False, 5),        # a table built for a 5 x 5 board: offsets beyond its range are clamped
    (1, 21, 22, 1, False, None),   # 462 tokens: the most the kernel takes (480 key slots + nothing to spare)
    (1, 1, 1, 2, False, None),     # a single token
    (40, 15, 15, 8, False, None),  # 320 (head, item) pairs: more than one per CTA of the persistent kernel, both of its groups at work
    (170, 5, 6, 2, True, None),    # 340 pairs of one query tile each, q = k
    (37, 12, 13, 5, False, None),  # 185 pairs of 156 tokens (160 keys: a last chunk of 32), ranges of one and two pairs per CTA
    (3, 5, 6, 2, False, 15),       # a table built for a 15 x 15 board on a 5 x 6 one: the kernel copies the window of offsets it can reach
    (2, 15, 15, 8, False, 20),     # the same on the benchmark's board (table of 39 x 39 entries)
])
def test_multi_head_attention_tcgen05_shapes(ctx, oracle, cfg):
    """Head dimension 32 in fp16 -- the shapes that run on the tcgen05 kernel (scores in tensor memory) -- against the oracle, with
    and without the relative-position table, over the token counts at which its tiling changes."""
    from minml_b200 import backend as B
    b, h, w, heads, symmetric, table_board = cfg
    d = 32
    r = np.random.default_rng(h * 100 + w)
    parts = 2 if symmetric else 3
    x = r.standard_normal((b, h, w, parts * heads * d)).astype(np.float16).astype(np.float32)
    n = 2 * (table_board or max(h, w)) - 1
    table = (r.standard_normal((heads, n, (n + 3) // 4 * 4)) * 0.5).astype(np.float16).astype(np.float32)
    try:
        for kernel in (0, 1, 2, 3):  # by shape, tcgen05 wherever possible, tcgen05 with one CTA per pair, never tcgen05
            B.set_attention_kernel(kernel)
            for t in (table, None):
                y = torch.full((b, h, w, heads * d), float("nan"), device="cuda", dtype=torch.float16)
                B.multiHeadAttentionForward(ctx, dev(x, torch.float16), y, None if t is None else dev(t, torch.float16), heads, symmetric)
                ctx.synchronize()
                want = oracle.mha_forward(x, heads, t, symmetric)
                assert max_rel_err(host(y), want) <= FP16_REL, "kernel %d, table %s" % (kernel, t is not None)
    finally:
        B.set_attention_kernel(0)
