"""Batch norm at inference time, depthwise convolution (fp and int8) and channel scaling against the oracle
(reference tests: test/backend/test_batchnorm.cpp, test/backend/test_depthwise_conv.cpp, test/backend/test_global_pooling.cpp)."""
import os

import numpy as np
import pytest
import torch

from tests.util import FP16_REL, dev, host, max_rel_err

pytestmark = pytest.mark.gpu


def _tol(dtype, got, want):
    if dtype == torch.float32:
        return np.max(np.abs(got - want)) <= 2e-5 * max(1.0, np.max(np.abs(want)))
    return max_rel_err(got, want) <= FP16_REL


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(4, 15, 15, 128), (3, 7, 5, 36), (5, 33)])
def test_batchnorm_inference(ctx, oracle, dtype, shape):
    from minml_b200 import backend as B
    r = np.random.default_rng(sum(shape))
    c = shape[-1]
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == torch.float16 else (lambda a: a.astype(np.float32))
    x, y0 = rnd(r.standard_normal(shape)), rnd(r.standard_normal(shape))
    gamma, beta_bn = rnd(r.uniform(0.5, 1.5, c)), rnd(r.standard_normal(c))
    avg_var = np.stack([r.standard_normal(c), r.uniform(0.2, 2.0, c)]).astype(np.float32)
    for act, alpha, beta, with_params in (("relu", 1.0, 0.0, True), ("linear", 1.0, 0.0, False), ("sigmoid", 0.5, 0.25, True), ("leaky_relu", 1.0, 0.0, True)):
        y = dev(y0, dtype)
        B.batchnormInference(ctx, dev(x, dtype), y, dev(gamma, dtype) if with_params else None, dev(beta_bn, dtype) if with_params else None,
                             dev(avg_var), act, alpha, beta)
        ctx.synchronize()
        want = oracle.batchnorm_inference(x, gamma if with_params else None, beta_bn if with_params else None, avg_var, act, alpha, beta, y0)
        assert _tol(dtype, host(y), want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(64, 3, 3, 32), (128, 1, 1, 64), (40, 24), (7, 7, 96), (3, 3, 20)])
def test_fold_batchnorm(ctx, oracle, dtype, shape):
    from minml_b200 import backend as B
    r = np.random.default_rng(sum(shape))
    c = shape[-1] if len(shape) == 3 else shape[0]
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == torch.float16 else (lambda a: a.astype(np.float32))
    w, b = rnd(r.standard_normal(shape)), rnd(r.standard_normal(c))
    gamma, beta_bn = rnd(r.uniform(0.5, 1.5, c)), rnd(r.standard_normal(c))
    avg_var = np.stack([r.standard_normal(c), r.uniform(0.2, 2.0, c)]).astype(np.float32)
    wd, bd = dev(w, dtype), dev(b, dtype)
    B.foldBatchnorm(ctx, wd, bd, dev(gamma, dtype), dev(beta_bn, dtype), dev(avg_var))
    ctx.synchronize()
    want_w, want_b = oracle.fold_batchnorm(w, b, gamma, beta_bn, avg_var)
    assert _tol(dtype, host(wd), want_w) and _tol(dtype, host(bd), want_b)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("k", [3, 5, 7])
@pytest.mark.parametrize("shape", [(3, 15, 15, 128), (2, 20, 20, 64), (2, 5, 3, 20), (1, 9, 11, 7)])
def test_depthwise_conv(ctx, oracle, dtype, k, shape):
    from minml_b200 import backend as B
    r = np.random.default_rng(sum(shape) + k)
    c = shape[-1]
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == torch.float16 else (lambda a: a.astype(np.float32))
    x, y0 = rnd(r.standard_normal(shape)), rnd(r.standard_normal(shape))
    w, bias = rnd(r.standard_normal((k, k, c)) * 0.2), rnd(r.standard_normal(c))
    for alpha, beta, with_bias in ((1.0, 0.0, True), (1.0, 1.0, True), (0.5, 0.0, False)):
        y = dev(y0, dtype)
        B.depthwiseConvForward(ctx, dev(x, dtype), dev(w, dtype), y, dev(bias, dtype) if with_bias else None, alpha, beta)
        ctx.synchronize()
        want = oracle.depthwise_conv(x, w, bias if with_bias else None, alpha, beta, y0)
        assert _tol(dtype, host(y), want)


@pytest.mark.parametrize("k", [3, 5, 7])
@pytest.mark.parametrize("shape", [(3, 15, 15, 128), (2, 6, 7, 24), (1, 20, 20, 200)])
def test_quantized_depthwise_conv(ctx, oracle, k, shape):
    """int8 outputs equal the oracle's (the arithmetic is integer up to one fp32 multiply-add pair written without FMA)."""
    from minml_b200 import backend as B
    r = np.random.default_rng(sum(shape) + k)
    c = shape[-1]
    x = r.integers(-128, 128, shape, dtype=np.int8)
    w = r.integers(-127, 128, (k, k, c), dtype=np.int8)
    scales = r.uniform(1e-4, 3e-4, c).astype(np.float32)
    bias = (r.standard_normal(c) * 0.1).astype(np.float32)
    for out_qd, zero in (((0.01, 0.0), 0), ((0.012, 0.07), -5)):
        y = torch.zeros(shape, dtype=torch.int8, device="cuda")
        B.quantized_depthwise_conv_forward(ctx, dev(x), dev(w), dev(scales), dev(bias), y, out_qd, zero)
        ctx.synchronize()
        want8, _ = oracle.depthwise_conv_int8(x, w, scales, bias, out_qd, zero)
        assert np.array_equal(host(y), want8)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(4, 15, 15, 128), (3, 5, 7, 20), (2, 9, 33)])
def test_channel_scaling(ctx, oracle, dtype, shape):
    from minml_b200 import backend as B
    r = np.random.default_rng(sum(shape))
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == torch.float16 else (lambda a: a.astype(np.float32))
    x, y0 = rnd(r.standard_normal(shape)), rnd(r.standard_normal(shape))
    s = rnd(r.uniform(0, 1, (shape[0], shape[-1])))
    for alpha, beta in ((1.0, 0.0), (0.5, 0.5)):
        y = dev(y0, dtype)
        B.channelScalingForward(ctx, dev(x, dtype), dev(s, dtype), y, alpha, beta)
        ctx.synchronize()
        assert _tol(dtype, host(y), oracle.channel_scaling(x, s, alpha, beta, y0))


def test_squeeze_and_excitation_block(ctx, oracle):
    """GlobalAveragePooling -> Dense (ReLU) -> Dense (sigmoid) -> ChannelScaling, the SE block of minml's current architectures,
    after a depthwise 7x7 convolution with folded batch norm."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    r = np.random.default_rng(3)
    b, h, w, c, red = 8, 15, 15, 128, 32
    h16 = lambda a: a.astype(np.float16).astype(np.float32)
    x = h16(r.standard_normal((b, h, w, c)))
    wd, bd = h16(r.standard_normal((7, 7, c)) * 0.1), h16(r.standard_normal(c) * 0.1)
    gamma, beta_bn = h16(r.uniform(0.5, 1.5, c)), h16(r.standard_normal(c) * 0.1)
    avg_var = np.stack([r.standard_normal(c) * 0.1, r.uniform(0.5, 1.5, c)]).astype(np.float32)
    w1, b1 = h16(r.standard_normal((red, c)) * 0.1), h16(r.standard_normal(red) * 0.1)
    w2, b2 = h16(r.standard_normal((c, red)) * 0.1), h16(r.standard_normal(c) * 0.1)
    f16 = torch.float16
    wdd, bdd = dev(wd, f16), dev(bd, f16)
    B.foldBatchnorm(ctx, wdd, bdd, dev(gamma, f16), dev(beta_bn, f16), dev(avg_var))
    t = torch.empty((b, h, w, c), device="cuda", dtype=f16)
    B.depthwiseConvForward(ctx, dev(x, f16), wdd, t, bdd)
    pooled = torch.empty((b, c), device="cuda", dtype=f16)
    L.GlobalAveragePooling(ctx).forward([t], pooled)
    hid, gate = torch.empty((b, red), device="cuda", dtype=f16), torch.empty((b, c), device="cuda", dtype=f16)
    L.Dense(ctx, w1, b1, "relu", f16).forward([pooled], hid)
    L.Dense(ctx, w2, b2, "sigmoid", f16).forward([hid], gate)
    y = torch.empty_like(t)
    B.channelScalingForward(ctx, t, gate, y)
    ctx.synchronize()
    t_ref = oracle.batchnorm_inference(oracle.depthwise_conv(x, wd, bd), gamma, beta_bn, avg_var)
    p_ref = oracle.global_average_pooling(t_ref)
    hid_ref = oracle.add_bias_act(oracle.gemm("n", p_ref, "t", w1), b1, "relu")
    gate_ref = oracle.add_bias_act(oracle.gemm("n", hid_ref, "t", w2), b2, "sigmoid")
    assert max_rel_err(host(y), oracle.channel_scaling(t_ref, gate_ref)) <= FP16_REL


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_fused_conv_block_call_sequence(ctx, oracle, dtype):
    """FusedConvBlock::forward on a CUDA device (src/layers/FusedConvBlock.cpp:192-213): depthwise 7x7 convolution with bias,
    1x1 convolution + ReLU into the workspace, 1x1 convolution back with the block's input as the residual -- three ABI
    calls, the last two each one fused tensor-core kernel."""
    from minml_b200 import backend as B
    r = np.random.default_rng(11)
    b, h, w, c = 4, 15, 15, 128
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == torch.float16 else (lambda a: a.astype(np.float32))
    x = rnd(r.standard_normal((b, h, w, c)))
    wd, bd = rnd(r.standard_normal((7, 7, c)) * 0.1), rnd(r.standard_normal(c) * 0.1)
    w1, b1 = rnd(r.standard_normal((c, c)) * 0.1), rnd(r.standard_normal(c) * 0.1)
    w2, b2 = rnd(r.standard_normal((c, c)) * 0.1), rnd(r.standard_normal(c) * 0.1)
    xd = dev(x, dtype)
    out = torch.empty((b, h, w, c), device="cuda", dtype=dtype)
    tmp = torch.empty((b * h * w, c), device="cuda", dtype=dtype)
    B.depthwiseConvForward(ctx, xd, dev(wd, dtype), out, dev(bd, dtype))
    before = B.launch_count()
    B.gemm_ex(ctx, tmp, 1.0, "n", out.view(b * h * w, c), "t", dev(w1, dtype), 0.0, tmp, dev(b1, dtype), "relu")
    B.gemm_ex(ctx, out.view(b * h * w, c), 1.0, "n", tmp, "t", dev(w2, dtype), 1.0, xd.view(b * h * w, c), dev(b2, dtype), "linear")
    ctx.synchronize()
    if not (dtype == torch.float32 and os.environ.get("MINML_B200_FP32_SIMT", "0")[:1] == "1"):  # (the plain fp32 engine adds bias and activation in kernels of their own)
        assert B.launch_count() - before == 2
    t = oracle.depthwise_conv(x, wd, bd).reshape(b * h * w, c)
    t = oracle.add_bias_act(oracle.gemm("n", t, "t", w1), b1, "relu")
    want = oracle.add_bias_act(oracle.gemm("n", t, "t", w2) + x.reshape(b * h * w, c), b2, "linear").reshape(b, h, w, c)
    assert _tol(dtype, host(out), want)
