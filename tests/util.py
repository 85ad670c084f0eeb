"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype).contiguous() if dtype is not None else t.contiguous()


def host(t):
    return t.detach().float().cpu().numpy() if t.dtype in (torch.float16, torch.float32, torch.float64) else t.detach().cpu().numpy()


def init_for_test(shape, shift=0.0, scale=1.0):
    n = int(np.prod(shape))
    return (np.sin(np.arange(n, dtype=np.float32) / 10.0 + shift) * scale).astype(np.float32).reshape(shape)


def mean_abs_diff(a, b):
    return float(np.mean(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))))


def max_rel_err(got, want):
    """max |got - want| / max |want|: the relative error measure of the parity bar (1e-2 for fp16, 2e-2 for dequantised int8)."""
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - want)) / max(np.max(np.abs(want)), 1e-30))


# tolerances of the parity bar
FP32_TOL = 1e-4   # mean absolute difference, as the reference's fp32 tests use
FP16_REL = 1e-2
INT8_REL = 2e-2


def oracle_trunk(oracle, weights, x, blocks):
    """fp32 forward of the ResNet trunk topology with the oracle's direct convolution: (policy [b,h,w,1], value [b,3])."""
    a = oracle.conv2d(x, weights["stem_w"], weights["stem_b"], None, "relu")
    for i in range(blocks):
        t = oracle.conv2d(a, weights["b%d_w1" % i], weights["b%d_b1" % i], None, "relu")
        a = oracle.conv2d(t, weights["b%d_w2" % i], weights["b%d_b2" % i], a, "relu")
    policy = oracle.conv2d(a, weights["policy_w"], weights["policy_b"], None, "linear")
    pooled = oracle.global_average_pooling(a)
    value = oracle.add_bias_act(oracle.gemm("n", pooled, "t", weights["value_w"]), weights["value_b"], "linear")
    return policy, value


def pack_planes(x01):
    """[..., c] array of {0, 1} -> uint32 words [..., ceil(c / 32)], channel j in bit j % 32 of word j // 32."""
    c = x01.shape[-1]
    words = (c + 31) // 32
    out = np.zeros(x01.shape[:-1] + (words,), np.uint32)
    for j in range(c):
        out[..., j // 32] |= (x01[..., j].astype(np.uint32) & 1) << np.uint32(j % 32)
    return out
