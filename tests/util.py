"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

from minml_b200.synthetic import pack_planes  # noqa: F401  (the tests import it from here)
from tests.util_cpu import (forward_loaded_network_on_cpu, load_int8_conv_cases, oracle_hybrid, oracle_quantized_trunk,  # noqa: F401
                            oracle_trunk)


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
