"""mb200_convolution_forward_noalloc -- the convolution entry point for hosts that may not allocate device memory.

Some users of this library run it inside a process that has already handed all GPU memory to its own arena, or inside a
serving loop where the device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.  For them the library keeps
the Winograd scratch (transformed weights, transformed input, products) in a fixed 16 MiB array of its own image.  This
test drives that entry point through the C ABI, twice in a row on changing inputs, and checks every result against
cuda_convolution_implicit_gemm_forward, the allocating entry point that computes the same convolution, and against the
CPU oracle's direct convolution; it also checks that free device memory does not shrink across the calls and that a
problem too large for the array is refused.

The file sorts last on purpose: a `pytest -x` run reaches it only after every other test has run.
"""
import ctypes

import numpy as np
import pytest
import torch

from tests.util import dev, host, max_rel_err

pytestmark = pytest.mark.gpu


def _call(B, ctx, fn, x, w, y, bias, add, act):
    fn(ctx.handle, B.dtype_of(x), B.shape_of(x), B.shape_of(w), B.ptr(x), B.ptr(w), B.ptr(y), B.ptr(bias), B.ptr(add), B.act_code(act))
    ctx.check()


# fp32: the allocating entry point runs small layers like this one as the fused split-TF32 kernel, the no-allocation one as F(4x4,3x3)
# Winograd; both are fp32-accurate and differ by rounding (a few 1e-6 of the largest value).  fp16: the Winograd path's bound.
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float16, 2.5e-2)])
def test_noalloc_matches_allocating_entry_point(ctx, oracle, dtype, tol):
    from minml_b200 import backend as B
    noalloc = B.lib.mb200_convolution_forward_noalloc
    reference_entry = B.lib.cuda_convolution_implicit_gemm_forward
    b, h, w_, cin, cout = 3, 15, 15, 64, 48
    rng = np.random.default_rng(2024)
    wt = dev((rng.standard_normal((cout, 3, 3, cin)) * np.sqrt(2.0 / (9 * cin))).astype(np.float32), dtype)
    bias = dev((rng.standard_normal(cout) * 0.01).astype(np.float32), dtype)
    # warm both paths up once so that one-time work (workspace growth of the allocating path, symbol lookup) is behind us
    x0 = dev(rng.uniform(-1, 1, (b, h, w_, cin)).astype(np.float32), dtype)
    y0 = torch.empty((b, h, w_, cout), device="cuda", dtype=dtype)
    _call(B, ctx, reference_entry, x0, wt, y0, bias, None, "relu")
    _call(B, ctx, noalloc, x0, wt, y0, bias, None, "relu")
    ctx.synchronize()
    # every tensor of both rounds exists before the free-memory reading, so torch's own allocator is quiet in between
    rounds = []
    for round_index in range(2):
        rounds.append(dict(
            x=dev(rng.uniform(-1, 1, (b, h, w_, cin)).astype(np.float32), dtype),
            add=dev(rng.uniform(-1, 1, (b, h, w_, cout)).astype(np.float32), dtype),
            want=torch.full((b, h, w_, cout), float("nan"), device="cuda", dtype=dtype),
            got=torch.full((b, h, w_, cout), float("nan"), device="cuda", dtype=dtype),
            act="relu" if round_index == 0 else "linear"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for r in rounds:  # two calls in a row: the array still holds the previous call's U, V and M
        _call(B, ctx, noalloc, r["x"], wt, r["got"], bias, r["add"], r["act"])
    ctx.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    # (another process may release memory on a shared GPU meanwhile; what must not happen is that these calls take any)
    assert free_after >= free_before, "device memory was allocated during the no-alloc calls"
    for index, r in enumerate(rounds):
        _call(B, ctx, reference_entry, r["x"], wt, r["want"], bias, r["add"], r["act"])
        ctx.synchronize()
        assert not torch.isnan(r["got"]).any()
        assert max_rel_err(host(r["got"]), host(r["want"])) <= tol, "call %d" % index
        # and against the oracle's direct convolution on the same (rounded) operands: fp32 by the reference's own measure (mean
        # absolute difference <= 1e-4), fp16 within the bound of the Winograd path with fp16 intermediates
        direct = oracle.conv2d(host(r["x"]), host(wt), host(bias), host(r["add"]), r["act"])
        if dtype == torch.float32:
            assert float(np.mean(np.abs(host(r["got"]) - direct))) <= 1e-4, "call %d against the oracle" % index
        else:
            assert max_rel_err(host(r["got"]), direct) <= 2.5e-2, "call %d against the oracle" % index


def test_noalloc_refuses_what_does_not_fit(ctx):
    from minml_b200 import backend as B
    noalloc = B.lib.mb200_convolution_forward_noalloc
    # 36 * 4 bytes * (256*256 + 2*tiles*256) with tiles = 64 * 25 = 1600 is far beyond 16 MiB
    x = torch.zeros((64, 20, 20, 256), device="cuda")
    w = torch.zeros((256, 3, 3, 256), device="cuda")
    y = torch.full((64, 20, 20, 256), 7.0, device="cuda")
    with pytest.raises(B.BackendError, match="scratch"):
        _call(B, ctx, noalloc, x, w, y, None, None, "linear")
    ctx.synchronize()
    assert torch.all(y == 7.0)  # nothing was launched
