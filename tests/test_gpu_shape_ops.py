"""RMS normalisation, space-to-depth and depth-to-space through the C ABI against the oracle
(reference tests: test/backend/test_normalization.cpp:977-1013,1071-1103; test/backend/test_convert.cpp:282-360)."""
import numpy as np
import pytest
import torch

from tests.util import FP16_REL, dev, host, init_for_test, max_rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(123, 43), (57, 256), (4, 15, 15, 128), (33, 1024), (9, 1032), (5, 2048), (3, 4100)])
@pytest.mark.parametrize("with_gamma", [True, False])
def test_rmsnorm_forward(ctx, oracle, dtype, shape, with_gamma):
    from minml_b200 import backend as B
    r = np.random.default_rng(sum(shape))
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == torch.float16 else (lambda a: a.astype(np.float32))
    x = rnd(r.standard_normal(shape) * 2.0)
    gamma = rnd(r.uniform(0.5, 1.5, shape[-1])) if with_gamma else None
    y = torch.full(shape, float("nan"), device="cuda", dtype=dtype)
    B.rmsnormForward(ctx, dev(x, dtype), y, None if gamma is None else dev(gamma, dtype))
    ctx.synchronize()
    want = oracle.rmsnorm(x, gamma)
    if dtype == torch.float32:
        assert np.abs(host(y) - want).max() <= 1e-5  # fp32: sums in a different order only
    else:
        assert max_rel_err(host(y), want) <= FP16_REL


def test_rmsnorm_reference_test_shape(ctx, oracle):
    """test_normalization.cpp:977-1013: 123 x 43, weights = sin fill + 1.1, mean absolute difference <= 1e-4."""
    from minml_b200 import backend as B
    x, gamma = init_for_test((123, 43)), init_for_test((43,)) + 1.1
    y = torch.zeros((123, 43), device="cuda")
    B.rmsnormForward(ctx, dev(x), y, dev(gamma))
    ctx.synchronize()
    assert np.abs(host(y) - oracle.rmsnorm(x, gamma)).mean() <= 1e-4


CASES = [((3, 8, 8, 5), (4, 4)), ((2, 15, 15, 4), (8, 8)), ((2, 13, 14, 3), (5, 7)), ((1, 6, 9, 2), (6, 3)), ((4, 20, 20, 32), (10, 10)),
         ((2, 15, 15, 128), (4, 4))]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int8])
@pytest.mark.parametrize("case", CASES)
def test_space_to_depth_and_back_are_exact(ctx, oracle, dtype, case):
    from minml_b200 import backend as B
    (b, h, w, c), (oh, ow) = case
    r = np.random.default_rng(h * w + c)
    if dtype == torch.int8:
        x = r.integers(-128, 128, (b, h, w, c), dtype=np.int8)
    else:
        x = r.standard_normal((b, h, w, c)).astype(np.float16 if dtype == torch.float16 else np.float32)
    want = oracle.space_to_depth(x, (oh, ow))
    xd = torch.from_numpy(x).cuda()
    deep = torch.full(want.shape, 77, device="cuda", dtype=dtype)  # stale values must be overwritten, zero fill included
    B.spaceToDepth(ctx, xd, deep)
    ctx.synchronize()
    assert np.array_equal(deep.cpu().numpy(), want)
    back = torch.full((b, h, w, c), 77, device="cuda", dtype=dtype)
    B.depthToSpace(ctx, deep, back)
    ctx.synchronize()
    assert np.array_equal(back.cpu().numpy(), x)


def test_unaligned_views_use_narrower_pieces(ctx, oracle):
    """A tensor that starts 2 bytes into an allocation: the 16-byte pieces are not usable and the result must not change."""
    from minml_b200 import backend as B
    x = np.random.default_rng(5).standard_normal((2, 8, 8, 8)).astype(np.float16)
    buf = torch.zeros(x.size + 1, device="cuda", dtype=torch.float16)
    xd = buf[1:].view(2, 8, 8, 8)
    xd.copy_(torch.from_numpy(x))
    deep = torch.zeros((2, 4, 4, 32), device="cuda", dtype=torch.float16)
    B.spaceToDepth(ctx, xd, deep)
    ctx.synchronize()
    assert np.array_equal(deep.cpu().numpy(), oracle.space_to_depth(x, (4, 4)))


def test_shapes_that_do_not_fit_are_refused(ctx):
    from minml_b200 import backend as B
    x = torch.zeros((1, 10, 10, 2), device="cuda")
    with pytest.raises(B.BackendError):
        B.spaceToDepth(ctx, x, torch.zeros((1, 4, 6, 12), device="cuda"))
    with pytest.raises(B.BackendError):
        B.spaceToDepth(ctx, x, torch.zeros((1, 5, 5, 6), device="cuda"))  # 2 x 2 patches of 2 channels are 8, not 6
    ctx.synchronize()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", [(4, 15, 15, 128), (7, 33), (1, 5)])
def test_multiply_tensors(ctx, dtype, shape):
    """cuda_multiply_tensors (the Multiply layer): dst = src1 * src2; one rounding of the exact product in the tensor's type
    (the reference's CPU twin: src/backend/cpu/training.cpp:102-121)."""
    from minml_b200 import backend as B
    r = np.random.default_rng(sum(shape))
    np_dtype = {torch.float32: np.float32, torch.float16: np.float16, torch.float64: np.float64}[dtype]
    a, b = r.standard_normal(shape).astype(np_dtype), r.standard_normal(shape).astype(np_dtype)
    y = torch.full(shape, float("nan"), device="cuda", dtype=dtype)
    B.multiplyTensors(ctx, y, torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    ctx.synchronize()
    want = (a.astype(np.float64) * b.astype(np.float64)).astype(np_dtype)
    assert np.array_equal(y.cpu().numpy(), want)
