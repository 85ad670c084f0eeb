"""The backward-pass Winograd transforms and the fused activation / bias-gradient step against the oracle, and the whole
Conv2D::backward sequence (src/layers/Conv2D.cpp:383-448) against the direct formulas for dx and dw
(reference tests: test/backend/test_winograd.cpp cudaGradientTransform / cudaUpdateTransform, test/backend/test_conv2D.cpp:630-733)."""
import numpy as np
import pytest
import torch

from tests.util import FP16_REL, dev, host, max_rel_err

pytestmark = pytest.mark.gpu


def _rnd(dtype):
    return (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == torch.float16 else (lambda a: a.astype(np.float32))


def _ok(dtype, got, want):
    if dtype == torch.float32:
        return np.max(np.abs(got - want)) <= 2e-5 * max(1.0, np.max(np.abs(want)))
    return max_rel_err(got, want) <= FP16_REL


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("tile,k", [(4, 3), (2, 3), (2, 5)])
@pytest.mark.parametrize("shape", [(3, 9, 11, 35), (2, 15, 15, 128), (1, 4, 4, 8)])
def test_gradient_transform(ctx, oracle, dtype, tile, k, shape):
    from minml_b200 import backend as B
    b, h, w, c = shape
    dy = _rnd(dtype)(np.random.default_rng(sum(shape)).standard_normal(shape))
    p = tile + k - 1
    tiles = b * ((h + tile - 1) // tile) * ((w + tile - 1) // tile)
    m = torch.full((p * p, tiles, c), float("nan"), device="cuda", dtype=dtype)
    B.winogradGradientTransform(ctx, (c, k, k, 1), dev(dy, dtype), m, tile)
    ctx.synchronize()
    assert _ok(dtype, host(m), oracle.winograd_gradient_transform(dy, tile, k))


@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32), (torch.float16, torch.float16), (torch.float16, torch.float32)])
@pytest.mark.parametrize("tile,k", [(4, 3), (2, 3), (2, 5)])
@pytest.mark.parametrize("cout,cin", [(21, 35), (128, 128)])
def test_update_transform(ctx, oracle, dtypes, tile, k, cout, cin):
    from minml_b200 import backend as B
    p = tile + k - 1
    m = _rnd(dtypes[0])(np.random.default_rng(cout + cin).standard_normal((p * p, cout, cin)))
    dw = torch.full((cout, k, k, cin), float("nan"), device="cuda", dtype=dtypes[1])
    B.winogradUpdateTransform(ctx, dev(m, dtypes[0]), dw, tile)
    ctx.synchronize()
    assert _ok(dtypes[1], host(dw), oracle.winograd_update_transform(m, tile, k))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(4, 15, 15, 128), (3, 5, 7, 20), (33, 10)])
@pytest.mark.parametrize("act", ["linear", "relu", "sigmoid", "tanh", "leaky_relu"])
def test_fused_act_bias_copy_backward(ctx, oracle, dtype, shape, act):
    from minml_b200 import backend as B
    r = np.random.default_rng(sum(shape))
    rnd = _rnd(dtype)
    dy, y = rnd(r.standard_normal(shape)), rnd(r.uniform(-1, 1, shape))
    dx0, db0 = rnd(r.standard_normal(shape)), rnd(r.standard_normal(shape[-1]))
    for beta_dx, beta_db, with_dx in ((0.0, 0.0, True), (0.5, 1.0, True), (0.0, 0.25, False)):
        dyd, dxd, dbd = dev(dy, dtype), dev(dx0, dtype) if with_dx else None, dev(db0, dtype)
        B.fusedBiasActCopyBackward(ctx, dyd, dev(y, dtype), dxd, dbd, act, beta_dx, beta_db)
        ctx.synchronize()
        want_dy, want_dx, want_db = oracle.act_bias_copy_backward(dy, y, dx0, db0, beta_dx, beta_db, act, with_dx=with_dx)
        assert _ok(dtype, host(dyd), want_dy)
        if with_dx:
            assert _ok(dtype, host(dxd), want_dx)
        # column sums over many rows: fp16 adds one rounding per block and channel
        assert max_rel_err(host(dbd), want_db) <= (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("tile", [4, 2])
def test_conv2d_backward_sequence_fp32(ctx, oracle, tile):
    """dx = conv(dy, flipped w^T) and dw = correlation(x, dy), computed the way Conv2D::backward does: gradient transform, batched
    'n','n' product with the transformed (non-inverted: the host inverts) weights, output transform; and input transform, batched
    't','n' product, update transform."""
    from minml_b200 import backend as B
    r = np.random.default_rng(7)
    b, h, w, cin, cout, k = 2, 8, 8, 12, 20, 3
    p = tile + k - 1
    x = r.standard_normal((b, h, w, cin)).astype(np.float32)
    wt = (r.standard_normal((cout, k, k, cin)) * 0.2).astype(np.float32)
    dy = r.standard_normal((b, h, w, cout)).astype(np.float32)
    tiles = b * ((h + tile - 1) // tile) * ((w + tile - 1) // tile)
    f32 = torch.float32
    ctx.set_fusion(False)
    # ---- dw
    v = torch.empty((p * p, tiles, cin), device="cuda", dtype=f32)
    g = torch.empty((p * p, tiles, cout), device="cuda", dtype=f32)
    m = torch.empty((p * p, cout, cin), device="cuda", dtype=f32)
    dw = torch.empty((cout, k, k, cin), device="cuda", dtype=f32)
    B.winogradInputTransform(ctx, wt.shape, dev(x), v, tile)
    B.winogradGradientTransform(ctx, wt.shape, dev(dy), g, tile)
    B.gemmBatched(ctx, "t", g, "n", v, m)
    B.winogradUpdateTransform(ctx, m, dw, tile)
    ctx.synchronize()
    xp = np.pad(x, ((0, 0), (1, 1), (1, 1), (0, 0)))
    want_dw = np.zeros_like(wt)
    for i in range(k):
        for j in range(k):
            want_dw[:, i, j, :] = np.einsum("bhwo,bhwc->oc", dy, xp[:, i:i + h, j:j + w, :])
    assert np.max(np.abs(host(dw) - want_dw)) <= 1e-3 * np.max(np.abs(want_dw))
    # ---- dx: the convolution of dy with the spatially flipped weights, input and output channels exchanged
    u_inv = torch.empty((p * p, cout, cin), device="cuda", dtype=f32)
    B.winogradWeightTransform(ctx, dev(wt), u_inv, True, tile)
    gd = torch.empty((p * p, tiles, cout), device="cuda", dtype=f32)
    md = torch.empty((p * p, tiles, cin), device="cuda", dtype=f32)
    dx = torch.empty((b, h, w, cin), device="cuda", dtype=f32)
    B.winogradInputTransform(ctx, wt.shape, dev(dy), gd, tile)
    B.gemmBatched(ctx, "n", gd, "n", u_inv, md)
    B.winogradOutputTransform(ctx, wt.shape, md, dx, None, None, "linear", tile)
    ctx.synchronize()
    ctx.set_fusion(True)
    w_back = np.ascontiguousarray(np.flip(wt, (1, 2)).transpose(3, 1, 2, 0))  # [cin, k, k, cout]
    want_dx = oracle.conv2d(dy, w_back, None, None, "linear")
    assert np.max(np.abs(host(dx) - want_dx)) <= 1e-3 * np.max(np.abs(want_dx))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("act", ["linear", "relu", "sigmoid", "tanh", "leaky_relu"])
def test_activation_backward(ctx, oracle, dtype, act):
    from minml_b200 import backend as B
    r = np.random.default_rng(3)
    rnd = _rnd(dtype)
    shape = (3, 7, 5, 36)
    dy, y, dx0 = rnd(r.standard_normal(shape)), rnd(r.uniform(-1, 1, shape)), rnd(r.standard_normal(shape))
    for alpha, beta in ((1.0, 0.0), (0.5, 0.25)):
        dx = dev(dx0, dtype)
        B.activationBackward(ctx, dev(dy, dtype), dev(y, dtype), dx, act, alpha, beta)
        ctx.synchronize()
        scaled, _, _ = oracle.act_bias_copy_backward(dy, y, act=act, with_dx=False, with_db=False)
        assert _ok(dtype, host(dx), alpha * scaled + beta * dx0)
