"""The benchmark configurations at their FULL sizes.  The oracle is scalar C, so a whole full-size tensor is out of its reach;
what is checked instead holds at any size:

  * positions (batch items) are independent, so the oracle on a handful of SAMPLED items -- first, last, and items that
    straddle tile boundaries of the kernels -- is an exact reference for those items of the full-size launch;
  * permuting the batch permutes the result BIT FOR BIT (every output element sees the same operands in the same order
    wherever its tile lands), which exercises the tile / cluster scheduling over the whole tensor;
  * linearity of the convolution in its input (linear activation), within the fp16 tolerance.

Tolerances: fp16 max |d| / max |ref| <= 1e-2 per layer, int32 accumulators bit-exact; the 41-layer trunk accumulates fp16
rounding layer after layer, its bound (3e-2 at the heads) is stated in the test.
"""
import numpy as np
import pytest
import torch

from tests.util import FP16_REL, host, max_rel_err, oracle_hybrid, oracle_trunk, pack_planes

pytestmark = pytest.mark.gpu


def _sample_items(batch):
    return sorted({0, 1, batch // 3, batch // 2 - 1, batch // 2, batch - 2, batch - 1})


def _perm(batch, seed):
    return torch.from_numpy(np.random.default_rng(seed).permutation(batch)).cuda()


def test_config3_layer_full_size(ctx, oracle):
    """One residual-block layer of config 3: 1024 x 20 x 20 x 256 -> 256, bias + residual + ReLU (fused, CTA pairs)."""
    from minml_b200 import layers as L
    b, h, w, c = 1024, 20, 20, 256
    r = np.random.default_rng(31)
    wt = (r.standard_normal((c, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float16).astype(np.float32)
    bias = (r.standard_normal(c) * 0.01).astype(np.float16).astype(np.float32)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.rand((b, h, w, c), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    res = (torch.rand((b, h, w, c), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    conv = L.Conv2D(ctx, wt, bias, "relu", torch.float16)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(x.shape))
    y = torch.full_like(x, float("nan"))
    conv.forward([x, res], y, ws)
    ctx.synchronize()
    assert bool(torch.isfinite(y).all())
    items = _sample_items(b)
    want = oracle.conv2d(host(x[items]), wt, bias, host(res[items]), "relu")
    assert max_rel_err(host(y[items]), want) <= FP16_REL
    # batch permutation: bit-exact
    perm = _perm(b, 1)
    xp, rp = x[perm].contiguous(), res[perm].contiguous()
    yp = torch.empty_like(y)
    conv.forward([xp, rp], yp, ws)
    ctx.synchronize()
    assert torch.equal(yp, y[perm])
    # linearity (no bias, no residual, linear activation): conv(x + x2) = conv(x) + conv(x2) up to fp16 rounding of the three results
    lin = L.Conv2D(ctx, wt, None, "linear", torch.float16)
    x2 = (torch.rand((b, h, w, c), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    xs = (x.float() + x2.float()).to(torch.float16)
    y1, y2, y12 = torch.empty_like(y), torch.empty_like(y), torch.empty_like(y)
    lin.forward([x], y1, ws)
    lin.forward([x2], y2, ws)
    lin.forward([xs], y12, ws)
    ctx.synchronize()
    # what separates the two sides: the fp16 rounding of xs (2^-11 relative per element) and of the three outputs
    err = (y12.float() - y1.float() - y2.float()).abs().max().item()
    assert err / y12.float().abs().max().item() <= FP16_REL


def test_config2_int8_layer_full_size(ctx, oracle):
    """One layer of config 2: 512 x 20 x 20 x 128 -> 128 int8; identity requantisation to fp32 exposes the int32 accumulators."""
    from minml_b200 import layers as L
    b, h, w, c = 512, 20, 20, 128
    r = np.random.default_rng(32)
    q = r.integers(-127, 128, (c, 3, 3, c), dtype=np.int8)
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randint(-128, 128, (b, h, w, c), device="cuda", dtype=torch.int8, generator=g)
    ones, zeros = np.ones(c, np.float32), np.zeros(c, np.float32)
    conv = L.QuantizedConv2D(ctx, q, ones, zeros, (1.0, 0.0), (1.0, 0.0), "linear", torch.float32)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(x.shape))
    y = torch.zeros((b, h, w, c), device="cuda", dtype=torch.float32)
    conv.forward([x], y, ws)
    ctx.synchronize()
    items = _sample_items(b)
    _, _, acc = oracle.conv2d_int8(host(x[items]), q, ones, zeros, 0)
    assert np.max(np.abs(acc)) < 2 ** 24  # exactly representable in fp32
    assert np.array_equal(host(y[items]).astype(np.int64), acc.astype(np.int64))
    perm = _perm(b, 2)
    yp = torch.zeros_like(y)
    conv.forward([x[perm].contiguous()], yp, ws)
    ctx.synchronize()
    assert torch.equal(yp, y[perm])
    # the int8 -> int8 epilogue with residual and ReLU at full size, against the oracle on the sampled items
    scales = (r.uniform(0.5, 1.5, c) * 2e-4).astype(np.float32)
    shifts = (r.standard_normal(c) * 0.05).astype(np.float32)
    ext = torch.randint(-128, 128, (b, h, w, c), device="cuda", dtype=torch.int8, generator=g)
    qconv = L.QuantizedConv2D(ctx, q, scales, shifts, (1.0, 0.0), (0.02, 0.0), "relu", torch.int8)
    y8 = torch.zeros((b, h, w, c), device="cuda", dtype=torch.int8)
    qconv.forward([x, ext], y8, ws, (0.01, 0.0))
    ctx.synchronize()
    want8, _, _ = oracle.conv2d_int8(host(x[items]), q, scales, shifts, 0, (0.02, 0.0), "relu", host(ext[items]), (0.01, 0.0))
    diff = np.abs(host(y8[items]).astype(np.int32) - want8.astype(np.int32))
    assert diff.max() <= 1
    assert (diff != 0).mean() < 1e-3  # ties of the rounding only


def test_config3_trunk_full_size(ctx, oracle):
    """The whole config-3 trunk (20 blocks x 256 channels, batch 1024): batch permutation bit-exact at the heads, and two sampled
    positions against the fp32 oracle trunk.  41 fp16 layers accumulate rounding: bound 3e-2 at the heads."""
    from minml_b200 import layers as L
    b, h, w, planes, channels, blocks = 1024, 20, 20, 32, 256, 20
    weights = L.make_trunk_weights(1237, planes, channels, blocks)
    weights16 = {k: v.astype(np.float16).astype(np.float32) for k, v in weights.items()}
    x = (np.random.default_rng(8).random((b, h, w, planes)) < 0.3).astype(np.float32)
    net = L.ResNetTrunk(ctx, weights, b, h, w, planes, channels, blocks)
    packed = torch.from_numpy(pack_planes(x).view(np.int32)).cuda()
    policy, value = net.predict(packed)
    ctx.synchronize()
    policy, value = policy.clone(), value.clone()
    assert bool(torch.isfinite(policy).all()) and bool(torch.isfinite(value).all())
    perm = _perm(b, 3)
    policy_p, value_p = net.predict(packed[perm].contiguous())
    ctx.synchronize()
    assert torch.equal(policy_p, policy[perm]) and torch.equal(value_p, value[perm])
    items = [0, b - 1]
    want_p, want_v = oracle_trunk(oracle, weights16, x[items], blocks)
    assert max_rel_err(host(policy[items]), want_p) <= 3e-2
    assert max_rel_err(host(value[items]), want_v) <= 3e-2


def test_config4_block_full_size(ctx, oracle):
    """The conv + attention block of config 4 at batch 256: permutation bit-exact, sampled items against the fp32 oracle."""
    from minml_b200 import layers as L
    b, h, w, embed, heads, ffn = 256, 15, 15, 256, 8, 1024
    weights = L.make_hybrid_weights(1237, embed, heads, ffn, max(h, w))
    weights16 = {k: v.astype(np.float16).astype(np.float32) for k, v in weights.items()}
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((b, h, w, embed), device="cuda", generator=g).to(torch.float16)
    block = L.HybridBlock(ctx, weights, b, h, w, embed, heads, ffn)
    out = block.predict(x)
    ctx.synchronize()
    out = out.clone()
    assert bool(torch.isfinite(out).all())
    perm = _perm(b, 4)
    xp = x[perm].contiguous()
    out_p = block.predict(xp)
    ctx.synchronize()
    assert torch.equal(out_p, out[perm])
    items = [0, b // 2, b - 1]
    want = oracle_hybrid(oracle, weights16, host(x[items]), heads)
    assert max_rel_err(host(out[items]), want) <= FP16_REL


def test_winograd_gemm_full_size(ctx, oracle):
    """The 36 batched products of the three-kernel path at config-3 size ([36, 25600, 256] x [36, 256, 256]^T): sampled rows of
    sampled matrices against the oracle (rows of a product are independent)."""
    from minml_b200 import backend as B
    tiles, c = 1024 * 25, 256
    g = torch.Generator(device="cuda").manual_seed(10)
    v = (torch.rand((36, tiles, c), device="cuda", generator=g) - 0.5).to(torch.float16)
    u = (torch.rand((36, c, c), device="cuda", generator=g) - 0.5).to(torch.float16)
    m = torch.full((36, tiles, c), float("nan"), device="cuda", dtype=torch.float16)
    ctx.set_fusion(False)
    B.gemmBatched(ctx, "n", v, "t", u, m)
    ctx.synchronize()
    ctx.set_fusion(True)
    assert bool(torch.isfinite(m).all())
    rows = np.unique(np.concatenate([np.arange(0, 130), np.arange(tiles - 130, tiles), np.random.default_rng(1).integers(0, tiles, 64)]))
    for mat in (0, 17, 35):
        want = oracle.gemm("n", host(v[mat][rows]), "t", host(u[mat]))
        assert max_rel_err(host(m[mat][rows]), want) <= FP16_REL
