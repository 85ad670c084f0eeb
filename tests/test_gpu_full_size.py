"""The benchmark configurations at their FULL sizes.  The oracle is scalar C, so a whole full-size tensor is out of its reach;
what is checked instead holds at any size:

  * positions (batch items) are independent, so the oracle on a handful of SAMPLED items -- first, last, and items that
    straddle tile boundaries of the kernels -- is an exact reference for those items of the full-size launch;
  * permuting the batch permutes the result BIT FOR BIT (every output element sees the same operands in the same order
    wherever its tile lands), which exercises the tile / cluster scheduling over the whole tensor;
  * linearity of the convolution in its input (linear activation), within the fp16 tolerance.

Tolerances: fp32 mean |d| <= 1e-4 (the reference's own metric and threshold); fp16 max |d| / max |ref| <= 1e-2 per layer and
for the whole trunks of configs 1 (21 layers) and 3 (41 layers); int32 accumulators bit-exact.  The trunk tests print the
measured errors (run with -s); for config 3 also against an oracle chain that stores every activation in fp16 like the
device does, which attributes the error to the storage format.
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


def test_config0_layer_full_size(ctx, oracle, refcpu):
    """Benchmark configuration 0 at its stated size: fp32, batch 64, 15x15, 128 -> 128, y = ReLU(conv + bias), through the
    reference's own call triple and through the single-call entry; against the oracle on every item (it is small enough) and
    against minml's CPU backend (its F(4x4,3x3) Winograd path), mean absolute difference <= 1e-4, the threshold of the
    reference's own test of this path (test/backend/test_conv2D.cpp:580-629)."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    b, h, w, c = 64, 15, 15, 128
    r = np.random.default_rng(1234)
    x = r.uniform(-1, 1, (b, h, w, c)).astype(np.float32)
    wt = (r.standard_normal((c, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float32)
    bias = (r.standard_normal(c) * 0.01).astype(np.float32)
    want = oracle.conv2d(x, wt, bias, None, "relu")
    assert np.mean(np.abs(want - refcpu.conv3x3_winograd(x, wt, bias, None, "relu", 4))) <= 1e-4  # oracle and reference agree here
    conv = L.Conv2D(ctx, wt, bias, "relu", torch.float32)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(x.shape))
    xd = torch.from_numpy(x).cuda()
    for fusion in (True, False):
        ctx.set_fusion(fusion)
        y = torch.full((b, h, w, c), float("nan"), device="cuda")
        before = B.launch_count()
        conv.forward([xd], y, ws)
        ctx.synchronize()
        print("config 0, fusion %s: %d launches, mean |d| %.3g, max |d| %.3g" % (fusion, B.launch_count() - before,
              np.mean(np.abs(host(y) - want)), np.max(np.abs(host(y) - want))))
        assert np.mean(np.abs(host(y) - want)) <= 1e-4
        assert np.max(np.abs(host(y) - want)) <= 1e-3
    ctx.set_fusion(True)
    y = torch.full((b, h, w, c), float("nan"), device="cuda")
    B.convolutionImplicitGemmForward(ctx, xd, conv.weights, y, conv.bias, None, "relu")
    ctx.synchronize()
    assert np.mean(np.abs(host(y) - want)) <= 1e-4
    perm = _perm(b, 7)
    yp = torch.empty_like(y)
    B.convolutionImplicitGemmForward(ctx, xd[perm].contiguous(), conv.weights, yp, conv.bias, None, "relu")
    ctx.synchronize()
    assert torch.equal(yp, y[perm])


def test_config1_trunk_full_size(ctx, oracle):
    """The whole config-1 trunk at its stated size (batch 256, 15x15, 32 planes, 10 blocks x 128 channels, fp16): batch
    permutation bit-exact at the heads, eight sampled positions within 1e-2 of the fp32 oracle trunk."""
    from minml_b200 import layers as L
    b, h, w, planes, channels, blocks = 256, 15, 15, 32, 128, 10
    weights = L.make_trunk_weights(1235, planes, channels, blocks)
    weights16 = {k: v.astype(np.float16).astype(np.float32) for k, v in weights.items()}
    x = (np.random.default_rng(18).random((b, h, w, planes)) < 0.3).astype(np.float32)
    net = L.ResNetTrunk(ctx, weights, b, h, w, planes, channels, blocks)
    packed = torch.from_numpy(pack_planes(x).view(np.int32)).cuda()
    policy, value = net.predict(packed)
    ctx.synchronize()
    policy, value = policy.clone(), value.clone()
    assert bool(torch.isfinite(policy).all()) and bool(torch.isfinite(value).all())
    perm = _perm(b, 13)
    policy_p, value_p = net.predict(packed[perm].contiguous())
    ctx.synchronize()
    assert torch.equal(policy_p, policy[perm]) and torch.equal(value_p, value[perm])
    items = sorted(set(_sample_items(b) + [b // 4]))
    assert len(items) >= 8
    want_p, want_v = oracle_trunk(oracle, weights16, x[items], blocks)
    ep, ev = max_rel_err(host(policy[items]), want_p), max_rel_err(host(value[items]), want_v)
    print("config 1 trunk against the fp32 oracle: policy %.3g value %.3g" % (ep, ev))
    assert ep <= FP16_REL and ev <= FP16_REL


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
    """The whole config-3 trunk (20 blocks x 256 channels, batch 1024): batch permutation bit-exact at the heads, and eight
    sampled positions within 1e-2 of the fp32 oracle trunk.  A second oracle trunk that rounds every activation to fp16, as the
    device must (the ABI's tensors are fp16), shows where the error comes from: that storage alone moves the oracle as far from
    its fp32 self as the device is."""
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
    items = sorted(set(_sample_items(b) + [b // 4]))
    assert len(items) >= 8
    want_p, want_v = oracle_trunk(oracle, weights16, x[items], blocks)
    stored_p, stored_v = oracle_trunk(oracle, weights16, x[items], blocks, fp16_storage=True)
    got_p, got_v = host(policy[items]), host(value[items])
    storage_p, storage_v = max_rel_err(stored_p, want_p), max_rel_err(stored_v, want_v)  # what fp16 activations cost the oracle itself
    ep, ev = max_rel_err(got_p, want_p), max_rel_err(got_v, want_v)
    sp, sv = max_rel_err(got_p, stored_p), max_rel_err(got_v, stored_v)
    print("config 3 trunk, %d positions: against the fp32 oracle policy %.3g value %.3g; against the oracle with fp16 activations "
          "policy %.3g value %.3g; fp16 storage alone costs the oracle policy %.3g value %.3g" % (len(items), ep, ev, sp, sv, storage_p, storage_v))
    # the bar itself: within 1e-2 of the fp32 oracle at the heads of all 41 layers (measured: policy 3.5e-3, value 6e-4) ...
    assert ep <= FP16_REL and ev <= FP16_REL
    # ... and of the size that rounding every activation to fp16 costs the oracle's own chain (measured 3.6e-3 / 6e-4): the two
    # fp16-storage chains round independently, so they sit about sqrt(2) of that apart (measured 5.6e-3 / 9e-4)
    assert ep <= 2 * storage_p + 1e-3 and ev <= 2 * storage_v + 1e-3
    assert sp <= 2 * storage_p + 1e-3 and sv <= 2 * storage_v + 1e-3


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
