"""Convolutions on the GPU, driven the way minml's Conv2D layer drives its backend, against the oracle
(reference tests: test/backend/test_conv2D.cpp:204-248,580-629, test/backend/test_quantization.cpp:56-240)."""
import os

import numpy as np
import pytest
import torch

from tests.util import FP16_REL, INT8_REL, dev, host, max_rel_err, mean_abs_diff, oracle_trunk, pack_planes

pytestmark = pytest.mark.gpu


def _case(seed, b, h, w, cin, cout, k=3):
    r = np.random.default_rng(seed)
    x = r.uniform(-1, 1, (b, h, w, cin)).astype(np.float32)
    wt = (r.standard_normal((cout, k, k, cin)) * np.sqrt(2.0 / (k * k * cin))).astype(np.float32)
    bias = (r.standard_normal(cout) * 0.01).astype(np.float32)
    ext = r.uniform(-1, 1, (b, h, w, cout)).astype(np.float32)
    return x, wt, bias, ext


def test_config0_fp32_three_call_path(ctx, oracle, refcpu):
    """Benchmark configuration 0 at a reduced batch: fp32, 15x15, 128 -> 128, bias + ReLU, via the reference's own call triple."""
    from minml_b200 import layers as L
    x, wt, bias, _ = _case(1234, 8, 15, 15, 128, 128)
    conv = L.Conv2D(ctx, wt, bias, "relu", torch.float32)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(x.shape))
    y = torch.full((8, 15, 15, 128), float("nan"), device="cuda")
    conv.forward([dev(x)], y, ws)
    ctx.synchronize()
    want = oracle.conv2d(x, wt, bias, None, "relu")
    assert np.max(np.abs(host(y) - want)) <= 1e-4
    assert np.max(np.abs(host(y) - refcpu.conv3x3_winograd(x, wt, bias, None, "relu"))) <= 1e-4


@pytest.mark.parametrize("fusion", [False, True])
@pytest.mark.parametrize("shape", [(4, 15, 15, 128, 128), (2, 20, 20, 256, 256), (3, 9, 11, 35, 21), (2, 15, 15, 32, 128), (1, 7, 5, 64, 192)])
@pytest.mark.parametrize("act,use_ext", [("relu", False), ("relu", True), ("linear", True), ("sigmoid", False)])
def test_fp16_conv3x3(ctx, oracle, fusion, shape, act, use_ext):
    from minml_b200 import layers as L
    b, h, w, cin, cout = shape
    x, wt, bias, ext = [t.astype(np.float16).astype(np.float32) for t in _case(sum(shape), b, h, w, cin, cout)]
    ctx.set_fusion(fusion)
    conv = L.Conv2D(ctx, wt, bias, act, torch.float16)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(x.shape))
    y = torch.full((b, h, w, cout), float("nan"), device="cuda", dtype=torch.float16)
    inputs = [dev(x, torch.float16)] + ([dev(ext, torch.float16)] if use_ext else [])
    conv.forward(inputs, y, ws)
    conv.forward(inputs, y, ws)  # second call reuses the cached transformed weights
    ctx.synchronize()
    ctx.set_fusion(True)
    want = oracle.conv2d(x, wt, bias, ext if use_ext else None, act)
    # The fused kernel accumulates in fp32 and rounds once: it must meet the 1e-2 bar.  With fusion off the three
    # kernels exchange V and M in fp16, as the reference's ABI prescribes; F(4x4,3x3) amplifies that rounding, and the
    # reference's own fp16 tests allow for it (test/backend/test_winograd.cpp:974-1090 use thresholds up to 1e-1).
    assert max_rel_err(host(y), want) <= (FP16_REL if fusion else 2.5 * FP16_REL)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("k,shape", [(3, (2, 15, 15, 128, 128)), (3, (1, 6, 7, 12, 20)), (1, (3, 15, 15, 128, 1)), (1, (2, 9, 9, 64, 96))])
def test_single_call_fused_entry(ctx, oracle, dtype, k, shape):
    """cuda_convolution_implicit_gemm_forward: y = act(conv(x, w) + bias + add) on raw weights."""
    from minml_b200 import backend as B
    b, h, w, cin, cout = shape
    x, wt, bias, ext = _case(7, b, h, w, cin, cout, k)
    if dtype == torch.float16:
        x, wt, bias, ext = [t.astype(np.float16).astype(np.float32) for t in (x, wt, bias, ext)]
    for act, use in (("relu", True), ("linear", False)):
        y = torch.full((b, h, w, cout), float("nan"), device="cuda", dtype=dtype)
        B.convolutionImplicitGemmForward(ctx, dev(x, dtype), dev(wt, dtype), y, dev(bias, dtype), dev(ext, dtype) if use else None, act)
        ctx.synchronize()
        want = oracle.conv2d(x, wt, bias, ext if use else None, act)
        if dtype == torch.float16:
            assert max_rel_err(host(y), want) <= FP16_REL
        else:
            assert np.max(np.abs(host(y) - want)) <= 2e-4


@pytest.mark.parametrize("fusion", [False, True])
@pytest.mark.parametrize("k,shape", [(3, (4, 20, 20, 128, 128)), (3, (2, 20, 20, 32, 128)), (3, (11, 12, 13, 36, 44)), (1, (11, 12, 13, 36, 44)),
                                     (3, (2, 7, 5, 16, 24))])
@pytest.mark.parametrize("zero_shift", [True, False])
def test_int8_conv(ctx, oracle, fusion, k, shape, zero_shift):
    """The integer branch of Conv2D::forward: int32 accumulators bit-exact, int8 outputs within one step, dequantised within 2e-2."""
    from minml_b200 import layers as L
    b, h, w, cin, cout = shape
    r = np.random.default_rng(sum(shape) + k)
    wf = (r.standard_normal((cout, k, k, cin)) * np.sqrt(2.0 / (k * k * cin))).astype(np.float32)
    bias = (r.standard_normal(cout) * 0.01).astype(np.float32)
    in_qd = (1.0 / 127.0, 0.0) if zero_shift else (0.011, 0.37)
    ext_qd = (0.013, 0.05)
    xq = r.integers(-128, 128, (b, h, w, cin), dtype=np.int8)
    extq = r.integers(-128, 128, (b, h, w, cout), dtype=np.int8)
    q, cs, qb = oracle.quantize_weights(wf, bias, *in_qd)
    input_zero = int(np.clip(np.round(-np.float32(in_qd[1]) / np.float32(in_qd[0])), -128, 127))
    ctx.set_fusion(fusion)
    for act, use_ext, out_dtype in (("relu", True, torch.int8), ("linear", False, torch.int8), ("relu", False, torch.float32)):
        # calibrate the output transform on the fp32 result so that nothing saturates (per-tensor max-abs rule)
        _, calib, _ = oracle.conv2d_int8(xq, q, cs, qb, input_zero, (1.0, 0.0), act, extq if use_ext else None, ext_qd)
        if zero_shift:
            out_qd = (float(np.max(np.abs(calib))) / 127.0, 0.0)
        else:
            lo, hi = float(calib.min()), float(calib.max())
            out_qd = ((hi - lo) / 254.0, (hi + lo) / 2.0)
        conv = L.QuantizedConv2D(ctx, q, cs, qb, in_qd, out_qd, act, out_dtype)
        ws = L.Workspace()
        ws.reserve(conv.workspace_bytes(xq.shape))
        y = torch.zeros((b, h, w, cout), device="cuda", dtype=out_dtype)
        conv.forward([dev(xq)] + ([dev(extq)] if use_ext else []), y, ws, ext_qd)
        ctx.synchronize()
        want8, wantf, want_acc = oracle.conv2d_int8(xq, q, cs, qb, conv.input_zero, out_qd, act, extq if use_ext else None, ext_qd)
        if not fusion:  # the eager path leaves the int32 accumulators in the workspace: they must match bit for bit
            acc = ws.view((b * h * w, cout), torch.int32)
            assert np.array_equal(host(acc).reshape(want_acc.shape), want_acc)
        if out_dtype == torch.int8:
            got = host(y).astype(np.int32)
            assert np.max(np.abs(got - want8.astype(np.int32))) <= 1
            deq_got = got * out_qd[0] + out_qd[1]
            assert max_rel_err(deq_got, wantf) <= INT8_REL
        else:
            assert max_rel_err(host(y), wantf) <= 1e-5
    ctx.set_fusion(True)


@pytest.mark.parametrize("fusion", [False, True])
def test_int8_conv_against_the_reference_layer(ctx, fusion):
    """Every int8 path of the library against the outputs minml's own Conv2D computed on its CPU device
    (tests/golden/int8_conv_cases.bin, the scalar loop of src/layers/Conv2D.cpp:240-308): with ReLU or no activation the int8 and
    fp32 outputs are equal BIT FOR BIT -- same accumulators, same requantisation formula and rounding order on every path;
    with sigmoid / tanh (different exp implementations on the two machines) within one int8 step, and nearly all equal.
    36-channel cases take the three kernels also with fusion on; the 32- and 128-channel cases run the fused kernel (gather and
    copy-engine operand paths, the latter with the border corrections of a non-zero quantised zero)."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    from tests.util import load_int8_conv_cases
    ctx.set_fusion(fusion)
    for name, c in load_int8_conv_cases().items():
        out_dtype = torch.int8 if c["output"].dtype == np.int8 else torch.float32
        conv = L.QuantizedConv2D(ctx, c["weights"], c["channel_scales"], c["bias"], c["in_qd"], c["out_qd"], c["activation"], out_dtype)
        assert conv.input_zero == c["input_zero"], name
        ws = L.Workspace()
        ws.reserve(conv.workspace_bytes(c["input"].shape))
        y = torch.zeros(c["output"].shape, device="cuda", dtype=out_dtype)
        before = B.launch_count()
        conv.forward([dev(c["input"])] + ([dev(c["ext"])] if c["ext"] is not None else []), y, ws, c["ext_qd"])
        ctx.synchronize()
        launches = B.launch_count() - before
        if fusion and c["kernel"] == 3 and c["input"].shape[-1] % 16 == 0:
            assert launches <= 2, "%s: expected the fused kernel (+ border table), saw %d launches" % (name, launches)
        got = host(y)
        if c["activation"] in ("relu", "linear"):
            if out_dtype == torch.int8:
                assert np.array_equal(got, c["output"]), "%s: %d of %d int8 outputs differ" % (name, int(np.sum(got != c["output"])), got.size)
            else:
                assert np.array_equal(got.view(np.uint32), c["output"].view(np.uint32)), name
        else:
            diff = np.abs(got.astype(np.int32) - c["output"].astype(np.int32))
            assert diff.max() <= 1 and np.mean(diff != 0) <= 0.01, "%s: max step %d, %.4f differ" % (name, diff.max(), np.mean(diff != 0))
    ctx.set_fusion(True)


def test_int8_fused_and_eager_outputs_are_identical(ctx):
    """One requantisation formula on every path: the fused kernel's fast path (cout a multiple of 16, aligned rows), its general
    path (a column tail; an output tensor that does not start on a 16-byte boundary) and the three eager kernels give the same
    int8 bits, with ReLU and a residual input."""
    from minml_b200 import layers as L
    r = np.random.default_rng(77)
    for (b, h, w, cin, cout), offset in (((3, 9, 10, 64, 128), 0), ((3, 9, 10, 64, 104), 0), ((2, 8, 8, 128, 128), 8), ((2, 8, 8, 32, 40), 4)):
        q = r.integers(-127, 128, (cout, 3, 3, cin), dtype=np.int8)
        cs = r.uniform(2e-4, 6e-4, cout).astype(np.float32)
        qb = (r.standard_normal(cout) * 0.3).astype(np.float32)
        xq = dev(r.integers(-128, 128, (b, h, w, cin), dtype=np.int8))
        extq = dev(r.integers(-128, 128, (b, h, w, cout), dtype=np.int8))
        conv = L.QuantizedConv2D(ctx, q, cs, qb, (0.02, 0.5), (0.031, 1.7), "relu", torch.int8)
        ws = L.Workspace()
        ws.reserve(conv.workspace_bytes(xq.shape))
        outs = []
        for fusion in (True, False):
            ctx.set_fusion(fusion)
            flat = torch.zeros(b * h * w * cout + 64, device="cuda", dtype=torch.int8)
            y = flat[offset:offset + b * h * w * cout].view(b, h, w, cout)
            conv.forward([xq, extq], y, ws, (0.027, -0.4))
            ctx.synchronize()
            outs.append(host(y).copy())
        ctx.set_fusion(True)
        assert len(np.unique(outs[0])) > 50
        assert np.array_equal(outs[0], outs[1]), "cout %d offset %d: %d differ" % (cout, offset, int(np.sum(outs[0] != outs[1])))


def test_int8_accumulators_fused_path_bit_exact(ctx, oracle):
    """With a requantisation that is the identity on integers (scale 1, shift 0, fp32 out) the fused kernel's output IS the int32 accumulator."""
    from minml_b200 import layers as L
    b, h, w, cin, cout = 3, 20, 20, 64, 128
    r = np.random.default_rng(99)
    q = r.integers(-127, 128, (cout, 3, 3, cin), dtype=np.int8)
    xq = r.integers(-128, 128, (b, h, w, cin), dtype=np.int8)
    conv = L.QuantizedConv2D(ctx, q, np.ones(cout, np.float32), np.zeros(cout, np.float32), (1.0, 0.0), (1.0, 0.0), "linear", torch.float32)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(xq.shape))
    y = torch.zeros((b, h, w, cout), device="cuda", dtype=torch.float32)
    conv.forward([dev(xq)], y, ws)
    ctx.synchronize()
    _, _, want_acc = oracle.conv2d_int8(xq, q, np.ones(cout, np.float32), np.zeros(cout, np.float32), 0)
    assert np.max(np.abs(want_acc)) < 2 ** 24  # exactly representable in fp32
    assert np.array_equal(host(y).astype(np.int64), want_acc.astype(np.int64))


@pytest.mark.parametrize("shape", [(3, 20, 20, 128, 128), (2, 15, 15, 256, 256), (5, 7, 9, 128, 64), (1, 2, 2, 128, 128), (100, 20, 20, 128, 128)])
@pytest.mark.parametrize("zero", [-128, -37, 55])
def test_int8_accumulators_with_a_nonzero_quantised_zero_are_bit_exact(ctx, oracle, shape, zero):
    """Asymmetric activations: positions outside the image hold the quantised zero, not 0. The copy engine can only fill with
    zeros, so the fused kernel adds zero * (sum of the weights of the taps that fell outside) per kind of border position;
    with an identity requantisation its fp32 output is the accumulator, which must equal the padded reference bit for bit.
    Shapes: one-row-tile, CTA-pair (256 columns), ragged, the smallest board with borders, and the two-row-tile variant."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    b, h, w, cin, cout = shape
    r = np.random.default_rng(sum(shape) + zero)
    q = r.integers(-20, 21, (cout, 3, 3, cin), dtype=np.int8)  # |acc| <= 9 * 256 * 20 * 128 < 2^24: exact in fp32
    xq = r.integers(-128, 128, (b, h, w, cin), dtype=np.int8)
    conv = L.QuantizedConv2D(ctx, q, np.ones(cout, np.float32), np.zeros(cout, np.float32), (1.0, float(-zero)), (1.0, 0.0), "linear", torch.float32)
    assert conv.input_zero == zero
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(xq.shape))
    y = torch.zeros((b, h, w, cout), device="cuda", dtype=torch.float32)
    before = B.launch_count()
    conv.forward([dev(xq)], y, ws)
    ctx.synchronize()
    # the table of border corrections and the fused kernel (the operand still comes by TMA); a board of fewer than 9 positions
    # leaves no room for the table in the accumulator scratch and takes the gather variant
    forced_gather = os.environ.get("MINML_B200_CONV_GATHER", "0")[:1] == "1"  # the measurement switch that forces the slower variant
    assert B.launch_count() - before == (2 if b * h * w >= 9 and not forced_gather else 1)
    _, _, want_acc = oracle.conv2d_int8(xq, q, np.ones(cout, np.float32), np.zeros(cout, np.float32), zero)
    assert np.max(np.abs(want_acc)) < 2 ** 24
    assert np.array_equal(host(y).astype(np.int64), want_acc.astype(np.int64))


@pytest.mark.parametrize("cfg", [(4, 15, 15, 32, 128, 2), (2, 20, 20, 32, 256, 2)])
def test_trunk_matches_fp32_oracle(ctx, oracle, cfg):
    """The benchmark topology end to end (packed planes in, policy and value out) against the fp32 oracle."""
    from minml_b200 import layers as L
    b, h, w, planes, channels, blocks = cfg
    weights = L.make_trunk_weights(1235, planes, channels, blocks)
    weights16 = {k: v.astype(np.float16).astype(np.float32) for k, v in weights.items()}
    x = (np.random.default_rng(1).random((b, h, w, planes)) < 0.3).astype(np.float32)
    net = L.ResNetTrunk(ctx, weights, b, h, w, planes, channels, blocks)
    policy, value = net.predict(dev(pack_planes(x).view(np.int32)))
    ctx.synchronize()
    want_p, want_v = oracle_trunk(oracle, weights16, x, blocks)
    assert max_rel_err(host(policy), want_p) <= FP16_REL
    assert max_rel_err(host(value), want_v) <= FP16_REL


@pytest.mark.parametrize("cfg", [(2, 15, 15, 256, 8, 1024), (1, 9, 7, 64, 4, 128)])
def test_hybrid_block_matches_fp32_oracle(ctx, oracle, cfg):
    """Benchmark configuration 4 topology (3x3 residual block, pre-LN attention with relative-position bias, ReLU feed-forward) at a small batch."""
    from minml_b200 import layers as L
    from tests.util import oracle_hybrid
    b, h, w, embed, heads, ffn = cfg
    weights = L.make_hybrid_weights(4321, embed, heads, ffn, max(h, w))
    weights16 = {k: v.astype(np.float16).astype(np.float32) for k, v in weights.items()}
    x = np.random.default_rng(3).standard_normal((b, h, w, embed)).astype(np.float16).astype(np.float32)
    block = L.HybridBlock(ctx, weights, b, h, w, embed, heads, ffn)
    xd = dev(x, torch.float16)
    out = block.predict(xd)
    ctx.synchronize()
    want = oracle_hybrid(oracle, weights16, x, heads)
    assert max_rel_err(host(out), want) <= FP16_REL


@pytest.mark.parametrize("calibrator", ["max_abs", "histogram"])
@pytest.mark.parametrize("cfg", [(4, 15, 15, 32, 128, 2), (2, 20, 20, 32, 256, 3)])
def test_quantized_trunk(ctx, oracle, cfg, calibrator):
    """Benchmark configuration 2 topology (int8 activations and weights between the 3x3 layers, fp16 heads): the heads' outputs against the
    oracle's integer chain with the same calibrated scales, and, loosely, against the fp32 trunk (the quantisation error itself)."""
    from minml_b200 import layers as L
    from minml_b200 import networks as N
    from tests.util import oracle_quantized_trunk
    b, h, w, planes, channels, blocks = cfg
    weights = {k: v.astype(np.float16).astype(np.float32) for k, v in L.make_trunk_weights(1235, planes, channels, blocks).items()}
    x = (np.random.default_rng(1).random((b, h, w, planes)) < 0.3).astype(np.float32)
    net = N.QuantizedTrunk(ctx, weights, b, h, w, planes, channels, blocks, calibration_batches=1 if calibrator == "max_abs" else 200,
                           calibrator=calibrator)
    if calibrator == "histogram":  # after a ReLU minml's calibrator puts real 0 at the bottom of the int8 range
        assert all(abs(shift / scale - 128.0) < 1e-3 for scale, shift in net.transforms)
    policy, value = net.predict(dev(pack_planes(x).view(np.int32)))
    ctx.synchronize()
    want_p, want_v = oracle_quantized_trunk(oracle, weights, x, blocks, net.transforms)
    # one int8 step of disagreement per layer (the oracle and the device round ties alike, but the fused kernel's fp32 sum can differ
    # in the last bit) moves the heads by far less than the fp16 tolerance
    assert max_rel_err(host(policy), want_p) <= FP16_REL
    assert max_rel_err(host(value), want_v) <= FP16_REL
    ref_p, ref_v = oracle_trunk(oracle, weights, x, blocks)
    # the quantisation error itself; the histogram calibrator clips the tails of the activations on purpose, so its worst element
    # can be further off than the max-abs rule's bound (measured 0.15 on the smaller configuration)
    loose = 0.1 if calibrator == "max_abs" else 0.25
    assert max_rel_err(host(policy), ref_p) <= loose
    assert max_rel_err(host(value), ref_v) <= loose


def test_trunk_step_replayed_as_cuda_graph(ctx, oracle):
    """The calls of one trunk step recorded into a CUDA graph on the context's stream and replayed on new input give the same bits
    as issuing them one by one (the deferred call triples are resolved at record time; nothing in the path allocates or
    synchronises once the layers are warm)."""
    from minml_b200 import layers as L
    b, h, w, planes, channels, blocks = 8, 15, 15, 32, 128, 2
    weights = L.make_trunk_weights(99, planes, channels, blocks)
    net = L.ResNetTrunk(ctx, weights, b, h, w, planes, channels, blocks)
    rng = np.random.default_rng(5)
    x1 = (rng.random((b, h, w, planes)) < 0.3).astype(np.float32)
    x2 = (rng.random((b, h, w, planes)) < 0.3).astype(np.float32)
    stage = dev(pack_planes(x1).view(np.int32))
    policy, value = net.predict(stage)  # warm: transformed weights, kernel attributes
    ctx.synchronize()
    stream = ctx.torch_stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        policy, value = net.predict(stage)
    results = []
    for x in (x1, x2):
        stage.copy_(dev(pack_planes(x).view(np.int32)))
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            graph.replay()
        ctx.synchronize()
        replayed = (policy.clone(), value.clone())
        eager = net.predict(stage)
        ctx.synchronize()
        assert torch.equal(replayed[0], eager[0]) and torch.equal(replayed[1], eager[1])
        results.append(replayed)
    assert not torch.equal(results[0][0], results[1][0])  # the replay really consumed the new input
    weights16 = {k: v.astype(np.float16).astype(np.float32) for k, v in weights.items()}
    want_p, want_v = oracle_trunk(oracle, weights16, x2, blocks)
    assert max_rel_err(host(results[1][0]), want_p) <= FP16_REL and max_rel_err(host(results[1][1]), want_v) <= FP16_REL


# ------------------------------------------------------------------------------------------- snapshot semantics, aliasing, threads
def test_fused_path_uses_a_snapshot_of_the_weights(ctx, oracle):
    """In the reference the transformed matrices are a snapshot of the weights at transform time.  The fused kernel reads raw
    weights, so the library keeps its own copy made by cuda_winograd_weight_transform: overwriting (or freeing) the host's
    weight tensor afterwards must not change the result, with fusion on exactly as with fusion off."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    x, wt, bias, ext = _case(501, 3, 10, 11, 64, 64)
    conv = L.Conv2D(ctx, wt, bias, "relu", torch.float16)
    ws = L.Workspace(ctx)
    ws.reserve(conv.workspace_bytes(x.shape))
    xd, extd = dev(x, torch.float16), dev(ext, torch.float16)
    want = oracle.conv2d(host(xd), host(conv.weights), host(conv.bias), host(extd), "relu")
    outs = {}
    for fusion in (True, False):
        ctx.set_fusion(fusion)
        y = torch.zeros((3, 10, 11, 64), device="cuda", dtype=torch.float16)
        conv.forward([xd, extd], y, ws)  # first call: transforms the weights (and takes the snapshot)
        ctx.synchronize()
        conv.weights.normal_()  # the host reuses the raw weight tensor for something else
        torch.cuda.synchronize()
        before = B.launch_count()
        y.zero_()
        conv.forward([xd, extd], y, ws)
        ctx.synchronize()
        assert B.launch_count() - before == (1 if fusion else 3)
        outs[fusion] = host(y)
        assert max_rel_err(outs[fusion], want) <= (FP16_REL if fusion else 2.5e-2), "fusion %s" % fusion
        # restore for the next round: a new transform replaces the snapshot
        conv.weights.copy_(dev(wt, torch.float16))
        conv.transformed = None
    ctx.set_fusion(True)


def test_writing_into_the_transformed_weights_drops_the_snapshot(ctx, oracle):
    """A host that loads transformed weights directly (a copy through the ABI into the matrices) makes the snapshot stale: the
    sequence must then run on the three eager kernels, which read the matrices as they are."""
    import ctypes
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    x, wt, bias, _ = _case(502, 2, 8, 8, 32, 32)
    x2, wt2, _, _ = _case(503, 2, 8, 8, 32, 32)
    conv = L.Conv2D(ctx, wt, bias, "linear", torch.float16)
    other = L.Conv2D(ctx, wt2, bias, "linear", torch.float16)
    ws = L.Workspace(ctx)
    ws.reserve(conv.workspace_bytes(x.shape))
    xd = dev(x, torch.float16)
    y = torch.zeros((2, 8, 8, 32), device="cuda", dtype=torch.float16)
    conv.forward([xd], y, ws)
    other.forward([xd], y, ws)
    ctx.synchronize()
    nbytes = other.transformed.numel() * 2
    B.lib.cuda_memcpy_within_device(ctx.handle, ctypes.c_void_p(conv.transformed.data_ptr()), 0, ctypes.c_void_p(other.transformed.data_ptr()), 0, nbytes)
    before = B.launch_count()
    conv.forward([xd], y, ws)
    ctx.synchronize()
    assert B.launch_count() - before == 3  # eager: the snapshot no longer describes the matrices
    want = oracle.conv2d(host(xd), host(other.weights), host(conv.bias), None, "linear")
    assert max_rel_err(host(y), want) <= 2.5e-2


@pytest.mark.parametrize("fusion", [True, False])
def test_convolution_in_place(ctx, oracle, fusion):
    """y aliasing x: correct on the three-kernel path (the transformed input is complete before y is written); the fused kernel
    would read neighbourhoods that other CTAs overwrite, so such calls are routed to the eager kernels, also with fusion on."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    x, wt, bias, _ = _case(504, 4, 12, 12, 64, 64)
    conv = L.Conv2D(ctx, wt, bias, "relu", torch.float16)
    ws = L.Workspace(ctx)
    ws.reserve(conv.workspace_bytes(x.shape))
    xd = dev(x, torch.float16)
    want = oracle.conv2d(host(xd), host(conv.weights), host(conv.bias), None, "relu")
    ctx.set_fusion(fusion)
    conv.forward([xd], xd, ws)
    ctx.synchronize()
    assert max_rel_err(host(xd), want) <= 2.5e-2
    xd2 = dev(x, torch.float16)
    B.convolutionImplicitGemmForward(ctx, xd2, conv.weights, xd2, conv.bias, None, "relu")
    ctx.synchronize()
    assert max_rel_err(host(xd2), want) <= 2.5e-2
    ctx.set_fusion(True)


def test_two_threads_two_contexts(oracle):
    """One context per host thread, as minml's search code runs its networks: thread A loops fused convolutions (the recorded call
    triple) on its context while thread B allocates, fills and frees tensors through the ABI -- cuda_free and the null-context
    memset flush EVERY context's recorded calls.  Both must see correct results throughout."""
    import ctypes
    import threading
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    ctx_a, ctx_b = B.Context(0), B.Context(0)
    x, wt, bias, ext = _case(505, 2, 9, 9, 32, 32)
    conv = L.Conv2D(ctx_a, wt, bias, "relu", torch.float16)
    ws = L.Workspace(ctx_a)
    ws.reserve(conv.workspace_bytes(x.shape))
    xd, extd = dev(x, torch.float16), dev(ext, torch.float16)
    want = oracle.conv2d(host(xd), host(conv.weights), host(conv.bias), host(extd), "relu")
    stop = threading.Event()
    errors = []

    def allocator():
        B.lib.cuda_malloc.restype = ctypes.c_void_p
        try:
            while not stop.is_set():
                p = B.lib.cuda_malloc(0, 4096)
                B.lib.cuda_memset(None, ctypes.c_void_p(p), 0, 4096, None, 0)  # null context: flushes every context
                B.lib.cuda_free(ctypes.c_void_p(p))
        except Exception as exc:  # pragma: no cover
            errors.append(exc)

    t = threading.Thread(target=allocator)
    t.start()
    try:
        for i in range(200):
            y = torch.zeros((2, 9, 9, 32), device="cuda", dtype=torch.float16)
            conv.forward([xd, extd], y, ws)
            ctx_a.synchronize()
            err = max_rel_err(host(y), want)
            assert err <= 2.5e-2, "iteration %d: %g" % (i, err)  # fused (1e-2) or, when the other thread flushed in between, eager
    finally:
        stop.set()
        t.join()
    assert errors == []
    # and a plain GEMM on the second context still works
    a = dev(np.random.default_rng(1).standard_normal((64, 32)).astype(np.float32), torch.float16)
    c = torch.zeros((64, 64), device="cuda", dtype=torch.float16)
    B.gemm(ctx_b, "n", a, "t", dev(np.eye(64, 32, dtype=np.float32), torch.float16), c)
    ctx_b.synchronize()
    assert np.allclose(host(c)[:, :32], host(a), atol=1e-3)
    ctx_a.close()
    ctx_b.close()


@pytest.mark.parametrize("tf32", [False, True])
@pytest.mark.parametrize("shape", [(8, 15, 15, 128, 128), (3, 9, 11, 32, 40), (2, 20, 20, 64, 256), (1, 5, 7, 96, 300)])
@pytest.mark.parametrize("act,use_ext", [("relu", False), ("linear", True)])
def test_fp32_conv3x3_fused(oracle, tf32, shape, act, use_ext):
    """fp32 3x3 layers whose channel count the copy-engine operand path takes (a multiple of 32) run as ONE kernel launched by the
    reference's call triple: at fp32 accuracy by default (three TF32 products of split operands: mean |d| <= 1e-4, the
    reference's threshold, and max |d| / max |ref| <= 1e-5), as one TF32 product when the host allowed TF32 on the context
    (as cuBLAS would use it: relative error of the order of 2^-11)."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    b, h, w, cin, cout = shape
    x, wt, bias, ext = _case(sum(shape) + 7, b, h, w, cin, cout)
    ctx = B.Context(0)
    ctx.enable_tf32(tf32)
    conv = L.Conv2D(ctx, wt, bias, act, torch.float32)
    ws = L.Workspace(ctx)
    ws.reserve(conv.workspace_bytes(x.shape))
    y = torch.full((b, h, w, cout), float("nan"), device="cuda")
    inputs = [dev(x)] + ([dev(ext)] if use_ext else [])
    conv.forward(inputs, y, ws)  # transforms the weights
    before = B.launch_count()
    conv.forward(inputs, y, ws)
    ctx.synchronize()
    mode = os.environ.get("MINML_B200_FP32_FUSED", "")[:1]
    # without TF32 permission only layers of up to 128 channels take the fused kernel (wider ones are faster on the Winograd path)
    fused = os.environ.get("MINML_B200_EAGER", "0")[:1] != "1" and mode != "n" and (tf32 or mode == "a" or (cin <= 128 and cout <= 128))
    forced_eager = not fused
    assert B.launch_count() - before == (1 if fused else 3)
    want = oracle.conv2d(x, wt, bias, ext if use_ext else None, act)
    if tf32:  # one TF32 product per slice when fused; the Winograd path with TF32 products otherwise (F(4x4,3x3) amplifies the 2^-11)
        assert max_rel_err(host(y), want) <= (2e-3 if fused else 3e-2)
    else:
        assert mean_abs_diff(host(y), want) <= 1e-4
        assert max_rel_err(host(y), want) <= 1e-5
    # the single-call entry takes the same kernel
    y2 = torch.full((b, h, w, cout), float("nan"), device="cuda")
    B.convolutionImplicitGemmForward(ctx, inputs[0], conv.weights, y2, conv.bias, inputs[1] if use_ext else None, act)
    ctx.synchronize()
    if fused and not tf32:
        assert torch.equal(y2, y)  # same kernel on the same weight planes
    else:  # with TF32 the call triple reads weights rounded to TF32 at transform time, the single call lets the tensor core truncate them
        assert max_rel_err(host(y2), want) <= ((2e-3 if fused else 3e-2) if tf32 else 1e-5)
    ctx.close()


def test_border_table_of_an_asymmetric_int8_layer_is_cached(ctx, oracle):
    """The corrections for a non-zero quantised zero depend only on the weights and the padding value: the first call of a layer
    computes them (two launches), later calls reuse them (one launch), and telling the library that the weights changed
    (mb200_forget_range; cuda_free and the ABI's copies do it themselves) makes the next call compute them again."""
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    if os.environ.get("MINML_B200_CONV_GATHER", "0")[:1] == "1" or os.environ.get("MINML_B200_EAGER", "0")[:1] == "1":
        pytest.skip("the measurement switch in force keeps this layer off the copy-engine operand path")
    b, h, w, cin, cout, zero = 2, 9, 9, 128, 128, -37
    r = np.random.default_rng(5150)
    xq = r.integers(-128, 128, (b, h, w, cin), dtype=np.int8)
    conv = None
    for round_index in range(2):
        q = r.integers(-20, 21, (cout, 3, 3, cin), dtype=np.int8)
        if conv is None:
            conv = L.QuantizedConv2D(ctx, q, np.ones(cout, np.float32), np.zeros(cout, np.float32), (1.0, float(-zero)), (1.0, 0.0), "linear", torch.float32)
        else:  # new weights written in place by something the library cannot see (a torch copy), then announced
            conv.weights.copy_(torch.from_numpy(q))
            torch.cuda.synchronize()
            B.lib.mb200_forget_range(B.ptr(conv.weights, ctx), conv.weights.numel())
        ws = L.Workspace(ctx)
        ws.reserve(conv.workspace_bytes(xq.shape))
        _, _, want_acc = oracle.conv2d_int8(xq, q, np.ones(cout, np.float32), np.zeros(cout, np.float32), zero)
        for call, expected_launches in enumerate((2, 1, 1)):
            y = torch.zeros((b, h, w, cout), device="cuda", dtype=torch.float32)
            before = B.launch_count()
            conv.forward([dev(xq)], y, ws)
            ctx.synchronize()
            assert B.launch_count() - before == expected_launches, "round %d call %d" % (round_index, call)
            assert np.array_equal(host(y).astype(np.int64), want_acc.astype(np.int64))
