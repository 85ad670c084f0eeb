"""Pins the oracle: (1) against the known-answer vectors the reference's own tests hold for the Winograd transforms,
(2) against minml's CPU backend compiled from the reference sources, op by op, on seeded inputs.  CPU only."""
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def rng(seed):
    return np.random.default_rng(seed)


def init_for_test(shape, shift=0.0, scale=1.0):
    """sin(i / 10 + shift) * scale -- the deterministic fill of the reference's tests (src/utils/testing_util.cpp:31-55)."""
    n = int(np.prod(shape))
    return (np.sin(np.arange(n, dtype=np.float32) / 10.0 + shift) * scale).astype(np.float32).reshape(shape)


def mean_abs_diff(a, b):
    """The reference's test metric (src/utils/testing_util.cpp:73-107)."""
    return float(np.mean(np.abs(a.astype(np.float64) - b.astype(np.float64))))


# ------------------------------------------------------------------------------------------ known-answer vectors
def _tile(matrices, channel):
    p = int(round(matrices.shape[0] ** 0.5))
    return matrices[:, 0, channel].reshape(p, p)


def test_known_answers_input(oracle):
    ka = json.load(open(os.path.join(GOLDEN, "winograd_known_answers.json")))["input_transform"]
    ones = np.ones((1, 4, 4, 2), np.float32)
    ramp = np.repeat(np.arange(1, 17, dtype=np.float32).reshape(1, 4, 4, 1), 2, axis=3)
    for x, case in zip((ones, ramp), ka):
        v = oracle.winograd_input_transform(x)
        for ch in range(2):
            assert mean_abs_diff(_tile(v, ch), np.array(case["tile_6x6"], np.float32)) <= 1e-4


def test_known_answers_output(oracle):
    ka = json.load(open(os.path.join(GOLDEN, "winograd_known_answers.json")))["output_transform"]
    ones = np.ones((36, 1, 2), np.float32)
    ramp = np.repeat(np.arange(1, 37, dtype=np.float32).reshape(36, 1, 1), 2, axis=2)
    for m, case in zip((ones, ramp), ka):
        y = oracle.winograd_output_transform(m, (1, 4, 4, 2))
        for ch in range(2):
            assert mean_abs_diff(y[0, :, :, ch], np.array(case["tile_4x4"], np.float32)) <= 1e-4


def test_known_answers_weight(oracle):
    ka = json.load(open(os.path.join(GOLDEN, "winograd_known_answers.json")))["weight_transform"]
    nines = np.full((1, 3, 3, 2), 9.0, np.float32)
    ramp = np.repeat(np.arange(1, 10, dtype=np.float32).reshape(1, 3, 3, 1), 2, axis=3)
    for w, case in zip((nines, ramp), ka):
        u = oracle.winograd_weight_transform(w)
        for ch in range(2):
            assert mean_abs_diff(u[:, 0, ch].reshape(6, 6), np.array(case["tile_6x6"], np.float32)) <= 1e-4


# ------------------------------------------------------------------------------------------ oracle vs reference CPU backend
@pytest.mark.parametrize("tile", [4])
def test_winograd_transforms_match_reference(oracle, refcpu, tile):
    # the odd shapes of the reference's own tests: test/backend/test_winograd.cpp:396-470 (3 x 9 x 11 x 35, 35 -> 21 filters)
    x = init_for_test((3, 9, 11, 35))
    w = init_for_test((21, 3, 3, 35), 1.0)
    assert mean_abs_diff(oracle.winograd_input_transform(x, tile), refcpu.winograd_input_transform(x, w.shape, tile)) <= 1e-5
    assert mean_abs_diff(oracle.winograd_weight_transform(w, tile), refcpu.winograd_weight_transform(w, tile)) <= 1e-5
    tiles = 3 * 3 * 3
    m = init_for_test((36, tiles, 21), 2.0)
    bias = init_for_test((21,), 3.0)
    ext = init_for_test((3, 9, 11, 21), 4.0)
    for act in ("linear", "relu", "sigmoid", "tanh"):
        a = oracle.winograd_output_transform(m, (3, 9, 11, 21), bias, ext, act, tile)
        b = refcpu.winograd_output_transform(m, w.shape, (3, 9, 11, 21), bias, ext, act, tile)
        assert mean_abs_diff(a, b) <= 1e-5, act


def test_winograd_conv_equals_direct_conv(oracle, refcpu):
    # reference: TestConv2D winograd_conv2D_3x3_forward, test/backend/test_conv2D.cpp:580-629 (bias + sigmoid)
    r = rng(1)
    x = r.uniform(-1, 1, (2, 13, 17, 35)).astype(np.float32)
    w = (r.standard_normal((21, 3, 3, 35)) * 0.1).astype(np.float32)
    bias = (r.standard_normal(21) * 0.1).astype(np.float32)
    ext = r.uniform(-1, 1, (2, 13, 17, 21)).astype(np.float32)
    direct = oracle.conv2d(x, w, bias, ext, "sigmoid")
    ref = refcpu.conv3x3_winograd(x, w, bias, ext, "sigmoid")
    assert np.max(np.abs(direct - ref)) <= 1e-4
    u = oracle.winograd_weight_transform(w)
    v = oracle.winograd_input_transform(x)
    m = np.stack([oracle.gemm("n", v[p], "t", u[p]) for p in range(36)])
    mine = oracle.winograd_output_transform(m, direct.shape, bias, ext, "sigmoid")
    assert np.max(np.abs(direct - mine)) <= 1e-4


@pytest.mark.parametrize("ops", [("n", "n"), ("n", "t"), ("t", "n"), ("t", "t")])
def test_gemm_matches_reference(oracle, refcpu, ops):
    # reference: test/backend/test_gemms.cpp:178-374, M=23 N=29 K=37, alpha=1.1 beta=0.1
    m, n, k = 23, 29, 37
    a = init_for_test((k, m) if ops[0] == "t" else (m, k))
    b = init_for_test((n, k) if ops[1] == "t" else (k, n), 1.0)
    c = init_for_test((m, n), 2.0)
    got = oracle.gemm(ops[0], a, ops[1], b, c, 1.1, 0.1)
    ref = refcpu.gemm(ops[0], a, ops[1], b, c, 1.1, 0.1)
    assert mean_abs_diff(got, ref) <= 1e-4


def test_gemm_ex_matches_reference(oracle, refcpu):
    a = init_for_test((23, 37))
    b = init_for_test((29, 37), 1.0)
    bias = init_for_test((29,), 2.0)
    ref = refcpu.gemm_ex(a, b, bias, "relu")
    got = oracle.add_bias_act(oracle.gemm("n", a, "t", b), bias, "relu")
    assert mean_abs_diff(got, ref) <= 1e-4


def test_misc_ops_match_reference(oracle, refcpu):
    r = rng(2)
    x = r.standard_normal((3, 5, 7, 36)).astype(np.float32)
    assert mean_abs_diff(oracle.global_average_pooling(x), refcpu.global_average_pooling(x)) <= 1e-5
    gamma = r.standard_normal(36).astype(np.float32)
    beta = r.standard_normal(36).astype(np.float32)
    ext = r.standard_normal(x.shape).astype(np.float32)
    assert mean_abs_diff(oracle.layernorm(x, gamma, beta), refcpu.layernorm(x, gamma, beta)) <= 1e-5
    assert mean_abs_diff(oracle.layernorm(x, gamma, beta, ext), refcpu.layernorm(x, gamma, beta, ext)) <= 1e-5
    bias = r.standard_normal(36).astype(np.float32)
    for act in ("linear", "relu", "sigmoid", "tanh"):
        assert mean_abs_diff(oracle.add_bias_act(x, bias, act), refcpu.add_bias_act(x, bias, act)) <= 1e-5
    packed = r.integers(0, 2 ** 32, size=(4 * 6 * 2,), dtype=np.uint64).astype(np.uint32)
    assert np.array_equal(oracle.unpack_input(packed, (4, 6, 35)), refcpu.unpack_input(packed, (4, 6, 35)))
    assert np.array_equal(oracle.im2row(x, 3), refcpu.im2row(x, 3))


def test_attention_matches_reference(oracle, refcpu):
    r = rng(3)
    heads, d, h, w = 2, 8, 5, 6
    x = r.standard_normal((2, h, w, 3 * heads * d)).astype(np.float32)
    n = 2 * max(h, w) - 1
    table = (r.standard_normal((heads, n, (n + 3) // 4 * 4)) * 0.5).astype(np.float32)
    assert mean_abs_diff(oracle.mha_forward(x, heads, None), refcpu.mha_forward(x, heads, None)) <= 1e-5
    assert mean_abs_diff(oracle.mha_forward(x, heads, table), refcpu.mha_forward(x, heads, table)) <= 1e-5


# ------------------------------------------------------------------------------------------ int8 restatement
def test_int8_conv_self_consistency(oracle):
    """int32 accumulators equal an int64 numpy convolution; padding uses the quantised zero; requantisation follows the formulas."""
    r = rng(4)
    x = r.integers(-128, 128, (2, 6, 7, 12), dtype=np.int8)
    wq = r.integers(-127, 128, (9, 3, 3, 12), dtype=np.int8)
    scales = r.uniform(0.001, 0.01, 9).astype(np.float32)
    bias = r.standard_normal(9).astype(np.float32)
    zero = -3
    y8, yf, acc = oracle.conv2d_int8(x, wq, scales, bias, zero, (0.05, 0.1), "relu")
    xp = np.full((2, 8, 9, 12), zero, np.int64)
    xp[:, 1:-1, 1:-1, :] = x
    ref = np.zeros((2, 6, 7, 9), np.int64)
    for i in range(3):
        for j in range(3):
            ref += np.einsum("bhwc,oc->bhwo", xp[:, i:i + 6, j:j + 7, :], wq[:, i, j, :].astype(np.int64))
    assert np.array_equal(acc, ref.astype(np.int32))
    f = np.maximum(acc.astype(np.float32) * scales + bias, 0.0)
    assert np.allclose(yf, f, atol=1e-6)
    # im2row (padded with the quantised zero) followed by the int8 GEMM gives the same accumulators
    rows = oracle.im2row(x, 3, pad=np.int8(zero))
    assert np.array_equal(oracle.gemm_i8_nt(rows, wq.reshape(9, -1)).reshape(acc.shape), acc)
    y8b, yfb = oracle.scale_shift_act(acc, scales, bias, (0.05, 0.1), "relu")
    assert np.array_equal(yfb, yf)
    assert np.max(np.abs(y8b.astype(np.int32) - y8.astype(np.int32))) <= 1  # (x - z) / s  versus  x * (1/s) - z/s


def test_int8_conv_bit_for_bit_against_the_reference_layer(oracle):
    """The restatement of the integer convolution against the outputs of minml's own Conv2D on Device::cpu() (the scalar loop
    of src/layers/Conv2D.cpp:240-308 after Layer::setupQuantization), committed as tests/golden/int8_conv_cases.bin: quantised
    weights, channel scales, absorbed bias, int8 and fp32 outputs are all equal bit for bit -- 3x3 and 1x1, zero and non-zero
    quantised zeros (padding), with and without a residual input, every activation the loop handles."""
    from tests.util import load_int8_conv_cases
    cases = load_int8_conv_cases()
    assert sorted(cases) == ["k1_sigmoid_ext_i8", "k3_linear_f32", "k3_linear_f32_c128", "k3_relu_ext_i8", "k3_relu_ext_i8_c128",
                             "k3_relu_ext_i8_c32", "k3_relu_min_i8", "k3_tanh_sym_i8"]
    assert [cases[n]["input_zero"] for n in sorted(cases)] == [-7, 55, 55, -37, -128, -37, -128, 0]
    for name, c in cases.items():
        if c["raw_weights"] is not None:  # the wide cases keep only the quantised parameters
            from minml_b200.networks import quantize_weights  # the numpy restatement the int8 trunk is built with
            for fn in (oracle.quantize_weights, quantize_weights):
                q, cs, qb = fn(c["raw_weights"], c["raw_bias"], *c["in_qd"])
                assert np.array_equal(q, c["weights"]), name
                assert np.array_equal(cs.view(np.uint32), c["channel_scales"].view(np.uint32)), name
                assert np.array_equal(qb.view(np.uint32), c["bias"].view(np.uint32)), name
        y8, yf, _ = oracle.conv2d_int8(c["input"], c["weights"], c["channel_scales"], c["bias"], c["input_zero"], c["out_qd"], c["activation"],
                                       c["ext"], c["ext_qd"])
        if c["output"].dtype == np.int8:
            assert np.array_equal(y8, c["output"]), "%s: %d of %d int8 outputs differ" % (name, int(np.sum(y8 != c["output"])), y8.size)
            assert len(np.unique(y8)) > 20  # not saturated: the comparison means something
        else:
            assert np.array_equal(yf.view(np.uint32), c["output"].view(np.uint32)), name


def test_quantize_weights(oracle):
    r = rng(5)
    w = (r.standard_normal((8, 3, 3, 4)) * 0.2).astype(np.float32)
    bias = r.standard_normal(8).astype(np.float32)
    q, cs, qb = oracle.quantize_weights(w, bias, 0.02, 0.3)
    for co in range(8):
        s = 127.0 / np.abs(w[co]).max()
        assert np.array_equal(q[co], np.clip(np.round(w[co] * np.float32(s)), -128, 127).astype(np.int8))
        assert abs(cs[co] - 0.02 / s) <= 1e-7
        assert abs(qb[co] - (0.3 / s * q[co].astype(np.int32).sum() + bias[co])) <= 1e-4


def test_host_weight_quantisation_matches_oracle(oracle):
    """minml_b200.networks.quantize_weights (numpy) against the oracle's restatement of src/layers/quantization.cpp:59-97."""
    from minml_b200.networks import quantize_weights
    r = np.random.default_rng(5)
    w = r.standard_normal((24, 3, 3, 16)).astype(np.float32)
    bias = r.standard_normal(24).astype(np.float32)
    for in_scale, in_shift in ((1.0, 0.0), (0.0131, 0.0), (0.02, 0.4)):
        q, cs, qb = quantize_weights(w, bias, in_scale, in_shift)
        q2, cs2, qb2 = oracle.quantize_weights(w, bias, in_scale, in_shift)
        assert np.array_equal(q, q2)
        assert np.allclose(cs, cs2, rtol=1e-6, atol=0)
        assert np.allclose(qb, qb2, rtol=1e-5, atol=1e-6)


def test_batchnorm_depthwise_and_channel_scaling_against_reference_cpu(oracle, refcpu):
    """The oracle's restatements of the layers next to the convolution path, op by op against minml's CPU backend."""
    r = np.random.default_rng(17)
    c = 128
    x = r.standard_normal((3, 9, 11, c)).astype(np.float32)
    gamma, beta_bn = r.uniform(0.5, 1.5, c).astype(np.float32), r.standard_normal(c).astype(np.float32)
    avg_var = np.stack([r.standard_normal(c), r.uniform(0.2, 2.0, c)]).astype(np.float32)
    for act in ("linear", "relu", "sigmoid", "tanh"):
        assert np.max(np.abs(oracle.batchnorm_inference(x, gamma, beta_bn, avg_var, act) - refcpu.batchnorm_inference(x, gamma, beta_bn, avg_var, act))) <= 1e-5
    # folding: [cout, k, k, cin] per output channel, [k, k, c] (depthwise) per channel
    for shape in ((c, 3, 3, 20), (7, 7, c)):
        w = r.standard_normal(shape).astype(np.float32)
        b = r.standard_normal(c).astype(np.float32)
        w1, b1 = oracle.fold_batchnorm(w, b, gamma, beta_bn, avg_var)
        w2, b2 = refcpu.fold_batchnorm(w, b, gamma, beta_bn, avg_var)
        assert np.max(np.abs(w1 - w2)) <= 1e-6 and np.max(np.abs(b1 - b2)) <= 1e-5
    # folding then convolving equals convolving then normalising
    w = (r.standard_normal((c, 1, 1, 16)) * 0.3).astype(np.float32)
    b = (r.standard_normal(c) * 0.1).astype(np.float32)
    x16 = r.standard_normal((2, 5, 5, 16)).astype(np.float32)
    wf, bf = oracle.fold_batchnorm(w, b, gamma, beta_bn, avg_var)
    direct = oracle.batchnorm_inference(oracle.conv2d(x16, w, b, None, "linear"), gamma, beta_bn, avg_var, "relu")
    assert np.max(np.abs(oracle.conv2d(x16, wf, bf, None, "relu") - direct)) <= 1e-4
    for k in (3, 5, 7):
        wd = (r.standard_normal((k, k, c)) * 0.2).astype(np.float32)
        bias = r.standard_normal(c).astype(np.float32)
        assert np.max(np.abs(oracle.depthwise_conv(x, wd, bias) - refcpu.depthwise_conv(x, wd, bias))) <= 1e-4
    s = r.uniform(0, 1, (3, c)).astype(np.float32)
    assert np.max(np.abs(oracle.channel_scaling(x, s) - refcpu.channel_scaling(x, s))) <= 1e-6


def test_int8_depthwise_restatement_matches_a_plain_numpy_loop(oracle):
    """The integer branch of DepthwiseConv2D::forward (src/layers/DepthwiseConv2D.cpp:104-140) written out once more in numpy."""
    r = np.random.default_rng(18)
    b, h, w, c, k = 2, 6, 7, 24, 7
    x = r.integers(-128, 128, (b, h, w, c), dtype=np.int8)
    wt = r.integers(-127, 128, (k, k, c), dtype=np.int8)
    scales = r.uniform(1e-4, 3e-4, c).astype(np.float32)
    bias = r.standard_normal(c).astype(np.float32) * 0.1
    zero, pad = -3, (k - 1) // 2
    xp = np.full((b, h + 2 * pad, w + 2 * pad, c), zero, np.int32)
    xp[:, pad:pad + h, pad:pad + w] = x
    acc = np.zeros((b, h, w, c), np.int32)
    for i in range(k):
        for j in range(k):
            acc += xp[:, i:i + h, j:j + w] * wt[i, j].astype(np.int32)
    want_f = acc.astype(np.float32) * scales + bias
    out_qd = (0.01, 0.05)
    t = want_f * np.float32(1.0 / np.float32(out_qd[0])) + np.float32(-np.float32(out_qd[1]) / np.float32(out_qd[0]))
    want_8 = np.clip(np.sign(t) * np.floor(np.abs(t) + np.float32(0.5)), -128, 127).astype(np.int8)
    y8, yf = oracle.depthwise_conv_int8(x, wt, scales, bias, out_qd, zero)
    assert np.array_equal(yf, want_f)
    assert np.array_equal(y8, want_8)


def test_gradient_and_update_transforms_against_reference_cpu(oracle, refcpu):
    """The backward-pass transforms against minml's CPU backend (F(4x4,3x3) and F(2x2,5x5), the two it implements), and the
    defining identity of the pair: sum over tiles of <gradient transform, input transform> pushed through the update transform is
    the weight gradient of the convolution."""
    r = np.random.default_rng(21)
    for tile, k in ((4, 3), (2, 5)):
        dy = r.standard_normal((3, 9, 11, 20)).astype(np.float32)
        wshape = (20, k, k, 12)
        assert np.max(np.abs(oracle.winograd_gradient_transform(dy, tile, k) - refcpu.winograd_gradient_transform(dy, wshape, tile))) <= 1e-5
        p = tile + k - 1
        m = r.standard_normal((p * p, 20, 12)).astype(np.float32)
        got, want = oracle.winograd_update_transform(m, tile, k), refcpu.winograd_update_transform(m, wshape, tile)
        assert np.max(np.abs(got - want)) <= 2e-6 * np.max(np.abs(want))  # the oracle sums in double, the backend in fp32
    # dL/dw of y = conv(x, w) for L = sum(y * dy), by the transforms and directly
    for tile, k in ((4, 3), (2, 3), (2, 5)):
        x = r.standard_normal((2, 8, 8, 5)).astype(np.float32)
        dy = r.standard_normal((2, 8, 8, 7)).astype(np.float32)
        v = oracle.winograd_input_transform(x, tile, k)         # [p*p, tiles, cin]
        g = oracle.winograd_gradient_transform(dy, tile, k)     # [p*p, tiles, cout]
        m = np.einsum("ptc,ptd->pcd", g, v).astype(np.float32)  # [p*p, cout, cin]
        dw = oracle.winograd_update_transform(m, tile, k)
        pad = k // 2
        xp = np.pad(x, ((0, 0), (pad, pad), (pad, pad), (0, 0)))
        want = np.zeros((7, k, k, 5), np.float32)
        for i in range(k):
            for j in range(k):
                want[:, i, j, :] = np.einsum("bhwo,bhwc->oc", dy, xp[:, i:i + 8, j:j + 8, :])
        assert np.max(np.abs(dw - want)) <= 1e-3 * np.max(np.abs(want))


def test_rmsnorm_and_space_depth_rearrangements_against_reference_cpu(oracle, refcpu):
    """The restatements against minml's own CPU functions (cpu_rmsnorm_forward, cpu_space_to_depth, cpu_depth_to_space), on the
    shapes of the reference's tests (test_normalization.cpp:977-1013: 123 x 43; test_convert.cpp:282-360: ragged patches)."""
    x = init_for_test((123, 43))
    gamma = init_for_test((43,)) + 1.1
    assert np.abs(oracle.rmsnorm(x, gamma) - refcpu.rmsnorm(x, gamma)).max() <= 1e-6
    assert np.abs(oracle.rmsnorm(x) - refcpu.rmsnorm(x)).max() <= 1e-6
    direct = gamma * x / (1e-6 + np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True)))
    assert np.abs(oracle.rmsnorm(x, gamma) - direct).max() <= 1e-6
    for (b, h, w, c), (oh, ow) in (((3, 8, 8, 5), (4, 4)), ((2, 15, 15, 4), (8, 8)), ((2, 13, 14, 3), (5, 7)), ((1, 6, 9, 2), (6, 3))):
        x = init_for_test((b, h, w, c))
        p, q = -(-h // oh), -(-w // ow)
        deep = oracle.space_to_depth(x, (oh, ow))
        assert deep.shape == (b, oh, ow, p * q * c)
        assert np.array_equal(deep, refcpu.space_to_depth(x, deep.shape))
        back = oracle.depth_to_space(deep, (h, w))
        assert np.array_equal(back, x)  # the round trip loses nothing: only the zero fill past the edge is dropped
        assert np.array_equal(back, refcpu.depth_to_space(deep, x.shape))
    with pytest.raises(ValueError):
        oracle.space_to_depth(init_for_test((1, 10, 10, 2)), (4, 6))  # ceil(10/3) = 4 but ceil(10/2) = 5, ceil(10/1) = 10: no patch gives 6


def test_space_to_depth_moves_bytes_for_any_element_size(oracle):
    x = np.arange(2 * 5 * 7 * 3, dtype=np.int8).reshape(2, 5, 7, 3)
    deep = oracle.space_to_depth(x, (3, 4))
    assert deep.dtype == np.int8 and deep.shape == (2, 3, 4, 2 * 2 * 3)
    assert np.array_equal(deep[1, 0, 0, :3], x[1, 0, 0]) and np.array_equal(deep[1, 0, 0, 3:6], x[1, 0, 1])
    assert np.array_equal(deep[1, 0, 0, 6:9], x[1, 1, 0]) and np.array_equal(deep[0, 2, 3, 3:], np.zeros(9, np.int8))  # past both edges
    assert np.array_equal(oracle.depth_to_space(deep, (5, 7)), x)


def test_round_half_away_from_zero_in_three_operations():
    """The int8 kernels round with trunc(y + copysign(0.49999997, y)) instead of roundf (epilogue.cuh: requant_round).  The two agree
    for every float -- the exhaustive check over all 2.5e9 floats with |y| < 2^23 takes a minute; here: every float around the
    half-integers up to 130 (where the outputs saturate), the neighbours of one half, and a stride through everything else."""
    magic = np.nextafter(np.float32(0.5), np.float32(0))
    assert magic.view(np.uint32) == 0x3EFFFFFF
    halves = (np.arange(0, 131, dtype=np.float32) + np.float32(0.5))
    near = [halves.view(np.uint32).astype(np.int64) + k for k in range(-3, 4)]
    samples = [np.concatenate(near).astype(np.uint32).view(np.float32)]
    samples.append(np.arange(0, 150 << 23, 9973, dtype=np.uint32).view(np.float32))  # a stride through every binade below 2^23
    samples.append(np.array([0.0, 0.49999997, 0.5, 0.50000006, 0.99999994, 1.0, 126.5, 127.49999, 127.5, 128.5, 8388607.5, 1e9], np.float32))
    y = np.concatenate(samples)
    y = np.concatenate([y, -y])
    got = np.trunc(y + np.copysign(magic, y))  # float32 arithmetic, round to nearest even: what the device does
    want = np.trunc(y.astype(np.float64) + np.copysign(0.5, y.astype(np.float64)))  # exact in double
    assert np.array_equal(got.astype(np.float64), want)
