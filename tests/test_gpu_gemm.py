"""Matrix products on the GPU against the oracle (reference tests: test/backend/test_gemms.cpp:178-374,
test/backend/test_conv2D.cpp:204-248, test/backend/test_quantization.cpp:173-240)."""
import os

import numpy as np
import pytest
import torch

from tests.util import FP16_REL, FP32_TOL, dev, host, init_for_test, max_rel_err, mean_abs_diff

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
@pytest.mark.parametrize("ops", [("n", "n"), ("n", "t"), ("t", "n"), ("t", "t")])
def test_gemm_all_transpositions(ctx, oracle, dtype, ops):
    from minml_b200 import backend as B
    m, n, k = 23, 29, 37
    a = init_for_test((k, m) if ops[0] == "t" else (m, k))
    b = init_for_test((n, k) if ops[1] == "t" else (k, n), 1.0)
    c = init_for_test((m, n), 2.0)
    if dtype == torch.float16:
        a, b, c = [t.astype(np.float16).astype(np.float32) for t in (a, b, c)]
    cd = dev(c, dtype)
    B.gemm(ctx, ops[0], dev(a, dtype), ops[1], dev(b, dtype), cd, 1.1, 0.1)
    ctx.synchronize()
    want = oracle.gemm(ops[0], a, ops[1], b, c, 1.1, 0.1)
    if dtype == torch.float16:
        assert max_rel_err(host(cd), want) <= FP16_REL
    else:
        assert mean_abs_diff(host(cd), want) <= FP32_TOL
    # the legacy entry point gives the same result
    cd2 = dev(c, dtype)
    B.gemm_legacy(ctx, ops[0], dev(a, dtype), ops[1], dev(b, dtype), cd2, 1.1, 0.1)
    ctx.synchronize()
    assert torch.equal(cd, cd2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("ops", [("n", "n"), ("t", "n"), ("t", "t"), ("n", "t")])
@pytest.mark.parametrize("shape", [(256, 256, 256), (136, 264, 200), (1000, 72, 136), (64, 520, 96), (8, 8, 8)])
def test_every_transposition_on_the_tensor_cores(ctx, oracle, dtype, ops, shape):
    """'t' on A and 'n' on B reach the tensor core as MN-major operands (the backward products of the training path,
    src/backend/cuda/gemms.cpp:183-259): row counts that are multiples of 8 (16-byte rows in either storage order), ragged against
    the 128 x 256 tile and the 64-element K slice in every dimension; batched with beta; fp32 both as split operands and as TF32."""
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(m + 3 * n + 7 * k + ord(ops[0]) + 2 * ord(ops[1]))
    batch = 3
    a = r.uniform(-1, 1, (batch, k, m) if ops[0] == "t" else (batch, m, k)).astype(np.float32)
    b = r.uniform(-1, 1, (batch, n, k) if ops[1] == "t" else (batch, k, n)).astype(np.float32)
    c = r.uniform(-1, 1, (batch, m, n)).astype(np.float32)
    if dtype == torch.float16:
        a, b, c = [t.astype(np.float16).astype(np.float32) for t in (a, b, c)]
    before = B.launch_count()
    for tf32 in ((False, True) if dtype == torch.float32 else (False,)):
        ctx.enable_tf32(tf32)
        try:
            cd = dev(c, dtype)
            B.gemmBatched(ctx, ops[0], dev(a, dtype), ops[1], dev(b, dtype), cd, 0.5, 0.25)
            ctx.synchronize()
            c1 = dev(c[0], dtype)
            B.gemm(ctx, ops[0], dev(a[0], dtype), ops[1], dev(b[0], dtype), c1, 0.5, 0.25)
            ctx.synchronize()
        finally:
            ctx.enable_tf32(False)
        for i in range(batch):
            want = oracle.gemm(ops[0], a[i], ops[1], b[i], c[i], 0.5, 0.25)
            if dtype == torch.float16:
                assert max_rel_err(host(cd)[i], want) <= FP16_REL
            elif tf32:
                assert max_rel_err(host(cd)[i], want) <= 2e-3
            else:
                assert mean_abs_diff(host(cd)[i], want) <= FP32_TOL
        assert torch.equal(c1, cd[0])
    # one kernel per product (this does not tell the engines apart: the CUDA-core engine is also one launch here; which engine ran is
    # what kernel_bench's 'n','n' and 't','n' lines show, 720 against 41 TFLOP/s)
    assert B.launch_count() - before == (4 if dtype == torch.float32 else 2)


# (M, N, K): aligned, ragged in every dimension, K not a multiple of the 64-element stage, N beyond one tile, tiny
TC_SHAPES = [(256, 256, 256), (300, 72, 40), (129, 130, 72), (1000, 384, 136), (5, 3, 8), (128, 1, 128), (64, 3, 256), (4096, 128, 128)]


@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_fp16_nt_tensor_core_path(ctx, oracle, shape, out_dtype):
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(m * 7 + n * 3 + k)
    a = r.uniform(-1, 1, (m, k)).astype(np.float16)
    b = r.uniform(-1, 1, (n, k)).astype(np.float16)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype)
    B.gemm(ctx, "n", dev(a), "t", dev(b), c)
    ctx.synchronize()
    want = oracle.gemm("n", a.astype(np.float32), "t", b.astype(np.float32))
    assert max_rel_err(host(c), want) <= (2e-3 if out_dtype == torch.float16 else 1e-5)


@pytest.mark.parametrize("broadcast_b", [False, True])
def test_fp16_batched_nt(ctx, oracle, broadcast_b):
    # the shape family of the Winograd products: [36, tiles, cin] x [36, cout, cin]^T
    from minml_b200 import backend as B
    batch, m, n, k = 36, 200, 96, 64
    r = np.random.default_rng(11)
    a = r.uniform(-1, 1, (batch, m, k)).astype(np.float16)
    b = r.uniform(-1, 1, (n, k) if broadcast_b else (batch, n, k)).astype(np.float16)
    c = torch.full((batch, m, n), float("nan"), device="cuda", dtype=torch.float16)
    B.gemmBatched(ctx, "n", dev(a), "t", dev(b), c)
    ctx.synchronize()
    got = host(c)
    for i in (0, 17, 35):
        want = oracle.gemm("n", a[i].astype(np.float32), "t", (b if broadcast_b else b[i]).astype(np.float32))
        assert max_rel_err(got[i], want) <= 2e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_batched_generic_and_beta(ctx, oracle, dtype):
    from minml_b200 import backend as B
    batch, m, n, k = 5, 23, 29, 37
    a = init_for_test((batch, m, k))
    b = init_for_test((batch, k, n), 1.0)
    c = init_for_test((batch, m, n), 2.0)
    if dtype == torch.float16:
        a, b, c = [t.astype(np.float16).astype(np.float32) for t in (a, b, c)]
    cd = dev(c, dtype)
    B.gemmBatched(ctx, "n", dev(a, dtype), "n", dev(b, dtype), cd, 1.1, 0.1)
    ctx.synchronize()
    for i in range(batch):
        want = oracle.gemm("n", a[i], "n", b[i], c[i], 1.1, 0.1)
        if dtype == torch.float16:
            assert max_rel_err(host(cd)[i], want) <= FP16_REL
        else:
            assert mean_abs_diff(host(cd)[i], want) <= FP32_TOL


@pytest.mark.parametrize("shape", [(1024, 128, 1152), (300, 44, 36), (77, 200, 288), (256, 256, 128), (9, 5, 16)])
def test_int8_nt_accumulators_are_exact(ctx, oracle, shape):
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(m + n + k)
    a = r.integers(-128, 128, (m, k), dtype=np.int8)
    b = r.integers(-128, 128, (n, k), dtype=np.int8)
    c = torch.full((m, n), -1, device="cuda", dtype=torch.int32)
    B.gemm(ctx, "n", dev(a), "t", dev(b), c)
    ctx.synchronize()
    assert np.array_equal(host(c), oracle.gemm_i8_nt(a, b))


def test_int8_k_not_multiple_of_16_uses_generic_engine(ctx, oracle):
    from minml_b200 import backend as B
    r = np.random.default_rng(5)
    a = r.integers(-128, 128, (33, 20), dtype=np.int8)
    b = r.integers(-128, 128, (17, 20), dtype=np.int8)
    c = torch.zeros(33, 17, device="cuda", dtype=torch.int32)
    B.gemm(ctx, "n", dev(a), "t", dev(b), c)
    ctx.synchronize()
    assert np.array_equal(host(c), oracle.gemm_i8_nt(a, b))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(23, 29, 37), (450, 128, 64), (225, 3, 128), (400, 1, 256),
                                   # many rows and a short K: in fp16 the weight-resident variant, whose epilogue moves C and D as boxes
                                   # through tensor maps -- column tails (200 = 6 x 32 + 8, 72, 264 = 256 + 8), row tails, 128- and
                                   # 256-wide tiles; 100 columns make rows that do not start on 16 bytes (the general variant)
                                   (1100, 200, 256), (1333, 72, 192), (1024, 264, 256), (2000, 100, 128)])
@pytest.mark.parametrize("act", ["linear", "relu", "sigmoid"])
def test_gemm_ex_bias_residual_activation(ctx, oracle, dtype, shape, act):
    # D = act(alpha * A B^T + beta * C + bias): 1x1 convolutions and dense layers (src/core/math.cpp:682-702)
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(m + n)
    a = r.uniform(-1, 1, (m, k)).astype(np.float32)
    b = (r.standard_normal((n, k)) * 0.1).astype(np.float32)
    c = r.uniform(-1, 1, (m, n)).astype(np.float32)
    bias = r.standard_normal(n).astype(np.float32)
    if dtype == torch.float16:
        a, b, c, bias = [t.astype(np.float16).astype(np.float32) for t in (a, b, c, bias)]
    for beta, use_bias in ((0.0, True), (1.0, True), (1.0, False), (0.0, False)):
        d = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
        B.gemm_ex(ctx, d, 1.0, "n", dev(a, dtype), "t", dev(b, dtype), beta, dev(c, dtype), dev(bias, dtype) if use_bias else None, act)
        ctx.synchronize()
        pre = oracle.gemm("n", a, "t", b, c, 1.0, beta)
        want = oracle.add_bias_act(pre, bias if use_bias else None, act)
        if dtype == torch.float16:
            assert max_rel_err(host(d), want) <= FP16_REL
        else:
            assert mean_abs_diff(host(d), want) <= FP32_TOL


@pytest.mark.parametrize("shape", [(1100, 200, 256), (2048, 256, 128), (1333, 72, 192)])
def test_weight_resident_variant_in_place(ctx, oracle, shape):
    """C = alpha A B^T + beta C with C read and written in place, on shapes that take the weight-resident variant: its epilogue
    fetches the box of C for the next chunk while the box of D of the current one is on its way out."""
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(m + n + k)
    a = r.uniform(-1, 1, (m, k)).astype(np.float16).astype(np.float32)
    b = (r.standard_normal((n, k)) * 0.1).astype(np.float16).astype(np.float32)
    c = r.uniform(-1, 1, (m, n)).astype(np.float16).astype(np.float32)
    cd = dev(c, torch.float16)
    B.gemm(ctx, "n", dev(a, torch.float16), "t", dev(b, torch.float16), cd, 0.75, 0.5)
    ctx.synchronize()
    assert max_rel_err(host(cd), oracle.gemm("n", a, "t", b, c, 0.75, 0.5)) <= FP16_REL


def test_shape_mismatch_is_reported(ctx):
    from minml_b200 import backend as B
    with pytest.raises(B.BackendError):
        B.gemm(ctx, "n", torch.zeros(4, 5, device="cuda"), "n", torch.zeros(6, 7, device="cuda"), torch.zeros(4, 7, device="cuda"))
    ctx.synchronize()


TF32_REL = 2e-3  # 10 explicit mantissa bits on each operand, fp32 accumulation
FP32_SIMT = os.environ.get("MINML_B200_FP32_SIMT", "0")[:1] == "1"


@pytest.mark.parametrize("shape", [(300, 200, 128), (129, 257, 40), (4096, 256, 256)])
def test_fp32_nt_on_tensor_cores_when_tf32_is_enabled(ctx, oracle, shape):
    """cuda_enable_tf32 moves fp32 'n','t' products to tcgen05 kind::tf32 (the reference then asks cuBLAS for FAST_TF32,
    src/backend/cuda/gemms.cpp:150-153); with it off the result is plain fp32."""
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(sum(shape))
    a, b = r.standard_normal((m, k)).astype(np.float32), r.standard_normal((n, k)).astype(np.float32)
    bias, c0 = r.standard_normal(n).astype(np.float32), r.standard_normal((m, n)).astype(np.float32)
    want = oracle.add_bias_act(oracle.gemm("n", a, "t", b) + c0, bias, "relu")
    launches = []
    for tf32 in (False, True):
        ctx.enable_tf32(tf32)
        d = torch.zeros((m, n), device="cuda")
        before = B.launch_count()
        B.gemm_ex(ctx, d, 1.0, "n", dev(a), "t", dev(b), 1.0, dev(c0), dev(bias), "relu")
        ctx.synchronize()
        launches.append(B.launch_count() - before)
        err = max_rel_err(host(d), want)
        assert err <= (TF32_REL if tf32 else 1e-5)
    ctx.enable_tf32(False)
    # one fused tensor-core kernel either way (split operands when TF32 is not allowed), unless the switch that sends plain fp32
    # products to the register-tiled engine is set
    assert launches[1] == 1 and (launches[0] == 1 or FP32_SIMT)


def test_fp32_winograd_layer_with_tf32(ctx, oracle):
    from minml_b200 import layers as L
    x = np.random.default_rng(2).uniform(-1, 1, (8, 15, 15, 128)).astype(np.float32)
    wt = (np.random.default_rng(3).standard_normal((128, 3, 3, 128)) * np.sqrt(2.0 / (9 * 128))).astype(np.float32)
    bias = (np.random.default_rng(4).standard_normal(128) * 0.01).astype(np.float32)
    conv = L.Conv2D(ctx, wt, bias, "relu", torch.float32)
    ws = L.Workspace()
    ws.reserve(conv.workspace_bytes(x.shape))
    y = torch.empty((8, 15, 15, 128), device="cuda")
    ctx.enable_tf32(True)
    conv.forward([dev(x)], y, ws)
    ctx.synchronize()
    ctx.enable_tf32(False)
    err = max_rel_err(host(y), oracle.conv2d(x, wt, bias, None, "relu"))
    assert err <= 1.5e-2  # measured 8.4e-3: F(4x4,3x3) amplifies the TF32 rounding of V and U (fp16 V / M give 1.2e-2 on such layers)


@pytest.mark.parametrize("ops", ["nn", "nt", "tn", "tt"])
@pytest.mark.parametrize("shape", [(300, 260, 72), (128, 128, 16), (515, 129, 203), (256, 384, 4)])
def test_fp32_register_tiled_engine(ctx, oracle, ops, shape):
    """fp32 products large enough for the 128 x 128 register-tiled kernel: every transposition, tails in all three dimensions,
    alpha / beta, and a batch."""
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(sum(shape) + ord(ops[0]))
    batch = 3
    a = r.standard_normal((batch, k, m) if ops[0] == "t" else (batch, m, k)).astype(np.float32)
    b = r.standard_normal((batch, n, k) if ops[1] == "t" else (batch, k, n)).astype(np.float32)
    c0 = r.standard_normal((batch, m, n)).astype(np.float32)
    c = dev(c0)
    B.gemmBatched(ctx, ops[0], dev(a), ops[1], dev(b), c, 1.1, 0.1)
    ctx.synchronize()
    for i in range(batch):
        want = 1.1 * oracle.gemm(ops[0], a[i], ops[1], b[i]) + 0.1 * c0[i]
        assert np.max(np.abs(host(c[i]) - want)) <= 1e-4 * max(1.0, np.max(np.abs(want)))
    c1 = torch.full((m, n), float("nan"), device="cuda")
    B.gemm(ctx, ops[0], dev(a[0]), ops[1], dev(b[0]), c1)
    ctx.synchronize()
    assert np.max(np.abs(host(c1) - oracle.gemm(ops[0], a[0], ops[1], b[0]))) <= 1e-4 * max(1.0, float(np.max(np.abs(host(c1)))))


@pytest.mark.parametrize("shape", [(1000, 256, 256), (130, 384, 36), (64, 72, 1024)])
def test_fp32_nt_split_operands_keep_fp32_accuracy(ctx, shape):
    """fp32 'n','t' products without TF32 permission run on the tensor cores as hi*hi + hi*lo + lo*hi of operands split into
    two TF32 terms. Checked against a float64 product, relative to sum |a||b|: the error has to stay at the level the other
    fp32 tests allow (1e-5), two orders of magnitude below plain TF32."""
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(k)
    a = (r.standard_normal((m, k)) * np.exp(r.uniform(-6, 6, (m, k)))).astype(np.float32)  # wide dynamic range
    b = (r.standard_normal((n, k)) * np.exp(r.uniform(-6, 6, (n, k)))).astype(np.float32)
    d = torch.full((m, n), float("nan"), device="cuda")
    before = B.launch_count()
    B.gemm(ctx, "n", dev(a), "t", dev(b), d)
    ctx.synchronize()
    assert B.launch_count() - before == 1
    if FP32_SIMT:
        pytest.skip("MINML_B200_FP32_SIMT=1: the split-operand kernel is switched off")
    exact = a.astype(np.float64) @ b.astype(np.float64).T
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).T
    err = float(np.max(np.abs(host(d) - exact) / scale))
    # measured 1.2e-6 (k = 36), 3.6e-6 (k = 256), 5.9e-6 (k = 1024): a few 2^-22 per product (dropped lo*lo, lo truncated to
    # TF32) plus the tensor core's truncating fp32 accumulation, which grows slowly with k; plain TF32 gives about 1e-3 here
    assert err <= 1e-5, err


@pytest.mark.parametrize("shape", [(57600, 1, 128), (1024, 3, 256), (777, 8, 520), (33, 5, 2048), (5, 2, 8)])
@pytest.mark.parametrize("act,use_c", [("linear", False), ("relu", True), ("sigmoid", False)])
def test_fp16_products_with_few_output_columns(ctx, oracle, shape, act, use_c):
    """The policy (N = 1) and value (N = 3) heads: gemm_ex with very few output columns, with bias, beta * C and an activation,
    in one kernel. (A streaming warp-per-row kernel for these shapes was tried and was slower than the tensor-core kernel with
    its mostly empty tile: 0.067 against 0.055 ms at 409600 x 256.)"""
    from minml_b200 import backend as B
    m, n, k = shape
    r = np.random.default_rng(m + n + k)
    h16 = lambda a: a.astype(np.float16).astype(np.float32)
    a, w = h16(r.standard_normal((m, k)) * 0.5), h16(r.standard_normal((n, k)) * 0.2)
    bias, c0 = h16(r.standard_normal(n) * 0.1), h16(r.standard_normal((m, n)))
    d = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float16)
    before = B.launch_count()
    B.gemm_ex(ctx, d, 1.1, "n", dev(a, torch.float16), "t", dev(w, torch.float16), 0.5 if use_c else 0.0, dev(c0, torch.float16) if use_c else None,
              dev(bias, torch.float16), act)
    ctx.synchronize()
    assert B.launch_count() - before == 1
    want = oracle.add_bias_act(1.1 * oracle.gemm("n", a, "t", w) + (0.5 * c0 if use_c else 0.0), bias, act)
    assert max_rel_err(host(d), want) <= FP16_REL
