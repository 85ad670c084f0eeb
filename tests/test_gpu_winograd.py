"""Winograd transforms on the GPU, through the C ABI, against the oracle (reference tests: test/backend/test_winograd.cpp)."""
import json
import os

import numpy as np
import pytest
import torch

from tests.util import FP16_REL, FP32_TOL, dev, host, init_for_test, max_rel_err, mean_abs_diff

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_known_answers_on_gpu(ctx):
    from minml_b200 import backend as B
    ka = json.load(open(os.path.join(GOLDEN, "winograd_known_answers.json")))
    ramp_x = np.repeat(np.arange(1, 17, dtype=np.float32).reshape(1, 4, 4, 1), 2, axis=3)
    for x, case in zip((np.ones((1, 4, 4, 2), np.float32), ramp_x), ka["input_transform"]):
        v = torch.zeros(36, 1, 2, device="cuda")
        B.winogradInputTransform(ctx, (1, 3, 3, 2), dev(x), v)
        ctx.synchronize()
        for ch in range(2):
            assert mean_abs_diff(host(v)[:, 0, ch].reshape(6, 6), case["tile_6x6"]) <= 1e-4
    ramp_m = np.repeat(np.arange(1, 37, dtype=np.float32).reshape(36, 1, 1), 2, axis=2)
    for m, case in zip((np.ones((36, 1, 2), np.float32), ramp_m), ka["output_transform"]):
        y = torch.zeros(1, 4, 4, 2, device="cuda")
        B.winogradOutputTransform(ctx, (1, 3, 3, 2), dev(m), y)
        ctx.synchronize()
        for ch in range(2):
            assert mean_abs_diff(host(y)[0, :, :, ch], case["tile_4x4"]) <= 1e-4
    ramp_w = np.repeat(np.arange(1, 10, dtype=np.float32).reshape(1, 3, 3, 1), 2, axis=3)
    for w, case in zip((np.full((1, 3, 3, 2), 9.0, np.float32), ramp_w), ka["weight_transform"]):
        u = torch.zeros(36, 1, 2, device="cuda")
        B.winogradWeightTransform(ctx, dev(w), u)
        ctx.synchronize()
        for ch in range(2):
            assert mean_abs_diff(host(u)[:, 0, ch].reshape(6, 6), case["tile_6x6"]) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("tile,k", [(4, 3), (2, 3), (2, 5)])
@pytest.mark.parametrize("shape", [(3, 9, 11, 35, 21), (2, 15, 15, 64, 32), (1, 20, 20, 8, 8), (2, 4, 4, 2, 2), (1, 1, 1, 3, 5)])
def test_transforms_against_oracle(ctx, oracle, dtype, tile, k, shape):
    from minml_b200 import backend as B
    b, h, w, cin, cout = shape
    p = tile + k - 1
    tiles = b * ((h + tile - 1) // tile) * ((w + tile - 1) // tile)
    x = init_for_test((b, h, w, cin))
    wt = init_for_test((cout, k, k, cin), 1.0)
    m = init_for_test((p * p, tiles, cout), 2.0)
    bias = init_for_test((cout,), 3.0)
    ext = init_for_test((b, h, w, cout), 4.0)
    if dtype == torch.float16:  # compare against the oracle run on the fp16-rounded inputs
        x, wt, m, bias, ext = [a.astype(np.float16).astype(np.float32) for a in (x, wt, m, bias, ext)]

    def close(got, want, what):
        if dtype == torch.float32:
            assert mean_abs_diff(got, want) <= FP32_TOL, what
        else:
            assert max_rel_err(got, want) <= FP16_REL, what

    v = torch.full((p * p, tiles, cin), float("nan"), device="cuda", dtype=dtype)
    xd = dev(x, dtype)  # stays alive until the synchronize below: the backend may defer the transform (see fusion.cu)
    B.winogradInputTransform(ctx, wt.shape, xd, v, tile_size=tile)
    u = torch.full((p * p, cout, cin), float("nan"), device="cuda", dtype=dtype)
    B.winogradWeightTransform(ctx, dev(wt, dtype), u, tile_size=tile)
    ctx.synchronize()
    close(host(v), oracle.winograd_input_transform(x, tile, k), "input")
    close(host(u), oracle.winograd_weight_transform(wt, tile), "weight")
    u2 = torch.empty_like(u)
    B.winogradWeightTransform(ctx, dev(wt, dtype), u2, invert=True, tile_size=tile)
    ctx.synchronize()
    close(host(u2), oracle.winograd_weight_transform(wt, tile, invert=True), "weight inverted")
    for act in ("linear", "relu", "sigmoid", "tanh", "leaky_relu"):
        for use_bias, use_ext in ((True, True), (False, False), (True, False)):
            y = torch.full((b, h, w, cout), float("nan"), device="cuda", dtype=dtype)
            B.winogradOutputTransform(ctx, wt.shape, dev(m, dtype), y, dev(bias, dtype) if use_bias else None,
                                      dev(ext, dtype) if use_ext else None, act, tile_size=tile)
            ctx.synchronize()
            want = oracle.winograd_output_transform(m, (b, h, w, cout), bias if use_bias else None, ext if use_ext else None, act, tile, k)
            close(host(y), want, "output %s" % act)


def test_output_does_not_write_outside(ctx):
    """Canary rows around the output buffer stay untouched for a board that is not a multiple of the tile."""
    from minml_b200 import backend as B
    b, h, w, c = 2, 7, 11, 20
    tiles = b * 2 * 3
    m = dev(init_for_test((36, tiles, c)))
    buf = torch.full((b * h * w * c + 256,), 777.0, device="cuda")
    y = buf[128:128 + b * h * w * c].view(b, h, w, c)
    B.winogradOutputTransform(ctx, (c, 3, 3, c), m, y)
    ctx.synchronize()
    assert torch.all(buf[:128] == 777.0) and torch.all(buf[-128:] == 777.0)
    assert not torch.any(y == 777.0)


def test_bad_arguments_record_an_error(ctx):
    from minml_b200 import backend as B
    x = torch.zeros(1, 4, 4, 8, device="cuda")
    with pytest.raises(B.BackendError):
        B.winogradInputTransform(ctx, (8, 3, 3, 8), x, torch.zeros(36, 2, 8, device="cuda"))  # wrong tile count
    with pytest.raises(B.BackendError):
        B.winogradInputTransform(ctx, (8, 3, 3, 8), x, torch.zeros(25, 1, 8, device="cuda"), tile_size=3)  # unsupported transform
    ctx.synchronize()
