"""One process, contexts on two devices -- how minml's own multi-GPU host code uses the backend (one mlContext_t per
device, src/backend/cuda/cuda_context.cpp).  Skipped on a single-GPU box."""
import numpy as np
import pytest
import torch

from tests.util import FP16_REL, host, max_rel_err

pytestmark = pytest.mark.gpu


def test_fused_conv_and_gemm_on_two_devices_of_one_process(oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from minml_b200 import backend as B
    from minml_b200 import layers as L
    r = np.random.default_rng(11)
    b, h, w, c = 3, 20, 20, 256
    x = r.uniform(-1, 1, (b, h, w, c)).astype(np.float16).astype(np.float32)
    wt = (r.standard_normal((c, 3, 3, c)) * np.sqrt(2.0 / (9 * c))).astype(np.float16).astype(np.float32)
    bias = (r.standard_normal(c) * 0.01).astype(np.float16).astype(np.float32)
    w1 = (r.standard_normal((64, 1, 1, c)) * 0.05).astype(np.float16).astype(np.float32)
    want = oracle.conv2d(x, wt, bias, x, "relu")
    want1 = oracle.conv2d(want.astype(np.float16).astype(np.float32), w1, None, None, "linear")
    outputs = []
    # torch's current device stays 0 throughout: the layers must allocate on their context's device, not on the current one
    for device in (1, 0, 1):  # device 1 first: per-device kernel attributes must not be cached from device 0
        ctx = B.Context(device)
        conv = L.Conv2D(ctx, wt, bias, "relu", torch.float16)
        head = L.Conv2D(ctx, w1, None, "linear", torch.float16)
        assert conv.weights.device.index == device
        ws = L.Workspace(ctx)
        ws.reserve(conv.workspace_bytes(x.shape))
        xd = torch.from_numpy(x).to("cuda:%d" % device, torch.float16)
        y = torch.empty((b, h, w, c), device="cuda:%d" % device, dtype=torch.float16)
        y1 = torch.empty((b, h, w, 64), device="cuda:%d" % device, dtype=torch.float16)
        conv.forward([xd, xd], y, ws)
        head.forward([y], y1, ws)
        ctx.synchronize()
        assert max_rel_err(host(y), want) <= FP16_REL
        assert max_rel_err(host(y1), want1) <= FP16_REL
        outputs.append(host(y1))
        if device == 1:  # a tensor of the other GPU is refused on the host, before any launch
            with pytest.raises(B.BackendError, match="passed to a context"):
                B.activationForward(ctx, torch.zeros(8, device="cuda:0"), torch.zeros(8, device="cuda:0"), "relu")
        ctx.close()
    assert np.array_equal(outputs[0], outputs[2])


def test_noalloc_entry_point_on_two_devices(oracle):
    """The no-allocation convolution resolves the address of its built-in scratch array once per device, with that device
    current: device 1 first, then device 0, then device 1 again, each against the oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from minml_b200 import backend as B
    r = np.random.default_rng(12)
    b, h, w, cin, cout = 2, 9, 10, 24, 40
    x = r.uniform(-1, 1, (b, h, w, cin)).astype(np.float32)
    wt = (r.standard_normal((cout, 3, 3, cin)) * np.sqrt(2.0 / (9 * cin))).astype(np.float32)
    bias = (r.standard_normal(cout) * 0.01).astype(np.float32)
    want = oracle.conv2d(x, wt, bias, None, "relu")
    for device in (1, 0, 1):
        ctx = B.Context(device)
        to = lambda a: torch.from_numpy(a).to("cuda:%d" % device)  # noqa: E731
        xd, wd, bd = to(x), to(wt), to(bias)
        y = torch.full((b, h, w, cout), float("nan"), device="cuda:%d" % device)
        B.lib.mb200_convolution_forward_noalloc(ctx.handle, B.dtype_of(xd), B.shape_of(xd), B.shape_of(wd), B.ptr(xd, ctx), B.ptr(wd, ctx),
                                                B.ptr(y, ctx), B.ptr(bd, ctx), None, B.act_code("relu"))
        ctx.check()
        ctx.synchronize()
        assert float(np.mean(np.abs(host(y) - want))) <= 1e-4, "device %d" % device
        ctx.close()
