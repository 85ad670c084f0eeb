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
    for device in (1, 0, 1):  # device 1 first: per-device kernel attributes must not be cached from device 0
        with torch.cuda.device(device):
            ctx = B.Context(device)
            conv = L.Conv2D(ctx, wt, bias, "relu", torch.float16)
            head = L.Conv2D(ctx, w1, None, "linear", torch.float16)
            ws = L.Workspace()
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
            ctx.close()
    assert np.array_equal(outputs[0], outputs[2])
