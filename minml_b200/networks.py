"""The int8 trunk of benchmark configuration 2, assembled the way minml's `Quantize` graph pass assembles it
(src/graph/graph_optimizers.cpp:220-242, src/layers/Layer.cpp:147-160, src/layers/quantization.cpp:59-97):

  * weights: per-output-channel symmetric int8, q = clamp(round(w * 127 / max|w_co|)); channel_scale = s_in * max|w_co| / 127;
    the bias absorbs the input zero point (here 0: activations are symmetric per-tensor, shift = 0);
  * activations: per-tensor int8, calibrated on seeded batches run through the fp16 trunk, either with scale = max|activation| / 127
    and shift 0 (`calibrator="max_abs"`, the rule the benchmark configuration states) or with minml's own histogram calibrator
    (`calibrator="histogram"`, minml_b200.calibration: the Kullback-Leibler range search of src/graph/Histogram.cpp), which for
    tensors after a ReLU gives an asymmetric transform (real 0 = int8 -128); the layers then pad with that quantised zero;
  * every 3x3 layer issues im2row -> int8 GEMM -> quantized_scale_shift_act (the integer branch of Conv2D::forward,
    src/layers/Conv2D.cpp:211-239), which the backend runs as one fused kernel; the last block writes fp16 for the heads,
    which stay in floating point (`quantizable(false)` in the reference).
"""
import numpy as np
import torch

from . import backend as B
from . import layers as L


def quantize_weights(weights, bias, in_scale, in_shift):
    """Host-side restatement of quantize_weights (src/layers/quantization.cpp:59-97), mode per_first_dim, 8 bits."""
    cout = weights.shape[0]
    flat = weights.reshape(cout, -1).astype(np.float32)
    max_abs = np.abs(flat).max(axis=1)
    s = (np.float32(127.0) / max_abs).astype(np.float32)
    q = np.clip(np.sign(flat * s[:, None]) * np.floor(np.abs(flat * s[:, None]) + np.float32(0.5)), -128, 127).astype(np.int8)  # std::round
    channel_scales = (np.float32(in_scale) / s).astype(np.float32)
    q_bias = (np.float32(in_shift) / s * q.astype(np.int32).sum(axis=1).astype(np.float32) + (0 if bias is None else bias)).astype(np.float32)
    return q.reshape(weights.shape), channel_scales, q_bias


class QuantizedTrunk:
    """Same topology as layers.ResNetTrunk; activations between the 3x3 layers are int8."""

    def __init__(self, ctx, weights, batch, height, width, in_planes, channels, blocks, calibration_batches=4, seed=77, calibrator="max_abs"):
        assert calibrator in ("max_abs", "histogram")
        self.ctx = ctx
        self.batch, self.height, self.width = batch, height, width
        self.in_planes, self.channels, self.blocks = in_planes, channels, blocks
        # ---- calibration: max |activation| of every tensor, from the fp16 trunk on seeded Bernoulli(0.3) planes
        calib_batch = min(batch, 64)
        ref = L.ResNetTrunk(ctx, weights, calib_batch, height, width, in_planes, channels, blocks)
        maxima = np.zeros(1 + 2 * blocks, np.float64)
        table = None
        if calibrator == "histogram":
            from . import calibration as K
            table = K.CalibrationTable(1 + 2 * blocks)
            for hist in table.histograms:
                hist.set_hint("relu")  # every tensor between the 3x3 layers follows a ReLU
        rng = np.random.default_rng(seed)
        from .layers import _dev
        for _ in range(calibration_batches):
            planes = (rng.random((calib_batch, height, width, in_planes)) < 0.3).astype(np.float32)
            x0 = _dev(ctx, planes, torch.float16)
            ref.stem.forward([x0], ref.a, ref.workspace)
            ctx.synchronize()
            maxima[0] = max(maxima[0], float(ref.a.abs().max()))
            if table is not None:
                table[0].collect_statistics(ref.a.float().cpu().numpy())
            cur, tmp, nxt = ref.a, ref.b, ref.c
            for i, (c1, c2) in enumerate(ref.convs):
                c1.forward([cur], tmp, ref.workspace)
                c2.forward([tmp, cur], nxt, ref.workspace)
                ctx.synchronize()
                maxima[1 + 2 * i] = max(maxima[1 + 2 * i], float(tmp.abs().max()))
                maxima[2 + 2 * i] = max(maxima[2 + 2 * i], float(nxt.abs().max()))
                if table is not None:
                    table[1 + 2 * i].collect_statistics(tmp.float().cpu().numpy())
                    table[2 + 2 * i].collect_statistics(nxt.float().cpu().numpy())
                cur, nxt = nxt, cur
            if table is not None and table.is_ready():
                break  # minml's Graph::calibrate stops feeding once every histogram reports ready
        # tensor t: real = q * transforms[t][0] + transforms[t][1]
        if table is not None and table.is_ready():
            self.transforms = [h.get_transform() for h in table.histograms]
        else:
            if table is not None:
                raise RuntimeError("the histograms did not settle within %d calibration batches" % calibration_batches)
            self.transforms = [(float(m) / 127.0, 0.0) for m in maxima]
        self.scales = [t[0] for t in self.transforms]
        del ref

        # ---- layers.  The packed planes unpack to {0, 1} int8, i.e. scale 1, shift 0.
        def qconv(wn, bn, in_qd, out_qd, act, out_dtype=torch.int8):
            q, cs, qb = quantize_weights(weights[wn], weights[bn], in_qd[0], in_qd[1])
            return L.QuantizedConv2D(ctx, q, cs, qb, in_qd, out_qd, act, out_dtype)
        self.stem = qconv("stem_w", "stem_b", (1.0, 0.0), self.transforms[0], "relu")
        self.convs = []
        for i in range(blocks):
            s_in = self.transforms[2 * i]
            s_mid, s_out = self.transforms[1 + 2 * i], self.transforms[2 + 2 * i]
            last = i == blocks - 1
            self.convs.append((qconv("b%d_w1" % i, "b%d_b1" % i, s_in, s_mid, "relu"),
                               qconv("b%d_w2" % i, "b%d_b2" % i, s_mid, s_out, "relu", torch.float16 if last else torch.int8), s_in))
        self.policy = L.Conv2D(ctx, weights["policy_w"], weights["policy_b"], "linear", torch.float16)
        self.gap = L.GlobalAveragePooling(ctx)
        self.value = L.Dense(ctx, weights["value_w"], weights["value_b"], "linear", torch.float16)

        def act8():
            return torch.empty((batch, height, width, channels), dtype=torch.int8, device=ctx.device)
        self.words = (in_planes + 31) // 32
        self.packed = torch.empty((batch, height, width, self.words), dtype=torch.int32, device=ctx.device)
        self.x0 = torch.empty((batch, height, width, in_planes), dtype=torch.int8, device=ctx.device)
        self.a, self.b, self.c = act8(), act8(), act8()
        self.last = torch.empty((batch, height, width, channels), dtype=torch.float16, device=ctx.device)
        self.policy_out = torch.empty((batch, height, width, 1), dtype=torch.float16, device=ctx.device)
        self.pooled = torch.empty((batch, channels), dtype=torch.float16, device=ctx.device)
        self.value_out = torch.empty((batch, 3), dtype=torch.float16, device=ctx.device)
        self.workspace = L.Workspace(ctx)
        self.workspace.reserve(self.convs[0][0].workspace_bytes(self.a.shape))

    def predict(self, packed_input=None):
        if packed_input is not None:
            self.packed = packed_input
        B.unpackInput(self.ctx, self.packed, self.x0)
        self.stem.forward([self.x0], self.a, self.workspace)
        cur, tmp, nxt = self.a, self.b, self.c
        for i, (c1, c2, s_in) in enumerate(self.convs):
            c1.forward([cur], tmp, self.workspace)
            out = self.last if i == self.blocks - 1 else nxt
            c2.forward([tmp, cur], out, self.workspace, s_in)  # the skip input carries its own transform
            cur, nxt = out, cur
        self.policy.forward([self.last], self.policy_out, None)
        self.gap.forward([self.last], self.pooled)
        self.value.forward([self.pooled], self.value_out)
        return self.policy_out, self.value_out
