"""Host-side mirror of the reference's layer code for the inference path.

The classes below issue exactly the backend calls that the corresponding minml layers issue, in the same order and with
the same workspace layout, so that what the tests and the benchmark exercise is what minml's unchanged C++ host code
would drive:

  Conv2D                  src/layers/Conv2D.cpp:209-382 (algorithm choice :450-530, workspace :141-191, int8 :211-239)
  Dense                   src/layers/Dense.cpp:90-101
  GlobalAveragePooling    src/layers/GlobalAveragePooling.cpp:51-55
  Add                     src/layers/Add.cpp:50-60
  LayerNormalization      src/layers/LayerNormalization.cpp:86-95
  MultiHeadAttention      src/layers/MultiHeadAttention.cpp:92-101
  ResNetTrunk / HybridBlock   the node loop of Graph::predict (src/graph/Graph.cpp:241-248) over the benchmark topologies,
                          after the FoldAdd pass (src/graph/graph_optimizers.cpp:186-218): the skip connection rides in
                          the second convolution of a block as its `ext` input.

torch supplies device memory only; every computation is a call into libminml_b200.so.
"""
import numpy as np
import torch

from . import backend as B
from .synthetic import he_normal, make_hybrid_weights, make_trunk_weights  # noqa: F401  (re-exported: callers build networks from them)


def _dev(ctx, a, dtype):
    """numpy array -> tensor of `dtype` on the context's device (never torch's current device: a context of GPU 1 must not be
    handed GPU 0's memory)."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(ctx.device).to(dtype).contiguous()


class Workspace:
    """The single scratch tensor a Graph shares between its layers (src/graph/Graph.cpp:578-587), on the device of the context
    that will use it (`ctx=None`: torch's current device)."""

    def __init__(self, ctx=None):
        self.buffer = None
        self.device = ctx.device if ctx is not None else None

    def reserve(self, nbytes):
        if self.buffer is None or self.buffer.numel() < nbytes:
            self.buffer = torch.empty(int(nbytes), dtype=torch.uint8, device=self.device if self.device is not None else "cuda")

    def view(self, shape, dtype, byte_offset=0):
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return self.buffer[byte_offset:byte_offset + n].view(dtype).view(*shape)


class Conv2D:
    def __init__(self, ctx, weights, bias, activation="linear", dtype=torch.float16):
        """weights [cout, k, k, cin] and bias [cout] as numpy fp32 (converted to `dtype` on the device)."""
        self.ctx = ctx
        self.dtype = dtype
        self.activation = activation
        self.kernel = weights.shape[1]
        self.cout, self.cin = weights.shape[0], weights.shape[3]
        self.weights = _dev(ctx, weights, dtype)
        self.bias = None if bias is None else _dev(ctx, bias, dtype)
        self.transformed = None  # cached, as m_transformed_weights in the reference (Conv2D.cpp:356-363)
        self.tile = 4            # CUDA, 3x3 -> WINOGRAD_NON_FUSED with F(4x4,3x3) (Conv2D.cpp:494-498)

    def workspace_bytes(self, in_shape):
        if self.kernel == 1:
            return 0
        b, h, w, _ = in_shape
        tiles = b * ((h + self.tile - 1) // self.tile) * ((w + self.tile - 1) // self.tile)
        elem = torch.empty((), dtype=self.dtype).element_size()
        return (36 * tiles * self.cin + 36 * tiles * self.cout + 1024) * elem  # Conv2D.cpp:173

    def forward(self, inputs, output, workspace):
        x = inputs[0]
        ext = inputs[1] if len(inputs) > 1 else None
        b, h, w, _ = x.shape
        if self.kernel == 1:
            # explicit_gemm_forward, src/core/math.cpp:1595-1626: the input is viewed as [b*h*w, cin]
            a = x.view(b * h * w, self.cin)
            d = output.view(b * h * w, self.cout)
            c = None if ext is None else ext.view(b * h * w, self.cout)
            B.gemm_ex(self.ctx, d, 1.0, "n", a, "t", self.weights.view(self.cout, self.cin), 0.0 if ext is None else 1.0, c, self.bias,
                      self.activation)
            return
        assert self.kernel == 3
        if self.transformed is None:
            self.transformed = torch.empty((36, self.cout, self.cin), dtype=self.dtype, device=self.ctx.device)
            B.winogradWeightTransform(self.ctx, self.weights, self.transformed, False, self.tile)
        tiles = b * ((h + self.tile - 1) // self.tile) * ((w + self.tile - 1) // self.tile)
        elem = torch.empty((), dtype=self.dtype).element_size()
        v = workspace.view((36, tiles, self.cin), self.dtype)
        m = workspace.view((36, tiles, self.cout), self.dtype, 36 * tiles * self.cin * elem)
        B.winogradInputTransform(self.ctx, self.weights.shape, x, v, self.tile)
        B.gemmBatched(self.ctx, "n", v, "t", self.transformed, m)
        B.winogradOutputTransform(self.ctx, self.weights.shape, m, output, self.bias, ext, self.activation, self.tile)


class QuantizedConv2D:
    """The integer branch of Conv2D::forward on a CUDA device (src/layers/Conv2D.cpp:211-239): im2row padded with the
    quantised zero, int8 x int8 -> int32 product into the workspace, then scale / shift / activation / requantisation."""

    def __init__(self, ctx, q_weights, channel_scales, q_bias, input_qd, output_qd, activation="linear", out_dtype=torch.int8):
        self.ctx = ctx
        self.kernel = q_weights.shape[1]
        self.cout, self.cin = q_weights.shape[0], q_weights.shape[3]
        self.weights = torch.from_numpy(np.ascontiguousarray(q_weights)).to(ctx.device)
        # torch's allocator hands out addresses again without the library seeing a free: whatever it cached for weights that lay here goes
        B.lib.mb200_forget_range(B.ptr(self.weights, ctx), self.weights.numel())
        self.channel_scales = _dev(ctx, channel_scales, torch.float32)
        self.bias = _dev(ctx, q_bias, torch.float32)
        self.input_qd, self.output_qd = input_qd, output_qd
        self.activation = activation
        self.out_dtype = out_dtype
        # int8 value that dequantises to 0: round(-shift / scale), AffineTransform::get_inverse()(0) (quantization.hpp:52-63)
        self.input_zero = int(np.clip(np.round(-np.float32(input_qd[1]) / np.float32(input_qd[0])), -128, 127))

    def workspace_bytes(self, in_shape):
        b, h, w, _ = in_shape
        rows = b * h * w
        return rows * self.cout * 4 + (rows * self.kernel * self.kernel * self.cin if self.kernel > 1 else 0) + 1024

    def forward(self, inputs, output, workspace, ext_qd=(1.0, 0.0)):
        x = inputs[0]
        ext = inputs[1] if len(inputs) > 1 else None
        b, h, w, _ = x.shape
        rows = b * h * w
        acc = workspace.view((rows, self.cout), torch.int32)
        wm = self.weights.view(self.cout, self.kernel * self.kernel * self.cin)
        if self.kernel == 1:
            a = x.view(rows, self.cin)
        else:
            a = workspace.view((rows, self.kernel * self.kernel * self.cin), torch.int8, rows * self.cout * 4)
            B.im2row(self.ctx, x, a, self.kernel, False, np.int8(self.input_zero))
        B.gemm(self.ctx, "n", a, "t", wm, acc)
        B.quantized_scale_shift_act(self.ctx, output, self.output_qd, acc, self.channel_scales, self.bias, self.activation, ext, ext_qd)


class Dense:
    def __init__(self, ctx, weights, bias, activation="linear", dtype=torch.float16):
        self.ctx = ctx
        self.weights = _dev(ctx, weights, dtype)  # [out, in]
        self.bias = None if bias is None else _dev(ctx, bias, dtype)
        self.activation = activation

    def forward(self, inputs, output, workspace=None):
        x = inputs[0].view(inputs[0].shape[0], -1)
        B.gemm_ex(self.ctx, output, 1.0, "n", x, "t", self.weights, 0.0, None, self.bias, self.activation)


class GlobalAveragePooling:
    def __init__(self, ctx):
        self.ctx = ctx

    def forward(self, inputs, output, workspace=None):
        B.globalAveragePoolingForward(self.ctx, inputs[0], output)


class Add:
    def __init__(self, ctx, activation="linear"):
        self.ctx = ctx
        self.activation = activation

    def forward(self, inputs, output, workspace=None):
        B.addTensors(self.ctx, output, 1.0, inputs[0], 1.0, inputs[1])
        if self.activation != "linear":
            B.activationForward(self.ctx, output, output, self.activation)


class LayerNormalization:
    def __init__(self, ctx, gamma, beta, dtype=torch.float16):
        self.ctx = ctx
        self.gamma, self.beta = _dev(ctx, gamma, dtype), _dev(ctx, beta, dtype)

    def forward(self, inputs, output, workspace=None):
        B.layernormForward(self.ctx, inputs[0], output, self.gamma, self.beta, inputs[1] if len(inputs) > 1 else None)


class MultiHeadAttention:
    def __init__(self, ctx, num_heads, table, dtype=torch.float16):
        self.ctx = ctx
        self.num_heads = num_heads
        self.table = None if table is None else _dev(ctx, table, dtype)  # [heads, 2R-1, round_up(2R-1, 4)]

    def forward(self, inputs, output, workspace=None):
        B.multiHeadAttentionForward(self.ctx, inputs[0], output, self.table, self.num_heads, False)


# ------------------------------------------------------------------------------------------------------ topologies
class ResNetTrunk:
    """Bit-packed input planes -> stem 3x3 -> `blocks` residual blocks of two 3x3 convolutions -> 1x1 policy head and
    global-average-pool + dense value head.  `predict` walks the nodes in insertion order like Graph::predict."""

    def __init__(self, ctx, weights, batch, height, width, in_planes, channels, blocks, dtype=torch.float16):
        self.ctx, self.dtype = ctx, dtype
        self.batch, self.height, self.width = batch, height, width
        self.in_planes, self.channels, self.blocks = in_planes, channels, blocks
        self.stem = Conv2D(ctx, weights["stem_w"], weights["stem_b"], "relu", dtype)
        self.convs = []
        for i in range(blocks):
            self.convs.append((Conv2D(ctx, weights["b%d_w1" % i], weights["b%d_b1" % i], "relu", dtype),
                               Conv2D(ctx, weights["b%d_w2" % i], weights["b%d_b2" % i], "relu", dtype)))
        self.policy = Conv2D(ctx, weights["policy_w"], weights["policy_b"], "linear", dtype)
        self.gap = GlobalAveragePooling(ctx)
        self.value = Dense(ctx, weights["value_w"], weights["value_b"], "linear", dtype)

        def act():
            return torch.empty((batch, height, width, channels), dtype=dtype, device=ctx.device)
        self.words = (in_planes + 31) // 32
        self.packed = torch.empty((batch, height, width, self.words), dtype=torch.int32, device=ctx.device)
        self.x0 = torch.empty((batch, height, width, in_planes), dtype=dtype, device=ctx.device)
        self.a, self.b, self.c = act(), act(), act()
        self.policy_out = torch.empty((batch, height, width, 1), dtype=dtype, device=ctx.device)
        self.pooled = torch.empty((batch, channels), dtype=dtype, device=ctx.device)
        self.value_out = torch.empty((batch, 3), dtype=dtype, device=ctx.device)
        self.workspace = Workspace(ctx)
        self.workspace.reserve(max(self.stem.workspace_bytes(self.x0.shape), self.convs[0][0].workspace_bytes(self.a.shape) if blocks else 0))

    def conv_flops_per_position(self):
        """Direct-convolution FLOPs per batch item: 2 * H * W * k^2 * cin * cout per convolution + 2 * in * out per dense row."""
        hw = self.height * self.width
        f = 2 * hw * 9 * self.in_planes * self.channels
        f += self.blocks * 2 * (2 * hw * 9 * self.channels * self.channels)
        f += 2 * hw * self.channels * 1 + 2 * self.channels * 3
        return f

    def predict(self, packed_input=None):
        """packed_input: int32 device tensor [batch, h, w, words] of bit planes, or None to reuse the resident one."""
        if packed_input is not None:
            self.packed = packed_input
        B.unpackInput(self.ctx, self.packed, self.x0)
        self.stem.forward([self.x0], self.a, self.workspace)
        cur, tmp, nxt = self.a, self.b, self.c
        for c1, c2 in self.convs:
            c1.forward([cur], tmp, self.workspace)
            c2.forward([tmp, cur], nxt, self.workspace)  # FoldAdd: the skip input is the convolution's second input
            cur, nxt = nxt, cur
        self.policy.forward([cur], self.policy_out, None)
        self.gap.forward([cur], self.pooled)
        self.value.forward([self.pooled], self.value_out)
        return self.policy_out, self.value_out


# ------------------------------------------------------------------------------------------------------ hybrid block
class HybridBlock:
    """x -> 3x3 residual block -> x + proj(MHA(qkv(LN(x)))) -> x + FFN(LN(x)), every layer through the calls minml's
    Conv2D (k = 3 and k = 1), LayerNormalization and MultiHeadAttention layers make; skips ride in the convolutions' `ext`."""

    def __init__(self, ctx, weights, batch, height, width, embed, heads, ffn, dtype=torch.float16):
        self.ctx = ctx
        self.conv1 = Conv2D(ctx, weights["c1_w"], weights["c1_b"], "relu", dtype)
        self.conv2 = Conv2D(ctx, weights["c2_w"], weights["c2_b"], "relu", dtype)
        self.ln1 = LayerNormalization(ctx, weights["ln1_g"], weights["ln1_b"], dtype)
        self.qkv = Conv2D(ctx, weights["qkv_w"], weights["qkv_b"], "linear", dtype)
        self.mha = MultiHeadAttention(ctx, heads, weights["table"], dtype)
        self.proj = Conv2D(ctx, weights["proj_w"], weights["proj_b"], "linear", dtype)
        self.ln2 = LayerNormalization(ctx, weights["ln2_g"], weights["ln2_b"], dtype)
        self.ffn1 = Conv2D(ctx, weights["ffn1_w"], weights["ffn1_b"], "relu", dtype)
        self.ffn2 = Conv2D(ctx, weights["ffn2_w"], weights["ffn2_b"], "linear", dtype)

        def buf(c):
            return torch.empty((batch, height, width, c), dtype=dtype, device=ctx.device)
        self.t1, self.a, self.n1, self.att, self.a2, self.n2, self.out = (buf(embed) for _ in range(7))
        self.qkv_out, self.f1 = buf(3 * embed), buf(ffn)
        self.workspace = Workspace(ctx)
        self.workspace.reserve(self.conv1.workspace_bytes((batch, height, width, embed)))
        self.flops_per_item = (2 * 2 * height * width * 9 * embed * embed + 2 * height * width * embed * (3 * embed + embed + 2 * ffn)
                               + 4 * (height * width) ** 2 * embed)

    def predict(self, x):
        ws = self.workspace
        self.conv1.forward([x], self.t1, ws)
        self.conv2.forward([self.t1, x], self.a, ws)
        self.ln1.forward([self.a], self.n1)
        self.qkv.forward([self.n1], self.qkv_out, ws)
        self.mha.forward([self.qkv_out], self.att)
        self.proj.forward([self.att, self.a], self.a2, ws)
        self.ln2.forward([self.a2], self.n2)
        self.ffn1.forward([self.n2], self.f1, ws)
        self.ffn2.forward([self.f1, self.a2], self.out, ws)
        return self.out
