"""Oracle-side helpers of the parity tests that need numpy only (no torch, no CUDA library): the benchmark topologies
evaluated layer by layer on the CPU oracle, and the reader of the int8 fixture.  bench.py's CPU arm uses them too."""
import numpy as np


def load_int8_conv_cases():
    """The cases of tests/golden/int8_conv_cases.bin (written by minml's own Conv2D on its CPU device, see make_int8_conv.cpp):
    name -> dict with numpy arrays `raw_weights`, `raw_bias`, `weights`, `bias`, `channel_scales`, `input`, `ext` (or None),
    `output`, the (scale, shift) pairs `in_qd`, `ext_qd`, `out_qd`, and `kernel`, `activation`, `input_zero`."""
    import os
    from minml_b200 import checkpoint as C
    description, blob = C.load_file(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "int8_conv_cases.bin"))
    cases = {}
    for name, entry in description.items():
        case = {k: C.read_tensor(entry[k], blob) for k in ("raw_weights", "raw_bias", "weights", "bias", "channel_scales", "input", "ext", "output")}
        t = C.read_tensor(entry["transforms"], blob)
        case["in_qd"], case["ext_qd"], case["out_qd"] = [(float(t[i, 0]), float(t[i, 1])) for i in range(3)]
        case["kernel"], case["activation"], case["input_zero"] = int(entry["kernel"]), entry["activation"], int(entry["input_zero"])
        cases[name] = case
    return cases


def oracle_trunk(oracle, weights, x, blocks, fp16_storage=False):
    """fp32 forward of the ResNet trunk topology with the oracle's direct convolution: (policy [b,h,w,1], value [b,3]).
    `fp16_storage=True` rounds every layer's output to fp16, which is what storing activations in fp16 between layers does to
    the otherwise exact chain: the difference between the two runs is the share of a device-versus-oracle error that the fp16
    tensors of the ABI account for, whatever the kernels do."""
    def store(t):
        return t.astype(np.float16).astype(np.float32) if fp16_storage else t
    a = store(oracle.conv2d(x, weights["stem_w"], weights["stem_b"], None, "relu"))
    for i in range(blocks):
        t = store(oracle.conv2d(a, weights["b%d_w1" % i], weights["b%d_b1" % i], None, "relu"))
        a = store(oracle.conv2d(t, weights["b%d_w2" % i], weights["b%d_b2" % i], a, "relu"))
    policy = store(oracle.conv2d(a, weights["policy_w"], weights["policy_b"], None, "linear"))
    pooled = store(oracle.global_average_pooling(a))
    value = store(oracle.add_bias_act(oracle.gemm("n", pooled, "t", weights["value_w"]), weights["value_b"], "linear"))
    return policy, value


def oracle_quantized_trunk(oracle, weights, x01, blocks, transforms):
    """The int8 trunk (minml_b200.networks.QuantizedTrunk) layer by layer on the oracle's integer convolution.
    `transforms[t]` is the per-tensor (scale, shift) of tensor t (stem output, then two per block), or a bare scale (shift 0)."""
    qd = [t if isinstance(t, tuple) else (t, 0.0) for t in transforms]

    def zero_of(t):  # the int8 value that dequantises to 0, as layers.QuantizedConv2D computes it
        return int(np.clip(np.round(-np.float32(t[1]) / np.float32(t[0])), -128, 127))

    def qconv(xq, wn, bn, t_in, t_out, ext=None, t_ext=(1.0, 0.0)):
        q, cs, qb = oracle.quantize_weights(weights[wn], weights[bn], t_in[0], t_in[1])
        return oracle.conv2d_int8(xq, q, cs, qb, zero_of(t_in), t_out, "relu", ext, t_ext)
    a, _, _ = qconv(x01.astype(np.int8), "stem_w", "stem_b", (1.0, 0.0), qd[0])
    real = None
    for i in range(blocks):
        t_in, t_mid, t_out = qd[2 * i], qd[1 + 2 * i], qd[2 + 2 * i]
        t, _, _ = qconv(a, "b%d_w1" % i, "b%d_b1" % i, t_in, t_mid)
        a, real, _ = qconv(t, "b%d_w2" % i, "b%d_b2" % i, t_mid, t_out, a, t_in)
    real = real.astype(np.float16).astype(np.float32)  # the last block hands fp16 to the heads
    policy = oracle.conv2d(real, weights["policy_w"], weights["policy_b"], None, "linear")
    pooled = oracle.global_average_pooling(real)
    value = oracle.add_bias_act(oracle.gemm("n", pooled, "t", weights["value_w"]), weights["value_b"], "linear")
    return policy, value


def oracle_hybrid(oracle, w, x, heads):
    """fp32 forward of the conv + attention block (same topology as minml_b200.layers.HybridBlock)."""
    def conv1x1(t, wn, bn, ext=None, act="linear"):
        b, h, ww, c = t.shape
        out = oracle.gemm("n", t.reshape(-1, c), "t", w[wn].reshape(w[wn].shape[0], -1))
        if ext is not None:
            out = out + ext.reshape(out.shape)
        return oracle.add_bias_act(out, w[bn], act).reshape(b, h, ww, -1)
    t1 = oracle.conv2d(x, w["c1_w"], w["c1_b"], None, "relu")
    a = oracle.conv2d(t1, w["c2_w"], w["c2_b"], x, "relu")
    n1 = oracle.layernorm(a, w["ln1_g"], w["ln1_b"])
    att = oracle.mha_forward(conv1x1(n1, "qkv_w", "qkv_b"), heads, w["table"])
    a2 = conv1x1(att, "proj_w", "proj_b", a)
    n2 = oracle.layernorm(a2, w["ln2_g"], w["ln2_b"])
    return conv1x1(conv1x1(n2, "ffn1_w", "ffn1_b", None, "relu"), "ffn2_w", "ffn2_b", a2)


def forward_loaded_network_on_cpu(oracle, description, blob, x):
    """Runs a network file (minml_b200.checkpoint's description + blob) through the CPU oracle, node by node; returns the
    output nodes' values. Only the layer kinds of the convolution path."""
    from minml_b200 import checkpoint as C
    values = []
    nodes = C.nodes_of(description)
    for node in nodes:
        layer, ins = node["layer"], node["input_nodes"]
        kind, act = layer["name"], layer["nonlinearity"]
        w, b = C.read_tensor(layer.get("weights"), blob), C.read_tensor(layer.get("bias"), blob)
        if kind == "Input":
            y = x
        elif kind == "Conv2D":
            y = oracle.conv2d(values[ins[0]], w, b if b is not None else np.zeros(w.shape[0], np.float32), None, act)
        elif kind == "BatchNormalization":
            y = oracle.batchnorm_inference(values[ins[0]], w, b, C.read_tensor(layer["avg_var"], blob), act)
        elif kind == "Add":
            y = oracle.add_bias_act(values[ins[0]] + values[ins[1]], np.zeros(values[ins[0]].shape[-1], np.float32), act)
        elif kind == "GlobalAveragePooling":
            y = oracle.global_average_pooling(values[ins[0]])
        elif kind == "Dense":
            rows = values[ins[0]].reshape(values[ins[0]].shape[0], -1)
            y = oracle.add_bias_act(oracle.gemm("n", rows, "t", w), b if b is not None else np.zeros(w.shape[0], np.float32), act)
        elif kind == "Softmax":
            y = oracle.softmax(values[ins[0]].reshape(values[ins[0]].shape[0], -1))
        elif kind == "DepthwiseConv2D":
            y = oracle.depthwise_conv(values[ins[0]], w, b)
        elif kind == "RMSNormalization":
            y = oracle.rmsnorm(values[ins[0]], w)
        elif kind == "ChannelScaling":
            y = oracle.channel_scaling(values[ins[0]], values[ins[1]])
        elif kind == "SpaceToDepth":
            h, wd = values[ins[0]].shape[1:3]
            y = oracle.space_to_depth(values[ins[0]], (-(-h // int(layer["patch_size_h"])), -(-wd // int(layer["patch_size_w"]))))
        elif kind == "DepthToSpace":
            y = oracle.depth_to_space(values[ins[0]], tuple(int(v) for v in layer["output_shape"]))
        else:
            raise NotImplementedError(kind)
        values.append(np.asarray(y, np.float32))
    return [values[i] for i, n in enumerate(nodes) if n["is_output_node"]]
