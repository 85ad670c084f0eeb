"""Reader of minml's on-disk network format and a runner for the layer kinds of the convolution path.

The format (reference: `src/utils/file_util.cpp:28-38` FileSaver::save, `:44-95` FileLoader; `src/graph/Graph.cpp:476-539`
Graph::save / Graph::load; `src/core/Tensor.cpp:786-831` Tensor::serialize / unserialize):

    <Json text> '\\n' <binary blob>            optionally zlib-compressed as a whole

The Json part ends where its outermost bracket closes (FileLoader::find_split_point counts brackets); one byte is skipped
and the rest is the blob. A tensor is `{"shape": [...], "dtype": "FLOAT32", "binary_offset": n}` and its values are
`volume * sizeof(dtype)` bytes of the blob from `n`. A network is `{"dtype", "is_trainable", "nodes": [...]}` (or, in old
files, the bare array of nodes); a node is `{"is_input_node", "is_output_node", "input_nodes": [indices], "layer": {...}}`
and a layer carries its configuration (`Layer::getConfig`, `src/layers/Layer.cpp:162-174`, plus the keys of its kind) and
its parameters `weights` / `bias` (`{"param": tensor, ...}`), `channel_scales`, and `avg_var` for batch normalisation.

`load_file` parses a file; `LoadedNetwork` runs the layer kinds this library accelerates (Input, Conv2D, Dense, Add,
BatchNormalization, GlobalAveragePooling, Softmax, DepthwiseConv2D, RMSNormalization, ChannelScaling, SpaceToDepth,
DepthToSpace) through the C ABI, in fp32 or fp16. Any other layer kind raises.
"""
import json
import zlib

import numpy as np

_DTYPES = {"FLOAT16": np.float16, "FLOAT32": np.float32, "FLOAT64": np.float64, "INT8": np.int8, "INT16": np.int16, "INT32": np.int32,
           "UINT8": np.uint8}


def split_point(data):
    """Index just past the closing bracket of the leading Json value (FileLoader::find_split_point, file_util.cpp:83-95).
    Like the reference it counts brackets only; a bracket inside a Json string would confuse both."""
    depth = 0
    for i, ch in enumerate(data):
        if ch in b"{[":
            depth += 1
        elif ch in b"}]":
            depth -= 1
            if depth == 0:
                return i + 1
    return len(data)


def load_bytes(data, uncompress=None):
    """(description, blob) of a file's content. `uncompress=None` detects zlib by trying it when the content does not
    start like Json (the reference is told by its caller, file_util.cpp:44-58)."""
    if uncompress is None:
        uncompress = not data.lstrip()[:1] in (b"{", b"[")
    if uncompress:
        # ZipWrapper::compress ends its last chunk with a partial flush (flush = 1), not Z_FINISH (src/utils/ZipWrapper.cpp:38-42),
        # so the stream has no final block and no checksum; like ZipWrapper::uncompress, take whatever inflates
        data = zlib.decompressobj().decompress(data)
    cut = split_point(data)
    description = json.loads(data[:cut].decode("utf-8"))
    return description, data[cut + 1:]  # the byte after the Json text is the separating newline


def load_file(path, uncompress=None):
    with open(path, "rb") as f:
        return load_bytes(f.read(), uncompress)


def read_tensor(desc, blob):
    """numpy array of a serialised tensor, or None for a null / empty one (Tensor::unserialize, Tensor.cpp:807-831)."""
    if desc is None:
        return None
    if "param" in desc:  # a Parameter wraps its tensor (src/layers/Parameter.cpp)
        desc = desc["param"]
    shape = [int(d) for d in desc["shape"]]
    if len(shape) == 0:
        return None
    dtype = np.dtype(_DTYPES[desc["dtype"]])
    count = int(np.prod(shape))
    offset = int(desc["binary_offset"])
    if offset + count * dtype.itemsize > len(blob):
        raise ValueError("tensor of shape %s at offset %d runs past the end of the blob (%d bytes)" % (shape, offset, len(blob)))
    return np.frombuffer(blob, dtype, count, offset).reshape(shape).copy()


def nodes_of(description):
    return description if isinstance(description, list) else description["nodes"]


SUPPORTED = ("Input", "Conv2D", "Dense", "Add", "BatchNormalization", "GlobalAveragePooling", "Softmax", "DepthwiseConv2D",
             "RMSNormalization", "ChannelScaling", "SpaceToDepth", "DepthToSpace")


class LoadedNetwork:
    """Runs a loaded network on one GPU through the C ABI, node by node in file order (minml's Graph::predict does the same,
    `src/graph/Graph.cpp:241-248`). Parameters are uploaded once; activations live in buffers allocated at construction for
    the file's own input shape."""

    def __init__(self, ctx, description, blob, dtype=None):
        import torch
        from . import layers as L
        self.ctx = ctx
        self.torch = torch
        self.dtype = dtype if dtype is not None else torch.float32
        self.nodes = nodes_of(description)
        self.workspace = L.Workspace(ctx)
        self.steps = []
        self.outputs = []
        self.shapes = []
        self.input_index = None
        dev = "cuda:%d" % ctx.device_index
        need = 0
        for index, node in enumerate(self.nodes):
            layer = node["layer"]
            kind = layer["name"]
            if kind not in SUPPORTED:
                raise NotImplementedError("layer kind '%s' (node %d) is outside the convolution path this library covers" % (kind, index))
            ins = [int(i) for i in node["input_nodes"]]
            act = layer.get("nonlinearity", "linear")
            w, b = read_tensor(layer.get("weights"), blob), read_tensor(layer.get("bias"), blob)
            if kind == "Input":
                shape = tuple(int(d) for d in layer["input_shape"])
                self.input_index = index
                step = None
            elif kind == "Conv2D":
                if int(layer.get("groups", 1)) != 1:
                    raise NotImplementedError("grouped convolution (node %d)" % index)
                bsz, h, wd, _ = self.shapes[ins[0]]
                shape = (bsz, h, wd, int(layer["output_filters"]))
                if w.shape[1] not in (1, 3) or w.shape[1] != w.shape[2]:
                    raise NotImplementedError("%dx%d convolution (node %d)" % (w.shape[1], w.shape[2], index))
                conv = L.Conv2D(ctx, w, b, act, self.dtype)
                need = max(need, conv.workspace_bytes(self.shapes[ins[0]]))
                step = ("conv", conv, ins)
            elif kind == "Dense":
                shape = (self.shapes[ins[0]][0], int(layer["neurons"]))  # everything after the batch axis is one row
                dense = L.Dense(ctx, w, b, act, self.dtype)
                step = ("dense", dense, ins)
            elif kind == "Add":
                shape = self.shapes[ins[0]]
                step = ("add", act, ins)
            elif kind == "BatchNormalization":
                shape = self.shapes[ins[0]]
                channels = shape[-1]
                stats = read_tensor(layer.get("avg_var"), blob)
                gamma = w if w is not None else np.ones(channels, np.float32)
                beta = b if b is not None else np.zeros(channels, np.float32)
                params = [torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(dev) for a in (gamma, beta, stats)]
                params[0], params[1] = params[0].to(self.dtype), params[1].to(self.dtype)
                step = ("batchnorm", params, act, ins)
            elif kind == "GlobalAveragePooling":
                shape = (self.shapes[ins[0]][0], self.shapes[ins[0]][-1])
                step = ("pool", ins)
            elif kind == "DepthwiseConv2D":
                shape = self.shapes[ins[0]]
                params = [torch.from_numpy(np.ascontiguousarray(w, np.float32)).to(dev).to(self.dtype),
                          None if b is None else torch.from_numpy(np.ascontiguousarray(b, np.float32)).to(dev).to(self.dtype)]
                step = ("depthwise", params, ins)
            elif kind == "RMSNormalization":
                shape = self.shapes[ins[0]]
                gamma = None if w is None else torch.from_numpy(np.ascontiguousarray(w, np.float32)).to(dev).to(self.dtype)
                step = ("rmsnorm", gamma, ins)
            elif kind == "ChannelScaling":
                shape = self.shapes[ins[0]]
                step = ("channel_scaling", ins)
            elif kind == "SpaceToDepth":
                bsz, h, wd, c = self.shapes[ins[0]]
                ph, pw = int(layer["patch_size_h"]), int(layer["patch_size_w"])
                shape = (bsz, -(-h // ph), -(-wd // pw), c * ph * pw)
                step = ("space_to_depth", ins)
            elif kind == "DepthToSpace":
                bsz, h, wd, c = self.shapes[ins[0]]
                ph, pw = int(layer["patch_size_h"]), int(layer["patch_size_w"])
                out_h, out_w = (int(v) for v in layer["output_shape"])
                shape = (bsz, out_h, out_w, c // (ph * pw))
                step = ("depth_to_space", ins)
            else:  # Softmax over all the axes after the first: rows of the flattened rest
                axis = [int(a) for a in layer.get("axis", [])]
                rank = len(self.shapes[ins[0]])
                if axis != list(range(1, rank)):
                    raise NotImplementedError("softmax over axes %s of a rank-%d tensor (node %d)" % (axis, rank, index))
                full = self.shapes[ins[0]]
                shape = (full[0], int(np.prod(full[1:])))
                step = ("softmax", ins)
            self.shapes.append(tuple(shape))
            self.steps.append(step)
            self.outputs.append(torch.empty(tuple(shape), device=dev, dtype=self.dtype))
        self.workspace.reserve(need)
        self.output_nodes = [i for i, n in enumerate(self.nodes) if n["is_output_node"]]

    def forward(self, x):
        """x: numpy array of the file's input shape; returns the output nodes' values as fp32 numpy arrays, in node order."""
        from . import backend as B
        torch = self.torch
        ctx = self.ctx
        out = self.outputs
        out[self.input_index].copy_(torch.from_numpy(np.ascontiguousarray(x, np.float32)).to(out[self.input_index].device).to(self.dtype))
        for index, step in enumerate(self.steps):
            if step is None:
                continue
            if step[0] == "conv":
                step[1].forward([out[i] for i in step[2]], out[index], self.workspace)
            elif step[0] == "dense":
                step[1].forward([out[step[2][0]]], out[index])
            elif step[0] == "add":
                a, b = (out[i] for i in step[2])
                B.addTensors(ctx, out[index], 1.0, a, 1.0, b)
                if step[1] != "linear":
                    B.activationForward(ctx, out[index], out[index], step[1])
            elif step[0] == "batchnorm":
                gamma, beta, stats = step[1]
                B.batchnormInference(ctx, out[step[3][0]], out[index], gamma, beta, stats, step[2])
            elif step[0] == "pool":
                B.globalAveragePoolingForward(ctx, out[step[1][0]], out[index])
            elif step[0] == "depthwise":
                B.depthwiseConvForward(ctx, out[step[2][0]], step[1][0], out[index], step[1][1])
            elif step[0] == "rmsnorm":
                B.rmsnormForward(ctx, out[step[2][0]], out[index], step[1])
            elif step[0] == "channel_scaling":
                B.channelScalingForward(ctx, out[step[1][0]], out[step[1][1]], out[index])
            elif step[0] == "space_to_depth":
                B.spaceToDepth(ctx, out[step[1][0]], out[index])
            elif step[0] == "depth_to_space":
                B.depthToSpace(ctx, out[step[1][0]], out[index])
            elif step[0] == "softmax":
                src = out[step[1][0]]
                B.softmaxForward(ctx, src.view(src.shape[0], -1), out[index])
        ctx.synchronize()
        return [out[i].float().cpu().numpy() for i in self.output_nodes]
