"""The reader of minml's network files against a fixture written by minml's own host code (tests/golden/make_checkpoint.cpp):
the container format, the tensors, and -- through the CPU oracle -- the outputs minml's CPU backend computed."""
import os
import zlib

import numpy as np
import pytest

from minml_b200 import checkpoint as C
from tests.util import forward_loaded_network_on_cpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def golden(name):
    return os.path.join(GOLDEN, name)


def test_plain_and_compressed_files_hold_the_same_network():
    d1, b1 = C.load_file(golden("toy_network.bin"))
    d2, b2 = C.load_file(golden("toy_network_compressed.bin"))
    assert d1 == d2 and b1 == b2
    assert d1["dtype"] == "FLOAT32" and d1["is_trainable"] is False
    kinds = [n["layer"]["name"] for n in C.nodes_of(d1)]
    assert kinds == ["Input", "Conv2D", "BatchNormalization", "Conv2D", "Conv2D", "Add", "Conv2D", "Conv2D", "Add", "Conv2D", "Softmax",
                     "GlobalAveragePooling", "Dense", "Softmax"]
    assert [n["input_nodes"] for n in C.nodes_of(d1)][5] == [4, 2]  # the residual connection
    # explicit flags agree with the detection
    assert C.load_file(golden("toy_network.bin"), uncompress=False)[1] == b1
    assert C.load_file(golden("toy_network_compressed.bin"), uncompress=True)[1] == b1


def test_compressed_stream_is_unfinished_as_the_reference_writes_it():
    """ZipWrapper::compress never passes Z_FINISH, so a strict inflate refuses the file; the reader must not."""
    raw = open(golden("toy_network_compressed.bin"), "rb").read()
    with pytest.raises(zlib.error):
        zlib.decompress(raw)
    assert len(C.load_bytes(raw)[1]) == 59152


def test_tensors_of_the_file():
    d, blob = C.load_file(golden("toy_network.bin"))
    nodes = C.nodes_of(d)
    stem = nodes[1]["layer"]
    w = C.read_tensor(stem["weights"], blob)
    assert w.shape == (16, 3, 3, 4) and w.dtype == np.float32
    assert C.read_tensor(stem["bias"], blob) is None  # use_bias = false: an empty tensor
    assert np.abs(w).max() <= np.sqrt(6.0 / 36) + 1e-6 and np.abs(w).mean() > 0.1  # the generator's He-uniform draw
    bn = nodes[2]["layer"]
    stats = C.read_tensor(bn["avg_var"], blob)
    assert stats.shape == (2, 16) and np.all(stats[1] >= 0.5) and np.all(np.abs(stats[0]) <= 0.5)
    assert C.read_tensor(bn["weights"], blob).shape == (16,)
    assert C.read_tensor(nodes[12]["layer"]["weights"], blob).shape == (3, 16)
    with pytest.raises(ValueError):
        C.read_tensor({"shape": [1 << 20], "dtype": "FLOAT32", "binary_offset": 0}, blob)


def test_split_point_counts_brackets_like_the_reference():
    assert C.split_point(b'{"a": [1, {"b": 2}]}\nxyz') == 20
    assert C.split_point(b'[{"a": 1}]\n\x00\x01') == 10
    assert C.load_bytes(b'[{"a": 1}]\n\x00\x01', uncompress=False) == ([{"a": 1}], b"\x00\x01")


@pytest.mark.parametrize("name", ["toy_network", "toy_block_network"])
def test_oracle_forward_of_the_file_matches_the_outputs_minml_computed(oracle, name):
    """toy_network: the trunk's layer kinds; toy_block_network: space-to-depth, depthwise 7x7, RMS norm, 1x1 convolutions, a
    squeeze-and-excitation branch with channel scaling, depth-to-space (the block of minml's current architectures)."""
    d, blob = C.load_file(golden(name + ".bin"))
    io, io_blob = C.load_file(golden(name + "_io.bin"))
    x = C.read_tensor(io["input"], io_blob)
    policy, value = forward_loaded_network_on_cpu(oracle, d, blob, x)
    want_policy, want_value = C.read_tensor(io["policy"], io_blob), C.read_tensor(io["value"], io_blob)
    assert want_policy.shape == ((3, 81) if name == "toy_network" else (2, 144)) and want_value.shape[1] == 3
    assert float(want_value.max()) > 0.4 and np.ptp(want_value, axis=0).max() > 1e-3  # far from uniform, and the items differ
    assert np.abs(policy - want_policy).max() <= 1e-5
    assert np.abs(value - want_value).max() <= 1e-5


def test_old_format_and_other_dtypes():
    """Files written before the header existed are the bare array of nodes (Graph::load, src/graph/Graph.cpp:502-510); tensors
    may be fp16 or int8 (a quantised network)."""
    import json
    d, blob = C.load_file(golden("toy_network.bin"))
    old = json.dumps(d["nodes"]).encode() + b"\n" + blob
    d2, blob2 = C.load_bytes(old)
    assert isinstance(d2, list) and C.nodes_of(d2) == d["nodes"] and blob2 == blob
    half = np.arange(6, dtype=np.float16).tobytes()
    q = np.array([-128, -1, 0, 127], np.int8).tobytes()
    payload = half + q
    t16 = C.read_tensor({"shape": [2, 3], "dtype": "FLOAT16", "binary_offset": 0}, payload)
    t8 = C.read_tensor({"param": {"shape": [4], "dtype": "INT8", "binary_offset": len(half)}}, payload)
    assert t16.dtype == np.float16 and t16.tolist() == [[0, 1, 2], [3, 4, 5]]
    assert t8.dtype == np.int8 and t8.tolist() == [-128, -1, 0, 127]
    assert C.read_tensor(None, payload) is None
