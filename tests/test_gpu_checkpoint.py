"""A network file written by minml's own host code, loaded by minml_b200.checkpoint and run through the C ABI, against the
outputs minml's CPU backend computed for the same input (tests/golden/make_checkpoint.cpp)."""
import os

import numpy as np
import pytest
import torch

from minml_b200 import checkpoint as C

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", ["toy_network.bin", "toy_network_compressed.bin", "toy_block_network.bin"])
@pytest.mark.parametrize("dtype,tolerance", [(torch.float32, 1e-4), (torch.float16, 1e-2)])
@pytest.mark.parametrize("fused", [False, True])
def test_loaded_network_reproduces_the_outputs_minml_computed(ctx, name, dtype, tolerance, fused):
    d, blob = C.load_file(os.path.join(GOLDEN, name))
    io, io_blob = C.load_file(os.path.join(GOLDEN, "toy_block_network_io.bin" if "block" in name else "toy_network_io.bin"))
    x = C.read_tensor(io["input"], io_blob)
    ctx.set_fusion(fused)
    try:
        net = C.LoadedNetwork(ctx, d, blob, dtype)
        policy, value = net.forward(x)
        again = net.forward(x)
    finally:
        ctx.set_fusion(True)
    want_policy, want_value = C.read_tensor(io["policy"], io_blob), C.read_tensor(io["value"], io_blob)
    # softmax outputs: absolute differences against probabilities in [0, 1]; fp32 bound as for every fp32 parity test here,
    # fp16 bound as for the fp16 ones (relative to the largest value, which is close to 1)
    assert np.abs(policy - want_policy).max() <= tolerance * max(1.0, float(want_policy.max()))
    assert np.abs(value - want_value).max() <= tolerance
    assert np.array_equal(again[0], policy) and np.array_equal(again[1], value)


def test_unknown_layer_kind_is_refused(ctx):
    d, blob = C.load_file(os.path.join(GOLDEN, "toy_network.bin"))
    C.nodes_of(d)[3]["layer"]["name"] = "MixtureOfExperts"
    with pytest.raises(NotImplementedError):
        C.LoadedNetwork(ctx, d, blob)
