"""minml's own host code driving the library: oracle/_ref/trunk_dropin is the reference's unmodified Graph / layers / core
sources (compiled in place from the reference checkout by `make -C oracle dropin`) linked against libminml_b200.so instead
of src/backend/cuda.  The program builds the trunk through minml's Graph API, runs it on minml's CPU backend in fp32 and on
this backend, and reports the largest relative difference of each output."""
import json
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
BINARY = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "trunk_dropin")


def run(*args, env=None):
    if not os.path.exists(BINARY):
        pytest.skip("oracle/_ref/trunk_dropin not built (needs the reference checkout: make -C oracle dropin)")
    e = dict(os.environ)
    e.update(env or {})
    out = subprocess.run([BINARY] + [str(a) for a in args], capture_output=True, text=True, timeout=600, env=e)
    assert out.returncode == 0, out.stdout + out.stderr
    return json.loads(out.stdout.strip().splitlines()[-1])


@pytest.mark.parametrize("fusion", ["0", "1"])
@pytest.mark.parametrize("cfg", [(4, 15, 15, 32, 128, 2), (2, 20, 20, 32, 256, 2), (3, 9, 11, 8, 24, 1)])
def test_reference_graph_fp16(cfg, fusion):
    r = run(*cfg, "fp16", env={"MINML_B200_EAGER": "0" if fusion == "1" else "1"})
    assert r["nodes"] == 1 + 1 + 2 * cfg[5] + 3  # input, stem, two convolutions per block (Add folded away), policy, pooling, dense
    assert r["policy_rel_err"] <= (1e-2 if fusion == "1" else 2.5e-2)
    assert r["value_rel_err"] <= (1e-2 if fusion == "1" else 2.5e-2)


def test_reference_graph_fp32():
    r = run(2, 15, 15, 32, 64, 2, "fp32")
    assert r["policy_rel_err"] <= 1e-4 and r["value_rel_err"] <= 1e-4
