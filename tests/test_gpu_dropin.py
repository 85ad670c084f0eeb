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


# ------------------------------------------------------------------------------------------- the reference's own test suite
TESTS_BINARY = os.path.join(os.path.dirname(BINARY), "minml_tests")

# tests of the reference whose device half exercises the inference path of this backend: all of them must pass
IN_SCOPE = """
TestConv2D.explicit_gemm_conv2D_1x1_forward_fp32 TestConv2D.explicit_gemm_conv2D_5x5_forward_fp32 TestConv2D.winograd_conv2D_3x3_forward
TestConv2D.winograd_conv2D_5x5_forward TestConv2D.im2row3x3 TestConv2D.im2row3x3_invert TestConv2D.im2row5x5 TestConv2D.im2row5x5_invert
TestGemm.float32_NN TestGemm.float32_NT TestGemm.float32_TN TestGemm.float32_TT TestGemm.float16_NN TestGemm.float16_NT TestGemm.float16_TN
TestGemm.float16_TT TestGemmEx.float32_NT TestGemmEx.float16_NT TestGlobalAveragePooling.forward_fp32 TestGlobalAveragePooling.forward_fp16
TestSoftmax.ForwardOnCUDA_fp32 TestSoftmax.ForwardOnCUDA_fp16 TestLayerNorm.forward TestQuantization.conv2D_1x1_forward
TestTensorOp.setall_cuda TestTensorOp.addBiasAct_fp32 TestTensorOp.addBiasAct_fp16 TestTensorOp.addTensors
TestWinograd3x3_4x4.cudaInputTransform TestWinograd3x3_4x4.cudaOutputTransform TestWinograd3x3_4x4.cudaWeightTransform
TestWinograd5x5_2x2.cudaInputTransform TestWinograd5x5_2x2.cudaOutputTransform TestWinograd5x5_2x2.cudaWeightTransform
TestWinograd3x3_4x4.cudaInputTransform_fp16 TestWinograd3x3_4x4.cudaOutputTransform_fp16 TestWinograd3x3_4x4.cudaWeightTransform_fp16
TestWinograd5x5_2x2.cudaInputTransform_fp16 TestWinograd5x5_2x2.cudaOutputTransform_fp16 TestWinograd5x5_2x2.cudaWeightTransform_fp16
TestBatchNorm.inference TestBatchNorm.inference_fp16 TestChannelScaling.forward_fp32 TestChannelScaling.forward_fp16
TestQuantization.depthwise_conv2D_forward TestSpaceToDepth.forward TestDepthToSpace.forward TestRMSNorm.forward TestRMSNorm.forward_no_gamma
TestWinograd3x3_4x4.cudaGradientTransform TestWinograd3x3_4x4.cudaUpdateTransform TestWinograd5x5_2x2.cudaGradientTransform
TestWinograd5x5_2x2.cudaUpdateTransform TestConv2D.winograd_conv2D_3x3_backward TestConv2D.winograd_conv2D_3x3_update
TestConv2D.winograd_conv2D_5x5_backward TestConv2D.winograd_conv2D_5x5_update TestConv2D.explicit_gemm_conv2D_1x1_backward
TestConv2D.explicit_gemm_conv2D_1x1_update TestConv2D.explicit_gemm_conv2D_5x5_update
""".split()

# tests that call entry points this backend exports as stubs (pooling / scaling variants and their backward passes, batch-norm
# training and RMS norm, window and transpose operations, the explicit-GEMM 5x5 backward path), plus one test that fails on the
# reference's own CPU backend as well (TestMultiHeadAttention.forward passes the bias table in the wrong argument)
OUT_OF_SCOPE_PREFIXES = (
    "TestMultiHeadAttention.forward", "TestConv2D.explicit_gemm_conv2D_5x5_backward", "TestGlobalAveragePooling.backward", "TestChannelScaling.backward",
    "TestChannelAveragePooling.", "TestSpatialScaling.", "TestBatchNorm.forward", "TestBatchNorm.backward", "TestLayerNorm.backward", "TestRMSNorm.backward",
    "TestTensorOp.sumOverFirstDim", "TestTensorOp.window_", "TestTensorOp.transpose",
)


def test_reference_test_suite_against_this_backend():
    """test/backend/*.cpp of the reference, compiled unchanged (against a stand-in gtest header), with this library as the CUDA backend."""
    if not os.path.exists(TESTS_BINARY):
        pytest.skip("oracle/_ref/minml_tests not built (needs the reference checkout: make -C oracle reftests)")
    out = subprocess.run([TESTS_BINARY], capture_output=True, text=True, timeout=900)
    lines = out.stdout.strip().splitlines()
    summary = json.loads(lines[-1])
    passed = {l.split("]", 1)[1].strip() for l in lines if l.startswith("[ OK")}
    missing = [t for t in IN_SCOPE if t not in passed]
    assert missing == [], "in-scope reference tests that did not pass: %s" % missing
    unexpected = [t for t in summary["failed_tests"] if not t.startswith(OUT_OF_SCOPE_PREFIXES)]
    assert unexpected == [], "reference tests failed outside the stubbed set: %s" % unexpected
