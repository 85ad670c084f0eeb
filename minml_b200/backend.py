"""Python mirror of the reference's dispatcher functions (include/minml/core/math.hpp:28-225) for the inference path.

Each function takes torch CUDA tensors, builds the POD descriptors and calls the matching `cuda_*` entry point of
libminml_b200.so through ctypes -- the same calls, in the same argument order, that src/core/math.cpp makes.
torch is used for device memory only.  After every call the context's sticky error is checked and raised.
"""
import ctypes

import torch

from . import _abi
from ._abi import (ACTIVATION_LINEAR, ACTIVATION_RELU, ACTIVATION_SIGMOID, ACTIVATION_TANH,  # noqa: F401
                   ACTIVATION_LEAKY_RELU, ACTIVATION_EXP, mlQuantizationData_t, mlShape_t, mlTensor_t)

lib = _abi.load()

_DTYPES = {
    torch.float16: _abi.DTYPE_FLOAT16, torch.float32: _abi.DTYPE_FLOAT32, torch.float64: _abi.DTYPE_FLOAT64,
    torch.uint8: _abi.DTYPE_UINT8, torch.int8: _abi.DTYPE_INT8, torch.int16: _abi.DTYPE_INT16, torch.int32: _abi.DTYPE_INT32,
}
ACTIVATIONS = {"linear": ACTIVATION_LINEAR, "sigmoid": ACTIVATION_SIGMOID, "tanh": ACTIVATION_TANH, "relu": ACTIVATION_RELU,
               "leaky_relu": ACTIVATION_LEAKY_RELU, "exp": ACTIVATION_EXP}


class BackendError(RuntimeError):
    pass


def dtype_of(t):
    return _DTYPES[t.dtype]


def shape_of(t_or_dims):
    dims = list(t_or_dims.shape) if isinstance(t_or_dims, torch.Tensor) else list(t_or_dims)
    s = mlShape_t()
    s.rank = len(dims)
    for i, d in enumerate(dims):
        s.dim[i] = int(d)
    return s


def _check_device(t, ctx):
    """A tensor handed to a context must live on that context's device: a kernel launched on one GPU's stream with another GPU's
    pointer faults (or, with peer access, silently reads across NVLink).  Raised here, on the host, before any launch."""
    if ctx is not None and t.is_cuda and t.device.index != ctx.device_index:
        raise BackendError("tensor on cuda:%d passed to a context of cuda:%d" % (t.device.index, ctx.device_index))


def desc(t, ctx=None):
    """mlTensor_t for a dense torch tensor; None gives the empty descriptor (null data, rank 0)."""
    d = mlTensor_t()
    if t is None:
        d.data = None
        d.dtype = _abi.DTYPE_UNKNOWN
        d.rank = 0
        return d
    assert t.is_contiguous(), "the backend ABI addresses dense row-major tensors only"
    _check_device(t, ctx)
    d.data = t.data_ptr()
    d.dtype = dtype_of(t)
    d.rank = t.dim()
    for i, n in enumerate(t.shape):
        d.dim[i] = int(n)
    return d


def ptr(t, ctx=None):
    if t is None:
        return None
    _check_device(t, ctx)
    return ctypes.c_void_p(t.data_ptr())


def act_code(act):
    return ACTIVATIONS[act] if isinstance(act, str) else int(act)


class Context:
    """ml::Context on Device::cuda(index) (reference: src/core/Context.cpp:20-60)."""

    def __init__(self, device_index=0):
        n = lib.cuda_get_number_of_devices()
        if n == 0:
            raise BackendError("no CUDA device: libminml_b200 has no CPU fallback")
        self.device_index = device_index
        self.device = torch.device("cuda", device_index)  # where tensors handed to this context must live
        self.handle = lib.cuda_create_context(device_index)
        if not self.handle:
            raise BackendError("cuda_create_context failed: %s" % _last_error(None))

    def synchronize(self):
        lib.cuda_synchronize_with_context(self.handle)
        self.check()

    def check(self):
        msg = _last_error(self.handle)
        if msg:
            lib.mb200_clear_last_error(self.handle)
            raise BackendError(msg)

    def set_fusion(self, enabled):
        lib.mb200_set_fusion(self.handle, 1 if enabled else 0)

    def enable_tf32(self, enabled):
        """ml::Context::enableTF32: fp32 matrix products may then run on the tensor cores in TF32 (off by default, as in the reference)."""
        lib.cuda_enable_tf32(self.handle, bool(enabled))

    def torch_stream(self):
        """The context's own CUDA stream as a torch stream object (for graph capture, or for queuing torch work behind backend calls)."""
        lib.mb200_get_stream.restype = ctypes.c_void_p
        return torch.cuda.ExternalStream(int(lib.mb200_get_stream(self.handle)), device=torch.device("cuda", self.device_index))

    def hold_stream(self, milliseconds):
        """Queues a busy-wait of about `milliseconds` on the context's stream, so that launches issued right after it pile up behind
        it and then run back to back: device time of short kernels can then be measured without the host's launch pace in it."""
        with torch.cuda.stream(self.torch_stream()):
            torch.cuda._sleep(int(milliseconds * 1.5e6))

    def wait_for_torch(self):
        """Orders this context's stream after work torch has queued on its current stream."""
        torch.cuda.current_stream().synchronize()

    def close(self):
        if self.handle:
            lib.cuda_destroy_context(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _last_error(handle):
    msg = lib.mb200_get_last_error(handle)
    return msg.decode() if msg else None


def set_attention_kernel(kernel):
    """Attention kernel for fp16, head dimension 32.  0: by shape (default: the persistent tcgen05 kernel up to 256 tokens, else the
    warp-level kernel); 1: tcgen05 wherever possible; 2: the one-CTA-per-head tcgen05 kernel; 3: never tcgen05."""
    lib.mb200_set_attention_kernel(int(kernel))


def launch_count():
    return int(lib.mb200_get_launch_count())


# ---------------------------------------------------------------------------------------------- Winograd
def winogradWeightTransform(ctx, weight, matrices, invert=False, tile_size=None):
    tile = tile_size if tile_size is not None else _tile_size(matrices, weight.shape[1])
    lib.cuda_winograd_weight_transform(ctx.handle, tile, desc(weight, ctx), desc(matrices, ctx), bool(invert))
    ctx.check()


def winogradInputTransform(ctx, weight_shape, x, matrices, tile_size=None):
    tile = tile_size if tile_size is not None else _tile_size(matrices, weight_shape[1])
    lib.cuda_winograd_input_transform(ctx.handle, tile, desc(x, ctx), desc(matrices, ctx))
    ctx.check()


def winogradOutputTransform(ctx, weight_shape, matrices, output, bias=None, ext=None, act="linear", tile_size=None):
    tile = tile_size if tile_size is not None else _tile_size(matrices, weight_shape[1])
    lib.cuda_winograd_output_transform(ctx.handle, tile, desc(matrices, ctx), desc(bias, ctx), desc(ext, ctx), desc(output, ctx), act_code(act))
    ctx.check()


def _tile_size(matrices, kernel):
    # reference: math.cpp:107-118 -- tile = sqrt(matrices.dim[0]) - (kernel - 1)
    p = int(round(matrices.shape[0] ** 0.5))
    return p - (kernel - 1)


# ---------------------------------------------------------------------------------------------- GEMM
def gemm(ctx, opA, A, opB, B, C, alpha=1.0, beta=0.0):
    lib.cuda_gemm_v2(ctx.handle, opA.encode(), opB.encode(), alpha, desc(A, ctx), desc(B, ctx), beta, desc(C, ctx))
    ctx.check()


def gemmBatched(ctx, opA, A, opB, B, C, alpha=1.0, beta=0.0):
    lib.cuda_gemm_batched_v2(ctx.handle, opA.encode(), opB.encode(), alpha, desc(A, ctx), desc(B, ctx), beta, desc(C, ctx))
    ctx.check()


def gemm_legacy(ctx, opA, A, opB, B, C, alpha=1.0, beta=0.0, batched=False):
    fn = lib.cuda_gemm_batched if batched else lib.cuda_gemm
    fn(ctx.handle, dtype_of(C), shape_of(C), ptr(C, ctx), shape_of(A), ptr(A, ctx), shape_of(B), ptr(B, ctx), opA.encode(), opB.encode(), alpha, beta)
    ctx.check()


def gemm_ex(ctx, D, alpha, opA, A, opB, B, beta, C, bias, act):
    lib.cuda_gemm_ex(ctx.handle, dtype_of(D), shape_of(D), ptr(D, ctx), alpha, opA.encode(), shape_of(A), ptr(A, ctx), opB.encode(), shape_of(B), ptr(B, ctx),
                     beta, shape_of(C if C is not None else D), ptr(C, ctx), ptr(bias, ctx), act_code(act))
    ctx.check()


# ---------------------------------------------------------------------------------------------- fused convolution
def convolutionImplicitGemmForward(ctx, x, weights, output, bias=None, add=None, act="linear"):
    lib.cuda_convolution_implicit_gemm_forward(ctx.handle, dtype_of(x), shape_of(x), shape_of(weights), ptr(x, ctx), ptr(weights, ctx), ptr(output, ctx),
                                               ptr(bias, ctx), ptr(add, ctx), act_code(act))
    ctx.check()


# ---------------------------------------------------------------------------------------------- elementwise
def addBiasAct(ctx, x, bias, y, act="linear", alpha=1.0, beta=0.0):
    lib.cuda_add_bias_act(ctx.handle, alpha, desc(x, ctx), desc(bias, ctx), beta, desc(y, ctx), act_code(act))
    ctx.check()


def activationForward(ctx, x, y, act, alpha=1.0, beta=0.0):
    lib.cuda_activation_forward(ctx.handle, alpha, desc(x, ctx), beta, desc(y, ctx), act_code(act))
    ctx.check()


def addTensors(ctx, y, alpha1=0.0, x1=None, alpha2=0.0, x2=None, alpha3=0.0, x3=None, beta=0.0):
    lib.cuda_add_tensors(ctx.handle, alpha1, desc(x1, ctx), alpha2, desc(x2, ctx), alpha3, desc(x3, ctx), beta, desc(y, ctx))
    ctx.check()


def multiplyTensors(ctx, dst, src1, src2):
    """ml::multiplyTensors: dst = src1 * src2 element by element (the Multiply layer)."""
    lib.cuda_multiply_tensors(ctx.handle, dtype_of(dst), shape_of(dst), ptr(dst, ctx), ptr(src1, ctx), ptr(src2, ctx))
    ctx.check()


def globalAveragePoolingForward(ctx, x, y, alpha=1.0, beta=0.0):
    lib.cuda_global_average_pooling_forward(ctx.handle, alpha, desc(x, ctx), beta, desc(y, ctx))
    ctx.check()


def softmaxForward(ctx, x, y):
    lib.cuda_softmax_forward(ctx.handle, dtype_of(x), shape_of(x), ptr(y, ctx), ptr(x, ctx))
    ctx.check()


def unpackInput(ctx, packed, dst):
    lib.cuda_unpack_input(ctx.handle, shape_of(dst), dtype_of(dst), ptr(dst, ctx), ptr(packed, ctx))
    ctx.check()


def convertType(ctx, dst, src):
    lib.cuda_convert_type(ctx.handle, ptr(dst, ctx), dtype_of(dst), ptr(src, ctx), dtype_of(src), src.numel())
    ctx.check()


def transpose_021(ctx, src, dst):
    lib.cuda_transpose_021(ctx.handle, dtype_of(src), shape_of(src), ptr(src, ctx), ptr(dst, ctx))
    ctx.check()


# ---------------------------------------------------------------------------------------------- norms, attention
def layernormForward(ctx, x, y, weights, bias, ext=None):
    lib.cuda_layernorm_forward(ctx.handle, shape_of(x), dtype_of(x), ptr(x, ctx), ptr(y, ctx), ptr(weights, ctx), ptr(bias, ctx), ptr(ext, ctx))
    ctx.check()


def rmsnormForward(ctx, x, y, weights=None):
    """ml::rmsnormForward (src/core/math.cpp): y = weights * x / (1e-6 + rms(x)) over the last axis; weights may be None."""
    lib.cuda_rmsnorm_forward(ctx.handle, shape_of(x), dtype_of(x), ptr(x, ctx), ptr(y, ctx), ptr(weights, ctx))
    ctx.check()


def spaceToDepth(ctx, x, y):
    """ml::spaceToDepth: [b, h, w, c] -> [b, ceil(h/p), ceil(w/q), p*q*c]; the patch size follows from the two shapes."""
    lib.cuda_space_to_depth(ctx.handle, dtype_of(x), shape_of(x), ptr(x, ctx), shape_of(y), ptr(y, ctx))
    ctx.check()


def depthToSpace(ctx, x, y):
    """ml::depthToSpace: the inverse of spaceToDepth."""
    lib.cuda_depth_to_space(ctx.handle, dtype_of(x), shape_of(x), ptr(x, ctx), shape_of(y), ptr(y, ctx))
    ctx.check()


def multiHeadAttentionGetWorkspaceSize(x_shape, weights_shape, num_heads, training=False):
    return lib.cuda_multi_head_attention_get_workspace_size(shape_of(x_shape), shape_of(weights_shape), num_heads, training)


def multiHeadAttentionForward(ctx, x, y, weights, num_heads, symmetric=False, workspace=None):
    wshape = shape_of(weights) if weights is not None else shape_of([])
    lib.cuda_multi_head_attention_forward(ctx.handle, shape_of(x), wshape, shape_of([]), dtype_of(x), ptr(x, ctx), ptr(y, ctx), ptr(weights, ctx), None,
                                          ptr(workspace, ctx), None, num_heads, bool(symmetric))
    ctx.check()


# ---------------------------------------------------------------------------------------------- int8
def qdata(scale, shift):
    q = mlQuantizationData_t()
    q.scale = float(scale)
    q.shift = float(shift)
    return q


def im2row(ctx, x, output, kernel_size, invert=False, padding=None):
    """`padding` is a host scalar of x's dtype (numpy scalar or 0-d torch CPU tensor) or None for zero."""
    pad_ptr = None
    keep = None
    if padding is not None:
        keep = torch.as_tensor(padding, dtype=x.dtype, device="cpu").reshape(1).contiguous()
        pad_ptr = ctypes.c_void_p(keep.data_ptr())
    lib.cuda_im2row(ctx.handle, dtype_of(x), shape_of(x), ptr(output, ctx), ptr(x, ctx), kernel_size, bool(invert), pad_ptr)
    ctx.check()
    del keep


def quantized_scale_shift_act(ctx, output, output_qd, acc_i32, scales, bias, act="linear", ext=None, ext_qd=(1.0, 0.0)):
    lib.cuda_quantized_scale_shift_act(ctx.handle, dtype_of(output), shape_of(output), ptr(output, ctx), qdata(*output_qd), ptr(acc_i32, ctx), ptr(scales, ctx),
                                       ptr(bias, ctx), act_code(act), ptr(ext, ctx), qdata(*ext_qd))
    ctx.check()


def dequantize(ctx, src_i8, dst, scale, shift):
    lib.cuda_dequantize(ctx.handle, dtype_of(dst), ptr(src_i8, ctx), ptr(dst, ctx), src_i8.numel(), float(scale), float(shift))
    ctx.check()


# ---------------------------------------------------------------------------------------------- layers next to the convolution path
def batchnormInference(ctx, x, y, weights, bias, avg_var, act="linear", alpha=1.0, beta=0.0):
    """ml::batchnormInference (src/core/math.cpp): avg_var is fp32 [2, channels] = (mean, variance); weights / bias may be None."""
    lib.cuda_batchnorm_inference(ctx.handle, alpha, desc(x, ctx), desc(weights, ctx), desc(bias, ctx), desc(avg_var, ctx), beta, desc(y, ctx), act_code(act))
    ctx.check()


def foldBatchnorm(ctx, layer_weights, layer_bias, bn_weights, bn_bias, bn_avg_var):
    lib.cuda_fold_batchnorm(ctx.handle, desc(layer_weights, ctx), desc(layer_bias, ctx), desc(bn_weights, ctx), desc(bn_bias, ctx), desc(bn_avg_var, ctx))
    ctx.check()


def depthwiseConvForward(ctx, x, w, y, bias=None, alpha=1.0, beta=0.0):
    lib.cuda_depthwise_conv_forward(ctx.handle, alpha, desc(x, ctx), desc(w, ctx), desc(bias, ctx), beta, desc(y, ctx))
    ctx.check()


def quantized_depthwise_conv_forward(ctx, x, w, scales, bias, y, output_qd, padding_value=0):
    lib.cuda_quantized_depthwise_conv_forward(ctx.handle, dtype_of(x), shape_of(x), shape_of(w), ptr(x, ctx), ptr(w, ctx), ptr(scales, ctx), ptr(bias, ctx), ptr(y, ctx),
                                              qdata(*output_qd), int(padding_value))
    ctx.check()


def channelScalingForward(ctx, x, scales, y, alpha=1.0, beta=0.0):
    lib.cuda_channel_scaling_forward(ctx.handle, alpha, desc(x, ctx), desc(scales, ctx), beta, desc(y, ctx))
    ctx.check()


# ---------------------------------------------------------------------------------------------- backward pass of the Winograd convolution
def winogradGradientTransform(ctx, weight_shape, dy, matrices, tile_size=None):
    tile = tile_size if tile_size is not None else _tile_size(matrices, weight_shape[1])
    lib.cuda_winograd_gradient_transform(ctx.handle, tile, desc(dy, ctx), desc(matrices, ctx))
    ctx.check()


def winogradUpdateTransform(ctx, matrices, dw, tile_size=None):
    tile = tile_size if tile_size is not None else _tile_size(matrices, dw.shape[1])
    lib.cuda_winograd_update_transform(ctx.handle, tile, desc(matrices, ctx), desc(dw, ctx))
    ctx.check()


def fusedBiasActCopyBackward(ctx, dy, y, dx=None, db=None, act="linear", beta_dx=0.0, beta_db=0.0):
    """ml::fusedBiasActCopyBackward (src/core/math.cpp:1046-1063): dy is updated in place when act is not linear."""
    lib.cuda_fused_act_bias_copy_backward(ctx.handle, desc(dy, ctx), desc(y, ctx), beta_dx, desc(dx, ctx), beta_db, desc(db, ctx), act_code(act))
    ctx.check()


def activationBackward(ctx, dy, y, dx, act="linear", alpha=1.0, beta=0.0):
    lib.cuda_activation_backward(ctx.handle, alpha, desc(dy, ctx), desc(y, ctx), beta, desc(dx, ctx), act_code(act))
    ctx.check()
