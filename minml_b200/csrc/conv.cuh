/*
 * conv.cuh -- internal interface of the fused convolution kernels (conv_igemm.cu).
 */
#pragma once

#include "common.cuh"

namespace mb200
{
	/* True when an input tensor can be consumed by the fused 3x3 kernel (dtype, channel count, alignment). */
	bool conv_fused_input_supported(mlContext_t ctx, const mlTensor_t &x);
	/* True when a raw weight tensor [cout, 3, 3, cin] can be the B operand of the fused kernel (dtype, channel count). */
	bool conv_fused_weights_supported(const mlTensor_t &w);
	/* True when y = act(conv3x3(x, w) + bias + ext) can run as the fused kernel. */
	bool conv_fused_supported(mlContext_t ctx, const mlTensor_t &x, const mlTensor_t &w, const mlTensor_t &y, mlActivationType_t act);
	/* `prepared` = w.data points at what conv_fused_prepare_weights wrote (the library's snapshot), not at the host's raw tensor */
	bool conv_fused_run(mlContext_t ctx, const mlTensor_t &x, const mlTensor_t &w, const void *bias, const void *ext, const mlTensor_t &y,
			mlActivationType_t act, bool prepared);
	/* The form in which the fused kernel wants a layer's weights kept: a plain copy for fp16, two planes (w rounded to TF32, and the
	 * remainder) for fp32.  `prepared` must hold conv_fused_weight_bytes(w); the work is queued on the context's stream. */
	/* conv_slab.cu: the variant for fp16 layers of up to 128 channels (input band resident in shared memory, shifted operand descriptors) */
	bool conv_slab_supported(const mlTensor_t &x, const mlTensor_t &w, const mlTensor_t &y);
	bool conv_slab_run(mlContext_t ctx, const mlTensor_t &x, const mlTensor_t &w, const void *bias, const void *ext, const mlTensor_t &y,
			mlActivationType_t act);
	/* Drops what the library derived from int8 weights lying in [ptr, ptr + bytes): they are being freed or overwritten. */
	void conv_forget_range(const void *ptr, size_t bytes);
	size_t conv_fused_weight_bytes(const mlTensor_t &w);
	bool conv_fused_prepare_weights(mlContext_t ctx, const mlTensor_t &w, void *prepared);
} /* namespace mb200 */

namespace mb200
{
	/* Hooks of the deferred int8 sequence im2row -> int8 GEMM -> scale_shift_act (src/layers/Conv2D.cpp:214-239).
	 * Each returns true when it consumed the call. */
	bool im2row_defer(mlContext_t ctx, mlDataType_t dtype, const mlShape_t &input_shape, void *output, const void *input, int kernel_size,
			bool invert, const void *padding);
	bool int8_gemm_defer(mlContext_t ctx, char opA, char opB, const mlTensor_t &A, const mlTensor_t &B, const mlTensor_t &C);
	void flush_pending_int8(mlContext_t ctx);
	bool requant_complete_fused(mlContext_t ctx, mlDataType_t dtype, const mlShape_t &shape, void *output, mlQuantizationData_t output_qd,
			const void *input, const void *scales, const void *bias, mlActivationType_t act, const void *ext, mlQuantizationData_t ext_qd);
} /* namespace mb200 */
