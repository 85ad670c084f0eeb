/*
 * conv.cu -- cuda_convolution_implicit_gemm_forward: y = act(conv(x, w) + bias + add) in one call, on raw weights
 * w [cout, k, k, cin].
 *
 * In the reference this entry is backed by cuDNN / cublasLt when built with USE_CUDNN and is an empty function
 * otherwise (src/backend/cuda/cudnn_math.cpp:374-476,691-694).  Here:
 *   k = 1            one tensor-core GEMM over [b*h*w, cin] with bias, residual and activation in its epilogue;
 *   k = 3, fp16      the fused tcgen05 implicit-GEMM kernel (conv_igemm.cu) when its shape rules hold,
 *   k = 3 otherwise  F(4x4,3x3) Winograd through the context's scratch workspace (weight transform, input transform,
 *                    36 batched products, output transform with bias / residual / activation).
 */
#include "common.cuh"
#include "conv.cuh"
#include "winograd.cuh"

using namespace mb200;

extern "C"
{
	void cuda_convolution_implicit_gemm_forward(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape,
			const void *input, const void *weights, void *output, const void *bias, const void *add, mlActivationType_t act)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_convolution_implicit_gemm_forward: null context");
		if (volume(input_shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, input_shape.rank == 4 && weights_shape.rank == 4, "cuda_convolution_implicit_gemm_forward: rank-4 shapes expected");
		MB200_REQUIRE(context, input != nullptr && weights != nullptr && output != nullptr, "cuda_convolution_implicit_gemm_forward: null pointer");
		MB200_REQUIRE(context, dtype == DTYPE_FLOAT16 || dtype == DTYPE_FLOAT32, "cuda_convolution_implicit_gemm_forward: dtype %d not supported",
				static_cast<int>(dtype));
		const int batch = input_shape.dim[0], height = input_shape.dim[1], width = input_shape.dim[2], cin = input_shape.dim[3];
		const int cout = weights_shape.dim[0], kh = weights_shape.dim[1], kw = weights_shape.dim[2];
		MB200_REQUIRE(context, weights_shape.dim[3] == cin, "cuda_convolution_implicit_gemm_forward: weights expect %d input channels, input has %d",
				weights_shape.dim[3], cin);
		MB200_REQUIRE(context, kh == kw && (kh == 1 || kh == 3), "cuda_convolution_implicit_gemm_forward: %d x %d kernels not supported (1x1, 3x3)",
				kh, kw);
		if (batch == 0 || height == 0 || width == 0)
			return;
		flush_pending(context);
		const mlShape_t out_shape = make_shape( { batch, height, width, cout });
		if (kh == 1)
		{
			const mlShape_t a = make_shape( { batch * height * width, cin });
			const mlShape_t b = make_shape( { cout, cin });
			const mlShape_t d = make_shape( { batch * height * width, cout });
			cuda_gemm_ex(context, dtype, d, output, 1.0f, 'n', a, input, 't', b, weights, (add != nullptr) ? 1.0f : 0.0f, d, add, bias, act);
			return;
		}
		const mlTensor_t x = make_tensor(input, dtype, input_shape);
		const mlTensor_t w = make_tensor(weights, dtype, weights_shape);
		const mlTensor_t y = make_tensor(output, dtype, out_shape);
		// in place (y overlapping x) only the Winograd path below is correct: V is complete before y is written, whereas the fused
		// kernel reads the 3x3 neighbourhood of positions that other CTAs are writing
		const bool in_place = ranges_overlap(input, volume(x) * size_of(dtype), output, volume(y) * size_of(dtype));
		if (!in_place && conv_fused_supported(context, x, w, y, act))
		{
			conv_fused_run(context, x, w, bias, add, y, act, false);
			return;
		}
		/* Winograd through the scratch workspace: U | V | M */
		const int tiles = batch * ((height + 3) / 4) * ((width + 3) / 4);
		const size_t elem = size_of(dtype);
		const size_t u_bytes = (static_cast<size_t>(36) * cout * cin * elem + 255) / 256 * 256;
		const size_t v_bytes = (static_cast<size_t>(36) * tiles * cin * elem + 255) / 256 * 256;
		const size_t m_bytes = (static_cast<size_t>(36) * tiles * cout * elem + 255) / 256 * 256;
		uint8_t *ws = reinterpret_cast<uint8_t*>(get_workspace(context, u_bytes + v_bytes + m_bytes));
		if (ws == nullptr)
			return;
		const mlTensor_t u = make_tensor(ws, dtype, make_shape( { 36, cout, cin }));
		const mlTensor_t v = make_tensor(ws + u_bytes, dtype, make_shape( { 36, tiles, cin }));
		const mlTensor_t m = make_tensor(ws + u_bytes + v_bytes, dtype, make_shape( { 36, tiles, cout }));
		const mlTensor_t bias_t = make_tensor(bias, dtype, make_shape( { cout }));
		const mlTensor_t add_t = make_tensor(add, dtype, out_shape);
		Context *c = get(context);
		const bool fusion = c->fusion;
		c->fusion = false; // the three steps below must run eagerly
		winograd_weight_transform_eager(context, 4, w, u, false);
		winograd_input_transform_eager(context, 4, x, v);
		cuda_gemm_batched_v2(context, 'n', 't', 1.0f, v, u, 0.0f, m);
		winograd_output_transform_eager(context, 4, m, bias_t, add_t, y, act);
		c->fusion = fusion;
	}
}
