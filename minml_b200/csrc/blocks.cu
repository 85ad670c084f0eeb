/*
 * blocks.cu -- the layers either side of the 1x1 GEMMs in minml's current architectures (depthwise 7x7 convolution, two
 * 1x1 convolutions, squeeze-and-excitation), and batch normalisation as it exists at inference time:
 *
 *   cuda_batchnorm_inference       y = alpha * act(x * scale[c] + shift[c]) + beta * y,   scale = gamma / sqrt(var + 1e-6),
 *                                  shift = beta_bn - mean * scale      (src/backend/cuda/kernels/batchnorm.cu:58-100,358-398)
 *   cuda_fold_batchnorm            the same scale / shift folded into a layer's weights and bias, per output channel for
 *                                  [cout, ...] weights, per channel for depthwise [k, k, c] weights (batchnorm.cu:400-438,606-657)
 *   cuda_depthwise_conv_forward    y = alpha * dwconv(x, w) + b + beta * y, x [b,h,w,c], w [k,k,c], k in {3, 5, 7}, "same" padding
 *                                  (src/backend/cuda/kernels/depthwise_conv.cu:110-182,285-324,381-403)
 *   cuda_quantized_depthwise_conv_forward   int8: acc = sum q_w * q_x (padding with the quantised zero), x = acc * scale[c] + bias[c],
 *                                  requantised.  Follows the host's CPU loop (src/layers/DepthwiseConv2D.cpp:104-140): the accumulator
 *                                  starts at zero.  (The reference's CUDA kernel seeds it with the truncated bias, quantized.cu:185,
 *                                  which its own CPU path does not do.)
 *   cuda_channel_scaling_forward   y = alpha * x * s[b, c] + beta * y, x [b,h,w,c], s [b,c]   (global_pooling.cu:99-123,360-407)
 *
 * All of them are HBM-bound: every thread owns a 16-byte group of channels (8 halves / 4 floats / 16 int8), so a warp reads and
 * writes whole 128-byte lines along the channel axis; accumulation is fp32 (the reference accumulates fp16 depthwise convolutions
 * in half2).
 */
#include "common.cuh"

#include <cuda_fp16.h>

#include <algorithm>

using namespace mb200;

namespace
{
	template<typename T, int VEC>
	struct Pack;
	template<>
	struct Pack<__half, 8>
	{
			uint4 raw;
			__device__ void load(const __half *p) { raw = *reinterpret_cast<const uint4*>(p); }
			__device__ void store(__half *p) const { *reinterpret_cast<uint4*>(p) = raw; }
			__device__ float get(int i) const { return __half2float(reinterpret_cast<const __half*>(&raw)[i]); }
			__device__ void set(int i, float v) { reinterpret_cast<__half*>(&raw)[i] = __float2half_rn(v); }
	};
	template<>
	struct Pack<float, 4>
	{
			float4 raw;
			__device__ void load(const float *p) { raw = *reinterpret_cast<const float4*>(p); }
			__device__ void store(float *p) const { *reinterpret_cast<float4*>(p) = raw; }
			__device__ float get(int i) const { return reinterpret_cast<const float*>(&raw)[i]; }
			__device__ void set(int i, float v) { reinterpret_cast<float*>(&raw)[i] = v; }
	};
	template<typename T>
	struct Pack<T, 1>
	{
			T raw;
			__device__ void load(const T *p) { raw = *p; }
			__device__ void store(T *p) const { *p = raw; }
			__device__ float get(int) const { return static_cast<float>(raw); }
			__device__ void set(int, float v) { raw = static_cast<T>(v); }
	};

	inline int grid_for(long long work_items, int block, int sm_count)
	{
		const long long blocks = (work_items + block - 1) / block;
		return static_cast<int>(std::max<long long>(1, std::min<long long>(blocks, static_cast<long long>(sm_count) * 16)));
	}
	__device__ __forceinline__ float to_float(float v) { return v; }
	__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

	/* ------------------------------------------------------------------------------------------------ batch norm */
	template<typename T, int VEC>
	__global__ void kernel_batchnorm_inference(T *y, const T *x, const T *gamma, const T *beta_bn, const float *avg_var, long long rows,
			int channels, float alpha, float beta, int act)
	{
		const int groups = channels / VEC;
		const long long total = rows * groups;
		for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const int c0 = static_cast<int>(i % groups) * VEC;
			const long long off = (i / groups) * channels + c0;
			Pack<T, VEC> in, out;
			in.load(x + off);
			if (beta != 0.0f)
				out.load(y + off);
#pragma unroll
			for (int k = 0; k < VEC; k++)
			{
				const int c = c0 + k;
				const float g = (gamma != nullptr) ? to_float(gamma[c]) : 1.0f;
				const float b = (beta_bn != nullptr) ? to_float(beta_bn[c]) : 0.0f;
				const float scale = g / sqrtf(avg_var[channels + c] + 1.0e-6f);
				const float shift = -avg_var[c] * scale + b;
				float v = apply_activation(in.get(k) * scale + shift, act) * alpha;
				if (beta != 0.0f)
					v += beta * out.get(k);
				out.set(k, v);
			}
			out.store(y + off);
		}
	}
	/* weights viewed as [outer, inner]; channel = row (per_row) or column.  One thread per element; the bias is updated by the
	 * threads of the first column / row. */
	template<typename T>
	__global__ void kernel_fold_batchnorm(T *weights, T *bias, const T *gamma, const T *beta_bn, const float *avg_var, int outer, int inner,
			bool per_row)
	{
		const int channels = per_row ? outer : inner;
		const long long total = static_cast<long long>(outer) * inner;
		for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const int r = static_cast<int>(i / inner), col = static_cast<int>(i % inner);
			const int c = per_row ? r : col;
			const float g = (gamma != nullptr) ? to_float(gamma[c]) : 1.0f;
			const float scale = g / sqrtf(avg_var[channels + c] + 1.0e-6f);
			weights[i] = static_cast<T>(to_float(weights[i]) * scale);
			if ((per_row ? col : r) == 0 && bias != nullptr)
			{
				const float b = (beta_bn != nullptr) ? to_float(beta_bn[c]) : 0.0f;
				const float shift = -avg_var[c] * scale + b;
				bias[c] = static_cast<T>(to_float(bias[c]) * scale + shift);
			}
		}
	}

	/* ------------------------------------------------------------------------------------------------ channel scaling */
	template<typename T, int VEC>
	__global__ void kernel_channel_scaling(T *y, const T *x, const T *scales, int hw, int channels, float alpha, float beta)
	{
		const int groups = channels / VEC;
		const int b = blockIdx.y;
		const long long total = static_cast<long long>(hw) * groups;
		for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const int c0 = static_cast<int>(i % groups) * VEC;
			const long long off = (static_cast<long long>(b) * hw + i / groups) * channels + c0;
			Pack<T, VEC> in, out, s;
			in.load(x + off);
			s.load(scales + static_cast<long long>(b) * channels + c0);
			if (beta != 0.0f)
				out.load(y + off);
#pragma unroll
			for (int k = 0; k < VEC; k++)
			{
				float v = in.get(k) * s.get(k) * alpha;
				if (beta != 0.0f)
					v += beta * out.get(k);
				out.set(k, v);
			}
			out.store(y + off);
		}
	}

	/* ------------------------------------------------------------------------------------------------ depthwise convolution */
	/* grid (ceil(h / ROWS), batch), block (channel groups, ROWS): a thread owns one output row of one group of VEC channels and
	 * walks along it.  Input column ww contributes to the K output columns ww - PAD .. ww + PAD, whose partial sums sit in K
	 * register accumulators that shift by one per step: every input element is loaded once per filter row (K times in all, not
	 * K x K), the filter taps come from L1 (K x K x channels elements, read by every thread of the CTA). */
	template<typename T, int VEC, int K>
	__global__ void kernel_depthwise_conv(T *y, const T *x, const T *w, const T *bias, int height, int width, int channels, float alpha,
			float beta)
	{
		constexpr int PAD = (K - 1) / 2;
		const int groups = channels / VEC;
		const int h = blockIdx.x * blockDim.y + threadIdx.y;
		const int b = blockIdx.y;
		if (h >= height)
			return;
		for (int g = threadIdx.x; g < groups; g += blockDim.x)
		{
			const int c0 = g * VEC;
			float bv[VEC];
#pragma unroll
			for (int k = 0; k < VEC; k++)
				bv[k] = (bias != nullptr) ? to_float(bias[c0 + k]) : 0.0f;
			const T *xb = x + static_cast<long long>(b) * height * width * channels + c0;
			T *yb = y + static_cast<long long>(b) * height * width * channels + c0;
			const T *wb = w + c0;
			float acc[K][VEC]; // acc[s]: output column ww - PAD + s
#pragma unroll
			for (int s = 0; s < K; s++)
#pragma unroll
				for (int k = 0; k < VEC; k++)
					acc[s][k] = 0.0f;
			for (int ww = 0; ww < width + PAD; ww++)
			{
				if (ww < width)
				{
#pragma unroll
					for (int i = 0; i < K; i++)
					{
						const int hh = h + i - PAD;
						if (hh < 0 || hh >= height)
							continue;
						Pack<T, VEC> in;
						in.load(xb + (static_cast<long long>(hh) * width + ww) * channels);
#pragma unroll
						for (int s = 0; s < K; s++)
						{ // output ww - PAD + s sees this input through filter column K - 1 - s
							Pack<T, VEC> f;
							f.load(wb + static_cast<long long>(i * K + (K - 1 - s)) * channels);
#pragma unroll
							for (int k = 0; k < VEC; k++)
								acc[s][k] += in.get(k) * f.get(k);
						}
					}
				}
				const int col = ww - PAD; // complete: no later input column reaches it
				if (col >= 0)
				{
					const long long off = (static_cast<long long>(h) * width + col) * channels;
					Pack<T, VEC> out;
					if (beta != 0.0f)
						out.load(yb + off);
#pragma unroll
					for (int k = 0; k < VEC; k++)
					{
						float v = acc[0][k] * alpha + bv[k];
						if (beta != 0.0f)
							v += beta * out.get(k);
						out.set(k, v);
					}
					out.store(yb + off);
				}
#pragma unroll
				for (int s = 0; s + 1 < K; s++)
#pragma unroll
					for (int k = 0; k < VEC; k++)
						acc[s][k] = acc[s + 1][k];
#pragma unroll
				for (int k = 0; k < VEC; k++)
					acc[K - 1][k] = 0.0f;
			}
		}
	}
	/* int8: one thread per (row, channel); channels are consecutive across the threads of a warp (coalesced byte accesses). */
	template<int K>
	__global__ void kernel_depthwise_conv_int8(int8_t *y, const int8_t *x, const int8_t *w, const float *scales, const float *bias, int height,
			int width, int channels, float inv_scale, float inv_shift, int padding_value)
	{
		constexpr int PAD = (K - 1) / 2;
		const int h = blockIdx.x * blockDim.y + threadIdx.y;
		const int b = blockIdx.y;
		if (h >= height)
			return;
		for (int c = threadIdx.x; c < channels; c += blockDim.x)
		{
			int filt[K * K];
#pragma unroll
			for (int t = 0; t < K * K; t++)
				filt[t] = w[static_cast<long long>(t) * channels + c];
			const float scale = (scales != nullptr) ? scales[c] : 1.0f;
			const float shift = (bias != nullptr) ? bias[c] : 0.0f;
			const int8_t *xb = x + static_cast<long long>(b) * height * width * channels + c;
			int8_t *yb = y + static_cast<long long>(b) * height * width * channels + c;
			for (int col = 0; col < width; col++)
			{
				int acc = 0;
#pragma unroll
				for (int i = 0; i < K; i++)
				{
					const int hh = h + i - PAD;
#pragma unroll
					for (int j = 0; j < K; j++)
					{
						const int ww = col + j - PAD;
						const bool inside = hh >= 0 && hh < height && ww >= 0 && ww < width;
						const int v = inside ? static_cast<int>(xb[(static_cast<long long>(hh) * width + ww) * channels]) : padding_value;
						acc += filt[i * K + j] * v;
					}
				}
				const float t = __fadd_rn(__fmul_rn(static_cast<float>(acc), scale), shift);
				const float q = fmaxf(-128.0f, fminf(127.0f, roundf(__fadd_rn(__fmul_rn(t, inv_scale), inv_shift))));
				yb[(static_cast<long long>(h) * width + col) * channels] = static_cast<int8_t>(q);
			}
		}
	}

	template<typename T, int VEC>
	void launch_depthwise(cudaStream_t stream, int k, const mlTensor_t &x, const mlTensor_t &w, const mlTensor_t &b, mlTensor_t &y, float alpha,
			float beta)
	{
		const int batch = x.dim[0], height = x.dim[1], width = x.dim[2], channels = x.dim[3];
		const int groups = channels / VEC;
		const int tx = std::min(groups, 64);
		const int rows = std::max(1, 256 / tx);
		const dim3 block(tx, rows);
		const dim3 grid(ceil_div(height, rows), batch);
		T *yp = reinterpret_cast<T*>(y.data);
		const T *xp = reinterpret_cast<const T*>(x.data), *wp = reinterpret_cast<const T*>(w.data), *bp = reinterpret_cast<const T*>(b.data);
		switch (k)
		{
			case 3:
				kernel_depthwise_conv<T, VEC, 3> <<<grid, block, 0, stream>>>(yp, xp, wp, bp, height, width, channels, alpha, beta);
				break;
			case 5:
				kernel_depthwise_conv<T, VEC, 5> <<<grid, block, 0, stream>>>(yp, xp, wp, bp, height, width, channels, alpha, beta);
				break;
			default:
				kernel_depthwise_conv<T, VEC, 7> <<<grid, block, 0, stream>>>(yp, xp, wp, bp, height, width, channels, alpha, beta);
				break;
		}
	}
}

extern "C"
{
	void cuda_batchnorm_inference(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b,
			const mlTensor_t avg_var, float beta, mlTensor_t y, mlActivationType_t act)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_batchnorm_inference: null context");
		MB200_REQUIRE(context, x.data != nullptr && y.data != nullptr && avg_var.data != nullptr, "cuda_batchnorm_inference: null tensor");
		MB200_REQUIRE(context, x.dtype == y.dtype && volume(x) == volume(y), "cuda_batchnorm_inference: x and y do not match");
		MB200_REQUIRE(context, avg_var.dtype == DTYPE_FLOAT32 && volume(avg_var) == 2LL * last_dim(x),
				"cuda_batchnorm_inference: avg_var must be fp32 [2, channels]");
		MB200_REQUIRE(context, (w.data == nullptr || (w.dtype == x.dtype && volume(w) == last_dim(x)))
				&& (b.data == nullptr || (b.dtype == x.dtype && volume(b) == last_dim(x))), "cuda_batchnorm_inference: weights / bias must be [channels] of x's type");
		flush_pending(context);
		const long long rows = volume_without_last_dim(x);
		const int channels = last_dim(x);
		if (rows == 0 || channels == 0)
			return;
		cudaStream_t stream = use_stream(context);
		const float *av = reinterpret_cast<const float*>(avg_var.data);
		const int sms = get(context)->sm_count;
		switch (x.dtype)
		{
			case DTYPE_FLOAT16:
			{
				__half *yp = reinterpret_cast<__half*>(y.data);
				const __half *xp = reinterpret_cast<const __half*>(x.data), *wp = reinterpret_cast<const __half*>(w.data),
						*bp = reinterpret_cast<const __half*>(b.data);
				if (channels % 8 == 0 && aligned_to(xp, 16) && aligned_to(yp, 16))
					kernel_batchnorm_inference<__half, 8> <<<grid_for(rows * (channels / 8), 256, sms), 256, 0, stream>>>(yp, xp, wp, bp, av, rows,
							channels, alpha, beta, act);
				else
					kernel_batchnorm_inference<__half, 1> <<<grid_for(rows * channels, 256, sms), 256, 0, stream>>>(yp, xp, wp, bp, av, rows, channels,
							alpha, beta, act);
				break;
			}
			case DTYPE_FLOAT32:
			{
				float *yp = reinterpret_cast<float*>(y.data);
				const float *xp = reinterpret_cast<const float*>(x.data), *wp = reinterpret_cast<const float*>(w.data),
						*bp = reinterpret_cast<const float*>(b.data);
				if (channels % 4 == 0 && aligned_to(xp, 16) && aligned_to(yp, 16))
					kernel_batchnorm_inference<float, 4> <<<grid_for(rows * (channels / 4), 256, sms), 256, 0, stream>>>(yp, xp, wp, bp, av, rows,
							channels, alpha, beta, act);
				else
					kernel_batchnorm_inference<float, 1> <<<grid_for(rows * channels, 256, sms), 256, 0, stream>>>(yp, xp, wp, bp, av, rows, channels,
							alpha, beta, act);
				break;
			}
			default:
				record_error(context, "cuda_batchnorm_inference: dtype %d not supported", static_cast<int>(x.dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_batchnorm_inference");
	}
	void cuda_fold_batchnorm(mlContext_t context, mlTensor_t layer_weights, mlTensor_t layer_bias, const mlTensor_t bn_weights,
			const mlTensor_t bn_bias, const mlTensor_t bn_avg_var)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_fold_batchnorm: null context");
		MB200_REQUIRE(context, layer_weights.data != nullptr && bn_avg_var.data != nullptr && layer_weights.rank >= 2,
				"cuda_fold_batchnorm: weights and statistics are required");
		MB200_REQUIRE(context, bn_avg_var.dtype == DTYPE_FLOAT32, "cuda_fold_batchnorm: statistics must be fp32");
		flush_pending(context);
		const bool per_row = layer_weights.rank != 3; // [k, k, c] is a depthwise filter: one channel per column
		const int outer = per_row ? layer_weights.dim[0] : static_cast<int>(volume_without_last_dim(layer_weights));
		const int inner = per_row ? static_cast<int>(volume(layer_weights) / std::max(1, layer_weights.dim[0])) : last_dim(layer_weights);
		const int channels = per_row ? outer : inner;
		MB200_REQUIRE(context, volume(bn_avg_var) == 2LL * channels, "cuda_fold_batchnorm: statistics must be [2, %d]", channels);
		MB200_REQUIRE(context, layer_bias.data == nullptr || (volume(layer_bias) == channels && layer_bias.dtype == layer_weights.dtype),
				"cuda_fold_batchnorm: bias must be [%d] of the weights' type", channels);
		if (outer == 0 || inner == 0)
			return;
		cudaStream_t stream = use_stream(context);
		const int grid = grid_for(static_cast<long long>(outer) * inner, 256, get(context)->sm_count);
		const float *av = reinterpret_cast<const float*>(bn_avg_var.data);
		switch (layer_weights.dtype)
		{
			case DTYPE_FLOAT16:
				kernel_fold_batchnorm<__half> <<<grid, 256, 0, stream>>>(reinterpret_cast<__half*>(layer_weights.data),
						reinterpret_cast<__half*>(layer_bias.data), reinterpret_cast<const __half*>(bn_weights.data),
						reinterpret_cast<const __half*>(bn_bias.data), av, outer, inner, per_row);
				break;
			case DTYPE_FLOAT32:
				kernel_fold_batchnorm<float> <<<grid, 256, 0, stream>>>(reinterpret_cast<float*>(layer_weights.data),
						reinterpret_cast<float*>(layer_bias.data), reinterpret_cast<const float*>(bn_weights.data),
						reinterpret_cast<const float*>(bn_bias.data), av, outer, inner, per_row);
				break;
			default:
				record_error(context, "cuda_fold_batchnorm: dtype %d not supported", static_cast<int>(layer_weights.dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_fold_batchnorm");
	}
	void cuda_channel_scaling_forward(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t scales, float beta, mlTensor_t y)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_channel_scaling_forward: null context");
		MB200_REQUIRE(context, x.data != nullptr && y.data != nullptr && scales.data != nullptr && x.rank >= 2 && scales.rank == 2,
				"cuda_channel_scaling_forward: x [b, ..., c], scales [b, c]");
		MB200_REQUIRE(context, x.dtype == y.dtype && x.dtype == scales.dtype && volume(x) == volume(y) && scales.dim[0] == x.dim[0]
				&& scales.dim[1] == last_dim(x), "cuda_channel_scaling_forward: tensors do not match");
		flush_pending(context);
		const int batch = x.dim[0], channels = last_dim(x);
		if (volume(x) == 0)
			return;
		const int hw = static_cast<int>(volume(x) / (static_cast<long long>(batch) * channels));
		MB200_REQUIRE(context, batch <= 65535, "cuda_channel_scaling_forward: batch %d exceeds one launch", batch);
		cudaStream_t stream = use_stream(context);
		const int sms = get(context)->sm_count;
		switch (x.dtype)
		{
			case DTYPE_FLOAT16:
			{
				__half *yp = reinterpret_cast<__half*>(y.data);
				const __half *xp = reinterpret_cast<const __half*>(x.data), *sp = reinterpret_cast<const __half*>(scales.data);
				if (channels % 8 == 0 && aligned_to(xp, 16) && aligned_to(yp, 16) && aligned_to(sp, 16))
					kernel_channel_scaling<__half, 8> <<<dim3(std::max(1, grid_for(static_cast<long long>(hw) * (channels / 8), 256, sms) / batch + 1), batch), 256, 0,
							stream>>>(yp, xp, sp, hw, channels, alpha, beta);
				else
					kernel_channel_scaling<__half, 1> <<<dim3(std::max(1, grid_for(static_cast<long long>(hw) * channels, 256, sms) / batch + 1), batch), 256, 0,
							stream>>>(yp, xp, sp, hw, channels, alpha, beta);
				break;
			}
			case DTYPE_FLOAT32:
			{
				float *yp = reinterpret_cast<float*>(y.data);
				const float *xp = reinterpret_cast<const float*>(x.data), *sp = reinterpret_cast<const float*>(scales.data);
				if (channels % 4 == 0 && aligned_to(xp, 16) && aligned_to(yp, 16) && aligned_to(sp, 16))
					kernel_channel_scaling<float, 4> <<<dim3(std::max(1, grid_for(static_cast<long long>(hw) * (channels / 4), 256, sms) / batch + 1), batch), 256, 0,
							stream>>>(yp, xp, sp, hw, channels, alpha, beta);
				else
					kernel_channel_scaling<float, 1> <<<dim3(std::max(1, grid_for(static_cast<long long>(hw) * channels, 256, sms) / batch + 1), batch), 256, 0,
							stream>>>(yp, xp, sp, hw, channels, alpha, beta);
				break;
			}
			default:
				record_error(context, "cuda_channel_scaling_forward: dtype %d not supported", static_cast<int>(x.dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_channel_scaling_forward");
	}
	void cuda_depthwise_conv_forward(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b, float beta,
			mlTensor_t y)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_depthwise_conv_forward: null context");
		MB200_REQUIRE(context, x.rank == 4 && y.rank == 4 && w.rank == 3 && x.data != nullptr && y.data != nullptr && w.data != nullptr,
				"cuda_depthwise_conv_forward: x, y [b,h,w,c], w [k,k,c]");
		MB200_REQUIRE(context, w.dim[0] == w.dim[1] && (w.dim[0] == 3 || w.dim[0] == 5 || w.dim[0] == 7), "cuda_depthwise_conv_forward: filter %d x %d not supported (3, 5, 7)",
				w.dim[0], w.dim[1]);
		MB200_REQUIRE(context, w.dim[2] == x.dim[3] && volume(x) == volume(y) && x.dtype == y.dtype && w.dtype == x.dtype
				&& (b.data == nullptr || (b.dtype == x.dtype && volume(b) == x.dim[3])), "cuda_depthwise_conv_forward: tensors do not match");
		flush_pending(context);
		if (volume(x) == 0)
			return;
		MB200_REQUIRE(context, x.dim[0] <= 65535, "cuda_depthwise_conv_forward: batch %d exceeds one launch", x.dim[0]);
		cudaStream_t stream = use_stream(context);
		const int channels = x.dim[3];
		const bool aligned = aligned_to(x.data, 16) && aligned_to(y.data, 16) && aligned_to(w.data, 16);
		switch (x.dtype)
		{
			case DTYPE_FLOAT16:
				if (channels % 8 == 0 && aligned)
					launch_depthwise<__half, 8>(stream, w.dim[0], x, w, b, y, alpha, beta);
				else
					launch_depthwise<__half, 1>(stream, w.dim[0], x, w, b, y, alpha, beta);
				break;
			case DTYPE_FLOAT32:
				if (channels % 4 == 0 && aligned)
					launch_depthwise<float, 4>(stream, w.dim[0], x, w, b, y, alpha, beta);
				else
					launch_depthwise<float, 1>(stream, w.dim[0], x, w, b, y, alpha, beta);
				break;
			default:
				record_error(context, "cuda_depthwise_conv_forward: dtype %d not supported", static_cast<int>(x.dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_depthwise_conv_forward");
	}
	void cuda_quantized_depthwise_conv_forward(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape,
			const void *input, const void *weights, const void *scales, const void *bias, void *output, mlQuantizationData_t output_qd,
			int padding_value)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_quantized_depthwise_conv_forward: null context");
		MB200_REQUIRE(context, dtype == DTYPE_INT8, "cuda_quantized_depthwise_conv_forward: only int8 is supported");
		MB200_REQUIRE(context, input_shape.rank == 4 && weights_shape.rank == 3 && input != nullptr && weights != nullptr && output != nullptr,
				"cuda_quantized_depthwise_conv_forward: input [b,h,w,c], weights [k,k,c]");
		const int k = weights_shape.dim[0];
		MB200_REQUIRE(context, weights_shape.dim[1] == k && (k == 3 || k == 5 || k == 7) && weights_shape.dim[2] == input_shape.dim[3],
				"cuda_quantized_depthwise_conv_forward: filter shape not supported");
		MB200_REQUIRE(context, output_qd.scale != 0.0f, "cuda_quantized_depthwise_conv_forward: output scale is zero");
		flush_pending(context);
		const int batch = input_shape.dim[0], height = input_shape.dim[1], width = input_shape.dim[2], channels = input_shape.dim[3];
		if (volume(input_shape) == 0)
			return;
		MB200_REQUIRE(context, batch <= 65535, "cuda_quantized_depthwise_conv_forward: batch %d exceeds one launch", batch);
		cudaStream_t stream = use_stream(context);
		const int tx = std::min(channels, 128);
		const int rows = std::max(1, 256 / tx);
		const dim3 block(tx, rows), grid(ceil_div(height, rows), batch);
		const float inv_scale = 1.0f / output_qd.scale, inv_shift = -output_qd.shift / output_qd.scale; // AffineTransform::get_inverse
		int8_t *yp = reinterpret_cast<int8_t*>(output);
		const int8_t *xp = reinterpret_cast<const int8_t*>(input), *wp = reinterpret_cast<const int8_t*>(weights);
		const float *sp = reinterpret_cast<const float*>(scales), *bp = reinterpret_cast<const float*>(bias);
		switch (k)
		{
			case 3:
				kernel_depthwise_conv_int8<3> <<<grid, block, 0, stream>>>(yp, xp, wp, sp, bp, height, width, channels, inv_scale, inv_shift, padding_value);
				break;
			case 5:
				kernel_depthwise_conv_int8<5> <<<grid, block, 0, stream>>>(yp, xp, wp, sp, bp, height, width, channels, inv_scale, inv_shift, padding_value);
				break;
			default:
				kernel_depthwise_conv_int8<7> <<<grid, block, 0, stream>>>(yp, xp, wp, sp, bp, height, width, channels, inv_scale, inv_shift, padding_value);
				break;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_quantized_depthwise_conv_forward");
	}
}
