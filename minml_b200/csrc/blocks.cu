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
 * Batch norm and channel scaling are HBM-bound: a thread owns a fixed 16-byte group of channels (its scale and shift are computed
 * once) and strides over rows, so a warp reads and writes whole 128-byte lines.
 *
 * The depthwise convolutions are bound by the fp32 multiply-adds (k x k per output element, no reuse across channels, nothing for
 * the tensor cores): a thread owns one output row of a small group of channels and walks along it.  Input column ww feeds the k
 * output columns ww - pad .. ww + pad, whose partial sums sit in k register accumulators that shift by one per step; the k x k
 * filter taps of the thread's channels stay in registers as fp32 for the whole row.  Every input element is therefore loaded k
 * times (once per filter row), not k x k times, and the inner loop is k multiply-adds per loaded value.  fp32 tensors accumulate in
 * fp32; fp16 tensors by default multiply and accumulate in half2 like the reference's kernel (two channels per instruction, no
 * conversions in the inner loop), or in fp32 when MINML_B200_DEPTHWISE_FP32=1; the int8 variant runs on the fp32 path, which is
 * exact there: every partial sum is an integer below 49 * 128 * 128 < 2^24.
 */
#include "common.cuh"

#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

using namespace mb200;

namespace
{
	inline int grid_for(long long work_items, int block, int sm_count)
	{
		const long long blocks = (work_items + block - 1) / block;
		return static_cast<int>(std::max<long long>(1, std::min<long long>(blocks, static_cast<long long>(sm_count) * 16)));
	}
	__device__ __forceinline__ float to_float(float v) { return v; }
	__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
	__device__ __forceinline__ float to_float(int8_t v) { return static_cast<float>(static_cast<int>(v)); }
	template<typename T> __device__ __forceinline__ T from_float(float v);
	template<> __device__ __forceinline__ float from_float<float>(float v) { return v; }
	template<> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
	template<> __device__ __forceinline__ int8_t from_float<int8_t>(float v) { return static_cast<int8_t>(static_cast<int>(v)); }

	/* VEC consecutive elements moved with one load / store (the address must be aligned to VEC * sizeof(T)). */
	template<typename T, int VEC>
	struct alignas(sizeof(T) * VEC) Group
	{
			T v[VEC];
	};
	template<typename T, int VEC>
	__device__ __forceinline__ void load_group(const T *p, float (&out)[VEC])
	{
		const Group<T, VEC> g = *reinterpret_cast<const Group<T, VEC>*>(p);
#pragma unroll
		for (int k = 0; k < VEC; k++)
			out[k] = to_float(g.v[k]);
	}
	template<typename T, int VEC>
	__device__ __forceinline__ void store_group(T *p, const float (&in)[VEC])
	{
		Group<T, VEC> g;
#pragma unroll
		for (int k = 0; k < VEC; k++)
			g.v[k] = from_float<T>(in[k]);
		*reinterpret_cast<Group<T, VEC>*>(p) = g;
	}

	/* ------------------------------------------------------------------------------------------------ batch norm */
	/* block = (channel groups, rows): thread (tx, ty) owns channel group blockIdx.y * blockDim.x + tx and the rows ty, ty + step, ... */
	/* ACT is a compile-time class (0 linear, 1 ReLU, 2 decided at run time through a call): with the transcendental activations
	 * inlined per element and per unrolled row the kernel outgrew the instruction cache and stalled on instruction fetch. */
	__device__ __noinline__ float activation_by_call(float v, int act)
	{
		return apply_activation(v, act);
	}
	template<typename T, int VEC, int ACT>
	__global__ void __launch_bounds__(256) kernel_batchnorm_inference(T *y, const T *x, const T *gamma, const T *beta_bn, const float *avg_var,
			long long rows, int channels, float alpha, float beta, int act)
	{
		const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
		if (c0 >= channels)
			return;
		float scale[VEC], shift[VEC];
#pragma unroll
		for (int k = 0; k < VEC; k++)
		{
			const float g = (gamma != nullptr) ? to_float(gamma[c0 + k]) : 1.0f;
			const float b = (beta_bn != nullptr) ? to_float(beta_bn[c0 + k]) : 0.0f;
			scale[k] = g / sqrtf(avg_var[channels + c0 + k] + 1.0e-6f);
			shift[k] = -avg_var[c0 + k] * scale[k] + b;
		}
		// The per-channel constants take half of the registers a full-occupancy kernel may use, so fewer warps are resident;
		// each thread therefore keeps the loads of UNROLL rows in flight.
		constexpr int UNROLL = 2;
		const long long row_step = static_cast<long long>(gridDim.x) * blockDim.y;
		for (long long r0 = blockIdx.x * static_cast<long long>(blockDim.y) + threadIdx.y; r0 < rows; r0 += row_step * UNROLL)
		{
			float in[UNROLL][VEC], out[UNROLL][VEC];
#pragma unroll
			for (int u = 0; u < UNROLL; u++)
				if (r0 + u * row_step < rows)
				{
					const long long off = (r0 + u * row_step) * channels + c0;
					load_group<T, VEC>(x + off, in[u]);
					if (beta != 0.0f)
						load_group<T, VEC>(y + off, out[u]);
				}
#pragma unroll
			for (int u = 0; u < UNROLL; u++)
				if (r0 + u * row_step < rows)
				{
#pragma unroll
					for (int k = 0; k < VEC; k++)
					{
						float v = in[u][k] * scale[k] + shift[k];
						if (ACT == 1)
							v = fmaxf(v, 0.0f);
						else if (ACT == 2)
							v = activation_by_call(v, act);
						v *= alpha;
						out[u][k] = (beta != 0.0f) ? v + beta * out[u][k] : v;
					}
					store_group<T, VEC>(y + (r0 + u * row_step) * channels + c0, out[u]);
				}
		}
	}
	template<typename T, int VEC>
	void launch_batchnorm(cudaStream_t stream, int sm_count, T *y, const T *x, const T *w, const T *b, const float *av, long long rows, int channels,
			float alpha, float beta, int act)
	{
		const int groups = channels / VEC;
		const int tx = std::min(groups, 256);
		const int ty = std::max(1, 256 / tx);
		const dim3 block(tx, ty);
		const int row_blocks = static_cast<int>(std::max<long long>(1, std::min<long long>((rows + ty - 1) / ty, static_cast<long long>(sm_count) * 8)));
		const dim3 grid(row_blocks, ceil_div(groups, tx));
		if (act == ACTIVATION_LINEAR)
			kernel_batchnorm_inference<T, VEC, 0> <<<grid, block, 0, stream>>>(y, x, w, b, av, rows, channels, alpha, beta, act);
		else if (act == ACTIVATION_RELU)
			kernel_batchnorm_inference<T, VEC, 1> <<<grid, block, 0, stream>>>(y, x, w, b, av, rows, channels, alpha, beta, act);
		else
			kernel_batchnorm_inference<T, VEC, 2> <<<grid, block, 0, stream>>>(y, x, w, b, av, rows, channels, alpha, beta, act);
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
			weights[i] = from_float<T>(to_float(weights[i]) * scale);
			if ((per_row ? col : r) == 0 && bias != nullptr)
			{
				const float b = (beta_bn != nullptr) ? to_float(beta_bn[c]) : 0.0f;
				const float shift = -avg_var[c] * scale + b;
				bias[c] = from_float<T>(to_float(bias[c]) * scale + shift);
			}
		}
	}

	/* ------------------------------------------------------------------------------------------------ channel scaling */
	template<typename T, int VEC>
	__global__ void __launch_bounds__(256) kernel_channel_scaling(T *y, const T *x, const T *scales, int hw, int channels, float alpha,
			float beta)
	{
		const int groups = channels / VEC;
		const int b = blockIdx.y;
		const long long total = static_cast<long long>(hw) * groups;
		for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			const int c0 = static_cast<int>(i % groups) * VEC;
			const long long off = (static_cast<long long>(b) * hw + i / groups) * channels + c0;
			float in[VEC], s[VEC], out[VEC];
			load_group<T, VEC>(x + off, in);
			load_group<T, VEC>(scales + static_cast<long long>(b) * channels + c0, s);
			if (beta != 0.0f)
				load_group<T, VEC>(y + off, out);
#pragma unroll
			for (int k = 0; k < VEC; k++)
			{
				const float v = in[k] * s[k] * alpha;
				out[k] = (beta != 0.0f) ? v + beta * out[k] : v;
			}
			store_group<T, VEC>(y + off, out);
		}
	}

	/* ------------------------------------------------------------------------------------------------ depthwise convolution */
	struct DepthwiseParams
	{
			int height, width, channels;
			float alpha, beta; // floating point: y = alpha * conv + bias + beta * y
			const float *scales; // int8: x = acc * scales[c] + bias_f32[c]
			const float *bias_f32;
			float inv_scale, inv_shift; // int8 requantisation: q = clamp(round(x * inv_scale + inv_shift))
			float pad_value; // value of positions outside the image (the quantised zero; 0 for floating point)
	};
	constexpr int DEPTHWISE_SMEM_LIMIT = 96 * 1024;
	/* grid (row tiles x column tiles, batch, ceil(groups / blockDim.x)), block (32 channel groups, rows).  QUANT: int8 in / out.
	 * The CTA first copies its input patch -- (rows + K - 1) x (tile_w + K - 1) positions of its channels, positions outside the
	 * image holding the padding value -- into shared memory; the arithmetic then needs no bounds checks and no global latency.
	 * A thread owns R consecutive output rows of one group of VEC channels and walks along them: input column c feeds the K output columns
	 * c - K + 1 .. c through the K filter columns, so K partial sums live in a ring of register accumulators (the ring index is a
	 * compile-time constant because the column loop is unrolled K times). */
	/* H2 (fp16 only): taps, ring accumulators and multiply-adds in half2, two channels per instruction and no conversions in the
	 * inner loop; sums are then rounded to fp16 after every tap, as in the reference's kernel (depthwise_conv.cu accumulates fp16
	 * convolutions in half2), instead of being kept in fp32. Scaling, bias and the beta term stay in fp32. */
	template<typename T, int VEC, int K, int R, bool QUANT, bool H2 = false>
	__global__ void __launch_bounds__(256) kernel_depthwise_conv(T *y, const T *x, const T *w, const T *bias, const DepthwiseParams p,
			int tile_w, int tiles_w)
	{
		static_assert(!H2 || (sizeof(T) == 2 && VEC % 2 == 0 && !QUANT), "half2 arithmetic needs pairs of fp16 channels");
		constexpr int PAIRS = H2 ? VEC / 2 : 1;
		constexpr int PAD = (K - 1) / 2;
		extern __shared__ __align__(16) unsigned char smem_raw[];
		Group<T, VEC> *tile = reinterpret_cast<Group<T, VEC>*>(smem_raw);
		const int tx = threadIdx.x, ty = threadIdx.y, ntx = blockDim.x, nty = blockDim.y;
		const int h0 = (blockIdx.x / tiles_w) * nty * R, w0 = (blockIdx.x % tiles_w) * tile_w;
		const int c0 = (blockIdx.z * ntx + tx) * VEC;
		const bool lane_ok = c0 < p.channels;
		const int in_rows = nty * R + K - 1, in_cols = tile_w + K - 1;
		const long long image = static_cast<long long>(blockIdx.y) * p.height * p.width * p.channels + c0;
		const T *xb = x + image;
		T *yb = y + image;

		Group<T, VEC> pad_group;
#pragma unroll
		for (int k = 0; k < VEC; k++)
			pad_group.v[k] = from_float<T>(p.pad_value);
		for (int r = ty; r < in_rows; r += nty)
		{ // one patch row per step of threadIdx.y; the lanes of a warp copy consecutive channel groups of one position
			const int hh = h0 + r - PAD;
			const bool row_inside = lane_ok && hh >= 0 && hh < p.height;
			const T *src = xb + (static_cast<long long>(hh) * p.width + (w0 - PAD)) * p.channels;
			Group<T, VEC> *dst = tile + static_cast<long long>(r) * in_cols * ntx + tx;
			for (int cc = 0; cc < in_cols; cc++, src += p.channels, dst += ntx)
			{
				const int ww = w0 + cc - PAD;
				*dst = (row_inside && ww >= 0 && ww < p.width) ? *reinterpret_cast<const Group<T, VEC>*>(src) : pad_group;
			}
		}
		__syncthreads();
		const int h = h0 + ty * R; // first of this thread's R output rows
		if (!lane_ok || h >= p.height)
			return;

		float filt[H2 ? 1 : K * K][VEC];
		__half2 filt2[H2 ? K * K : 1][PAIRS];
#pragma unroll
		for (int t = 0; t < K * K; t++)
		{
			if constexpr (H2)
			{
				const Group<T, VEC> g = *reinterpret_cast<const Group<T, VEC>*>(w + static_cast<long long>(t) * p.channels + c0);
#pragma unroll
				for (int q = 0; q < PAIRS; q++)
					filt2[t][q] = reinterpret_cast<const __half2*>(&g)[q];
			}
			else
				load_group<T, VEC>(w + static_cast<long long>(t) * p.channels + c0, filt[t]);
		}
		float post_scale[VEC], post_shift[VEC];
#pragma unroll
		for (int k = 0; k < VEC; k++)
		{
			if (QUANT)
			{
				post_scale[k] = (p.scales != nullptr) ? p.scales[c0 + k] : 1.0f;
				post_shift[k] = (p.bias_f32 != nullptr) ? p.bias_f32[c0 + k] : 0.0f;
			}
			else
			{
				post_scale[k] = p.alpha;
				post_shift[k] = (bias != nullptr) ? to_float(bias[c0 + k]) : 0.0f;
			}
		}
		float acc[R][K][H2 ? 1 : VEC]; // per output row a ring: output column o of the tile lives in slot o mod K
		__half2 acc2[R][K][PAIRS];
#pragma unroll
		for (int r = 0; r < R; r++)
#pragma unroll
			for (int s = 0; s < K; s++)
			{
#pragma unroll
				for (int k = 0; k < (H2 ? 1 : VEC); k++)
					acc[r][s][k] = 0.0f;
#pragma unroll
				for (int q = 0; q < PAIRS; q++)
					acc2[r][s][q] = __float2half2_rn(0.0f);
			}

		const int out_cols = min(tile_w, p.width - w0);
		const int ncols = out_cols + K - 1; // input columns of the patch these rows need
		const Group<T, VEC> *row0 = tile + static_cast<long long>(ty) * R * in_cols * ntx + tx;
		for (int col0 = 0; col0 < ncols; col0 += K)
		{
#pragma unroll
			for (int u = 0; u < K; u++)
			{
				const int col = col0 + u;
				if (col < ncols)
				{
#pragma unroll
					for (int i = 0; i < K + R - 1; i++)
					{ // patch row i feeds output row r through filter row i - r
						float in[VEC];
						const Group<T, VEC> g = row0[(i * in_cols + col) * ntx];
						if constexpr (!H2)
						{
#pragma unroll
							for (int k = 0; k < VEC; k++)
								in[k] = to_float(g.v[k]);
						}
#pragma unroll
						for (int r = 0; r < R; r++)
						{
							if (i - r < 0 || i - r >= K)
								continue;
#pragma unroll
							for (int j = 0; j < K; j++) // filter column j: output column col - j, ring slot (u - j) mod K
							{
								if constexpr (H2)
								{
#pragma unroll
									for (int q = 0; q < PAIRS; q++)
										acc2[r][(u - j + K) % K][q] = __hfma2(reinterpret_cast<const __half2*>(&g)[q], filt2[(i - r) * K + j][q],
												acc2[r][(u - j + K) % K][q]);
								}
								else
								{
#pragma unroll
									for (int k = 0; k < VEC; k++)
										acc[r][(u - j + K) % K][k] = fmaf(in[k], filt[(i - r) * K + j][k], acc[r][(u - j + K) % K][k]);
								}
							}
						}
					}
#pragma unroll
					for (int r = 0; r < R; r++)
					{
						float done[VEC]; // output column col - (K - 1): complete after this input column
						if constexpr (H2)
						{
#pragma unroll
							for (int q = 0; q < PAIRS; q++)
							{
								const float2 f = __half22float2(acc2[r][(u + 1) % K][q]);
								done[2 * q] = f.x;
								done[2 * q + 1] = f.y;
							}
						}
						else
						{
#pragma unroll
							for (int k = 0; k < VEC; k++)
								done[k] = acc[r][(u + 1) % K][k];
						}
						if (col >= K - 1 && h + r < p.height)
						{
							const long long off = (static_cast<long long>(h + r) * p.width + (w0 + col - (K - 1))) * p.channels;
							float out[VEC];
							if (QUANT)
							{
#pragma unroll
								for (int k = 0; k < VEC; k++)
								{ // the host's CPU loop, operation for operation, without fused multiply-adds
									const float t = __fadd_rn(__fmul_rn(done[k], post_scale[k]), post_shift[k]);
									out[k] = fmaxf(-128.0f, fminf(127.0f, roundf(__fadd_rn(__fmul_rn(t, p.inv_scale), p.inv_shift))));
								}
							}
							else
							{
								if (p.beta != 0.0f)
									load_group<T, VEC>(yb + off, out);
#pragma unroll
								for (int k = 0; k < VEC; k++)
								{
									const float v = done[k] * post_scale[k] + post_shift[k];
									out[k] = (p.beta != 0.0f) ? v + p.beta * out[k] : v;
								}
							}
							store_group<T, VEC>(yb + off, out);
						}
						// the slot the next input column opens
#pragma unroll
						for (int k = 0; k < (H2 ? 1 : VEC); k++)
							acc[r][(u + 1) % K][k] = 0.0f;
#pragma unroll
						for (int q = 0; q < PAIRS; q++)
							acc2[r][(u + 1) % K][q] = __float2half2_rn(0.0f);
					}
				}
			}
		}
	}

	/* Shared-memory opt-in above 48 KB and the large carve-out, once per device and kernel instantiation. */
	template<typename T, int VEC, int K, int R, bool QUANT, bool H2>
	bool depthwise_opt_in(int device)
	{
		static bool done[MAX_DEVICES] = { false };
		if (device < 0 || device >= MAX_DEVICES)
			return false;
		if (!done[device])
		{
			if (cudaFuncSetAttribute(kernel_depthwise_conv<T, VEC, K, R, QUANT, H2>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEPTHWISE_SMEM_LIMIT)
					!= cudaSuccess || cudaFuncSetAttribute(kernel_depthwise_conv<T, VEC, K, R, QUANT, H2>, cudaFuncAttributePreferredSharedMemoryCarveout,
							cudaSharedmemCarveoutMaxShared) != cudaSuccess)
			{
				cudaGetLastError();
				return false;
			}
			done[device] = true;
		}
		return true;
	}
	template<typename T, int VEC, int K, bool QUANT, bool H2 = false>
	bool launch_depthwise_kv(cudaStream_t stream, int device, int batch, T *y, const T *x, const T *w, const T *bias, const DepthwiseParams &p)
	{
		constexpr int R = 2; // output rows per thread: every patch element read feeds two rows' multiply-adds
		const int groups = p.channels / VEC;
		const int tx = std::min(groups, 32);
		// rows of the image split evenly over as few CTAs as 8 x R rows each allow; then the widest column tile that fits
		const int max_ty = std::max(1, 256 / tx);
		const int row_blocks = ceil_div(p.height, std::min(8, max_ty) * R);
		int ty = ceil_div(ceil_div(p.height, row_blocks), R), tile_w = std::min(p.width, 32);
		auto patch_bytes = [&](int threads_y, int cols)
		{
			return static_cast<size_t>(threads_y * R + K - 1) * (cols + K - 1) * tx * VEC * sizeof(T);
		};
		while (patch_bytes(ty, tile_w) > static_cast<size_t>(DEPTHWISE_SMEM_LIMIT) && (ty > 1 || tile_w > 1))
		{
			if (tile_w >= ty * R && tile_w > 1)
				tile_w = (tile_w + 1) / 2;
			else
				ty = (ty + 1) / 2;
		}
		const size_t smem = patch_bytes(ty, tile_w);
		if (!depthwise_opt_in<T, VEC, K, R, QUANT, H2>(device)) // also asks for the large shared-memory carve-out: several patches per SM
			return false;
		const int tiles_w = ceil_div(p.width, tile_w);
		const dim3 block(tx, ty);
		const dim3 grid(ceil_div(p.height, ty * R) * tiles_w, batch, ceil_div(groups, tx));
		kernel_depthwise_conv<T, VEC, K, R, QUANT, H2> <<<grid, block, smem, stream>>>(y, x, w, bias, p, tile_w, tiles_w);
		return true;
	}
	/* The widest channel group that keeps the k x k fp32 filter taps in registers: 8 / 4 / 2 channels for k = 3 / 5 / 7. */
	template<typename T, bool QUANT>
	bool launch_depthwise(cudaStream_t stream, int device, int k, int batch, T *y, const T *x, const T *w, const T *bias, const DepthwiseParams &p)
	{
		auto ok = [&](int vec)
		{
			const size_t bytes = sizeof(T) * vec;
			return p.channels % vec == 0 && aligned_to(x, bytes) && aligned_to(y, bytes) && aligned_to(w, bytes);
		};
		constexpr int WIDEST = (sizeof(T) == 4) ? 4 : 8;
		if constexpr (sizeof(T) == 2 && !QUANT)
		{ // fp16: half2 arithmetic for the widest group of each kernel size, unless MINML_B200_DEPTHWISE_FP32=1 asks for fp32 sums
			static const bool fp32_sums = std::getenv("MINML_B200_DEPTHWISE_FP32") != nullptr && std::getenv("MINML_B200_DEPTHWISE_FP32")[0] == '1';
			if (!fp32_sums)
			{
				if (k == 3 && ok(8))
					return launch_depthwise_kv<T, 8, 3, QUANT, true>(stream, device, batch, y, x, w, bias, p);
				if (k == 5 && ok(4))
					return launch_depthwise_kv<T, 4, 5, QUANT, true>(stream, device, batch, y, x, w, bias, p);
				if (k == 7 && ok(2))
					return launch_depthwise_kv<T, 2, 7, QUANT, true>(stream, device, batch, y, x, w, bias, p);
			}
		}
		if (k == 3)
		{
			if (ok(WIDEST))
				return launch_depthwise_kv<T, WIDEST, 3, QUANT>(stream, device, batch, y, x, w, bias, p);
			else if (ok(2))
				return launch_depthwise_kv<T, 2, 3, QUANT>(stream, device, batch, y, x, w, bias, p);
			else
				return launch_depthwise_kv<T, 1, 3, QUANT>(stream, device, batch, y, x, w, bias, p);
		}
		else if (k == 5)
		{
			if (ok(4))
				return launch_depthwise_kv<T, 4, 5, QUANT>(stream, device, batch, y, x, w, bias, p);
			else if (ok(2))
				return launch_depthwise_kv<T, 2, 5, QUANT>(stream, device, batch, y, x, w, bias, p);
			else
				return launch_depthwise_kv<T, 1, 5, QUANT>(stream, device, batch, y, x, w, bias, p);
		}
		else
		{
			if (ok(2))
				return launch_depthwise_kv<T, 2, 7, QUANT>(stream, device, batch, y, x, w, bias, p);
			else
				return launch_depthwise_kv<T, 1, 7, QUANT>(stream, device, batch, y, x, w, bias, p);
		}
	}
}

extern "C"
{
	void cuda_batchnorm_inference(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b,
			const mlTensor_t avg_var, float beta, mlTensor_t y, mlActivationType_t act)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_batchnorm_inference: null context");
		if (volume(x) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
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
					launch_batchnorm<__half, 8>(stream, sms, yp, xp, wp, bp, av, rows, channels, alpha, beta, act);
				else
					launch_batchnorm<__half, 1>(stream, sms, yp, xp, wp, bp, av, rows, channels, alpha, beta, act);
				break;
			}
			case DTYPE_FLOAT32:
			{
				float *yp = reinterpret_cast<float*>(y.data);
				const float *xp = reinterpret_cast<const float*>(x.data), *wp = reinterpret_cast<const float*>(w.data),
						*bp = reinterpret_cast<const float*>(b.data);
				if (channels % 4 == 0 && aligned_to(xp, 16) && aligned_to(yp, 16))
					launch_batchnorm<float, 4>(stream, sms, yp, xp, wp, bp, av, rows, channels, alpha, beta, act);
				else
					launch_batchnorm<float, 1>(stream, sms, yp, xp, wp, bp, av, rows, channels, alpha, beta, act);
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
		if (volume(x) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
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
		auto blocks_per_image = [&](int vec)
		{
			return std::max(1, grid_for(static_cast<long long>(hw) * (channels / vec), 256, sms) / batch + 1);
		};
		switch (x.dtype)
		{
			case DTYPE_FLOAT16:
			{
				__half *yp = reinterpret_cast<__half*>(y.data);
				const __half *xp = reinterpret_cast<const __half*>(x.data), *sp = reinterpret_cast<const __half*>(scales.data);
				if (channels % 8 == 0 && aligned_to(xp, 16) && aligned_to(yp, 16) && aligned_to(sp, 16))
					kernel_channel_scaling<__half, 8> <<<dim3(blocks_per_image(8), batch), 256, 0, stream>>>(yp, xp, sp, hw, channels, alpha, beta);
				else
					kernel_channel_scaling<__half, 1> <<<dim3(blocks_per_image(1), batch), 256, 0, stream>>>(yp, xp, sp, hw, channels, alpha, beta);
				break;
			}
			case DTYPE_FLOAT32:
			{
				float *yp = reinterpret_cast<float*>(y.data);
				const float *xp = reinterpret_cast<const float*>(x.data), *sp = reinterpret_cast<const float*>(scales.data);
				if (channels % 4 == 0 && aligned_to(xp, 16) && aligned_to(yp, 16) && aligned_to(sp, 16))
					kernel_channel_scaling<float, 4> <<<dim3(blocks_per_image(4), batch), 256, 0, stream>>>(yp, xp, sp, hw, channels, alpha, beta);
				else
					kernel_channel_scaling<float, 1> <<<dim3(blocks_per_image(1), batch), 256, 0, stream>>>(yp, xp, sp, hw, channels, alpha, beta);
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
		if (volume(x) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
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
		DepthwiseParams p = { };
		p.height = x.dim[1];
		p.width = x.dim[2];
		p.channels = x.dim[3];
		p.alpha = alpha;
		p.beta = beta;
		bool launched = false;
		switch (x.dtype)
		{
			case DTYPE_FLOAT16:
				launched = launch_depthwise<__half, false>(stream, get(context)->device, w.dim[0], x.dim[0], reinterpret_cast<__half*>(y.data),
						reinterpret_cast<const __half*>(x.data), reinterpret_cast<const __half*>(w.data), reinterpret_cast<const __half*>(b.data), p);
				break;
			case DTYPE_FLOAT32:
				launched = launch_depthwise<float, false>(stream, get(context)->device, w.dim[0], x.dim[0], reinterpret_cast<float*>(y.data),
						reinterpret_cast<const float*>(x.data), reinterpret_cast<const float*>(w.data), reinterpret_cast<const float*>(b.data), p);
				break;
			default:
				record_error(context, "cuda_depthwise_conv_forward: dtype %d not supported", static_cast<int>(x.dtype));
				return;
		}
		MB200_REQUIRE(context, launched, "cuda_depthwise_conv_forward: shared-memory opt-in failed");
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_depthwise_conv_forward");
	}
	void cuda_quantized_depthwise_conv_forward(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape,
			const void *input, const void *weights, const void *scales, const void *bias, void *output, mlQuantizationData_t output_qd,
			int padding_value)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_quantized_depthwise_conv_forward: null context");
		if (volume(input_shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, dtype == DTYPE_INT8, "cuda_quantized_depthwise_conv_forward: only int8 is supported");
		MB200_REQUIRE(context, input_shape.rank == 4 && weights_shape.rank == 3 && input != nullptr && weights != nullptr && output != nullptr,
				"cuda_quantized_depthwise_conv_forward: input [b,h,w,c], weights [k,k,c]");
		const int k = weights_shape.dim[0];
		MB200_REQUIRE(context, weights_shape.dim[1] == k && (k == 3 || k == 5 || k == 7) && weights_shape.dim[2] == input_shape.dim[3],
				"cuda_quantized_depthwise_conv_forward: filter shape not supported");
		MB200_REQUIRE(context, output_qd.scale != 0.0f, "cuda_quantized_depthwise_conv_forward: output scale is zero");
		MB200_REQUIRE(context, padding_value >= -128 && padding_value <= 127, "cuda_quantized_depthwise_conv_forward: padding value %d is not an int8", padding_value);
		flush_pending(context);
		if (volume(input_shape) == 0)
			return;
		MB200_REQUIRE(context, input_shape.dim[0] <= 65535, "cuda_quantized_depthwise_conv_forward: batch %d exceeds one launch", input_shape.dim[0]);
		cudaStream_t stream = use_stream(context);
		DepthwiseParams p = { };
		p.height = input_shape.dim[1];
		p.width = input_shape.dim[2];
		p.channels = input_shape.dim[3];
		p.scales = reinterpret_cast<const float*>(scales);
		p.bias_f32 = reinterpret_cast<const float*>(bias);
		p.inv_scale = 1.0f / output_qd.scale; // AffineTransform::get_inverse (include/minml/layers/quantization.hpp:52-63)
		p.inv_shift = -output_qd.shift / output_qd.scale;
		p.pad_value = static_cast<float>(padding_value);
		const bool launched = launch_depthwise<int8_t, true>(stream, get(context)->device, k, input_shape.dim[0], reinterpret_cast<int8_t*>(output),
				reinterpret_cast<const int8_t*>(input), reinterpret_cast<const int8_t*>(weights), static_cast<const int8_t*>(nullptr), p);
		MB200_REQUIRE(context, launched, "cuda_quantized_depthwise_conv_forward: shared-memory opt-in failed");
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_quantized_depthwise_conv_forward");
	}
}
