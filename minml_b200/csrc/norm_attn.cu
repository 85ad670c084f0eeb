/*
 * norm_attn.cu -- layer normalisation and multi-head attention forward.
 *
 * Replaces src/backend/cuda/kernels/layernorm.cu:204-316,480-527 and src/backend/cuda/kernels/attention.cu:56-197,494-568.
 *
 * Layer norm: per row of the last dimension, mean and UNBIASED variance (divide by N - 1), eps = 1e-6 inside the
 * square root, then gamma * (x - mean) / stddev + beta.  When `ext` is given it is added to the input first -- the
 * behaviour of minml's CPU backend (src/backend/cpu/normalization.cpp:346-397), which is the parity target; the
 * reference's CUDA kernels accept the argument and ignore it.
 *
 * Attention: input [b, h, w, (3 - symmetric) * heads * d] packed as [q | k | v] x heads x d, output [b, h, w, heads * d].
 *   S = Q K^T / sqrt(d);  S[i, j] += table[head, r + clamp(hj - hi), r + clamp(wj - wi)]  (relative-position bias,
 *   table [heads, n, round_up(n, 4)], r = (n - 1) / 2);  P = softmax(S);  O = P V.
 * One CTA per (batch item, head) keeps K and V of that head in shared memory; each warp owns one query at a time,
 * so the [b, heads, T, T] score tensor the reference materialises in its workspace never exists.
 */
#include "common.cuh"

namespace mb200
{
	bool mha_forward_mma(mlContext_t ctx, void *output, const void *input, const void *table, int batch, int height, int width, int heads,
			int head_dim, int parts, int table_n, int table_pad); // attention_mma.cu
	bool mha_forward_tc(mlContext_t ctx, void *output, const void *input, const void *table, int batch, int height, int width, int heads,
			int head_dim, int parts, int table_n, int table_pad); // attention_tc.cu

	namespace
	{
		template<typename T>
		__global__ void __launch_bounds__(256) kernel_layernorm(T *__restrict__ output, const T *__restrict__ input, const T *__restrict__ gamma,
				const T *__restrict__ beta, const T *__restrict__ ext, long long rows, int channels)
		{
			const int lane = threadIdx.x % 32;
			const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x / 32);
			for (long long r = static_cast<long long>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32; r < rows; r += warps)
			{
				const T *px = input + r * channels;
				const T *pe = (ext != nullptr) ? ext + r * channels : nullptr;
				float sum = 0.0f;
				for (int j = lane; j < channels; j += 32)
					sum += to_float(px[j]) + (pe != nullptr ? to_float(pe[j]) : 0.0f);
				for (int k = 16; k >= 1; k /= 2)
					sum += __shfl_xor_sync(0xffffffffu, sum, k);
				const float mean = sum / static_cast<float>(channels);
				float var = 0.0f;
				for (int j = lane; j < channels; j += 32)
				{
					const float d = to_float(px[j]) + (pe != nullptr ? to_float(pe[j]) : 0.0f) - mean;
					var += d * d;
				}
				for (int k = 16; k >= 1; k /= 2)
					var += __shfl_xor_sync(0xffffffffu, var, k);
				const float inv_stddev = 1.0f / sqrtf(1.0e-6f + var / static_cast<float>(channels - 1));
				for (int j = lane; j < channels; j += 32)
				{
					const float x = to_float(px[j]) + (pe != nullptr ? to_float(pe[j]) : 0.0f);
					const float g = (gamma != nullptr) ? to_float(gamma[j]) : 1.0f;
					const float b = (beta != nullptr) ? to_float(beta[j]) : 0.0f;
					output[r * channels + j] = from_float<T>(g * (x - mean) * inv_stddev + b);
				}
			}
		}

		/* fp16 rows of 256 * ITERS channels: one warp per row, every lane keeps its 8 * ITERS values in registers (16-byte loads),
		 * so the row is read from memory once; the statistics are the same two passes (mean, then squared deviations) in fp32. */
		template<int ITERS, bool HAS_EXT>
		__global__ void __launch_bounds__(256) kernel_layernorm_rows_fp16(__half *__restrict__ output, const __half *__restrict__ input,
				const __half *__restrict__ gamma, const __half *__restrict__ beta, const __half *__restrict__ ext, long long rows)
		{
			constexpr int CHANNELS = 256 * ITERS;
			const int lane = threadIdx.x % 32;
			float g[ITERS][8], b[ITERS][8];
#pragma unroll
			for (int i = 0; i < ITERS; i++)
			{
				const int c = (i * 32 + lane) * 8;
				uint4 gr = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u), br = make_uint4(0, 0, 0, 0); // ones, zeros
				if (gamma != nullptr)
					gr = *reinterpret_cast<const uint4*>(gamma + c);
				if (beta != nullptr)
					br = *reinterpret_cast<const uint4*>(beta + c);
#pragma unroll
				for (int k = 0; k < 8; k++)
				{
					g[i][k] = __half2float(reinterpret_cast<const __half*>(&gr)[k]);
					b[i][k] = __half2float(reinterpret_cast<const __half*>(&br)[k]);
				}
			}
			// ROWS rows per pass, so that every lane has four 16-byte loads in flight whatever the row length
			constexpr int ROWS = (ITERS == 1) ? 4 : (ITERS == 2 ? 2 : 1);
			const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x / 32);
			for (long long r0 = static_cast<long long>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32; r0 < rows; r0 += warps * ROWS)
			{
				uint4 raw[ROWS][ITERS], er[HAS_EXT ? ROWS : 1][HAS_EXT ? ITERS : 1];
#pragma unroll
				for (int q = 0; q < ROWS; q++)
				{
					const long long r = r0 + q * warps;
#pragma unroll
					for (int i = 0; i < ITERS; i++)
					{
						const long long off = r * CHANNELS + (i * 32 + lane) * 8;
						raw[q][i] = make_uint4(0, 0, 0, 0);
						if (HAS_EXT)
							er[q][i] = make_uint4(0, 0, 0, 0);
						if (r < rows)
						{
							raw[q][i] = *reinterpret_cast<const uint4*>(input + off);
							if (HAS_EXT)
								er[q][i] = *reinterpret_cast<const uint4*>(ext + off);
						}
					}
				}
#pragma unroll
				for (int q = 0; q < ROWS; q++)
				{
					const long long r = r0 + q * warps;
					if (r >= rows)
						break; // warp-uniform
					float v[ITERS][8];
					float sum = 0.0f;
#pragma unroll
					for (int i = 0; i < ITERS; i++)
#pragma unroll
						for (int k = 0; k < 8; k++)
						{
							v[i][k] = __half2float(reinterpret_cast<const __half*>(&raw[q][i])[k]);
							if (HAS_EXT)
								v[i][k] += __half2float(reinterpret_cast<const __half*>(&er[q][i])[k]);
							sum += v[i][k];
						}
					for (int k = 16; k >= 1; k /= 2)
						sum += __shfl_xor_sync(0xffffffffu, sum, k);
					const float mean = sum / static_cast<float>(CHANNELS);
					float var = 0.0f;
#pragma unroll
					for (int i = 0; i < ITERS; i++)
#pragma unroll
						for (int k = 0; k < 8; k++)
						{
							const float d = v[i][k] - mean;
							var += d * d;
						}
					for (int k = 16; k >= 1; k /= 2)
						var += __shfl_xor_sync(0xffffffffu, var, k);
					const float inv_stddev = 1.0f / sqrtf(1.0e-6f + var / static_cast<float>(CHANNELS - 1));
#pragma unroll
					for (int i = 0; i < ITERS; i++)
					{
						uint4 out;
#pragma unroll
						for (int k = 0; k < 8; k++)
							reinterpret_cast<__half*>(&out)[k] = __float2half_rn(g[i][k] * (v[i][k] - mean) * inv_stddev + b[i][k]);
						*reinterpret_cast<uint4*>(output + r * CHANNELS + (i * 32 + lane) * 8) = out;
					}
				}
			}
		}

		constexpr int MHA_WARPS = 8;
		/* dynamic shared memory: K [tokens][d + 1] fp32, V [tokens][d] fp32, bias table [n * n_pad] fp32,
		 * per-warp: q [d] and p [tokens] */
		template<typename T>
		__global__ void __launch_bounds__(MHA_WARPS * 32) kernel_mha_forward(T *__restrict__ output, const T *__restrict__ input,
				const T *__restrict__ table, int height, int width, int heads, int head_dim, int parts, int table_n, int table_pad)
		{
			extern __shared__ float smem[];
			const int tokens = height * width;
			const int b = blockIdx.y, h = blockIdx.x;
			const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
			const int kd = head_dim + 1;
			float *sk = smem;
			float *sv = sk + tokens * kd;
			float *st = sv + tokens * head_dim;
			float *sq = st + ((table != nullptr) ? table_n * table_pad : 0) + warp * head_dim;
			float *sp = st + ((table != nullptr) ? table_n * table_pad : 0) + MHA_WARPS * head_dim + warp * tokens;

			const int stride = parts * heads * head_dim; // channels per token
			const T *base = input + static_cast<long long>(b) * tokens * stride;
			const int k_off = (parts == 3 ? 1 : 0) * heads * head_dim + h * head_dim; // symmetric: K is Q
			const int v_off = (parts - 1) * heads * head_dim + h * head_dim;
			for (int i = threadIdx.x; i < tokens * head_dim; i += blockDim.x)
			{
				const int t = i / head_dim, d = i % head_dim;
				sk[t * kd + d] = to_float(base[static_cast<long long>(t) * stride + k_off + d]);
				sv[t * head_dim + d] = to_float(base[static_cast<long long>(t) * stride + v_off + d]);
			}
			if (table != nullptr)
				for (int i = threadIdx.x; i < table_n * table_pad; i += blockDim.x)
					st[i] = to_float(table[static_cast<long long>(h) * table_n * table_pad + i]);
			__syncthreads();

			const float scale = 1.0f / sqrtf(static_cast<float>(head_dim));
			const int range = (table_n - 1) / 2;
			for (int qi = warp; qi < tokens; qi += MHA_WARPS)
			{
				for (int d = lane; d < head_dim; d += 32)
					sq[d] = to_float(base[static_cast<long long>(qi) * stride + h * head_dim + d]) * scale;
				__syncwarp();
				const int qh = qi / width, qw = qi % width;
				float max_value = -1.0e32f;
				for (int j = lane; j < tokens; j += 32)
				{
					float s = 0.0f;
					for (int d = 0; d < head_dim; d++)
						s += sq[d] * sk[j * kd + d];
					if (table != nullptr)
					{
						const int dh = min(max(j / width - qh, -range), range) + range;
						const int dw = min(max(j % width - qw, -range), range) + range;
						s += st[dh * table_pad + dw];
					}
					sp[j] = s;
					max_value = fmaxf(max_value, s);
				}
				for (int k = 16; k >= 1; k /= 2)
					max_value = fmaxf(max_value, __shfl_xor_sync(0xffffffffu, max_value, k));
				float sum = 0.0f;
				for (int j = lane; j < tokens; j += 32)
				{
					const float e = expf(sp[j] - max_value);
					sp[j] = e;
					sum += e;
				}
				for (int k = 16; k >= 1; k /= 2)
					sum += __shfl_xor_sync(0xffffffffu, sum, k);
				const float inv = 1.0f / sum;
				__syncwarp();
				for (int d = lane; d < head_dim; d += 32)
				{
					float o = 0.0f;
					for (int j = 0; j < tokens; j++)
						o += sp[j] * sv[j * head_dim + d];
					output[(static_cast<long long>(b) * tokens + qi) * heads * head_dim + h * head_dim + d] = from_float<T>(o * inv);
				}
				__syncwarp();
			}
		}
	}
} /* namespace mb200 */

using namespace mb200;

extern "C"
{
	void cuda_layernorm_forward(mlContext_t context, mlShape_t shape, mlDataType_t dtype, const void *input, void *output, const void *weights,
			const void *bias, const void *ext)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_layernorm_forward: null context");
		if (volume(shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, input != nullptr && output != nullptr, "cuda_layernorm_forward: null pointer");
		flush_pending(context);
		const long long rows = volume_without_last_dim(shape);
		const int channels = last_dim(shape);
		if (rows == 0 || channels == 0)
			return;
		MB200_REQUIRE(context, channels >= 2, "cuda_layernorm_forward: the unbiased variance needs at least 2 channels");
		cudaStream_t stream = use_stream(context);
		const int grid = static_cast<int>(std::min<long long>((rows + 7) / 8, static_cast<long long>(get(context)->sm_count) * 8));
		switch (dtype)
		{
			case DTYPE_FLOAT16:
			{
				__half *yp = reinterpret_cast<__half*>(output);
				const __half *xp = reinterpret_cast<const __half*>(input), *gp = reinterpret_cast<const __half*>(weights),
						*bp = reinterpret_cast<const __half*>(bias), *ep = reinterpret_cast<const __half*>(ext);
				const bool aligned = aligned_to(xp, 16) && aligned_to(yp, 16) && (gp == nullptr || aligned_to(gp, 16)) && (bp == nullptr || aligned_to(bp, 16))
						&& (ep == nullptr || aligned_to(ep, 16));
#define ROWS_KERNEL(I) do { if (ep != nullptr) kernel_layernorm_rows_fp16<I, true> <<<grid, 256, 0, stream>>>(yp, xp, gp, bp, ep, rows); \
		else kernel_layernorm_rows_fp16<I, false> <<<grid, 256, 0, stream>>>(yp, xp, gp, bp, ep, rows); } while (0)
				if (aligned && channels == 256)
					ROWS_KERNEL(1);
				else if (aligned && channels == 512)
					ROWS_KERNEL(2);
				else if (aligned && channels == 1024)
					ROWS_KERNEL(4);
				else
					kernel_layernorm<__half> <<<grid, 256, 0, stream>>>(yp, xp, gp, bp, ep, rows, channels);
				break;
			}
			case DTYPE_FLOAT32:
				kernel_layernorm<float> <<<grid, 256, 0, stream>>>(reinterpret_cast<float*>(output), reinterpret_cast<const float*>(input),
						reinterpret_cast<const float*>(weights), reinterpret_cast<const float*>(bias), reinterpret_cast<const float*>(ext), rows,
						channels);
				break;
			default:
				record_error(context, "cuda_layernorm_forward: dtype %d not supported", static_cast<int>(dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_layernorm_forward");
	}

	int cuda_multi_head_attention_get_workspace_size(mlShape_t input_shape, mlShape_t weights_shape, int num_heads, bool training)
	{
		// Same figure as the reference (src/backend/cuda/kernels/attention.cu:494-508) so the host sizes its buffers
		// identically; the forward kernel here does not touch the workspace.
		if (input_shape.rank != 4)
			return 0;
		const int batch_size = input_shape.dim[0];
		const int tokens = input_shape.dim[1] * input_shape.dim[2];
		int result = batch_size * num_heads * tokens * tokens;
		if (training)
		{
			result *= 2;
			if (weights_shape.rank == 3)
				result += batch_size * num_heads * weights_shape.dim[1] * weights_shape.dim[2];
		}
		return result;
	}
	void cuda_multi_head_attention_forward(mlContext_t context, mlShape_t input_shape, mlShape_t weights_shape, mlShape_t bias_shape,
			mlDataType_t dtype, const void *input, void *output, const void *weights, const void *bias, void *workspace, void *backward_data,
			int num_heads, bool symmetric)
	{
		(void) bias_shape;
		(void) bias;
		(void) workspace;
		(void) backward_data;
		MB200_REQUIRE(context, context != nullptr, "cuda_multi_head_attention_forward: null context");
		if (volume(input_shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, input_shape.rank == 4 && input != nullptr && output != nullptr,
				"cuda_multi_head_attention_forward: needs a rank-4 input and buffers");
		MB200_REQUIRE(context, num_heads > 0, "cuda_multi_head_attention_forward: %d heads", num_heads);
		flush_pending(context);
		const int batch = input_shape.dim[0], height = input_shape.dim[1], width = input_shape.dim[2];
		const int parts = symmetric ? 2 : 3;
		MB200_REQUIRE(context, input_shape.dim[3] % (parts * num_heads) == 0,
				"cuda_multi_head_attention_forward: %d channels do not split into %d parts x %d heads", input_shape.dim[3], parts, num_heads);
		const int head_dim = input_shape.dim[3] / (parts * num_heads);
		const int tokens = height * width;
		if (batch == 0 || tokens == 0)
			return;
		int table_n = 0, table_pad = 0;
		const void *table = nullptr;
		if (weights != nullptr && weights_shape.rank == 3)
		{
			MB200_REQUIRE(context, weights_shape.dim[0] == num_heads && weights_shape.dim[2] == ((weights_shape.dim[1] + 3) / 4) * 4,
					"cuda_multi_head_attention_forward: relative-position table must be [heads, n, round_up(n, 4)]");
			table = weights;
			table_n = weights_shape.dim[1];
			table_pad = weights_shape.dim[2];
		}
		// fp16, head dimension 32: the tcgen05 kernels as selected (by default the persistent one for boards of up to 256 tokens); fp16 with
		// a head dimension of 16, 32, 64 or 128: the warp-level tensor-core kernel; anything else: the generic kernel below
		if (dtype == DTYPE_FLOAT16 && mha_forward_tc(context, output, input, table, batch, height, width, num_heads, head_dim, parts, table_n,
				table_pad))
			return;
		if (dtype == DTYPE_FLOAT16 && mha_forward_mma(context, output, input, table, batch, height, width, num_heads, head_dim, parts, table_n,
				table_pad))
			return;
		const size_t smem = sizeof(float)
				* (static_cast<size_t>(tokens) * (head_dim + 1) + static_cast<size_t>(tokens) * head_dim + static_cast<size_t>(table_n) * table_pad
						+ static_cast<size_t>(MHA_WARPS) * head_dim + static_cast<size_t>(MHA_WARPS) * tokens);
		MB200_REQUIRE(context, smem <= 227 * 1024, "cuda_multi_head_attention_forward: %d tokens x head_dim %d need %zu bytes of shared memory", tokens,
				head_dim, smem);
		MB200_REQUIRE(context, batch <= 65535, "cuda_multi_head_attention_forward: batch %d exceeds one launch", batch);
		cudaStream_t stream = use_stream(context);
		dim3 grid(num_heads, batch);
		switch (dtype)
		{
			case DTYPE_FLOAT16:
				cudaFuncSetAttribute(kernel_mha_forward<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
				kernel_mha_forward<__half> <<<grid, MHA_WARPS * 32, smem, stream>>>(reinterpret_cast<__half*>(output),
						reinterpret_cast<const __half*>(input), reinterpret_cast<const __half*>(table), height, width, num_heads, head_dim, parts,
						table_n, table_pad);
				break;
			case DTYPE_FLOAT32:
				cudaFuncSetAttribute(kernel_mha_forward<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
				kernel_mha_forward<float> <<<grid, MHA_WARPS * 32, smem, stream>>>(reinterpret_cast<float*>(output),
						reinterpret_cast<const float*>(input), reinterpret_cast<const float*>(table), height, width, num_heads, head_dim, parts,
						table_n, table_pad);
				break;
			default:
				record_error(context, "cuda_multi_head_attention_forward: dtype %d not supported", static_cast<int>(dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_multi_head_attention_forward");
	}
}
