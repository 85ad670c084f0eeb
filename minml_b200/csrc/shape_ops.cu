/*
 * shape_ops.cu -- layers that sit between the convolution blocks of minml's current networks: RMS normalisation and the
 * space-to-depth / depth-to-space rearrangements. All three are bound by HBM traffic (every element read once, written once).
 *
 *   cuda_rmsnorm_forward   y[r, c] = gamma[c] * x[r, c] / (1e-6 + sqrt(mean_c x[r, c]^2))
 *                          replaces src/backend/cuda/kernels/rmsnorm.cu:32-84,219-257 (CPU twin: src/backend/cpu/normalization.cpp:452-486)
 *   cuda_space_to_depth    [b, h, w, c] -> [b, ceil(h/p), ceil(w/q), p*q*c]: out[b, i, j, (x*q + y)*c + k] = in[b, i*p + x, j*q + y, k],
 *                          zero where the patch hangs over the edge
 *   cuda_depth_to_space    the inverse: out[b, h, w, k] = in[b, h/p, w/q, ((h%p)*q + w%q)*c + k]
 *                          replaces src/backend/cuda/kernels/conversion.cu:100-150,308-389 (CPU twin: src/backend/cpu/dispatcher.cpp:190-247)
 *
 * The reference builds a table of offsets in the context workspace with one kernel and copies element by element with a second one;
 * here the index arithmetic is done in the copying kernel itself (once per channel block, not per element) and the block of
 * channels moves in pieces of up to 16 bytes. The patch size is not an argument: like the reference, it is the smallest p
 * with ceil(larger / p) == smaller.
 */
#include "common.cuh"

#include <cuda_fp16.h>

#include <algorithm>

using namespace mb200;

namespace
{
	__device__ __forceinline__ float to_f(float v) { return v; }
	__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
	template<typename T> __device__ __forceinline__ T from_f(float v);
	template<> __device__ __forceinline__ float from_f<float>(float v) { return v; }
	template<> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

	template<typename T, int VEC>
	struct alignas(sizeof(T) * VEC) Pack
	{
			T v[VEC];
	};

	/* One warp per row. Rows of up to 32 * VEC * ITERS channels stay in registers between the sum of squares and the scaling, so
	 * the row is read from memory once, and ROWS rows are in flight per warp (four 16-byte loads per lane whatever the row length);
	 * longer rows are read a second time (from L1 / L2). */
	template<typename T, int VEC, int ITERS, int ROWS>
	__global__ void __launch_bounds__(256) kernel_rmsnorm(T *__restrict__ output, const T *__restrict__ input, const T *__restrict__ gamma,
			long long rows, int channels)
	{
		const int lane = threadIdx.x % 32;
		const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x / 32);
		const bool cached = channels <= 32 * VEC * ITERS;
		for (long long r0 = static_cast<long long>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32; r0 < rows; r0 += warps * ROWS)
		{
			if (cached)
			{
				Pack<T, VEC> keep[ROWS][ITERS];
#pragma unroll
				for (int q = 0; q < ROWS; q++)
#pragma unroll
					for (int i = 0; i < ITERS; i++)
					{
						const int c = (i * 32 + lane) * VEC;
						if (r0 + q * warps < rows && c < channels)
							keep[q][i] = *reinterpret_cast<const Pack<T, VEC>*>(input + (r0 + q * warps) * channels + c);
					}
#pragma unroll
				for (int q = 0; q < ROWS; q++)
				{
					const long long r = r0 + q * warps;
					if (r >= rows)
						break; // warp-uniform
					float sum = 0.0f;
#pragma unroll
					for (int i = 0; i < ITERS; i++)
						if ((i * 32 + lane) * VEC < channels)
						{
#pragma unroll
							for (int k = 0; k < VEC; k++)
								sum += to_f(keep[q][i].v[k]) * to_f(keep[q][i].v[k]);
						}
					for (int k = 16; k >= 1; k /= 2)
						sum += __shfl_xor_sync(0xffffffffu, sum, k);
					const float inv_rms = 1.0f / (1.0e-6f + sqrtf(sum / static_cast<float>(channels)));
#pragma unroll
					for (int i = 0; i < ITERS; i++)
					{
						const int c = (i * 32 + lane) * VEC;
						if (c < channels)
						{
							Pack<T, VEC> g, out;
							if (gamma != nullptr)
								g = *reinterpret_cast<const Pack<T, VEC>*>(gamma + c);
#pragma unroll
							for (int k = 0; k < VEC; k++)
								out.v[k] = from_f<T>((gamma != nullptr ? to_f(g.v[k]) : 1.0f) * to_f(keep[q][i].v[k]) * inv_rms);
							*reinterpret_cast<Pack<T, VEC>*>(output + r * channels + c) = out;
						}
					}
				}
			}
			else
				for (int q = 0; q < ROWS; q++)
				{
					const long long r = r0 + q * warps;
					if (r >= rows)
						break;
					const T *px = input + r * channels;
					T *py = output + r * channels;
					float sum = 0.0f;
					for (int c = lane * VEC; c < channels; c += 32 * VEC)
					{
						const Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(px + c);
#pragma unroll
						for (int k = 0; k < VEC; k++)
							sum += to_f(p.v[k]) * to_f(p.v[k]);
					}
					for (int k = 16; k >= 1; k /= 2)
						sum += __shfl_xor_sync(0xffffffffu, sum, k);
					const float inv_rms = 1.0f / (1.0e-6f + sqrtf(sum / static_cast<float>(channels)));
					for (int c = lane * VEC; c < channels; c += 32 * VEC)
					{
						const Pack<T, VEC> p = *reinterpret_cast<const Pack<T, VEC>*>(px + c);
						Pack<T, VEC> g, out;
						if (gamma != nullptr)
							g = *reinterpret_cast<const Pack<T, VEC>*>(gamma + c);
#pragma unroll
						for (int k = 0; k < VEC; k++)
							out.v[k] = from_f<T>((gamma != nullptr ? to_f(g.v[k]) : 1.0f) * to_f(p.v[k]) * inv_rms);
						*reinterpret_cast<Pack<T, VEC>*>(py + c) = out;
					}
				}
		}
	}

	template<typename T>
	void launch_rmsnorm(mlContext_t context, cudaStream_t stream, void *output, const void *input, const void *weights, long long rows,
			int channels)
	{
		T *yp = reinterpret_cast<T*>(output);
		const T *xp = reinterpret_cast<const T*>(input), *gp = reinterpret_cast<const T*>(weights);
		const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((rows + 7) / 8, static_cast<long long>(get(context)->sm_count) * 8)));
		constexpr int WIDE = 16 / static_cast<int>(sizeof(T)); // elements per 16-byte access
		const bool wide = channels % WIDE == 0 && reinterpret_cast<uintptr_t>(xp) % 16 == 0 && reinterpret_cast<uintptr_t>(yp) % 16 == 0
				&& reinterpret_cast<uintptr_t>(gp) % 16 == 0;
		if (wide && channels <= 32 * WIDE)
			kernel_rmsnorm<T, WIDE, 1, 4> <<<grid, 256, 0, stream>>>(yp, xp, gp, rows, channels);
		else if (wide && channels <= 64 * WIDE)
			kernel_rmsnorm<T, WIDE, 2, 2> <<<grid, 256, 0, stream>>>(yp, xp, gp, rows, channels);
		else if (wide)
			kernel_rmsnorm<T, WIDE, 4, 1> <<<grid, 256, 0, stream>>>(yp, xp, gp, rows, channels);
		else
			kernel_rmsnorm<T, 1, 8, 1> <<<grid, 256, 0, stream>>>(yp, xp, gp, rows, channels);
		MB200_COUNT_LAUNCH();
	}

	/* The smallest p with ceil(larger / p) == smaller, 0 when there is none (src/backend/cpu/dispatcher.cpp:125-137). */
	int patch_size(int smaller, int larger)
	{
		if (smaller <= 0 || larger < smaller)
			return 0;
		for (int p = 1;; p++)
		{
			const int tmp = (larger + p - 1) / p;
			if (tmp == smaller)
				return p;
			if (tmp < smaller)
				return 0;
		}
	}

	struct Geometry
	{
			int batch, height, width; // of the spatially larger tensor
			int ph, pw; // patch size
			int coarse_h, coarse_w; // of the spatially smaller tensor
			int pieces; // pieces of V bytes per channel block of the larger tensor
			FastDiv by_pieces, by_pw, by_ph;
	};

	/* A block walks over rows of coarse pixels (batch item b, coarse row i); within one, consecutive threads take consecutive
	 * pieces of the deep tensor, which is contiguous there. TO_DEPTH picks the copy direction. */
	template<typename V, bool TO_DEPTH>
	__global__ void __launch_bounds__(256) kernel_rearrange(V *__restrict__ deep, V *__restrict__ flat, const Geometry g)
	{
		const uint32_t inner = static_cast<uint32_t>(g.coarse_w) * g.ph * g.pw * g.pieces;
		const int coarse_rows = g.batch * g.coarse_h;
		for (int row = blockIdx.x; row < coarse_rows; row += gridDim.x)
		{
			const int b = row / g.coarse_h, i = row - b * g.coarse_h;
			V *deep_row = deep + static_cast<long long>(row) * inner;
			V *flat_image = flat + static_cast<long long>(b) * g.height * g.width * g.pieces;
			for (uint32_t t = threadIdx.x; t < inner; t += blockDim.x)
			{
				uint32_t rest, piece, y, x, j;
				g.by_pieces.divmod(t, rest, piece);
				g.by_pw.divmod(rest, rest, y);
				g.by_ph.divmod(rest, j, x);
				const int h = i * g.ph + static_cast<int>(x), w = static_cast<int>(j) * g.pw + static_cast<int>(y);
				const bool inside = h < g.height && w < g.width;
				V *flat_at = flat_image + (static_cast<long long>(h) * g.width + w) * g.pieces + piece;
				if (TO_DEPTH)
				{
					V value;
					memset(&value, 0, sizeof(V));
					if (inside)
						value = *flat_at;
					deep_row[t] = value;
				}
				else if (inside)
					*flat_at = deep_row[t];
			}
		}
	}

	template<bool TO_DEPTH>
	void rearrange(mlContext_t context, const char *who, mlDataType_t dtype, const mlShape_t &flat_shape, const void *flat, const mlShape_t &deep_shape,
			const void *deep)
	{
		MB200_REQUIRE(context, context != nullptr, "%s: null context", who);
		MB200_REQUIRE(context, flat_shape.rank == 4 && deep_shape.rank == 4, "%s: both tensors must be [batch, height, width, channels]", who);
		if (volume(flat_shape) == 0 || volume(deep_shape) == 0)
			return; // an empty problem: nothing to validate or launch
		MB200_REQUIRE(context, flat != nullptr && deep != nullptr, "%s: null pointer", who);
		const int elem = size_of(dtype);
		MB200_REQUIRE(context, elem > 0, "%s: dtype %d not supported", who, static_cast<int>(dtype));
		Geometry g;
		g.batch = flat_shape.dim[0];
		g.height = flat_shape.dim[1];
		g.width = flat_shape.dim[2];
		g.coarse_h = deep_shape.dim[1];
		g.coarse_w = deep_shape.dim[2];
		g.ph = patch_size(g.coarse_h, g.height);
		g.pw = patch_size(g.coarse_w, g.width);
		MB200_REQUIRE(context, g.ph != 0 && g.pw != 0, "%s: %d x %d is not %d x %d divided into equal patches", who, g.coarse_h, g.coarse_w, g.height,
				g.width);
		MB200_REQUIRE(context, deep_shape.dim[0] == g.batch && static_cast<long long>(flat_shape.dim[3]) * g.ph * g.pw == deep_shape.dim[3],
				"%s: channels %d x patch %d x %d do not give %d", who, flat_shape.dim[3], g.ph, g.pw, deep_shape.dim[3]);
		flush_pending(context);
		const long long block_bytes = static_cast<long long>(flat_shape.dim[3]) * elem;
		const uintptr_t addresses = reinterpret_cast<uintptr_t>(flat) | reinterpret_cast<uintptr_t>(deep);
		int piece = 16;
		while (piece > 1 && (block_bytes % piece != 0 || addresses % piece != 0))
			piece /= 2;
		g.pieces = static_cast<int>(block_bytes / piece);
		g.by_pieces = FastDiv(static_cast<uint32_t>(g.pieces));
		g.by_pw = FastDiv(static_cast<uint32_t>(g.pw));
		g.by_ph = FastDiv(static_cast<uint32_t>(g.ph));
		const long long inner = static_cast<long long>(g.coarse_w) * g.ph * g.pw * g.pieces;
		MB200_REQUIRE(context, inner < (1ll << 31), "%s: a row of %lld pieces is too long", who, inner);
		const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(static_cast<long long>(g.batch) * g.coarse_h,
				static_cast<long long>(get(context)->sm_count) * 16)));
		cudaStream_t stream = use_stream(context);
		void *d = const_cast<void*>(deep), *f = const_cast<void*>(flat);
		switch (piece)
		{
			case 16:
				kernel_rearrange<uint4, TO_DEPTH> <<<grid, 256, 0, stream>>>(reinterpret_cast<uint4*>(d), reinterpret_cast<uint4*>(f), g);
				break;
			case 8:
				kernel_rearrange<uint2, TO_DEPTH> <<<grid, 256, 0, stream>>>(reinterpret_cast<uint2*>(d), reinterpret_cast<uint2*>(f), g);
				break;
			case 4:
				kernel_rearrange<uint32_t, TO_DEPTH> <<<grid, 256, 0, stream>>>(reinterpret_cast<uint32_t*>(d), reinterpret_cast<uint32_t*>(f), g);
				break;
			case 2:
				kernel_rearrange<uint16_t, TO_DEPTH> <<<grid, 256, 0, stream>>>(reinterpret_cast<uint16_t*>(d), reinterpret_cast<uint16_t*>(f), g);
				break;
			default:
				kernel_rearrange<uint8_t, TO_DEPTH> <<<grid, 256, 0, stream>>>(reinterpret_cast<uint8_t*>(d), reinterpret_cast<uint8_t*>(f), g);
				break;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), who);
	}
}

extern "C"
{
	void cuda_rmsnorm_forward(mlContext_t context, mlShape_t shape, mlDataType_t dtype, const void *input, void *output, const void *weights)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_rmsnorm_forward: null context");
		if (volume(shape) == 0)
			return; // an empty problem: nothing to validate or launch
		MB200_REQUIRE(context, input != nullptr && output != nullptr, "cuda_rmsnorm_forward: null pointer");
		flush_pending(context);
		const long long rows = volume_without_last_dim(shape);
		const int channels = last_dim(shape);
		cudaStream_t stream = use_stream(context);
		switch (dtype)
		{
			case DTYPE_FLOAT16:
				launch_rmsnorm<__half>(context, stream, output, input, weights, rows, channels);
				break;
			case DTYPE_FLOAT32:
				launch_rmsnorm<float>(context, stream, output, input, weights, rows, channels);
				break;
			default:
				record_error(context, "cuda_rmsnorm_forward: dtype %d not supported", static_cast<int>(dtype));
				return;
		}
		check_cuda(context, cudaGetLastError(), "cuda_rmsnorm_forward");
	}
	void cuda_space_to_depth(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, const void *input, mlShape_t output_shape, void *output)
	{
		rearrange<true>(context, "cuda_space_to_depth", dtype, input_shape, input, output_shape, output);
	}
	void cuda_depth_to_space(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, const void *input, mlShape_t output_shape, void *output)
	{
		rearrange<false>(context, "cuda_depth_to_space", dtype, output_shape, output, input_shape, input);
	}
}
