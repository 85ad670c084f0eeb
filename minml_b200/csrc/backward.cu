/*
 * backward.cu -- the mirror image of the Winograd forward path, for Conv2D::backward (src/layers/Conv2D.cpp:383-448):
 *
 *   cuda_winograd_gradient_transform   dy [b,h,w,cout] -> matrices [p*p, tiles, cout],  M = Gr d Gr^T on tile x tile pieces of dy
 *                                      (src/backend/cuda/kernels/winograd_nonfused.cu:182-212,472-489)
 *   cuda_winograd_update_transform     matrices [p*p, cout, cin] -> dw [cout,k,k,cin],  dw = Up M Up^T
 *                                      (winograd_nonfused.cu:214-239,490-510)
 *   cuda_activation_backward           dx = alpha * dy * act'(y) + beta * dx   (src/backend/cuda/kernels/activations.cu:50-62,216-245)
 *   cuda_fused_act_bias_copy_backward  dy <- dy * act'(y) in place; db <- beta_db * db + column sums of dy; dx <- dy + beta_dx * dx
 *                                      (src/backend/cuda/kernels/tensor_op.cu:195-270,527-580)
 *
 * The matrix products in between (gradient matrices x transformed weights, 'n','n'; gradient matrices^T x input matrices, 't','n')
 * go through cuda_gemm_batched_v2's generic engine.  Transform matrices: winograd_transforms.cuh:95-135,205-250,304-352.
 * All three kernels move each element once; arithmetic is fp32 whatever the storage type.
 */
#include "common.cuh"

#include <cuda_fp16.h>

#include <algorithm>

using namespace mb200;

namespace
{
	__device__ __forceinline__ float to_float(float v) { return v; }
	__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
	template<typename T> __device__ __forceinline__ T from_float(float v);
	template<> __device__ __forceinline__ float from_float<float>(float v) { return v; }
	template<> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

	/* Gr: (k + tile - 1) x tile, Up: k x (k + tile - 1); rows beyond a configuration's size are unused. */
	template<int K, int TILE> struct Backward;
	template<> struct Backward<3, 2>
	{
			__device__ static float gr(int r, int c)
			{
				const float m[4][2] = { { 1, 0 }, { 1, 1 }, { 1, -1 }, { 0, 1 } };
				return m[r][c];
			}
			__device__ static float up(int r, int c)
			{
				const float m[3][4] = { { 1, 0.5f, 0.5f, 0 }, { 0, 0.5f, -0.5f, 0 }, { 0, 0.5f, 0.5f, 1 } };
				return m[r][c];
			}
	};
	template<> struct Backward<3, 4>
	{
			__device__ static float gr(int r, int c)
			{
				const float a = 1.0f / 3.0f, b = 2.0f / 3.0f;
				const float m[6][4] = { { 1, 0, 0, 0 }, { b, b, b, b }, { b, -b, b, -b }, { a, 2 * a, 4 * a, 8 * a }, { a, -2 * a, 4 * a, -8 * a },
						{ 0, 0, 0, 2 } };
				return m[r][c];
			}
			__device__ static float up(int r, int c)
			{
				const float m[3][6] = { { 1, 1, 1, 0.25f, 0.25f, 0 }, { 0, 1, -1, 0.5f, -0.5f, 0 }, { 0, 1, 1, 1, 1, 2 } };
				return m[r][c];
			}
	};
	template<> struct Backward<5, 2>
	{
			__device__ static float gr(int r, int c)
			{
				const float a = 1.0f / 3.0f, b = 2.0f / 3.0f;
				const float m[6][2] = { { 1, 0 }, { b, b }, { b, -b }, { a, 2 * a }, { a, -2 * a }, { 0, 1 } };
				return m[r][c];
			}
			__device__ static float up(int r, int c)
			{
				const float m[5][6] = { { 1, 1, 1, 0.25f, 0.25f, 0 }, { 0, 1, -1, 0.5f, -0.5f, 0 }, { 0, 1, 1, 1, 1, 0 }, { 0, 1, -1, 2, -2, 0 },
						{ 0, 1, 1, 4, 4, 4 } };
				return m[r][c];
			}
	};

	/* grid (tiles_h, tiles_w, batch), threads over channels */
	template<typename T, int K, int TILE>
	__global__ void __launch_bounds__(128) kernel_gradient_transform(T *__restrict__ matrices, const T *__restrict__ dy, int height, int width,
			int channels)
	{
		constexpr int P = K + TILE - 1;
		const long long tiles = static_cast<long long>(gridDim.x) * gridDim.y * gridDim.z;
		const long long t = (static_cast<long long>(blockIdx.z) * gridDim.x + blockIdx.x) * gridDim.y + blockIdx.y;
		for (int c = threadIdx.x; c < channels; c += blockDim.x)
		{
			float d[TILE][TILE];
#pragma unroll
			for (int r = 0; r < TILE; r++)
#pragma unroll
				for (int q = 0; q < TILE; q++)
				{
					const int h = TILE * blockIdx.x + r, w = TILE * blockIdx.y + q;
					d[r][q] = (h < height && w < width) ? to_float(dy[((static_cast<long long>(blockIdx.z) * height + h) * width + w) * channels + c]) : 0.0f;
				}
			float tmp[P][TILE];
#pragma unroll
			for (int i = 0; i < P; i++)
#pragma unroll
				for (int q = 0; q < TILE; q++)
				{
					float s = 0.0f;
#pragma unroll
					for (int r = 0; r < TILE; r++)
						s += Backward<K, TILE>::gr(i, r) * d[r][q];
					tmp[i][q] = s;
				}
#pragma unroll
			for (int i = 0; i < P; i++)
#pragma unroll
				for (int j = 0; j < P; j++)
				{
					float s = 0.0f;
#pragma unroll
					for (int q = 0; q < TILE; q++)
						s += tmp[i][q] * Backward<K, TILE>::gr(j, q);
					matrices[(static_cast<long long>(i * P + j) * tiles + t) * channels + c] = from_float<T>(s);
				}
		}
	}
	/* grid (cout), threads over cin */
	template<typename T, typename U, int K, int TILE>
	__global__ void __launch_bounds__(128) kernel_update_transform(U *__restrict__ dw, const T *__restrict__ matrices, int cout, int cin)
	{
		constexpr int P = K + TILE - 1;
		const int co = blockIdx.x;
		for (int ci = threadIdx.x; ci < cin; ci += blockDim.x)
		{
			float d[P][P];
#pragma unroll
			for (int r = 0; r < P; r++)
#pragma unroll
				for (int q = 0; q < P; q++)
					d[r][q] = to_float(matrices[(static_cast<long long>(r * P + q) * cout + co) * cin + ci]);
			float tmp[K][P];
#pragma unroll
			for (int i = 0; i < K; i++)
#pragma unroll
				for (int q = 0; q < P; q++)
				{
					float s = 0.0f;
#pragma unroll
					for (int r = 0; r < P; r++)
						s += Backward<K, TILE>::up(i, r) * d[r][q];
					tmp[i][q] = s;
				}
#pragma unroll
			for (int i = 0; i < K; i++)
#pragma unroll
				for (int j = 0; j < K; j++)
				{
					float s = 0.0f;
#pragma unroll
					for (int q = 0; q < P; q++)
						s += tmp[i][q] * Backward<K, TILE>::up(j, q);
					dw[((static_cast<long long>(co) * K + i) * K + j) * cin + ci] = from_float<U>(s);
				}
		}
	}

	/* block (32 channels, 8 row lanes), grid (channel blocks, row blocks): column sums are reduced in shared memory and added to
	 * db with one atomic per block and channel (db has been scaled by beta_db beforehand). */
	template<typename T>
	__global__ void __launch_bounds__(256) kernel_act_bias_copy_backward(T *dy, const T *__restrict__ y, T *dx, T *db, float beta_dx, long long rows,
			int channels, int act)
	{
		__shared__ float partial[8][33];
		const int c = blockIdx.x * 32 + threadIdx.x;
		float sum = 0.0f;
		if (c < channels)
		{
			for (long long r = static_cast<long long>(blockIdx.y) * 8 + threadIdx.y; r < rows; r += static_cast<long long>(gridDim.y) * 8)
			{
				const long long i = r * channels + c;
				float g = to_float(dy[i]);
				if (act != ACTIVATION_LINEAR)
				{
					const float v = to_float(y[i]);
					switch (act)
					{
						case ACTIVATION_SIGMOID:
							g *= v * (1.0f - v);
							break;
						case ACTIVATION_TANH:
							g *= 1.0f - v * v;
							break;
						case ACTIVATION_RELU:
							g = (v > 0.0f) ? g : 0.0f;
							break;
						case ACTIVATION_LEAKY_RELU:
							g = (v > 0.0f) ? g : g * 0.1f;
							break;
						default:
							break;
					}
					dy[i] = from_float<T>(g);
					g = to_float(from_float<T>(g)); // what the next reader of dy sees
				}
				sum += g;
				if (dx != nullptr)
					dx[i] = from_float<T>((beta_dx != 0.0f) ? g + beta_dx * to_float(dx[i]) : g);
			}
		}
		if (db == nullptr)
			return;
		partial[threadIdx.y][threadIdx.x] = sum;
		__syncthreads();
		if (threadIdx.y == 0 && c < channels)
		{
			float total = 0.0f;
#pragma unroll
			for (int k = 0; k < 8; k++)
				total += partial[k][threadIdx.x];
			atomicAdd(db + c, from_float<T>(total));
		}
	}

	__device__ __forceinline__ float activation_derivative(float y, int act)
	{
		switch (act)
		{
			case ACTIVATION_SIGMOID:
				return y * (1.0f - y);
			case ACTIVATION_TANH:
				return 1.0f - y * y;
			case ACTIVATION_RELU:
				return (y > 0.0f) ? 1.0f : 0.0f;
			case ACTIVATION_LEAKY_RELU:
				return (y > 0.0f) ? 1.0f : 0.1f;
			case ACTIVATION_EXP:
				return y;
			default:
				return 1.0f;
		}
	}
	/* dx = alpha * dy * act'(y) + beta * dx  (src/backend/cuda/kernels/activations.cu:50-62,216-245) */
	template<typename T>
	__global__ void __launch_bounds__(256) kernel_activation_backward(T *dx, const T *__restrict__ dy, const T *__restrict__ y, long long elements,
			float alpha, float beta, int act)
	{
		for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < elements; i += static_cast<long long>(gridDim.x) * blockDim.x)
		{
			float g = to_float(dy[i]) * activation_derivative(to_float(y[i]), act) * alpha;
			if (beta != 0.0f)
				g += beta * to_float(dx[i]);
			dx[i] = from_float<T>(g);
		}
	}

	template<typename T>
	bool launch_gradient(cudaStream_t stream, int k, int tile, T *matrices, const T *dy, int batch, int height, int width, int channels)
	{
		const dim3 grid(ceil_div(height, tile), ceil_div(width, tile), batch);
		const int block = std::min(128, std::max(32, channels));
		if (k == 3 && tile == 2)
			kernel_gradient_transform<T, 3, 2> <<<grid, block, 0, stream>>>(matrices, dy, height, width, channels);
		else if (k == 3 && tile == 4)
			kernel_gradient_transform<T, 3, 4> <<<grid, block, 0, stream>>>(matrices, dy, height, width, channels);
		else if (k == 5 && tile == 2)
			kernel_gradient_transform<T, 5, 2> <<<grid, block, 0, stream>>>(matrices, dy, height, width, channels);
		else
			return false;
		return true;
	}
	template<typename T, typename U>
	bool launch_update(cudaStream_t stream, int k, int tile, U *dw, const T *matrices, int cout, int cin)
	{
		const int block = std::min(128, std::max(32, cin));
		if (k == 3 && tile == 2)
			kernel_update_transform<T, U, 3, 2> <<<cout, block, 0, stream>>>(dw, matrices, cout, cin);
		else if (k == 3 && tile == 4)
			kernel_update_transform<T, U, 3, 4> <<<cout, block, 0, stream>>>(dw, matrices, cout, cin);
		else if (k == 5 && tile == 2)
			kernel_update_transform<T, U, 5, 2> <<<cout, block, 0, stream>>>(dw, matrices, cout, cin);
		else
			return false;
		return true;
	}
	int patch_of(const mlTensor_t &matrices)
	{
		int p = 0;
		while (p * p < matrices.dim[0])
			p++;
		return (p * p == matrices.dim[0]) ? p : 0;
	}
}

extern "C"
{
	void cuda_winograd_gradient_transform(mlContext_t context, int tile_size, const mlTensor_t dy, mlTensor_t matrices)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_winograd_gradient_transform: null context");
		if (volume(dy) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, dy.rank == 4 && matrices.rank == 3 && dy.data != nullptr && matrices.data != nullptr && dy.dtype == matrices.dtype,
				"cuda_winograd_gradient_transform: dy [b,h,w,c] and matrices [p*p,tiles,c] of one type");
		const int p = patch_of(matrices), k = p - tile_size + 1;
		const long long tiles = static_cast<long long>(dy.dim[0]) * ceil_div(dy.dim[1], std::max(1, tile_size)) * ceil_div(dy.dim[2], std::max(1, tile_size));
		MB200_REQUIRE(context, p > 0 && tile_size > 0 && matrices.dim[1] == tiles && matrices.dim[2] == dy.dim[3],
				"cuda_winograd_gradient_transform: matrices do not match dy for tile size %d", tile_size);
		MB200_REQUIRE(context, dy.dim[0] <= 65535 && ceil_div(dy.dim[2], tile_size) <= 65535, "cuda_winograd_gradient_transform: too many tiles for one launch");
		flush_pending(context);
		if (volume(dy) == 0)
			return;
		cudaStream_t stream = use_stream(context);
		bool ok = false;
		if (dy.dtype == DTYPE_FLOAT16)
			ok = launch_gradient<__half>(stream, k, tile_size, reinterpret_cast<__half*>(matrices.data), reinterpret_cast<const __half*>(dy.data), dy.dim[0],
					dy.dim[1], dy.dim[2], dy.dim[3]);
		else if (dy.dtype == DTYPE_FLOAT32)
			ok = launch_gradient<float>(stream, k, tile_size, reinterpret_cast<float*>(matrices.data), reinterpret_cast<const float*>(dy.data), dy.dim[0],
					dy.dim[1], dy.dim[2], dy.dim[3]);
		MB200_REQUIRE(context, ok, "cuda_winograd_gradient_transform: kernel %d, tile %d, dtype %d not supported", k, tile_size, static_cast<int>(dy.dtype));
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_winograd_gradient_transform");
	}
	void cuda_winograd_update_transform(mlContext_t context, int tile_size, const mlTensor_t matrices, mlTensor_t dw)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_winograd_update_transform: null context");
		if (volume(dw) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, matrices.rank == 3 && dw.rank == 4 && matrices.data != nullptr && dw.data != nullptr,
				"cuda_winograd_update_transform: matrices [p*p,cout,cin] and dw [cout,k,k,cin]");
		const int p = patch_of(matrices), k = p - tile_size + 1;
		MB200_REQUIRE(context, p > 0 && dw.dim[1] == k && dw.dim[2] == k && matrices.dim[1] == dw.dim[0] && matrices.dim[2] == dw.dim[3],
				"cuda_winograd_update_transform: matrices do not match dw for tile size %d", tile_size);
		flush_pending(context);
		if (volume(dw) == 0)
			return;
		cudaStream_t stream = use_stream(context);
		const int cout = dw.dim[0], cin = dw.dim[3];
		bool ok = false;
		if (matrices.dtype == DTYPE_FLOAT16 && dw.dtype == DTYPE_FLOAT16)
			ok = launch_update<__half, __half>(stream, k, tile_size, reinterpret_cast<__half*>(dw.data), reinterpret_cast<const __half*>(matrices.data), cout, cin);
		else if (matrices.dtype == DTYPE_FLOAT16 && dw.dtype == DTYPE_FLOAT32)
			ok = launch_update<__half, float>(stream, k, tile_size, reinterpret_cast<float*>(dw.data), reinterpret_cast<const __half*>(matrices.data), cout, cin);
		else if (matrices.dtype == DTYPE_FLOAT32 && dw.dtype == DTYPE_FLOAT32)
			ok = launch_update<float, float>(stream, k, tile_size, reinterpret_cast<float*>(dw.data), reinterpret_cast<const float*>(matrices.data), cout, cin);
		MB200_REQUIRE(context, ok, "cuda_winograd_update_transform: kernel %d, tile %d or dtypes %d -> %d not supported", k, tile_size,
				static_cast<int>(matrices.dtype), static_cast<int>(dw.dtype));
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_winograd_update_transform");
	}
	void cuda_activation_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t y, float beta, mlTensor_t dx,
			mlActivationType_t act)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_activation_backward: null context");
		if (volume(dy) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, dy.data != nullptr && y.data != nullptr && dx.data != nullptr && volume(dy) == volume(y) && volume(dy) == volume(dx)
				&& dy.dtype == y.dtype && dy.dtype == dx.dtype, "cuda_activation_backward: dy, y and dx must match");
		flush_pending(context);
		const long long elements = volume(dy);
		if (elements == 0)
			return;
		cudaStream_t stream = use_stream(context);
		const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((elements + 255) / 256, static_cast<long long>(get(context)->sm_count) * 16)));
		if (dy.dtype == DTYPE_FLOAT16)
			kernel_activation_backward<__half> <<<grid, 256, 0, stream>>>(reinterpret_cast<__half*>(dx.data), reinterpret_cast<const __half*>(dy.data),
					reinterpret_cast<const __half*>(y.data), elements, alpha, beta, act);
		else if (dy.dtype == DTYPE_FLOAT32)
			kernel_activation_backward<float> <<<grid, 256, 0, stream>>>(reinterpret_cast<float*>(dx.data), reinterpret_cast<const float*>(dy.data),
					reinterpret_cast<const float*>(y.data), elements, alpha, beta, act);
		else
		{
			record_error(context, "cuda_activation_backward: dtype %d not supported", static_cast<int>(dy.dtype));
			return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_activation_backward");
	}
	void cuda_fused_act_bias_copy_backward(mlContext_t context, mlTensor_t dy, const mlTensor_t y, float beta_dx, mlTensor_t dx, float beta_dw,
			mlTensor_t dw, mlActivationType_t act)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_fused_act_bias_copy_backward: null context");
		if (volume(dy) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, dy.data != nullptr && y.data != nullptr && volume(dy) == volume(y) && dy.dtype == y.dtype,
				"cuda_fused_act_bias_copy_backward: dy and y must match");
		MB200_REQUIRE(context, dx.data == nullptr || (volume(dx) == volume(dy) && dx.dtype == dy.dtype),
				"cuda_fused_act_bias_copy_backward: dx must match dy");
		MB200_REQUIRE(context, dw.data == nullptr || (volume(dw) == last_dim(dy) && dw.dtype == dy.dtype),
				"cuda_fused_act_bias_copy_backward: the bias gradient must be [channels] of dy's type");
		flush_pending(context);
		const long long rows = volume_without_last_dim(dy);
		const int channels = last_dim(dy);
		if (rows == 0 || channels == 0)
			return;
		cudaStream_t stream = use_stream(context);
		if (dw.data != nullptr)
		{ // db <- beta * db first; the kernel then adds the column sums atomically
			if (beta_dw == 0.0f)
				check_cuda(context, cudaMemsetAsync(dw.data, 0, static_cast<size_t>(channels) * size_of(dw.dtype), stream), "cuda_fused_act_bias_copy_backward");
			else
				cuda_scale_tensor(context, beta_dw, dw);
		}
		const dim3 block(32, 8);
		const dim3 grid(ceil_div(channels, 32), static_cast<unsigned>(std::max<long long>(1, std::min<long long>((rows + 7) / 8, 1024))));
		if (dy.dtype == DTYPE_FLOAT16)
			kernel_act_bias_copy_backward<__half> <<<grid, block, 0, stream>>>(reinterpret_cast<__half*>(dy.data), reinterpret_cast<const __half*>(y.data),
					reinterpret_cast<__half*>(dx.data), reinterpret_cast<__half*>(dw.data), beta_dx, rows, channels, act);
		else if (dy.dtype == DTYPE_FLOAT32)
			kernel_act_bias_copy_backward<float> <<<grid, block, 0, stream>>>(reinterpret_cast<float*>(dy.data), reinterpret_cast<const float*>(y.data),
					reinterpret_cast<float*>(dx.data), reinterpret_cast<float*>(dw.data), beta_dx, rows, channels, act);
		else
		{
			record_error(context, "cuda_fused_act_bias_copy_backward: dtype %d not supported", static_cast<int>(dy.dtype));
			return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_fused_act_bias_copy_backward");
	}
}
