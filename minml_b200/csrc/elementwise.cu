/*
 * elementwise.cu -- bandwidth-bound entry points: bias + activation, activation, tensor sums, input unpacking,
 * dtype conversion, [d0,d1,d2] -> [d0,d2,d1] transposition, global average pooling and row softmax.
 *
 * Replaces src/backend/cuda/kernels/activations.cu:36-84,190-284, tensor_op.cu:290-363, conversion.cu:35-54,196-300,
 * global_pooling.cu:29-73,269-314 and softmax.cu:123-173 of the reference.
 *
 * Every kernel moves 16 bytes per thread per access when the pointers and the channel count allow it, keeps the
 * arithmetic in fp32, and is launched with a grid that is a multiple of the SM count (grid-stride loops).
 */
#include "common.cuh"

namespace mb200
{
	namespace
	{
		/* 16-byte packet of N elements of T, converted to and from fp32 */
		template<typename T> struct Vec16;
		template<> struct Vec16<float>
		{
				static constexpr int N = 4;
				__device__ static void load(const float *p, float (&v)[4])
				{
					const float4 t = *reinterpret_cast<const float4*>(p);
					v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
				}
				__device__ static void store(float *p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
		};
		template<> struct Vec16<__half>
		{
				static constexpr int N = 8;
				__device__ static void load(const __half *p, float (&v)[8])
				{
					const uint4 raw = *reinterpret_cast<const uint4*>(p);
					const uint32_t w[4] = { raw.x, raw.y, raw.z, raw.w };
#pragma unroll
					for (int i = 0; i < 4; i++)
					{
						const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
						v[2 * i] = f.x;
						v[2 * i + 1] = f.y;
					}
				}
				__device__ static void store(__half *p, const float (&v)[8])
				{
					uint32_t w[4];
#pragma unroll
					for (int i = 0; i < 4; i++)
					{
						const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
						w[i] = *reinterpret_cast<const uint32_t*>(&h);
					}
					*reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
				}
		};
		template<> struct Vec16<double>
		{
				static constexpr int N = 2;
				__device__ static void load(const double *p, float (&v)[2])
				{
					const double2 t = *reinterpret_cast<const double2*>(p);
					v[0] = static_cast<float>(t.x); v[1] = static_cast<float>(t.y);
				}
				__device__ static void store(double *p, const float (&v)[2]) { *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]); }
		};

		inline int grid_for(long long work_items, int block, int sm_count)
		{
			const long long blocks = (work_items + block - 1) / block;
			return static_cast<int>(std::max<long long>(1, std::min<long long>(blocks, static_cast<long long>(sm_count) * 16)));
		}

		/* y = act(x + bias[c]) * alpha + beta * y  over [rows, channels].
		 * These kernels are bound by instruction issue before they are bound by memory when written naively (a 64-bit modulo
		 * and a switch over the activation per element cost more than the 16-byte load they accompany), so: ACT is a compile-time
		 * class (0 linear, 1 ReLU, 2 decided at run time), PLAIN drops alpha and beta, and the channel offset of a thread's next
		 * packet is advanced by a precomputed step instead of being recomputed with a division. */
		template<typename T, bool VECTOR, int ACT, bool PLAIN>
		__global__ void __launch_bounds__(256) kernel_bias_act(T *__restrict__ y, const T *__restrict__ x, const T *__restrict__ bias, long long rows,
				int channels, float alpha, float beta, int act)
		{
			constexpr int N = VECTOR ? Vec16<T>::N : 1;
			const long long total = rows * channels / N;
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
			const int groups = channels / N; // packets per row
			int g = static_cast<int>(first % groups);
			const int g_step = static_cast<int>(stride % groups);
			for (long long i = first; i < total; i += stride)
			{
				const long long e = i * N;
				float v[N];
				if constexpr (VECTOR)
					Vec16<T>::load(x + e, reinterpret_cast<float (&)[Vec16<T>::N]>(v));
				else
					v[0] = to_float(x[e]);
				if (bias != nullptr)
				{
					float b[N];
					if constexpr (VECTOR)
						Vec16<T>::load(bias + g * N, reinterpret_cast<float (&)[Vec16<T>::N]>(b));
					else
						b[0] = to_float(bias[g]);
#pragma unroll
					for (int k = 0; k < N; k++)
						v[k] += b[k];
				}
#pragma unroll
				for (int k = 0; k < N; k++)
				{
					if (ACT == 1)
						v[k] = fmaxf(v[k], 0.0f);
					else if (ACT == 2)
						v[k] = apply_activation(v[k], act);
				}
				if (!PLAIN)
				{
#pragma unroll
					for (int k = 0; k < N; k++)
						v[k] *= alpha;
					if (beta != 0.0f)
					{
						float o[N];
						if constexpr (VECTOR)
							Vec16<T>::load(y + e, reinterpret_cast<float (&)[Vec16<T>::N]>(o));
						else
							o[0] = to_float(y[e]);
#pragma unroll
						for (int k = 0; k < N; k++)
							v[k] += beta * o[k];
					}
				}
				if constexpr (VECTOR)
					Vec16<T>::store(y + e, reinterpret_cast<const float (&)[Vec16<T>::N]>(v));
				else
					y[e] = from_float<T>(v[0]);
				g += g_step;
				if (g >= groups)
					g -= groups;
			}
		}
		template<typename T, bool VECTOR>
		void launch_bias_act_variant(cudaStream_t stream, int grid, T *y, const T *x, const T *bias, long long rows, int channels, float alpha,
				float beta, int act)
		{
			const bool plain = alpha == 1.0f && beta == 0.0f;
			const int cls = (act == ACTIVATION_LINEAR) ? 0 : (act == ACTIVATION_RELU ? 1 : 2);
#define VARIANT(A, P) kernel_bias_act<T, VECTOR, A, P> <<<grid, 256, 0, stream>>>(y, x, bias, rows, channels, alpha, beta, act)
			if (plain)
			{
				if (cls == 0)
					VARIANT(0, true);
				else if (cls == 1)
					VARIANT(1, true);
				else
					VARIANT(2, true);
			}
			else
			{
				if (cls == 1)
					VARIANT(1, false);
				else
					VARIANT(2, false); // apply_activation passes linear through
			}
#undef VARIANT
		}
		template<typename T>
		void launch_bias_act(mlContext_t ctx, void *y, const void *x, const void *bias, long long rows, int channels, float alpha, float beta,
				int act)
		{
			cudaStream_t stream = use_stream(ctx);
			const int sm = get(ctx)->sm_count;
			const bool vec = channels % Vec16<T>::N == 0 && aligned_to(y, 16) && aligned_to(x, 16) && (bias == nullptr || aligned_to(bias, 16));
			if (vec)
				launch_bias_act_variant<T, true>(stream, grid_for(rows * channels / Vec16<T>::N, 256, sm), reinterpret_cast<T*>(y),
						reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(bias), rows, channels, alpha, beta, act);
			else
				launch_bias_act_variant<T, false>(stream, grid_for(rows * channels, 256, sm), reinterpret_cast<T*>(y), reinterpret_cast<const T*>(x),
						reinterpret_cast<const T*>(bias), rows, channels, alpha, beta, act);
			MB200_COUNT_LAUNCH();
		}

		/* y = a1*x1 + a2*x2 + a3*x3 + beta*y */
		template<typename T, bool VECTOR>
		__global__ void __launch_bounds__(256) kernel_axpy3(T *y, const T *x1, const T *x2, const T *x3, float a1, float a2, float a3, float beta,
				long long elements)
		{
			constexpr int N = VECTOR ? Vec16<T>::N : 1;
			const long long total = elements / N;
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
			{
				const long long e = i * N;
				float acc[N];
#pragma unroll
				for (int k = 0; k < N; k++)
					acc[k] = 0.0f;
				const T *src[4] = { x1, x2, x3, y };
				const float coef[4] = { a1, a2, a3, beta };
#pragma unroll
				for (int s = 0; s < 4; s++)
					if (src[s] != nullptr && coef[s] != 0.0f)
					{
						float v[N];
						if constexpr (VECTOR)
							Vec16<T>::load(src[s] + e, reinterpret_cast<float (&)[Vec16<T>::N]>(v));
						else
							v[0] = to_float(src[s][e]);
#pragma unroll
						for (int k = 0; k < N; k++)
							acc[k] += coef[s] * v[k];
					}
				if constexpr (VECTOR)
					Vec16<T>::store(y + e, reinterpret_cast<const float (&)[Vec16<T>::N]>(acc));
				else
					y[e] = from_float<T>(acc[0]);
			}
		}
		template<typename T>
		void launch_axpy3(mlContext_t ctx, void *y, const void *x1, const void *x2, const void *x3, float a1, float a2, float a3, float beta,
				long long elements)
		{
			cudaStream_t stream = use_stream(ctx);
			const int sm = get(ctx)->sm_count;
			const bool vec = elements % Vec16<T>::N == 0 && aligned_to(y, 16) && (x1 == nullptr || aligned_to(x1, 16))
					&& (x2 == nullptr || aligned_to(x2, 16)) && (x3 == nullptr || aligned_to(x3, 16));
			if (vec)
				kernel_axpy3<T, true> <<<grid_for(elements / Vec16<T>::N, 256, sm), 256, 0, stream>>>(reinterpret_cast<T*>(y),
						reinterpret_cast<const T*>(x1), reinterpret_cast<const T*>(x2), reinterpret_cast<const T*>(x3), a1, a2, a3, beta, elements);
			else
				kernel_axpy3<T, false> <<<grid_for(elements, 256, sm), 256, 0, stream>>>(reinterpret_cast<T*>(y), reinterpret_cast<const T*>(x1),
						reinterpret_cast<const T*>(x2), reinterpret_cast<const T*>(x3), a1, a2, a3, beta, elements);
			MB200_COUNT_LAUNCH();
		}

		/* bit-packed planes -> {0, 1}: channel j of a position is bit (j % 32) of its word j / 32 */
		template<typename T> __device__ __forceinline__ T one_of() { return static_cast<T>(1); }
		template<> __device__ __forceinline__ __half one_of<__half>() { return __float2half(1.0f); }
		template<typename T> __device__ __forceinline__ T zero_of() { return static_cast<T>(0); }
		template<> __device__ __forceinline__ __half zero_of<__half>() { return __float2half(0.0f); }

		template<typename T>
		__global__ void __launch_bounds__(256) kernel_unpack(T *__restrict__ dst, const uint32_t *__restrict__ src, long long rows, int channels)
		{
			const int words = (channels + 31) / 32;
			const long long total = rows * channels;
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
			{
				const long long r = i / channels;
				const int j = static_cast<int>(i % channels);
				const uint32_t word = src[r * words + j / 32];
				dst[i] = ((word >> (j % 32)) & 1u) ? one_of<T>() : zero_of<T>();
			}
		}

		/* The same for 8 consecutive channels per thread (channels a multiple of 8, aligned destination): one byte of the
		 * position's word becomes one store of 8 elements; row and channel group advance without divisions. */
		template<typename T>
		struct alignas(sizeof(T) * 8 > 16 ? 16 : sizeof(T) * 8) Unpacked8
		{
				T v[8];
		};
		template<typename T>
		__global__ void __launch_bounds__(256) kernel_unpack_groups(T *__restrict__ dst, const uint32_t *__restrict__ src, long long rows, int channels)
		{
			const int words = (channels + 31) / 32;
			const int groups = channels / 8;
			const long long total = rows * groups;
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
			long long r = first / groups;
			int g = static_cast<int>(first - r * groups);
			const long long r_step = stride / groups;
			const int g_step = static_cast<int>(stride - r_step * groups);
			for (long long i = first; i < total; i += stride)
			{
				const uint32_t bits = src[r * words + g / 4] >> ((g % 4) * 8);
				Unpacked8<T> out;
#pragma unroll
				for (int k = 0; k < 8; k++)
					out.v[k] = ((bits >> k) & 1u) ? one_of<T>() : zero_of<T>();
				reinterpret_cast<Unpacked8<T>*>(dst)[i] = out;
				r += r_step;
				g += g_step;
				if (g >= groups)
				{
					g -= groups;
					r++;
				}
			}
		}
		template<typename T>
		void launch_unpack(cudaStream_t stream, int sm, void *dst, const uint32_t *src, long long rows, int channels)
		{
			if (channels % 8 == 0 && aligned_to(dst, 16))
				kernel_unpack_groups<T> <<<grid_for(rows * (channels / 8), 256, sm), 256, 0, stream>>>(reinterpret_cast<T*>(dst), src, rows, channels);
			else
				kernel_unpack<T> <<<grid_for(rows * channels, 256, sm), 256, 0, stream>>>(reinterpret_cast<T*>(dst), src, rows, channels);
		}

		template<typename T> __device__ __forceinline__ float as_float(T x) { return static_cast<float>(x); }
		template<> __device__ __forceinline__ float as_float<__half>(__half x) { return __half2float(x); }
		template<typename T> __device__ __forceinline__ T float_as(float x) { return static_cast<T>(x); }
		template<> __device__ __forceinline__ __half float_as<__half>(float x) { return __float2half_rn(x); }

		template<typename D, typename S>
		__global__ void __launch_bounds__(256) kernel_convert(D *__restrict__ dst, const S *__restrict__ src, long long elements)
		{
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += stride)
				dst[i] = float_as<D>(as_float<S>(src[i])); // always through fp32, as the reference does (conversion.cu:53)
		}
		/* The same in groups of 8 consecutive elements per thread, two groups loaded before the first is converted. */
		template<typename T>
		struct alignas(sizeof(T) * 8 > 16 ? 16 : sizeof(T) * 8) Group8
		{
				T v[8];
		};
		template<typename D, typename S>
		__global__ void __launch_bounds__(256) kernel_convert_groups(D *__restrict__ dst, const S *__restrict__ src, long long groups)
		{
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < groups; i += 2 * stride)
			{
				const bool second = i + stride < groups;
				const Group8<S> a = reinterpret_cast<const Group8<S>*>(src)[i];
				Group8<S> b;
				if (second)
					b = reinterpret_cast<const Group8<S>*>(src)[i + stride];
				Group8<D> out;
#pragma unroll
				for (int k = 0; k < 8; k++)
					out.v[k] = float_as<D>(as_float<S>(a.v[k]));
				reinterpret_cast<Group8<D>*>(dst)[i] = out;
				if (second)
				{
#pragma unroll
					for (int k = 0; k < 8; k++)
						out.v[k] = float_as<D>(as_float<S>(b.v[k]));
					reinterpret_cast<Group8<D>*>(dst)[i + stride] = out;
				}
			}
		}
		template<typename D, typename S>
		void launch_convert(cudaStream_t stream, int sm, void *dst, const void *src, long long elements)
		{
			if (elements % 8 == 0 && aligned_to(dst, 16) && aligned_to(src, 16))
				kernel_convert_groups<D, S> <<<grid_for(elements / 16, 256, sm), 256, 0, stream>>>(reinterpret_cast<D*>(dst),
						reinterpret_cast<const S*>(src), elements / 8);
			else
				kernel_convert<D, S> <<<grid_for(elements, 256, sm), 256, 0, stream>>>(reinterpret_cast<D*>(dst), reinterpret_cast<const S*>(src), elements);
		}
		template<typename D>
		bool convert_from(cudaStream_t stream, int sm, void *dst, const void *src, mlDataType_t src_dtype, long long elements)
		{
#define CASE(E, S) case E: launch_convert<D, S>(stream, sm, dst, src, elements); break
			switch (src_dtype)
			{
				CASE(DTYPE_FLOAT16, __half);
				CASE(DTYPE_FLOAT32, float);
				CASE(DTYPE_FLOAT64, double);
				CASE(DTYPE_UINT8, uint8_t);
				CASE(DTYPE_INT8, int8_t);
				CASE(DTYPE_INT16, int16_t);
				CASE(DTYPE_INT32, int32_t);
				default:
					return false;
			}
#undef CASE
			MB200_COUNT_LAUNCH();
			return true;
		}

		/* [d0, d1, d2] -> [d0, d2, d1] through a padded 32 x 32 shared tile */
		template<typename T>
		__global__ void __launch_bounds__(256) kernel_transpose_021(T *__restrict__ dst, const T *__restrict__ src, int d1, int d2)
		{
			__shared__ T tile[32][33];
			const long long base = static_cast<long long>(blockIdx.z) * d1 * d2;
			const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
			for (int r = threadIdx.y; r < 32; r += 8)
				if (r0 + r < d1 && c0 + threadIdx.x < d2)
					tile[r][threadIdx.x] = src[base + static_cast<long long>(r0 + r) * d2 + c0 + threadIdx.x];
			__syncthreads();
			for (int c = threadIdx.y; c < 32; c += 8)
				if (c0 + c < d2 && r0 + threadIdx.x < d1)
					dst[base + static_cast<long long>(c0 + c) * d1 + r0 + threadIdx.x] = tile[threadIdx.x][c];
		}

		/* [b, hw, c] -> [b, c] mean.  One CTA per (batch item, slab of 32 * N channels): 8 warps split the positions,
		 * each lane owns N consecutive channels, partial sums meet in shared memory. */
		template<typename T, int N>
		__global__ void __launch_bounds__(256) kernel_global_avg_pool(T *__restrict__ y, const T *__restrict__ x, int hw, int channels, float alpha,
				float beta)
		{
			__shared__ float partial[8][32 * N];
			const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
			const int c = (blockIdx.x * 32 + lane) * N;
			const int b = blockIdx.y;
			float acc[N];
#pragma unroll
			for (int k = 0; k < N; k++)
				acc[k] = 0.0f;
			if (c < channels)
			{
				const T *px = x + static_cast<long long>(b) * hw * channels + c;
				for (int i = warp; i < hw; i += 8)
				{
					if constexpr (N == 1)
						acc[0] += to_float(px[static_cast<long long>(i) * channels]);
					else
					{
						float v[N];
						Vec16<T>::load(px + static_cast<long long>(i) * channels, reinterpret_cast<float (&)[Vec16<T>::N]>(v));
#pragma unroll
						for (int k = 0; k < N; k++)
							acc[k] += v[k];
					}
				}
			}
#pragma unroll
			for (int k = 0; k < N; k++)
				partial[warp][lane * N + k] = acc[k];
			__syncthreads();
			for (int j = threadIdx.x; j < 32 * N; j += 256)
			{
				const int cc = blockIdx.x * 32 * N + j;
				if (cc < channels)
				{
					float s = 0.0f;
#pragma unroll
					for (int w = 0; w < 8; w++)
						s += partial[w][j];
					s *= alpha / static_cast<float>(hw);
					T *py = y + static_cast<long long>(b) * channels + cc;
					if (beta != 0.0f)
						s += beta * to_float(*py);
					*py = from_float<T>(s);
				}
			}
		}

		/* softmax over the last dimension, one warp per row */
		template<typename T>
		__global__ void __launch_bounds__(256) kernel_softmax(T *__restrict__ y, const T *__restrict__ x, long long rows, int channels)
		{
			const int lane = threadIdx.x % 32;
			const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x / 32);
			for (long long r = static_cast<long long>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32; r < rows; r += warps)
			{
				const T *px = x + r * channels;
				float m = -3.0e38f;
				for (int j = lane; j < channels; j += 32)
					m = fmaxf(m, to_float(px[j]));
				for (int k = 16; k >= 1; k /= 2)
					m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, k));
				float s = 0.0f;
				for (int j = lane; j < channels; j += 32)
					s += expf(to_float(px[j]) - m);
				for (int k = 16; k >= 1; k /= 2)
					s += __shfl_xor_sync(0xffffffffu, s, k);
				const float inv = 1.0f / s;
				for (int j = lane; j < channels; j += 32)
					y[r * channels + j] = from_float<T>(expf(to_float(px[j]) - m) * inv);
			}
		}
		/* Rows of up to 32 * N * ITERS channels (N elements per 16-byte access, channels a multiple of N): every lane keeps its
		 * pieces of the row in registers, so the row is read once and all of a lane's loads are in flight together. */
		template<typename T, int ITERS>
		__global__ void __launch_bounds__(256) kernel_softmax_rows(T *__restrict__ y, const T *__restrict__ x, long long rows, int channels)
		{
			constexpr int N = Vec16<T>::N;
			const int lane = threadIdx.x % 32;
			const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x / 32);
			for (long long r = static_cast<long long>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32; r < rows; r += warps)
			{
				float v[ITERS][N];
#pragma unroll
				for (int i = 0; i < ITERS; i++)
				{
					const int c = (i * 32 + lane) * N;
					if (c < channels)
						Vec16<T>::load(x + r * channels + c, reinterpret_cast<float (&)[Vec16<T>::N]>(v[i]));
				}
				float m = -3.0e38f;
#pragma unroll
				for (int i = 0; i < ITERS; i++)
					if ((i * 32 + lane) * N < channels)
					{
#pragma unroll
						for (int k = 0; k < N; k++)
							m = fmaxf(m, v[i][k]);
					}
				for (int k = 16; k >= 1; k /= 2)
					m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, k));
				float s = 0.0f;
#pragma unroll
				for (int i = 0; i < ITERS; i++)
					if ((i * 32 + lane) * N < channels)
					{
#pragma unroll
						for (int k = 0; k < N; k++)
						{
							v[i][k] = expf(v[i][k] - m);
							s += v[i][k];
						}
					}
				for (int k = 16; k >= 1; k /= 2)
					s += __shfl_xor_sync(0xffffffffu, s, k);
				const float inv = 1.0f / s;
#pragma unroll
				for (int i = 0; i < ITERS; i++)
				{
					const int c = (i * 32 + lane) * N;
					if (c < channels)
					{
#pragma unroll
						for (int k = 0; k < N; k++)
							v[i][k] *= inv;
						Vec16<T>::store(y + r * channels + c, reinterpret_cast<const float (&)[Vec16<T>::N]>(v[i]));
					}
				}
			}
		}
		template<typename T>
		void launch_softmax(cudaStream_t stream, int grid, void *output, const void *input, long long rows, int channels)
		{
			T *yp = reinterpret_cast<T*>(output);
			const T *xp = reinterpret_cast<const T*>(input);
			constexpr int N = Vec16<T>::N;
			const bool wide = channels % N == 0 && aligned_to(yp, 16) && aligned_to(xp, 16);
			if (wide && channels <= 32 * N)
				kernel_softmax_rows<T, 1> <<<grid, 256, 0, stream>>>(yp, xp, rows, channels);
			else if (wide && channels <= 64 * N)
				kernel_softmax_rows<T, 2> <<<grid, 256, 0, stream>>>(yp, xp, rows, channels);
			else if (wide && channels <= 128 * N)
				kernel_softmax_rows<T, 4> <<<grid, 256, 0, stream>>>(yp, xp, rows, channels);
			else
				kernel_softmax<T> <<<grid, 256, 0, stream>>>(yp, xp, rows, channels);
		}
		/* dst = src1 * src2, element by element (fp16 through fp32; fp64 stays fp64) */
		template<typename T>
		__global__ void __launch_bounds__(256) kernel_multiply_packets(T *__restrict__ dst, const T *__restrict__ a, const T *__restrict__ b, long long packets)
		{
			constexpr int N = Vec16<T>::N;
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < packets; i += stride)
			{
				float x[N], y[N];
				Vec16<T>::load(a + i * N, x);
				Vec16<T>::load(b + i * N, y);
#pragma unroll
				for (int k = 0; k < N; k++)
					x[k] *= y[k];
				Vec16<T>::store(dst + i * N, x);
			}
		}
		template<typename T, typename ACC>
		__global__ void __launch_bounds__(256) kernel_multiply_elements(T *__restrict__ dst, const T *__restrict__ a, const T *__restrict__ b, long long elements)
		{
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += stride)
				dst[i] = static_cast<T>(static_cast<ACC>(a[i]) * static_cast<ACC>(b[i]));
		}
	}
} /* namespace mb200 */

using namespace mb200;

extern "C"
{
	void cuda_add_bias_act(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t b, float beta, mlTensor_t y, mlActivationType_t act)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_add_bias_act: null context");
		if (volume(x) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, x.data != nullptr && y.data != nullptr && b.data != nullptr, "cuda_add_bias_act: null tensor data");
		MB200_REQUIRE(context, x.dtype == y.dtype && x.dtype == b.dtype, "cuda_add_bias_act: dtypes differ");
		MB200_REQUIRE(context, volume(x) == volume(y) && last_dim(b) == last_dim(x), "cuda_add_bias_act: shapes do not match");
		flush_pending(context);
		const long long rows = volume_without_last_dim(x);
		const int channels = last_dim(x);
		if (rows == 0 || channels == 0)
			return;
		switch (x.dtype)
		{
			case DTYPE_FLOAT16:
				launch_bias_act<__half>(context, y.data, x.data, b.data, rows, channels, alpha, beta, act);
				break;
			case DTYPE_FLOAT32:
				launch_bias_act<float>(context, y.data, x.data, b.data, rows, channels, alpha, beta, act);
				break;
			case DTYPE_FLOAT64:
				launch_bias_act<double>(context, y.data, x.data, b.data, rows, channels, alpha, beta, act);
				break;
			default:
				record_error(context, "cuda_add_bias_act: dtype %d not supported", static_cast<int>(x.dtype));
				return;
		}
		check_cuda(context, cudaGetLastError(), "cuda_add_bias_act");
	}
	void cuda_activation_forward(mlContext_t context, float alpha, const mlTensor_t x, float beta, mlTensor_t y, mlActivationType_t act)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_activation_forward: null context");
		if (volume(x) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, x.data != nullptr && y.data != nullptr, "cuda_activation_forward: null tensor data");
		MB200_REQUIRE(context, x.dtype == y.dtype && volume(x) == volume(y), "cuda_activation_forward: x and y differ in dtype or size");
		const long long elements = volume(x);
		if (elements == 0)
			return;
		if (act == ACTIVATION_LINEAR)
		{ // the reference copies and ignores alpha and beta (src/backend/cuda/kernels/activations.cu:194-197)
			if (x.data != y.data)
				cuda_memcpy_within_device(context, y.data, 0, x.data, 0, static_cast<size_t>(elements) * size_of(x.dtype));
			return;
		}
		flush_pending(context);
		// viewed as [elements / 8, 8] so the 16-byte path applies whenever the element count allows it
		const int act_channels = (elements % 8 == 0) ? 8 : 1;
		const long long act_rows = elements / act_channels;
		switch (x.dtype)
		{
			case DTYPE_FLOAT16:
				launch_bias_act<__half>(context, y.data, x.data, nullptr, act_rows, act_channels, alpha, beta, act);
				break;
			case DTYPE_FLOAT32:
				launch_bias_act<float>(context, y.data, x.data, nullptr, act_rows, act_channels, alpha, beta, act);
				break;
			case DTYPE_FLOAT64:
				launch_bias_act<double>(context, y.data, x.data, nullptr, act_rows, act_channels, alpha, beta, act);
				break;
			default:
				record_error(context, "cuda_activation_forward: dtype %d not supported", static_cast<int>(x.dtype));
				return;
		}
		check_cuda(context, cudaGetLastError(), "cuda_activation_forward");
	}
	void cuda_add_tensors(mlContext_t context, float alpha1, const mlTensor_t x1, float alpha2, const mlTensor_t x2, float alpha3,
			const mlTensor_t x3, float beta, mlTensor_t y)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_add_tensors: null context");
		if (volume(y) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		const long long elements = volume(y);
		if (elements == 0 || y.data == nullptr)
			return;
		MB200_REQUIRE(context, (x1.data == nullptr || (x1.dtype == y.dtype && volume(x1) == elements))
				&& (x2.data == nullptr || (x2.dtype == y.dtype && volume(x2) == elements))
				&& (x3.data == nullptr || (x3.dtype == y.dtype && volume(x3) == elements)), "cuda_add_tensors: inputs must match the output");
		flush_pending(context);
		switch (y.dtype)
		{
			case DTYPE_FLOAT16:
				launch_axpy3<__half>(context, y.data, x1.data, x2.data, x3.data, alpha1, alpha2, alpha3, beta, elements);
				break;
			case DTYPE_FLOAT32:
				launch_axpy3<float>(context, y.data, x1.data, x2.data, x3.data, alpha1, alpha2, alpha3, beta, elements);
				break;
			case DTYPE_FLOAT64:
				launch_axpy3<double>(context, y.data, x1.data, x2.data, x3.data, alpha1, alpha2, alpha3, beta, elements);
				break;
			default:
				record_error(context, "cuda_add_tensors: dtype %d not supported", static_cast<int>(y.dtype));
				return;
		}
		check_cuda(context, cudaGetLastError(), "cuda_add_tensors");
	}
	void cuda_scale_tensor(mlContext_t context, float alpha, mlTensor_t x)
	{
		mlTensor_t none;
		none.data = nullptr;
		none.dtype = x.dtype;
		none.rank = 0;
		for (int i = 0; i < 6; i++)
			none.dim[i] = 0;
		cuda_add_tensors(context, 0.0f, none, 0.0f, none, 0.0f, none, alpha, x);
	}
	void cuda_unpack_input(mlContext_t context, mlShape_t shape, mlDataType_t dst_dtype, void *dst, const void *src)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_unpack_input: null context");
		if (volume(shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, dst != nullptr && src != nullptr, "cuda_unpack_input: null pointer");
		flush_pending(context);
		const long long rows = volume_without_last_dim(shape);
		const int channels = last_dim(shape);
		if (rows == 0 || channels == 0)
			return;
		cudaStream_t stream = use_stream(context);
		const uint32_t *s = reinterpret_cast<const uint32_t*>(src);
#define CASE(E, T) case E: launch_unpack<T>(stream, get(context)->sm_count, dst, s, rows, channels); break
		switch (dst_dtype)
		{
			CASE(DTYPE_FLOAT16, __half);
			CASE(DTYPE_FLOAT32, float);
			CASE(DTYPE_FLOAT64, double);
			CASE(DTYPE_UINT8, uint8_t);
			CASE(DTYPE_INT8, int8_t);
			CASE(DTYPE_INT16, int16_t);
			CASE(DTYPE_INT32, int32_t);
			default:
				record_error(context, "cuda_unpack_input: dtype %d not supported", static_cast<int>(dst_dtype));
				return;
		}
#undef CASE
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_unpack_input");
	}
	void cuda_convert_type(mlContext_t context, void *dst, mlDataType_t dst_dtype, const void *src, mlDataType_t src_dtype, int elements)
	{
		if (elements == 0)
			return;
		MB200_REQUIRE(context, context != nullptr, "cuda_convert_type: null context");
		MB200_REQUIRE(context, dst != nullptr && src != nullptr && elements > 0, "cuda_convert_type: null pointer or negative size");
		if (dst_dtype == src_dtype)
		{
			if (dst != src)
				cuda_memcpy_within_device(context, dst, 0, src, 0, static_cast<size_t>(elements) * size_of(dst_dtype));
			return;
		}
		flush_pending(context);
		cudaStream_t stream = use_stream(context);
		const int sm = get(context)->sm_count;
		bool ok = false;
		switch (dst_dtype)
		{
			case DTYPE_FLOAT16:
				ok = convert_from<__half>(stream, sm, dst, src, src_dtype, elements);
				break;
			case DTYPE_FLOAT32:
				ok = convert_from<float>(stream, sm, dst, src, src_dtype, elements);
				break;
			case DTYPE_FLOAT64:
				ok = convert_from<double>(stream, sm, dst, src, src_dtype, elements);
				break;
			case DTYPE_UINT8:
				ok = convert_from<uint8_t>(stream, sm, dst, src, src_dtype, elements);
				break;
			case DTYPE_INT8:
				ok = convert_from<int8_t>(stream, sm, dst, src, src_dtype, elements);
				break;
			case DTYPE_INT16:
				ok = convert_from<int16_t>(stream, sm, dst, src, src_dtype, elements);
				break;
			case DTYPE_INT32:
				ok = convert_from<int32_t>(stream, sm, dst, src, src_dtype, elements);
				break;
			default:
				break;
		}
		MB200_REQUIRE(context, ok, "cuda_convert_type: conversion %d -> %d not supported", static_cast<int>(src_dtype), static_cast<int>(dst_dtype));
		check_cuda(context, cudaGetLastError(), "cuda_convert_type");
	}
	void cuda_transpose_021(mlContext_t context, mlDataType_t dtype, mlShape_t shape, const void *input, void *output)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_transpose_021: null context");
		if (volume(shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, shape.rank == 3 && input != nullptr && output != nullptr && input != output,
				"cuda_transpose_021: needs a rank-3 shape and distinct non-null buffers");
		flush_pending(context);
		const int d0 = shape.dim[0], d1 = shape.dim[1], d2 = shape.dim[2];
		if (d0 == 0 || d1 == 0 || d2 == 0)
			return;
		MB200_REQUIRE(context, d0 <= 65535 && ceil_div(d1, 32) <= 65535, "cuda_transpose_021: shape too large for one launch");
		cudaStream_t stream = use_stream(context);
		dim3 grid(ceil_div(d2, 32), ceil_div(d1, 32), d0), block(32, 8);
		switch (size_of(dtype))
		{
			case 1:
				kernel_transpose_021<uint8_t> <<<grid, block, 0, stream>>>(reinterpret_cast<uint8_t*>(output), reinterpret_cast<const uint8_t*>(input),
						d1, d2);
				break;
			case 2:
				kernel_transpose_021<uint16_t> <<<grid, block, 0, stream>>>(reinterpret_cast<uint16_t*>(output),
						reinterpret_cast<const uint16_t*>(input), d1, d2);
				break;
			case 4:
				kernel_transpose_021<uint32_t> <<<grid, block, 0, stream>>>(reinterpret_cast<uint32_t*>(output),
						reinterpret_cast<const uint32_t*>(input), d1, d2);
				break;
			case 8:
				kernel_transpose_021<uint64_t> <<<grid, block, 0, stream>>>(reinterpret_cast<uint64_t*>(output),
						reinterpret_cast<const uint64_t*>(input), d1, d2);
				break;
			default:
				record_error(context, "cuda_transpose_021: dtype %d not supported", static_cast<int>(dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_transpose_021");
	}
	void cuda_global_average_pooling_forward(mlContext_t context, float alpha, const mlTensor_t x, float beta, mlTensor_t y)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_global_average_pooling_forward: null context");
		if (volume(x) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, x.rank == 4 && y.rank == 2 && x.data != nullptr && y.data != nullptr,
				"cuda_global_average_pooling_forward: x must be [b,h,w,c] and y [b,c]");
		MB200_REQUIRE(context, x.dim[0] == y.dim[0] && x.dim[3] == y.dim[1] && x.dtype == y.dtype,
				"cuda_global_average_pooling_forward: x and y do not match");
		flush_pending(context);
		const int batch = x.dim[0], hw = x.dim[1] * x.dim[2], channels = x.dim[3];
		if (batch == 0 || hw == 0 || channels == 0)
			return;
		MB200_REQUIRE(context, batch <= 65535, "cuda_global_average_pooling_forward: batch %d exceeds one launch", batch);
		cudaStream_t stream = use_stream(context);
		switch (x.dtype)
		{
			case DTYPE_FLOAT16:
				if (channels % 8 == 0 && aligned_to(x.data, 16))
					kernel_global_avg_pool<__half, 8> <<<dim3(ceil_div(channels, 256), batch), 256, 0, stream>>>(reinterpret_cast<__half*>(y.data),
							reinterpret_cast<const __half*>(x.data), hw, channels, alpha, beta);
				else
					kernel_global_avg_pool<__half, 1> <<<dim3(ceil_div(channels, 32), batch), 256, 0, stream>>>(reinterpret_cast<__half*>(y.data),
							reinterpret_cast<const __half*>(x.data), hw, channels, alpha, beta);
				break;
			case DTYPE_FLOAT32:
				if (channels % 4 == 0 && aligned_to(x.data, 16))
					kernel_global_avg_pool<float, 4> <<<dim3(ceil_div(channels, 128), batch), 256, 0, stream>>>(reinterpret_cast<float*>(y.data),
							reinterpret_cast<const float*>(x.data), hw, channels, alpha, beta);
				else
					kernel_global_avg_pool<float, 1> <<<dim3(ceil_div(channels, 32), batch), 256, 0, stream>>>(reinterpret_cast<float*>(y.data),
							reinterpret_cast<const float*>(x.data), hw, channels, alpha, beta);
				break;
			default:
				record_error(context, "cuda_global_average_pooling_forward: dtype %d not supported", static_cast<int>(x.dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_global_average_pooling_forward");
	}
	void cuda_softmax_forward(mlContext_t context, mlDataType_t dtype, mlShape_t shape, void *output, const void *input)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_softmax_forward: null context");
		if (volume(shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, output != nullptr && input != nullptr, "cuda_softmax_forward: null pointer");
		flush_pending(context);
		const long long rows = volume_without_last_dim(shape);
		const int channels = last_dim(shape);
		if (rows == 0 || channels == 0)
			return;
		cudaStream_t stream = use_stream(context);
		const int grid = grid_for(rows * 32, 256, get(context)->sm_count);
		switch (dtype)
		{
			case DTYPE_FLOAT16:
				launch_softmax<__half>(stream, grid, output, input, rows, channels);
				break;
			case DTYPE_FLOAT32:
				launch_softmax<float>(stream, grid, output, input, rows, channels);
				break;
			default:
				record_error(context, "cuda_softmax_forward: dtype %d not supported", static_cast<int>(dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_softmax_forward");
	}
	void cuda_multiply_tensors(mlContext_t context, mlDataType_t dtype, mlShape_t shape, void *dst, const void *src1, const void *src2)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_multiply_tensors: null context");
		const long long elements = volume(shape);
		if (elements == 0)
			return; // an empty problem: nothing to validate or launch
		MB200_REQUIRE(context, dst != nullptr && src1 != nullptr && src2 != nullptr, "cuda_multiply_tensors: null pointer");
		flush_pending(context);
		cudaStream_t stream = use_stream(context);
		const int sm = get(context)->sm_count;
		const bool packets = aligned_to(dst, 16) && aligned_to(src1, 16) && aligned_to(src2, 16);
		switch (dtype)
		{
			case DTYPE_FLOAT16:
				if (packets && elements % 8 == 0)
					kernel_multiply_packets<__half> <<<grid_for(elements / 8, 256, sm), 256, 0, stream>>>(reinterpret_cast<__half*>(dst),
							reinterpret_cast<const __half*>(src1), reinterpret_cast<const __half*>(src2), elements / 8);
				else
					kernel_multiply_elements<__half, float> <<<grid_for(elements, 256, sm), 256, 0, stream>>>(reinterpret_cast<__half*>(dst),
							reinterpret_cast<const __half*>(src1), reinterpret_cast<const __half*>(src2), elements);
				break;
			case DTYPE_FLOAT32:
				if (packets && elements % 4 == 0)
					kernel_multiply_packets<float> <<<grid_for(elements / 4, 256, sm), 256, 0, stream>>>(reinterpret_cast<float*>(dst),
							reinterpret_cast<const float*>(src1), reinterpret_cast<const float*>(src2), elements / 4);
				else
					kernel_multiply_elements<float, float> <<<grid_for(elements, 256, sm), 256, 0, stream>>>(reinterpret_cast<float*>(dst),
							reinterpret_cast<const float*>(src1), reinterpret_cast<const float*>(src2), elements);
				break;
			case DTYPE_FLOAT64:
				kernel_multiply_elements<double, double> <<<grid_for(elements, 256, sm), 256, 0, stream>>>(reinterpret_cast<double*>(dst),
						reinterpret_cast<const double*>(src1), reinterpret_cast<const double*>(src2), elements);
				break;
			default:
				record_error(context, "cuda_multiply_tensors: dtype %d not supported", static_cast<int>(dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_multiply_tensors");
	}
}
