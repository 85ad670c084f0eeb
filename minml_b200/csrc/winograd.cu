/*
 * winograd.cu -- the three forward Winograd transforms of the C ABI.
 *
 * Replaces src/backend/cuda/kernels/winograd_nonfused.cu:48-179,417-471 and the constant sets of
 * src/backend/cuda/kernels/winograd_transforms.cuh:135-203 (F(4x4,3x3)), :40-95 (F(2x2,3x3)), :244-302 (F(2x2,5x5)).
 *
 *   weight:  U[p, co, ci] = (G g G^T)[p]            w [co, k, k, ci] -> matrices [(t+k-1)^2, co, ci]
 *   input :  V[p, tile, c] = (B^T d B)[p]           x [b, h, w, c], zero padded patches of (t+k-1)^2, stride t
 *   output:  y = act(A^T M A + ext + bias)          matrices [(t+k-1)^2, tiles, c] -> y [b, h, w, c], clipped at the border
 *
 * tile index = (b * tiles_h + th) * tiles_w + tw;  p = row * (t+k-1) + column.
 * The transform matrices are those pinned by the reference's known-answer tests (test/backend/test_winograd.cpp:218-394):
 * interpolation points 0, +-1, +-2, inf with rows of G scaled by 2/3, 1/3 and 2.
 *
 * All arithmetic is fp32 (fp16 data is converted on load and rounded to nearest on store), which is at least as
 * accurate as the reference's half2 arithmetic.  One thread owns VEC consecutive channels of one tile, so a warp
 * reads and writes 32 * VEC contiguous channels per access.
 */
#include "common.cuh"
#include "winograd.cuh"

namespace mb200
{
	namespace
	{
		/* ---- transform matrices as compile-time tables; fully unrolled loops fold the zeros and ones away ---- */
		template<int K, int T> struct WM;
		template<> struct WM<3, 4>
		{
				static constexpr int P = 6;
				__device__ static constexpr float bt(int r, int c)
				{
					constexpr float m[6][6] = { { 1.0f, 0.0f, -1.25f, 0.0f, 0.25f, 0.0f }, { 0.0f, 1.0f, 1.0f, -0.25f, -0.25f, 0.0f }, { 0.0f, -1.0f,
							1.0f, 0.25f, -0.25f, 0.0f }, { 0.0f, -1.0f, -0.5f, 1.0f, 0.5f, 0.0f }, { 0.0f, 1.0f, -0.5f, -1.0f, 0.5f, 0.0f }, { 0.0f,
							1.0f, 0.0f, -1.25f, 0.0f, 0.25f } };
					return m[r][c];
				}
				__device__ static constexpr float g(int r, int c)
				{
					constexpr float c13 = 1.0f / 3.0f, c23 = 2.0f / 3.0f;
					constexpr float m[6][3] = { { 1.0f, 0.0f, 0.0f }, { c23, c23, c23 }, { c23, -c23, c23 }, { c13, 2.0f * c13, 4.0f * c13 }, { c13,
							-2.0f * c13, 4.0f * c13 }, { 0.0f, 0.0f, 2.0f } };
					return m[r][c];
				}
				__device__ static constexpr float at(int r, int c)
				{
					constexpr float m[4][6] = { { 1.0f, 1.0f, 1.0f, 0.25f, 0.25f, 0.0f }, { 0.0f, 1.0f, -1.0f, 0.5f, -0.5f, 0.0f }, { 0.0f, 1.0f,
							1.0f, 1.0f, 1.0f, 0.0f }, { 0.0f, 1.0f, -1.0f, 2.0f, -2.0f, 2.0f } };
					return m[r][c];
				}
		};
		template<> struct WM<3, 2>
		{
				static constexpr int P = 4;
				__device__ static constexpr float bt(int r, int c)
				{
					constexpr float m[4][4] = { { 1.0f, 0.0f, -1.0f, 0.0f }, { 0.0f, 1.0f, 1.0f, 0.0f }, { 0.0f, -1.0f, 1.0f, 0.0f }, { 0.0f, -1.0f,
							0.0f, 1.0f } };
					return m[r][c];
				}
				__device__ static constexpr float g(int r, int c)
				{
					constexpr float m[4][3] = { { 1.0f, 0.0f, 0.0f }, { 0.5f, 0.5f, 0.5f }, { 0.5f, -0.5f, 0.5f }, { 0.0f, 0.0f, 1.0f } };
					return m[r][c];
				}
				__device__ static constexpr float at(int r, int c)
				{
					constexpr float m[2][4] = { { 1.0f, 1.0f, 1.0f, 0.0f }, { 0.0f, 1.0f, -1.0f, 1.0f } };
					return m[r][c];
				}
		};
		template<> struct WM<5, 2>
		{
				static constexpr int P = 6;
				__device__ static constexpr float bt(int r, int c)
				{
					return WM<3, 4>::bt(r, c); // same interpolation points, hence the same input transform
				}
				__device__ static constexpr float g(int r, int c)
				{
					constexpr float c16 = 1.0f / 6.0f, c23 = 2.0f / 3.0f;
					constexpr float m[6][5] = { { 1.0f, 0.0f, 0.0f, 0.0f, 0.0f }, { c23, c23, c23, c23, c23 }, { c23, -c23, c23, -c23, c23 }, { c16,
							2.0f * c16, 4.0f * c16, 8.0f * c16, 16.0f * c16 }, { c16, -2.0f * c16, 4.0f * c16, -8.0f * c16, 16.0f * c16 }, { 0.0f,
							0.0f, 0.0f, 0.0f, 2.0f } };
					return m[r][c];
				}
				__device__ static constexpr float at(int r, int c)
				{
					constexpr float m[2][6] = { { 1.0f, 1.0f, 1.0f, 0.5f, 0.5f, 0.0f }, { 0.0f, 1.0f, -1.0f, 1.0f, -1.0f, 2.0f } };
					return m[r][c];
				}
		};

		template<typename T, int VEC> struct Pack;
		template<> struct Pack<float, 1>
		{
				__device__ static void load(const float *p, float (&v)[1]) { v[0] = *p; }
				__device__ static void store(float *p, const float (&v)[1]) { *p = v[0]; }
		};
		template<> struct Pack<float, 4>
		{
				__device__ static void load(const float *p, float (&v)[4])
				{
					const float4 t = *reinterpret_cast<const float4*>(p);
					v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
				}
				__device__ static void store(float *p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
		};
		template<> struct Pack<__half, 1>
		{
				__device__ static void load(const __half *p, float (&v)[1]) { v[0] = __half2float(*p); }
				__device__ static void store(__half *p, const float (&v)[1]) { *p = __float2half_rn(v[0]); }
		};
		template<> struct Pack<__half, 2>
		{
				__device__ static void load(const __half *p, float (&v)[2])
				{
					const float2 t = __half22float2(*reinterpret_cast<const __half2*>(p));
					v[0] = t.x; v[1] = t.y;
				}
				__device__ static void store(__half *p, const float (&v)[2]) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(v[0], v[1]); }
		};
		template<> struct Pack<__half, 4>
		{
				__device__ static void load(const __half *p, float (&v)[4])
				{
					const uint2 raw = *reinterpret_cast<const uint2*>(p);
					const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
					const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
					v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
				}
				__device__ static void store(__half *p, const float (&v)[4])
				{
					const __half2 a = __floats2half2_rn(v[0], v[1]);
					const __half2 b = __floats2half2_rn(v[2], v[3]);
					uint2 raw;
					raw.x = *reinterpret_cast<const uint32_t*>(&a);
					raw.y = *reinterpret_cast<const uint32_t*>(&b);
					*reinterpret_cast<uint2*>(p) = raw;
				}
		};

		template<int K, int T, typename D, int VEC>
		__global__ void __launch_bounds__(128) kernel_weight_transform(D *__restrict__ matrices, const D *__restrict__ weights, int cout, int cin,
				bool invert)
		{
			using M = WM<K, T>;
			constexpr int P = M::P;
			const int cvecs = cin / VEC;
			const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
			if (idx >= static_cast<long long>(cout) * cvecs)
				return;
			const int co = static_cast<int>(idx / cvecs);
			const int ci = static_cast<int>(idx % cvecs) * VEC;

			float g[K][K][VEC];
#pragma unroll
			for (int r = 0; r < K; r++)
#pragma unroll
				for (int c = 0; c < K; c++)
				{
					const int rr = invert ? (K - 1 - r) : r;
					const int cc = invert ? (K - 1 - c) : c;
					Pack<D, VEC>::load(weights + ((static_cast<long long>(co) * K + rr) * K + cc) * cin + ci, g[r][c]);
				}
			// tmp = G g  (P x K), then U = tmp G^T (P x P)
			float tmp[P][K][VEC];
#pragma unroll
			for (int i = 0; i < P; i++)
#pragma unroll
				for (int c = 0; c < K; c++)
#pragma unroll
					for (int v = 0; v < VEC; v++)
					{
						float s = 0.0f;
#pragma unroll
						for (int r = 0; r < K; r++)
							s += M::g(i, r) * g[r][c][v];
						tmp[i][c][v] = s;
					}
#pragma unroll
			for (int i = 0; i < P; i++)
#pragma unroll
				for (int j = 0; j < P; j++)
				{
					float out[VEC];
#pragma unroll
					for (int v = 0; v < VEC; v++)
					{
						float s = 0.0f;
#pragma unroll
						for (int c = 0; c < K; c++)
							s += tmp[i][c][v] * M::g(j, c);
						out[v] = s;
					}
					Pack<D, VEC>::store(matrices + (static_cast<long long>(i * P + j) * cout + co) * cin + ci, out);
				}
		}

		/* Raw (unconverted) packet of VEC elements, so that a whole patch can be fetched before any arithmetic starts:
		 * all loads of a thread are independent and in flight together, which is what a bandwidth-bound kernel needs. */
		template<typename D, int VEC> struct Raw;
		template<> struct Raw<float, 1> { using type = float; };
		template<> struct Raw<float, 4> { using type = float4; };
		template<> struct Raw<__half, 1> { using type = unsigned short; };
		template<> struct Raw<__half, 2> { using type = unsigned int; };
		template<> struct Raw<__half, 4> { using type = uint2; };
		template<typename D, int VEC>
		__device__ __forceinline__ void unpack_raw(const typename Raw<D, VEC>::type &raw, float (&v)[VEC])
		{
			Pack<D, VEC>::load(reinterpret_cast<const D*>(&raw), v);
		}

		template<int K, int T, typename D, int VEC>
		__global__ void __launch_bounds__(128) kernel_input_transform(D *__restrict__ matrices, const D *__restrict__ input, int batch, int height,
				int width, int channels, int tiles_h, int tiles_w)
		{
			using M = WM<K, T>;
			using R = typename Raw<D, VEC>::type;
			constexpr int P = M::P;
			constexpr int PAD = K / 2;
			const int cvecs = channels / VEC;
			const long long total_tiles = static_cast<long long>(batch) * tiles_h * tiles_w;
			const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
			if (idx >= total_tiles * cvecs)
				return;
			// 32-bit index arithmetic (the launcher checks that the thread count fits): five 64-bit divisions cost about as many
			// instructions as the transform itself
			const unsigned idx32 = static_cast<unsigned>(idx);
			const unsigned tile32 = idx32 / static_cast<unsigned>(cvecs);
			const int c0 = static_cast<int>(idx32 - tile32 * static_cast<unsigned>(cvecs)) * VEC;
			const unsigned row32 = tile32 / static_cast<unsigned>(tiles_w);
			const int tw = static_cast<int>(tile32 - row32 * static_cast<unsigned>(tiles_w));
			const int b = static_cast<int>(row32 / static_cast<unsigned>(tiles_h));
			const int th = static_cast<int>(row32 - static_cast<unsigned>(b) * static_cast<unsigned>(tiles_h));
			const long long tile = tile32;

			// 1. fetch the whole zero-padded patch: P*P independent loads (a position outside the image reads element 0 and is masked)
			R raw[P][P];
			const R *src = reinterpret_cast<const R*>(input + c0);
			const long long pitch = channels / VEC; // packets per position
#pragma unroll
			for (int r = 0; r < P; r++)
			{
				const int h = T * th - PAD + r;
#pragma unroll
				for (int c = 0; c < P; c++)
				{
					const int w = T * tw - PAD + c;
					const bool inside = h >= 0 && h < height && w >= 0 && w < width;
					const long long off = inside ? ((static_cast<long long>(b) * height + h) * width + w) * pitch : 0;
					raw[r][c] = src[off];
					if (!inside)
						raw[r][c] = R();
				}
			}
			// 2. tmp = B^T d
			float tmp[P][P][VEC];
#pragma unroll
			for (int c = 0; c < P; c++)
			{
				float d[P][VEC];
#pragma unroll
				for (int r = 0; r < P; r++)
					unpack_raw<D, VEC>(raw[r][c], d[r]);
#pragma unroll
				for (int i = 0; i < P; i++)
#pragma unroll
					for (int v = 0; v < VEC; v++)
					{
						float s = 0.0f;
#pragma unroll
						for (int r = 0; r < P; r++)
							if (M::bt(i, r) != 0.0f)
								s += M::bt(i, r) * d[r][v];
						tmp[i][c][v] = s;
					}
			}
			// 3. V = tmp B, one store per matrix
#pragma unroll
			for (int i = 0; i < P; i++)
#pragma unroll
				for (int j = 0; j < P; j++)
				{
					float out[VEC];
#pragma unroll
					for (int v = 0; v < VEC; v++)
					{
						float s = 0.0f;
#pragma unroll
						for (int c = 0; c < P; c++)
							if (M::bt(j, c) != 0.0f)
								s += tmp[i][c][v] * M::bt(j, c);
						out[v] = s;
					}
					Pack<D, VEC>::store(matrices + (static_cast<long long>(i * P + j) * total_tiles + tile) * channels + c0, out);
				}
		}

		template<int K, int T, typename D, int VEC>
		__global__ void __launch_bounds__(128) kernel_output_transform(const D *__restrict__ matrices, D *__restrict__ output,
				const D *__restrict__ ext, const D *__restrict__ bias, int act, int batch, int height, int width, int channels, int tiles_h,
				int tiles_w)
		{
			using M = WM<K, T>;
			using R = typename Raw<D, VEC>::type;
			constexpr int P = M::P;
			const int cvecs = channels / VEC;
			const long long total_tiles = static_cast<long long>(batch) * tiles_h * tiles_w;
			const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
			if (idx >= total_tiles * cvecs)
				return;
			// 32-bit index arithmetic (the launcher checks that the thread count fits): five 64-bit divisions cost about as many
			// instructions as the transform itself
			const unsigned idx32 = static_cast<unsigned>(idx);
			const unsigned tile32 = idx32 / static_cast<unsigned>(cvecs);
			const int c0 = static_cast<int>(idx32 - tile32 * static_cast<unsigned>(cvecs)) * VEC;
			const unsigned row32 = tile32 / static_cast<unsigned>(tiles_w);
			const int tw = static_cast<int>(tile32 - row32 * static_cast<unsigned>(tiles_w));
			const int b = static_cast<int>(row32 / static_cast<unsigned>(tiles_h));
			const int th = static_cast<int>(row32 - static_cast<unsigned>(b) * static_cast<unsigned>(tiles_h));
			const long long tile = tile32;

			// 1. all P*P matrix elements and the T*T residual values of this tile are fetched before any arithmetic
			R raw[P][P];
			const R *src = reinterpret_cast<const R*>(matrices + c0);
			const long long pitch = channels / VEC;
#pragma unroll
			for (int r = 0; r < P; r++)
#pragma unroll
				for (int c = 0; c < P; c++)
					raw[r][c] = src[(static_cast<long long>(r * P + c) * total_tiles + tile) * pitch];
			R raw_ext[T][T];
			if (ext != nullptr)
			{
				const R *esrc = reinterpret_cast<const R*>(ext + c0);
#pragma unroll
				for (int i = 0; i < T; i++)
#pragma unroll
					for (int j = 0; j < T; j++)
					{
						const int h = T * th + i, w = T * tw + j;
						const bool inside = h < height && w < width;
						raw_ext[i][j] = esrc[inside ? ((static_cast<long long>(b) * height + h) * width + w) * pitch : 0];
					}
			}
			float bias_value[VEC];
			if (bias != nullptr)
				Pack<D, VEC>::load(bias + c0, bias_value);
			else
			{
#pragma unroll
				for (int v = 0; v < VEC; v++)
					bias_value[v] = 0.0f;
			}
			// 2. tmp = A^T M
			float tmp[T][P][VEC];
#pragma unroll
			for (int c = 0; c < P; c++)
			{
				float mcol[P][VEC];
#pragma unroll
				for (int r = 0; r < P; r++)
					unpack_raw<D, VEC>(raw[r][c], mcol[r]);
#pragma unroll
				for (int i = 0; i < T; i++)
#pragma unroll
					for (int v = 0; v < VEC; v++)
					{
						float s = 0.0f;
#pragma unroll
						for (int r = 0; r < P; r++)
							if (M::at(i, r) != 0.0f)
								s += M::at(i, r) * mcol[r][v];
						tmp[i][c][v] = s;
					}
			}
			// 3. y = tmp A + ext + bias, activation, clipped store
#pragma unroll
			for (int i = 0; i < T; i++)
			{
				const int h = T * th + i;
#pragma unroll
				for (int j = 0; j < T; j++)
				{
					const int w = T * tw + j;
					float out[VEC];
#pragma unroll
					for (int v = 0; v < VEC; v++)
					{
						float s = 0.0f;
#pragma unroll
						for (int c = 0; c < P; c++)
							if (M::at(j, c) != 0.0f)
								s += tmp[i][c][v] * M::at(j, c);
						out[v] = s;
					}
					if (ext != nullptr)
					{
						float e[VEC];
						unpack_raw<D, VEC>(raw_ext[i][j], e);
#pragma unroll
						for (int v = 0; v < VEC; v++)
							out[v] += e[v];
					}
#pragma unroll
					for (int v = 0; v < VEC; v++)
						out[v] = apply_activation(out[v] + bias_value[v], act);
					if (h < height && w < width)
						Pack<D, VEC>::store(output + ((static_cast<long long>(b) * height + h) * width + w) * channels + c0, out);
				}
			}
		}

		int kernel_size_of(const mlTensor_t &matrices, int tile_size)
		{ // reference: get_kernel_size, src/backend/cuda/kernels/winograd_nonfused.cu:258-262
			int p = 1;
			while (p * p < matrices.dim[0])
				p++;
			return p + 1 - tile_size;
		}
		bool supported(int kernel, int tile)
		{
			return (kernel == 3 && (tile == 2 || tile == 4)) || (kernel == 5 && tile == 2);
		}
		template<typename D, int VEC>
		bool vec_ok(int channels, const void *a, const void *b, const void *c = nullptr, const void *d = nullptr)
		{
			const size_t bytes = sizeof(D) * VEC;
			return channels % VEC == 0 && aligned_to(a, bytes) && aligned_to(b, bytes) && (c == nullptr || aligned_to(c, bytes))
					&& (d == nullptr || aligned_to(d, bytes));
		}

#define DISPATCH_KT(KERNEL, D, VEC, ...) \
		do { \
			if (kernel == 3 && tile_size == 4) KERNEL<3, 4, D, VEC> <<<grid, 128, 0, stream>>>(__VA_ARGS__); \
			else if (kernel == 3 && tile_size == 2) KERNEL<3, 2, D, VEC> <<<grid, 128, 0, stream>>>(__VA_ARGS__); \
			else KERNEL<5, 2, D, VEC> <<<grid, 128, 0, stream>>>(__VA_ARGS__); \
			MB200_COUNT_LAUNCH(); \
		} while (0)
	}

	void winograd_weight_transform_eager(mlContext_t ctx, int tile_size, const mlTensor_t w, mlTensor_t matrices, bool invert)
	{
		const int kernel = kernel_size_of(matrices, tile_size);
		const int cout = w.dim[0], cin = w.dim[3];
		cudaStream_t stream = use_stream(ctx);
		if (w.dtype == DTYPE_FLOAT16)
		{
			if (vec_ok<__half, 2>(cin, w.data, matrices.data))
			{
				const int grid = ceil_div(static_cast<long long>(cout) * (cin / 2), 128);
				DISPATCH_KT(kernel_weight_transform, __half, 2, reinterpret_cast<__half*>(matrices.data), reinterpret_cast<const __half*>(w.data),
						cout, cin, invert);
			}
			else
			{
				const int grid = ceil_div(static_cast<long long>(cout) * cin, 128);
				DISPATCH_KT(kernel_weight_transform, __half, 1, reinterpret_cast<__half*>(matrices.data), reinterpret_cast<const __half*>(w.data),
						cout, cin, invert);
			}
		}
		else
		{
			const int grid = ceil_div(static_cast<long long>(cout) * cin, 128);
			DISPATCH_KT(kernel_weight_transform, float, 1, reinterpret_cast<float*>(matrices.data), reinterpret_cast<const float*>(w.data), cout,
					cin, invert);
		}
		check_cuda(ctx, cudaGetLastError(), "cuda_winograd_weight_transform");
	}
	void winograd_input_transform_eager(mlContext_t ctx, int tile_size, const mlTensor_t x, mlTensor_t matrices)
	{
		const int kernel = kernel_size_of(matrices, tile_size);
		const int batch = x.dim[0], height = x.dim[1], width = x.dim[2], channels = x.dim[3];
		const int tiles_h = (height + tile_size - 1) / tile_size, tiles_w = (width + tile_size - 1) / tile_size;
		const long long tiles = static_cast<long long>(batch) * tiles_h * tiles_w;
		MB200_REQUIRE(ctx, tiles * channels < (1ll << 31), "cuda_winograd_input_transform: %lld tiles x %d channels exceed one launch", tiles, channels);
		cudaStream_t stream = use_stream(ctx);
#define ARGS(D) reinterpret_cast<D*>(matrices.data), reinterpret_cast<const D*>(x.data), batch, height, width, channels, tiles_h, tiles_w
		if (x.dtype == DTYPE_FLOAT16)
		{
			if (vec_ok<__half, 2>(channels, x.data, matrices.data))
			{
				const int grid = ceil_div(tiles * (channels / 2), 128);
				DISPATCH_KT(kernel_input_transform, __half, 2, ARGS(__half));
			}
			else
			{
				const int grid = ceil_div(tiles * channels, 128);
				DISPATCH_KT(kernel_input_transform, __half, 1, ARGS(__half));
			}
		}
		else
		{
			const int grid = ceil_div(tiles * channels, 128);
			DISPATCH_KT(kernel_input_transform, float, 1, ARGS(float));
		}
#undef ARGS
		check_cuda(ctx, cudaGetLastError(), "cuda_winograd_input_transform");
	}
	void winograd_output_transform_eager(mlContext_t ctx, int tile_size, const mlTensor_t matrices, const mlTensor_t bias, const mlTensor_t ext,
			mlTensor_t y, mlActivationType_t act)
	{
		const int kernel = kernel_size_of(matrices, tile_size);
		const int batch = y.dim[0], height = y.dim[1], width = y.dim[2], channels = y.dim[3];
		const int tiles_h = (height + tile_size - 1) / tile_size, tiles_w = (width + tile_size - 1) / tile_size;
		const long long tiles = static_cast<long long>(batch) * tiles_h * tiles_w;
		MB200_REQUIRE(ctx, tiles * channels < (1ll << 31), "cuda_winograd_output_transform: %lld tiles x %d channels exceed one launch", tiles, channels);
		cudaStream_t stream = use_stream(ctx);
#define ARGS(D) reinterpret_cast<const D*>(matrices.data), reinterpret_cast<D*>(y.data), reinterpret_cast<const D*>(ext.data), \
		reinterpret_cast<const D*>(bias.data), static_cast<int>(act), batch, height, width, channels, tiles_h, tiles_w
		if (y.dtype == DTYPE_FLOAT16)
		{
			if (vec_ok<__half, 2>(channels, y.data, matrices.data, ext.data, bias.data))
			{
				const int grid = ceil_div(tiles * (channels / 2), 128);
				DISPATCH_KT(kernel_output_transform, __half, 2, ARGS(__half));
			}
			else
			{
				const int grid = ceil_div(tiles * channels, 128);
				DISPATCH_KT(kernel_output_transform, __half, 1, ARGS(__half));
			}
		}
		else
		{
			const int grid = ceil_div(tiles * channels, 128);
			DISPATCH_KT(kernel_output_transform, float, 1, ARGS(float));
		}
#undef ARGS
		check_cuda(ctx, cudaGetLastError(), "cuda_winograd_output_transform");
	}

	bool winograd_check_common(mlContext_t ctx, const char *who, int tile_size, const mlTensor_t &matrices)
	{
		if (ctx == nullptr)
		{
			record_error(ctx, "%s: null context", who);
			return false;
		}
		if (matrices.rank != 3 || matrices.data == nullptr)
		{
			record_error(ctx, "%s: matrices must be a rank-3 tensor", who);
			return false;
		}
		if (matrices.dtype != DTYPE_FLOAT16 && matrices.dtype != DTYPE_FLOAT32)
		{
			record_error(ctx, "%s: dtype %d not supported (fp16 and fp32 are)", who, static_cast<int>(matrices.dtype));
			return false;
		}
		const int kernel = kernel_size_of(matrices, tile_size);
		const int p = tile_size + kernel - 1;
		if (p * p != matrices.dim[0] || !supported(kernel, tile_size))
		{
			record_error(ctx, "%s: %d matrices with tile size %d is not F(2x2,3x3), F(4x4,3x3) or F(2x2,5x5)", who, matrices.dim[0], tile_size);
			return false;
		}
		return true;
	}
} /* namespace mb200 */

using namespace mb200;

extern "C"
{
	void cuda_winograd_weight_transform(mlContext_t context, int tile_size, const mlTensor_t w, mlTensor_t matrices, bool invert)
	{
		if (!winograd_check_common(context, "cuda_winograd_weight_transform", tile_size, matrices))
			return;
		const int kernel = kernel_size_of(matrices, tile_size);
		MB200_REQUIRE(context, w.rank == 4 && w.data != nullptr && w.dtype == matrices.dtype,
				"cuda_winograd_weight_transform: weights must be a rank-4 tensor of the matrices' dtype");
		MB200_REQUIRE(context, w.dim[1] == kernel && w.dim[2] == kernel, "cuda_winograd_weight_transform: weights are %d x %d, expected %d x %d",
				w.dim[1], w.dim[2], kernel, kernel);
		MB200_REQUIRE(context, matrices.dim[1] == w.dim[0] && matrices.dim[2] == w.dim[3],
				"cuda_winograd_weight_transform: matrices [%d, %d, %d] do not match weights [%d, %d, %d, %d]", matrices.dim[0], matrices.dim[1],
				matrices.dim[2], w.dim[0], w.dim[1], w.dim[2], w.dim[3]);
		flush_pending(context);
		winograd_weight_transform_eager(context, tile_size, w, matrices, invert);
		winograd_register_weights(context, w, matrices, tile_size, invert);
	}
	void cuda_winograd_input_transform(mlContext_t context, int tile_size, const mlTensor_t x, mlTensor_t matrices)
	{
		if (context != nullptr && volume(x) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		if (!winograd_check_common(context, "cuda_winograd_input_transform", tile_size, matrices))
			return;
		MB200_REQUIRE(context, x.rank == 4 && x.data != nullptr && x.dtype == matrices.dtype,
				"cuda_winograd_input_transform: input must be a rank-4 tensor of the matrices' dtype");
		const long long tiles = static_cast<long long>(x.dim[0]) * ((x.dim[1] + tile_size - 1) / tile_size)
				* ((x.dim[2] + tile_size - 1) / tile_size);
		MB200_REQUIRE(context, matrices.dim[1] == tiles && matrices.dim[2] == x.dim[3],
				"cuda_winograd_input_transform: matrices [%d, %d, %d] do not match input [%d, %d, %d, %d] with tile size %d", matrices.dim[0],
				matrices.dim[1], matrices.dim[2], x.dim[0], x.dim[1], x.dim[2], x.dim[3], tile_size);
		flush_pending(context);
		if (winograd_defer_input(context, tile_size, x, matrices))
			return;
		winograd_input_transform_eager(context, tile_size, x, matrices);
	}
	void cuda_winograd_output_transform(mlContext_t context, int tile_size, const mlTensor_t matrices, const mlTensor_t bias, const mlTensor_t ext,
			mlTensor_t y, mlActivationType_t act)
	{
		if (context != nullptr && volume(y) == 0)
		{ // an empty problem: drop what an (equally empty) recorded input transform / product may have left pending
			flush_pending(context);
			return;
		}
		if (!winograd_check_common(context, "cuda_winograd_output_transform", tile_size, matrices))
			return;
		MB200_REQUIRE(context, y.rank == 4 && y.data != nullptr && y.dtype == matrices.dtype,
				"cuda_winograd_output_transform: output must be a rank-4 tensor of the matrices' dtype");
		const long long tiles = static_cast<long long>(y.dim[0]) * ((y.dim[1] + tile_size - 1) / tile_size)
				* ((y.dim[2] + tile_size - 1) / tile_size);
		MB200_REQUIRE(context, matrices.dim[1] == tiles && matrices.dim[2] == y.dim[3],
				"cuda_winograd_output_transform: matrices [%d, %d, %d] do not match output [%d, %d, %d, %d] with tile size %d", matrices.dim[0],
				matrices.dim[1], matrices.dim[2], y.dim[0], y.dim[1], y.dim[2], y.dim[3], tile_size);
		MB200_REQUIRE(context, bias.data == nullptr || (bias.dtype == y.dtype && last_dim(bias) == y.dim[3]),
				"cuda_winograd_output_transform: bias must hold %d values of the output dtype", y.dim[3]);
		MB200_REQUIRE(context, ext.data == nullptr || (ext.dtype == y.dtype && volume(ext) == volume(y)),
				"cuda_winograd_output_transform: ext must have the shape and dtype of the output");
		if (winograd_complete_fused(context, tile_size, matrices, bias, ext, y, act))
			return;
		flush_pending(context);
		winograd_output_transform_eager(context, tile_size, matrices, bias, ext, y, act);
	}
}
