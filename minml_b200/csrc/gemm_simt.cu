/*
 * gemm_simt.cu -- generic CUDA-core GEMM: every transposition, any shape or alignment, fp16 / fp32 / fp64 and
 * int8 -> int32.  It is the engine behind the GEMM entry points whenever the tensor-core kernel does not apply
 * (fp64 data, transposed int8 products, operands that TMA cannot address: rows that do not start on 16 bytes).  The reference
 * sends all of these to cuBLAS (src/backend/cuda/gemms.cpp:99-407).
 *
 * 64 x 64 output tile per CTA, 16 x 16 threads with a 4 x 4 register tile each, K staged through shared memory
 * in slabs of 16.  Accumulation: fp32 for fp16/fp32, fp64 for fp64, int32 for int8.
 */
#include "common.cuh"
#include "gemm.cuh"

#include <type_traits>

namespace mb200
{
	namespace
	{
		constexpr int TM = 64, TN = 64, TK = 16;

		template<typename T> struct AccOf { using type = float; };
		template<> struct AccOf<double> { using type = double; };
		template<> struct AccOf<int8_t> { using type = int; };

		template<typename T, typename Acc> __device__ __forceinline__ Acc load_as(const T *p) { return static_cast<Acc>(*p); }
		template<> __device__ __forceinline__ float load_as<__half, float>(const __half *p) { return __half2float(*p); }

		template<typename C, typename Acc> __device__ __forceinline__ C store_as(Acc x) { return static_cast<C>(x); }
		template<> __device__ __forceinline__ __half store_as<__half, float>(float x) { return __float2half_rn(x); }

		template<typename AB, typename C>
		__global__ void __launch_bounds__(256) kernel_gemm_simt(const AB *__restrict__ A, const AB *__restrict__ B, C *Cm, int rows, int cols, int K,
				int lda, int ldb, int ldc, long long stride_a, long long stride_b, long long stride_c, bool trans_a, bool trans_b, float alpha,
				float beta)
		{
			using Acc = typename AccOf<AB>::type;
			__shared__ Acc sa[TK][TM + 1];
			__shared__ Acc sb[TK][TN + 1];

			const int batch = blockIdx.z;
			A += batch * stride_a;
			B += batch * stride_b;
			Cm += batch * stride_c;

			const int row0 = blockIdx.y * TM;
			const int col0 = blockIdx.x * TN;
			const int tx = threadIdx.x % 16;
			const int ty = threadIdx.x / 16;

			Acc acc[4][4];
			for (int i = 0; i < 4; i++)
				for (int j = 0; j < 4; j++)
					acc[i][j] = Acc(0);

			for (int k0 = 0; k0 < K; k0 += TK)
			{
				// stage op(A)[row0.., k0..] as sa[k][m] and op(B)[k0.., col0..] as sb[k][n]
				for (int idx = threadIdx.x; idx < TM * TK; idx += 256)
				{
					int m, k;
					if (trans_a)
					{ // A stored [K, rows]: consecutive threads walk rows
						m = idx % TM;
						k = idx / TM;
					}
					else
					{ // A stored [rows, K]: consecutive threads walk K
						k = idx % TK;
						m = idx / TK;
					}
					const int gm = row0 + m, gk = k0 + k;
					Acc v = Acc(0);
					if (gm < rows && gk < K)
						v = trans_a ? load_as<AB, Acc>(A + static_cast<long long>(gk) * lda + gm) : load_as<AB, Acc>(
								A + static_cast<long long>(gm) * lda + gk);
					sa[k][m] = v;
				}
				for (int idx = threadIdx.x; idx < TN * TK; idx += 256)
				{
					int n, k;
					if (trans_b)
					{ // B stored [cols, K]
						k = idx % TK;
						n = idx / TK;
					}
					else
					{ // B stored [K, cols]
						n = idx % TN;
						k = idx / TN;
					}
					const int gn = col0 + n, gk = k0 + k;
					Acc v = Acc(0);
					if (gn < cols && gk < K)
						v = trans_b ? load_as<AB, Acc>(B + static_cast<long long>(gn) * ldb + gk) : load_as<AB, Acc>(
								B + static_cast<long long>(gk) * ldb + gn);
					sb[k][n] = v;
				}
				__syncthreads();
#pragma unroll
				for (int k = 0; k < TK; k++)
				{
					Acc a[4], b[4];
#pragma unroll
					for (int i = 0; i < 4; i++)
						a[i] = sa[k][ty + 16 * i];
#pragma unroll
					for (int j = 0; j < 4; j++)
						b[j] = sb[k][tx + 16 * j];
#pragma unroll
					for (int i = 0; i < 4; i++)
#pragma unroll
						for (int j = 0; j < 4; j++)
							acc[i][j] += a[i] * b[j];
				}
				__syncthreads();
			}
			for (int i = 0; i < 4; i++)
			{
				const int gm = row0 + ty + 16 * i;
				if (gm >= rows)
					continue;
				for (int j = 0; j < 4; j++)
				{
					const int gn = col0 + tx + 16 * j;
					if (gn >= cols)
						continue;
					C *dst = Cm + static_cast<long long>(gm) * ldc + gn;
					if (std::is_integral<Acc>::value)
					{ // integer accumulation: alpha = 1, beta = 0 (reference: src/backend/cuda/gemms.cpp:119-130)
						*dst = store_as<C, Acc>(acc[i][j]);
					}
					else
					{
						Acc v = static_cast<Acc>(alpha) * acc[i][j];
						if (beta != 0.0f)
							v += static_cast<Acc>(beta) * load_as<C, Acc>(dst);
						*dst = store_as<C, Acc>(v);
					}
				}
			}
		}

		/* fp32 x fp32 -> fp32 on the CUDA cores: 128 x 128 output tile per CTA, K in steps of 16, 8 x 8 outputs per thread read from
		 * shared memory as 16-byte vectors, the next K step prefetched into registers while the current one is multiplied.  The generic
		 * kernel above covers every other type and any alignment; this one serves fp32 products whose rows are 16-byte aligned when
		 * the tensor-core engine is switched off for them (MINML_B200_FP32_SIMT=1) or cannot address them.
		 * TA: A is stored [K, rows] (op 't'); TB: B is stored [cols, K] (op 't').  Needs 16-byte aligned operands and leading
		 * dimensions that are multiples of 4. */
		constexpr int FM = 128, FN = 128, FK = 16;
		template<bool TA, bool TB>
		__global__ void __launch_bounds__(256) kernel_sgemm_fp32(const float *__restrict__ A, const float *__restrict__ B, float *Cm, int rows, int cols,
				int K, int lda, int ldb, int ldc, long long stride_a, long long stride_b, long long stride_c, float alpha, float beta)
		{
			__shared__ __align__(16) float sa[2][FK][FM + 4];
			__shared__ __align__(16) float sb[2][FK][FN + 4];
			const int batch = blockIdx.z;
			A += batch * stride_a;
			B += batch * stride_b;
			Cm += batch * stride_c;
			const int row0 = blockIdx.y * FM, col0 = blockIdx.x * FN;
			const int t = threadIdx.x;
			const int tx = t % 16, ty = t / 16;

			// each thread fetches two 4-element groups of each operand tile per K step
			float4 ra[2], rb[2];
			auto fetch = [&](int k0)
			{
#pragma unroll
				for (int h = 0; h < 2; h++)
				{
					float v[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
					if (TA)
					{ // [K, rows]: 16 k-rows of 128 floats; thread -> (k = t / 32 + 8 h, m = 4 (t % 32))
						const int k = k0 + t / 32 + 8 * h, m = row0 + 4 * (t % 32);
						if (k < K)
						{
							const float *p = A + static_cast<long long>(k) * lda + m;
							if (m + 3 < rows)
								*reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(p);
							else
								for (int e = 0; e < 4; e++)
									if (m + e < rows)
										v[e] = p[e];
						}
					}
					else
					{ // [rows, K]: 128 rows of 16 floats; thread -> (m = t / 4 + 64 h, k = 4 (t % 4))
						const int m = row0 + t / 4 + 64 * h, k = k0 + 4 * (t % 4);
						if (m < rows)
						{
							const float *p = A + static_cast<long long>(m) * lda + k;
							if (k + 3 < K)
								*reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(p);
							else
								for (int e = 0; e < 4; e++)
									if (k + e < K)
										v[e] = p[e];
						}
					}
					ra[h] = make_float4(v[0], v[1], v[2], v[3]);
					float u[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
					if (!TB)
					{ // [K, cols]
						const int k = k0 + t / 32 + 8 * h, n = col0 + 4 * (t % 32);
						if (k < K)
						{
							const float *p = B + static_cast<long long>(k) * ldb + n;
							if (n + 3 < cols)
								*reinterpret_cast<float4*>(u) = *reinterpret_cast<const float4*>(p);
							else
								for (int e = 0; e < 4; e++)
									if (n + e < cols)
										u[e] = p[e];
						}
					}
					else
					{ // [cols, K]
						const int n = col0 + t / 4 + 64 * h, k = k0 + 4 * (t % 4);
						if (n < cols)
						{
							const float *p = B + static_cast<long long>(n) * ldb + k;
							if (k + 3 < K)
								*reinterpret_cast<float4*>(u) = *reinterpret_cast<const float4*>(p);
							else
								for (int e = 0; e < 4; e++)
									if (k + e < K)
										u[e] = p[e];
						}
					}
					rb[h] = make_float4(u[0], u[1], u[2], u[3]);
				}
			};
			auto stage = [&](int buf)
			{
#pragma unroll
				for (int h = 0; h < 2; h++)
				{
					if (TA)
						*reinterpret_cast<float4*>(&sa[buf][t / 32 + 8 * h][4 * (t % 32)]) = ra[h];
					else
					{
						const int m = t / 4 + 64 * h, k = 4 * (t % 4);
						sa[buf][k][m] = ra[h].x;
						sa[buf][k + 1][m] = ra[h].y;
						sa[buf][k + 2][m] = ra[h].z;
						sa[buf][k + 3][m] = ra[h].w;
					}
					if (!TB)
						*reinterpret_cast<float4*>(&sb[buf][t / 32 + 8 * h][4 * (t % 32)]) = rb[h];
					else
					{
						const int n = t / 4 + 64 * h, k = 4 * (t % 4);
						sb[buf][k][n] = rb[h].x;
						sb[buf][k + 1][n] = rb[h].y;
						sb[buf][k + 2][n] = rb[h].z;
						sb[buf][k + 3][n] = rb[h].w;
					}
				}
			};

			float acc[8][8];
#pragma unroll
			for (int i = 0; i < 8; i++)
#pragma unroll
				for (int j = 0; j < 8; j++)
					acc[i][j] = 0.0f;

			fetch(0);
			stage(0);
			__syncthreads();
			int buf = 0;
			for (int k0 = 0; k0 < K; k0 += FK)
			{
				const bool more = k0 + FK < K;
				if (more)
					fetch(k0 + FK);
#pragma unroll
				for (int k = 0; k < FK; k++)
				{
					const float4 a0 = *reinterpret_cast<const float4*>(&sa[buf][k][4 * ty]);
					const float4 a1 = *reinterpret_cast<const float4*>(&sa[buf][k][64 + 4 * ty]);
					const float4 b0 = *reinterpret_cast<const float4*>(&sb[buf][k][4 * tx]);
					const float4 b1 = *reinterpret_cast<const float4*>(&sb[buf][k][64 + 4 * tx]);
					const float a[8] = { a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w };
					const float b[8] = { b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w };
#pragma unroll
					for (int i = 0; i < 8; i++)
#pragma unroll
						for (int j = 0; j < 8; j++)
							acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
				}
				if (more)
				{
					stage(buf ^ 1);
					__syncthreads();
					buf ^= 1;
				}
			}
#pragma unroll
			for (int i = 0; i < 8; i++)
			{
				const int gm = row0 + (i < 4 ? 4 * ty + i : 64 + 4 * ty + i - 4);
				if (gm >= rows)
					continue;
#pragma unroll
				for (int jh = 0; jh < 2; jh++)
				{
					const int gn = col0 + 64 * jh + 4 * tx;
					float *dst = Cm + static_cast<long long>(gm) * ldc + gn;
					float v[4];
#pragma unroll
					for (int e = 0; e < 4; e++)
						v[e] = alpha * acc[i][4 * jh + e];
					if (gn + 3 < cols && (ldc % 4) == 0 && (reinterpret_cast<uintptr_t>(Cm) % 16) == 0)
					{
						if (beta != 0.0f)
						{
							const float4 c = *reinterpret_cast<const float4*>(dst);
							v[0] += beta * c.x;
							v[1] += beta * c.y;
							v[2] += beta * c.z;
							v[3] += beta * c.w;
						}
						*reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
					}
					else
					{
						for (int e = 0; e < 4; e++)
							if (gn + e < cols)
								dst[e] = (beta != 0.0f) ? v[e] + beta * dst[e] : v[e];
					}
				}
			}
		}
		bool sgemm_fp32_applicable(const GemmSimtProblem &g)
		{
			return g.ab_dtype == DTYPE_FLOAT32 && g.c_dtype == DTYPE_FLOAT32 && aligned_to(g.A, 16) && aligned_to(g.B, 16) && g.lda % 4 == 0
					&& g.ldb % 4 == 0 && g.stride_a % 4 == 0 && g.stride_b % 4 == 0 && static_cast<long long>(g.rows) * g.cols >= 128 * 128;
		}
		bool launch_sgemm_fp32(mlContext_t ctx, const GemmSimtProblem &g)
		{
			cudaStream_t stream = use_stream(ctx);
			dim3 grid(ceil_div(g.cols, FN), ceil_div(g.rows, FM), g.batch);
			if (grid.y > 65535 || grid.z > 65535)
				return false;
			const float *a = reinterpret_cast<const float*>(g.A), *b = reinterpret_cast<const float*>(g.B);
			float *c = reinterpret_cast<float*>(g.C);
			if (!g.trans_a && g.trans_b)
				kernel_sgemm_fp32<false, true> <<<grid, 256, 0, stream>>>(a, b, c, g.rows, g.cols, g.K, g.lda, g.ldb, g.ldc, g.stride_a, g.stride_b, g.stride_c,
						g.alpha, g.beta);
			else if (!g.trans_a && !g.trans_b)
				kernel_sgemm_fp32<false, false> <<<grid, 256, 0, stream>>>(a, b, c, g.rows, g.cols, g.K, g.lda, g.ldb, g.ldc, g.stride_a, g.stride_b, g.stride_c,
						g.alpha, g.beta);
			else if (g.trans_a && !g.trans_b)
				kernel_sgemm_fp32<true, false> <<<grid, 256, 0, stream>>>(a, b, c, g.rows, g.cols, g.K, g.lda, g.ldb, g.ldc, g.stride_a, g.stride_b, g.stride_c,
						g.alpha, g.beta);
			else
				kernel_sgemm_fp32<true, true> <<<grid, 256, 0, stream>>>(a, b, c, g.rows, g.cols, g.K, g.lda, g.ldb, g.ldc, g.stride_a, g.stride_b, g.stride_c,
						g.alpha, g.beta);
			MB200_COUNT_LAUNCH();
			return check_cuda(ctx, cudaGetLastError(), "sgemm_fp32 launch");
		}

		template<typename AB, typename C>
		bool launch(mlContext_t ctx, const GemmSimtProblem &g)
		{
			cudaStream_t stream = use_stream(ctx);
			dim3 grid(ceil_div(g.cols, TN), ceil_div(g.rows, TM), g.batch);
			if (grid.y > 65535 || grid.z > 65535)
			{
				record_error(ctx, "gemm: %d x %d x batch %d exceeds the grid limits of the generic kernel", g.rows, g.cols, g.batch);
				return false;
			}
			kernel_gemm_simt<AB, C> <<<grid, 256, 0, stream>>>(reinterpret_cast<const AB*>(g.A), reinterpret_cast<const AB*>(g.B),
					reinterpret_cast<C*>(g.C), g.rows, g.cols, g.K, g.lda, g.ldb, g.ldc, g.stride_a, g.stride_b, g.stride_c, g.trans_a, g.trans_b,
					g.alpha, g.beta);
			MB200_COUNT_LAUNCH();
			return check_cuda(ctx, cudaGetLastError(), "gemm_simt launch");
		}
	}

	bool gemm_simt_run(mlContext_t ctx, const GemmSimtProblem &g)
	{
		if (g.rows <= 0 || g.cols <= 0 || g.batch <= 0)
			return true;
		if (sgemm_fp32_applicable(g) && launch_sgemm_fp32(ctx, g))
			return true;
		if (g.ab_dtype == DTYPE_FLOAT32 && g.c_dtype == DTYPE_FLOAT32)
			return launch<float, float>(ctx, g);
		if (g.ab_dtype == DTYPE_FLOAT16 && g.c_dtype == DTYPE_FLOAT16)
			return launch<__half, __half>(ctx, g);
		if (g.ab_dtype == DTYPE_FLOAT16 && g.c_dtype == DTYPE_FLOAT32)
			return launch<__half, float>(ctx, g);
		if (g.ab_dtype == DTYPE_FLOAT64 && g.c_dtype == DTYPE_FLOAT64)
			return launch<double, double>(ctx, g);
		if (g.ab_dtype == DTYPE_INT8 && g.c_dtype == DTYPE_INT32)
			return launch<int8_t, int>(ctx, g);
		record_error(ctx, "gemm: unsupported dtype combination (operands %d, result %d)", static_cast<int>(g.ab_dtype),
				static_cast<int>(g.c_dtype));
		return false;
	}
} /* namespace mb200 */
