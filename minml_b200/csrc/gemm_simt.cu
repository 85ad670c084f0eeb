/*
 * gemm_simt.cu -- generic CUDA-core GEMM: every transposition, any shape or alignment, fp16 / fp32 / fp64 and
 * int8 -> int32.  It is the engine behind the GEMM entry points whenever the tensor-core kernel does not apply
 * (fp32 and fp64 data, 'n','n' / 't','n' / 't','t' products, operands that TMA cannot address).  The reference
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
