/*
 * gemm.cuh -- internal interface between the GEMM entry points (gemm_api.cu) and the two GEMM engines:
 * the tcgen05 kernel (gemm_tc.cu) and the generic SIMT kernel (gemm_simt.cu).
 */
#pragma once

#include "common.cuh"

namespace mb200
{
	/* Problem statement for the tensor-core engine: D[b] = epilogue(alpha * A[b] (M x K) * B[b]^T (N x K) + beta * C[b]).
	 * Leading dimensions and batch strides are in elements; a batch stride of 0 broadcasts the operand. */
	struct GemmTcProblem
	{
			int kind = 0; // 0: fp16 operands, fp32 accumulation; 1: int8 operands, int32 accumulation; 2: fp32 operands read as tf32;
			// 3: fp32 operands split into two tf32 terms each (three tensor-core products, close to fp32 accuracy)
			int M = 0, N = 0, K = 0, batch = 1;
			// Storage of the operands: A as [M, K] (false) or [K, M] (true: 't' on A); B as [N, K] (false: 't' on B) or [K, N] (true).
			// The transposed forms reach the tensor core as MN-major operands (kinds 0, 2, 3).
			bool a_mn = false, b_mn = false;
			const void *A = nullptr;
			int lda = 0;
			long long stride_a = 0;
			const void *B = nullptr;
			int ldb = 0;
			long long stride_b = 0;
			void *D = nullptr;
			int ldd = 0;
			long long stride_d = 0;
			const void *C = nullptr; // read only when beta != 0 (fp16 kind) -- same dtype as D
			int ldc = 0;
			long long stride_c = 0;
			const void *bias = nullptr; // [N], same dtype as D (fp16 kind)
			float alpha = 1.0f, beta = 0.0f;
			int act = ACTIVATION_LINEAR;
			mlDataType_t out_dtype = DTYPE_FLOAT16;
			/* int8 kind with out_dtype != INT32: fused requantisation epilogue
			 * x = acc * scales[n] + shifts[n] (+ ext * ext_scale + ext_shift); act; int8 out = clamp(round(x * (1 / out_scale) + (-out_shift / out_scale))),
			 * every step rounded on its own (epilogue.cuh) */
			const float *scales = nullptr;
			const float *shifts = nullptr;
			const int8_t *ext = nullptr; // indexed like C (ldc, stride_c)
			float ext_scale = 1.0f, ext_shift = 0.0f, out_scale = 1.0f, out_shift = 0.0f;
	};
	/* Kernel-side copy of the above (what the device needs). */
	struct GemmTcParams
	{
			int M, N, K, batch;
			int a_mn, b_mn;
			int a_broadcast, b_broadcast;
			void *D;
			int ldd;
			long long stride_d;
			const void *C;
			int ldc;
			long long stride_c;
			const void *bias;
			float alpha, beta;
			int act;
			int out_dtype;
			const float *scales;
			const float *shifts;
			const int8_t *ext;
			float ext_scale, ext_shift, inv_out_scale, inv_out_shift;
			int *status;
	};
	bool gemm_tc_supported(const GemmTcProblem &g);
	bool gemm_tc_run(mlContext_t ctx, const GemmTcProblem &g);

	/* Generic engine: any transposition, any shape, dtypes {fp16, fp32, fp64} and int8 -> int32.
	 * C[b] (rows x cols) = alpha * op(A[b]) * op(B[b]) + beta * C[b]; accumulation in fp32 (fp64 for fp64, int32 for int8). */
	struct GemmSimtProblem
	{
			mlDataType_t ab_dtype = DTYPE_FLOAT32;
			mlDataType_t c_dtype = DTYPE_FLOAT32;
			bool trans_a = false, trans_b = false;
			int rows = 0, cols = 0, K = 0, batch = 1;
			const void *A = nullptr;
			int lda = 0;
			long long stride_a = 0;
			const void *B = nullptr;
			int ldb = 0;
			long long stride_b = 0;
			void *C = nullptr;
			int ldc = 0;
			long long stride_c = 0;
			float alpha = 1.0f, beta = 0.0f;
	};
	bool gemm_simt_run(mlContext_t ctx, const GemmSimtProblem &g);
} /* namespace mb200 */
