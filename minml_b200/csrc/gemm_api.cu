/*
 * gemm_api.cu -- the matrix-multiplication entry points of the C ABI and their dispatch onto the two engines.
 *
 * Row-major semantics, identical to the reference wrappers (src/backend/cuda/gemms.cpp:99-407):
 *   C (rows x cols) = alpha * op(A) * op(B) + beta * C
 *   rows = opA == 't' ? columns(A) : rows(A);  cols = opB == 't' ? rows(B) : columns(B);  K = opB == 't' ? columns(B) : rows(B)
 * Batched variants take rank-3 tensors [batch, rows, columns]; a rank-2 operand is broadcast over the batch.
 * The result dtype selects the arithmetic: int32 <- int8 x int8 (alpha = 1, beta = 0), fp16 <- fp16, fp32 <- fp32 or fp16, fp64.
 *
 * 'n','t' products on fp16 or int8 data that TMA can address run on the tcgen05 kernel; everything else on the
 * generic kernel.  cuda_gemm_ex fuses beta * C, bias and activation into the tensor-core epilogue (the reference's
 * non-cuDNN build needs three extra passes over D: src/backend/cuda/cudnn_math.cpp:696-715).
 */
#include <cstdlib>
#include "common.cuh"
#include "gemm.cuh"
#include "winograd.cuh"
#include "conv.cuh"

using namespace mb200;

namespace
{
	struct Operand
	{
			const void *data;
			mlDataType_t dtype;
			int rows, cols;
			long long batch_stride;
			bool matrix; // rank 2 or 3
	};
	Operand operand_of(const mlTensor_t &t)
	{
		Operand r { t.data, t.dtype, 0, 0, 0, t.rank == 2 || t.rank == 3 };
		if (t.rank == 2)
		{
			r.rows = t.dim[0];
			r.cols = t.dim[1];
		}
		else if (t.rank == 3)
		{
			r.rows = t.dim[1];
			r.cols = t.dim[2];
			r.batch_stride = static_cast<long long>(t.dim[1]) * t.dim[2];
		}
		return r;
	}
	Operand operand_of(const void *data, mlDataType_t dtype, const mlShape_t &s)
	{
		return operand_of(make_tensor(data, dtype, s));
	}

	/* D = act(alpha * op(A) op(B) + beta * Cin + bias).  Cin may alias D.  bias/act are optional. */
	void run_gemm(mlContext_t ctx, const char *who, char opA, char opB, float alpha, const Operand &A, const Operand &B, float beta, const Operand &D,
			const void *Cin, const void *bias, mlActivationType_t act, int batch)
	{
		MB200_REQUIRE(ctx, ctx != nullptr, "%s: null context", who);
		MB200_REQUIRE(ctx, A.matrix && B.matrix && D.matrix, "%s: operands must have rank 2 or 3", who);
		if (static_cast<long long>(D.rows) * D.cols == 0 || batch == 0)
			return; // an empty product: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(ctx, A.data != nullptr && B.data != nullptr && D.data != nullptr, "%s: null tensor data", who);
		const bool ta = is_transpose(opA), tb = is_transpose(opB);
		const int rows = ta ? A.cols : A.rows;
		const int cols = tb ? B.rows : B.cols;
		const int K = tb ? B.cols : B.rows;
		const int Ka = ta ? A.rows : A.cols;
		MB200_REQUIRE(ctx, K == Ka, "%s: inner dimensions differ (%d vs %d)", who, Ka, K);
		MB200_REQUIRE(ctx, rows == D.rows && cols == D.cols, "%s: result is %d x %d but op(A) op(B) is %d x %d", who, D.rows, D.cols, rows, cols);
		MB200_REQUIRE(ctx, A.dtype == B.dtype, "%s: A and B must have the same dtype", who);
		const bool is_int = (D.dtype == DTYPE_INT32);
		if (is_int)
		{
			MB200_REQUIRE(ctx, A.dtype == DTYPE_INT8, "%s: int32 result needs int8 operands", who);
			MB200_REQUIRE(ctx, K % 4 == 0, "%s: int8 product needs K %% 4 == 0 (K = %d)", who, K);
			alpha = 1.0f;
			beta = 0.0f;
		}
		else if (D.dtype == DTYPE_FLOAT16)
			MB200_REQUIRE(ctx, A.dtype == DTYPE_FLOAT16, "%s: fp16 result needs fp16 operands", who);
		else if (D.dtype == DTYPE_FLOAT32)
			MB200_REQUIRE(ctx, A.dtype == DTYPE_FLOAT32 || A.dtype == DTYPE_FLOAT16, "%s: fp32 result needs fp32 or fp16 operands", who);
		else if (D.dtype == DTYPE_FLOAT64)
			MB200_REQUIRE(ctx, A.dtype == DTYPE_FLOAT64, "%s: fp64 result needs fp64 operands", who);
		else
			MB200_REQUIRE(ctx, false, "%s: unsupported result dtype %d", who, static_cast<int>(D.dtype));
		if (rows == 0 || cols == 0 || batch == 0)
			return;

		flush_pending(ctx);

		const void *c_in = (beta != 0.0f) ? (Cin != nullptr ? Cin : D.data) : nullptr;
		// fp32 operands are read as plain TF32 only when the host has allowed TF32 on this context (cuda_enable_tf32), the
		// condition under which the reference asks cuBLAS for CUBLAS_COMPUTE_32F_FAST_TF32 (src/backend/cuda/gemms.cpp:150-153);
		// otherwise they run as three TF32 products of split operands, which keeps the result within fp32 rounding noise
		// (MINML_B200_FP32_SIMT=1 sends them to the plain fp32 engine instead)
		static const bool fp32_simt = std::getenv("MINML_B200_FP32_SIMT") != nullptr && std::getenv("MINML_B200_FP32_SIMT")[0] == '1';
		const bool fp32 = A.dtype == DTYPE_FLOAT32 && D.dtype == DTYPE_FLOAT32;
		const bool tf32 = fp32 && get(ctx)->allow_tf32;
		// the tensor-core engine takes every transposition of fp16 and fp32 operands ('t' on A and 'n' on B as MN-major operands); int8
		// products only in the 'n','t' form
		if ((A.dtype == DTYPE_FLOAT16 || (A.dtype == DTYPE_INT8 && !ta && tb) || tf32 || (fp32 && !fp32_simt)) && A.dtype == B.dtype
				&& (D.dtype == DTYPE_FLOAT16 || D.dtype == DTYPE_FLOAT32 || D.dtype == DTYPE_INT32))
		{
			GemmTcProblem g;
			g.kind = (A.dtype == DTYPE_FLOAT16) ? 0 : (A.dtype == DTYPE_INT8 ? 1 : (tf32 ? 2 : 3));
			g.M = rows;
			g.N = cols;
			g.K = K;
			g.batch = batch;
			g.a_mn = ta;
			g.b_mn = !tb;
			g.A = A.data;
			g.lda = A.cols;
			g.stride_a = A.batch_stride;
			g.B = B.data;
			g.ldb = B.cols;
			g.stride_b = B.batch_stride;
			g.D = const_cast<void*>(D.data);
			g.ldd = D.cols;
			g.stride_d = D.batch_stride;
			g.C = c_in;
			g.ldc = D.cols;
			g.stride_c = D.batch_stride;
			g.bias = bias;
			g.alpha = alpha;
			g.beta = beta;
			g.act = act;
			g.out_dtype = D.dtype;
			if (gemm_tc_supported(g))
			{
				gemm_tc_run(ctx, g);
				return;
			}
		}

		/* generic engine; beta * C with C != D needs C copied into D first, bias/activation run as a second pass */
		if (c_in != nullptr && c_in != D.data)
			cuda_memcpy_within_device(ctx, const_cast<void*>(D.data), 0, c_in, 0,
					static_cast<size_t>(D.batch_stride > 0 ? D.batch_stride * batch : static_cast<long long>(rows) * cols) * size_of(D.dtype));
		GemmSimtProblem s;
		s.ab_dtype = A.dtype;
		s.c_dtype = D.dtype;
		s.trans_a = ta;
		s.trans_b = tb;
		s.rows = rows;
		s.cols = cols;
		s.K = K;
		s.batch = batch;
		s.A = A.data;
		s.lda = A.cols;
		s.stride_a = A.batch_stride;
		s.B = B.data;
		s.ldb = B.cols;
		s.stride_b = B.batch_stride;
		s.C = const_cast<void*>(D.data);
		s.ldc = D.cols;
		s.stride_c = D.batch_stride;
		s.alpha = alpha;
		s.beta = beta;
		if (!gemm_simt_run(ctx, s))
			return;
		if (bias != nullptr || act != ACTIVATION_LINEAR)
		{
			mlTensor_t xy;
			xy.data = const_cast<void*>(D.data);
			xy.dtype = D.dtype;
			xy.rank = 2;
			xy.dim[0] = (D.batch_stride > 0 ? batch : 1) * rows;
			xy.dim[1] = cols;
			for (int i = 2; i < 6; i++)
				xy.dim[i] = 0;
			if (bias != nullptr)
			{
				mlTensor_t b = make_tensor(bias, D.dtype, make_shape( { cols }));
				cuda_add_bias_act(ctx, 1.0f, xy, b, 0.0f, xy, act);
			}
			else
				cuda_activation_forward(ctx, 1.0f, xy, 0.0f, xy, act);
		}
	}
}

extern "C"
{
	void cuda_gemm_v2(mlContext_t context, char opA, char opB, float alpha, const mlTensor_t A, const mlTensor_t B, float beta, mlTensor_t C)
	{
		if (context != nullptr && mb200::int8_gemm_defer(context, opA, opB, A, B, C))
			return;
		run_gemm(context, "cuda_gemm_v2", opA, opB, alpha, operand_of(A), operand_of(B), beta, operand_of(C), nullptr, nullptr, ACTIVATION_LINEAR,
				1);
	}
	void cuda_gemm_batched_v2(mlContext_t context, char opA, char opB, float alpha, const mlTensor_t A, const mlTensor_t B, float beta, mlTensor_t C)
	{
		MB200_REQUIRE(context, C.rank == 3, "cuda_gemm_batched_v2: result must have rank 3");
		MB200_REQUIRE(context, A.rank == 3 || B.rank == 3, "cuda_gemm_batched_v2: at least one operand must have rank 3");
		MB200_REQUIRE(context, (A.rank != 3 || A.dim[0] == C.dim[0]) && (B.rank != 3 || B.dim[0] == C.dim[0]),
				"cuda_gemm_batched_v2: batch sizes differ");
		if (mb200::get(context) != nullptr && mb200::winograd_defer_gemm(context, opA, opB, alpha, A, B, beta, C))
			return;
		run_gemm(context, "cuda_gemm_batched_v2", opA, opB, alpha, operand_of(A), operand_of(B), beta, operand_of(C), nullptr, nullptr,
				ACTIVATION_LINEAR, C.dim[0]);
	}
	void cuda_gemm(mlContext_t context, mlDataType_t dtype, mlShape_t shape_C, void *C, mlShape_t shape_A, const void *A, mlShape_t shape_B,
			const void *B, char opA, char opB, float alpha, float beta)
	{
		// legacy form: one dtype names everything; int32 means int8 operands (reference: src/backend/cuda/gemms.cpp:281-290)
		const mlDataType_t ab = (dtype == DTYPE_INT32) ? DTYPE_INT8 : dtype;
		run_gemm(context, "cuda_gemm", opA, opB, alpha, operand_of(A, ab, shape_A), operand_of(B, ab, shape_B), beta, operand_of(C, dtype, shape_C),
				nullptr, nullptr, ACTIVATION_LINEAR, 1);
	}
	void cuda_gemm_batched(mlContext_t context, mlDataType_t dtype, mlShape_t shape_C, void *C, mlShape_t shape_A, const void *A, mlShape_t shape_B,
			const void *B, char opA, char opB, float alpha, float beta)
	{
		MB200_REQUIRE(context, shape_C.rank == 3, "cuda_gemm_batched: result must have rank 3");
		const mlDataType_t ab = (dtype == DTYPE_INT32) ? DTYPE_INT8 : dtype;
		run_gemm(context, "cuda_gemm_batched", opA, opB, alpha, operand_of(A, ab, shape_A), operand_of(B, ab, shape_B), beta,
				operand_of(C, dtype, shape_C), nullptr, nullptr, ACTIVATION_LINEAR, shape_C.dim[0]);
	}
	void cuda_gemm_ex(mlContext_t context, mlDataType_t dtype, mlShape_t shape_D, void *D, float alpha, char opA, mlShape_t shape_A, const void *A,
			char opB, mlShape_t shape_B, const void *B, float beta, mlShape_t shape_C, const void *C, const void *bias, mlActivationType_t act)
	{
		(void) shape_C;
		MB200_REQUIRE(context, dtype == DTYPE_FLOAT16 || dtype == DTYPE_FLOAT32 || dtype == DTYPE_FLOAT64,
				"cuda_gemm_ex: dtype %d is not a floating-point type", static_cast<int>(dtype));
		run_gemm(context, "cuda_gemm_ex", opA, opB, alpha, operand_of(A, dtype, shape_A), operand_of(B, dtype, shape_B), beta,
				operand_of(D, dtype, shape_D), (beta != 0.0f) ? C : nullptr, bias, act, 1);
	}
}
