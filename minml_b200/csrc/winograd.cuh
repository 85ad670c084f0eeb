/*
 * winograd.cuh -- internal interface of the Winograd path: the three eager transforms and the deferred
 * recognition of the reference's call triple (fusion.cu).
 */
#pragma once

#include "common.cuh"

namespace mb200
{
	void winograd_weight_transform_eager(mlContext_t ctx, int tile_size, const mlTensor_t w, mlTensor_t matrices, bool invert);
	void winograd_input_transform_eager(mlContext_t ctx, int tile_size, const mlTensor_t x, mlTensor_t matrices);
	void winograd_output_transform_eager(mlContext_t ctx, int tile_size, const mlTensor_t matrices, const mlTensor_t bias, const mlTensor_t ext,
			mlTensor_t y, mlActivationType_t act);

	/* Keeps a backend-owned snapshot of the raw weights a set of transformed matrices was computed from (what the fused kernel
	 * reads); dropped when the matrices are freed (forget_pointer) or written to through the ABI (forget_range). */
	void winograd_register_weights(mlContext_t ctx, const mlTensor_t &w, const mlTensor_t &matrices, int tile_size, bool invert);
	void winograd_forget_pointer(const void *ptr);
	void winograd_forget_range(const void *ptr, size_t bytes);

	/* The three hooks of the deferred sequence.  Each returns true when it consumed the call. */
	bool winograd_defer_input(mlContext_t ctx, int tile_size, const mlTensor_t &x, const mlTensor_t &matrices);
	bool winograd_defer_gemm(mlContext_t ctx, char opA, char opB, float alpha, const mlTensor_t &A, const mlTensor_t &B, float beta,
			const mlTensor_t &C);
	bool winograd_complete_fused(mlContext_t ctx, int tile_size, const mlTensor_t &matrices, const mlTensor_t &bias, const mlTensor_t &ext,
			const mlTensor_t &y, mlActivationType_t act);
} /* namespace mb200 */
