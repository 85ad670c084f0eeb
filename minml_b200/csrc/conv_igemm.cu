/*
 * conv_igemm.cu -- fused 3x3 convolution kernels (placeholder until the tcgen05 implicit-GEMM kernel lands).
 */
#include "common.cuh"
#include "conv.cuh"

namespace mb200
{
	bool conv_fused_input_supported(const mlTensor_t &x)
	{
		(void) x;
		return false;
	}
	bool conv_fused_supported(const mlTensor_t &x, const mlTensor_t &w, const mlTensor_t &y, mlActivationType_t act)
	{
		(void) x;
		(void) w;
		(void) y;
		(void) act;
		return false;
	}
	bool conv_fused_run(mlContext_t ctx, const mlTensor_t &x, const mlTensor_t &w, const void *bias, const void *ext, const mlTensor_t &y,
			mlActivationType_t act)
	{
		(void) x;
		(void) w;
		(void) bias;
		(void) ext;
		(void) y;
		(void) act;
		record_error(ctx, "fused convolution kernel not available");
		return false;
	}
	bool im2row_defer(mlContext_t ctx, mlDataType_t dtype, const mlShape_t &input_shape, void *output, const void *input, int kernel_size,
			bool invert, const void *padding)
	{
		(void) ctx; (void) dtype; (void) input_shape; (void) output; (void) input; (void) kernel_size; (void) invert; (void) padding;
		return false;
	}
	bool requant_complete_fused(mlContext_t ctx, mlDataType_t dtype, const mlShape_t &shape, void *output, mlQuantizationData_t output_qd,
			const void *input, const void *scales, const void *bias, mlActivationType_t act, const void *ext, mlQuantizationData_t ext_qd)
	{
		(void) ctx; (void) dtype; (void) shape; (void) output; (void) output_qd; (void) input; (void) scales; (void) bias; (void) act; (void) ext;
		(void) ext_qd;
		return false;
	}
} /* namespace mb200 */
