/*
 * stubs.cu -- entry points of the C ABI that are outside the convolution / matrix-multiply inference path
 * (training, mixture of experts, pooling and scaling variants, depthwise convolution, batch and RMS normalisation,
 * window operations).  They are exported so that minml's host library links against this backend exactly as it
 * links against src/backend/cuda or src/backend/cuda_dummy_backend.cpp; each records the sticky error
 * "<name>: not implemented by minml_b200" on its context and launches nothing.  The bracketed number is the line of
 * the declaration in the reference's include/minml/backend/cuda_backend.h.
 */
#include "common.cuh"

using namespace mb200;

#define NOT_IMPLEMENTED(ctx, name) record_error((ctx), "%s: not implemented by minml_b200", name)

extern "C"
{
	void cuda_depthwise_conv_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t w, float beta, mlTensor_t dx) /* [113] */
	{
		NOT_IMPLEMENTED(context, "cuda_depthwise_conv_backward");
	}
	void cuda_depthwise_conv_update(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t dy, float beta, mlTensor_t dw) /* [115] */
	{
		NOT_IMPLEMENTED(context, "cuda_depthwise_conv_update");
	}
	void cuda_average_pooling_forward(mlContext_t context, float alpha, const mlTensor_t x, float beta, mlTensor_t y, int size) /* [121] */
	{
		NOT_IMPLEMENTED(context, "cuda_average_pooling_forward");
	}
	void cuda_average_pooling_backward(mlContext_t context, float alpha, const mlTensor_t dy, float beta, mlTensor_t dx, int size) /* [122] */
	{
		NOT_IMPLEMENTED(context, "cuda_average_pooling_backward");
	}
	void cuda_global_average_pooling_backward(mlContext_t context, float alpha, const mlTensor_t dy, float beta, mlTensor_t dx) /* [128] */
	{
		NOT_IMPLEMENTED(context, "cuda_global_average_pooling_backward");
	}
	void cuda_channel_scaling_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t x, const mlTensor_t scales, float beta_dx, mlTensor_t dx, float beta_scales, mlTensor_t dscales) /* [131] */
	{
		NOT_IMPLEMENTED(context, "cuda_channel_scaling_backward");
	}
	void cuda_channel_average_pooling_forward(mlContext_t context, float alpha, const mlTensor_t x, float beta, mlTensor_t y) /* [137] */
	{
		NOT_IMPLEMENTED(context, "cuda_channel_average_pooling_forward");
	}
	void cuda_channel_average_pooling_backward(mlContext_t context, float alpha, const mlTensor_t dy, float beta, mlTensor_t dx) /* [138] */
	{
		NOT_IMPLEMENTED(context, "cuda_channel_average_pooling_backward");
	}
	void cuda_spatial_scaling_forward(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t scales, float beta, mlTensor_t y) /* [139] */
	{
		NOT_IMPLEMENTED(context, "cuda_spatial_scaling_forward");
	}
	void cuda_spatial_scaling_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t x, const mlTensor_t scales, float beta_dx, mlTensor_t dx, float beta_scales, mlTensor_t dscales) /* [141] */
	{
		NOT_IMPLEMENTED(context, "cuda_spatial_scaling_backward");
	}
	void cudnn_depthwise_conv_forward(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape, const void *input, const void *weights, const void *bias, void *output) /* [163] */
	{
		NOT_IMPLEMENTED(context, "cudnn_depthwise_conv_forward");
	}
	void cudnn_depthwise_conv_backward(mlContext_t context, mlShape_t input_shape, mlShape_t weights_shape, const void *gradient_next, const void *weights, void *gradient_prev) /* [165] */
	{
		NOT_IMPLEMENTED(context, "cudnn_depthwise_conv_backward");
	}
	void cudnn_depthwise_conv_update(mlContext_t context, mlShape_t input_shape, mlShape_t weights_shape, const void *input, const void *gradient_next, void *weights_update) /* [167] */
	{
		NOT_IMPLEMENTED(context, "cudnn_depthwise_conv_update");
	}
	void cuda_batchnorm_forward(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b, float beta, mlTensor_t y, mlTensor_t running_stats, mlActivationType_t act) /* [179] */
	{
		NOT_IMPLEMENTED(context, "cuda_batchnorm_forward");
	}
	void cuda_batchnorm_backward(mlContext_t context, float alpha, const mlTensor_t x, mlTensor_t dy, const mlTensor_t w, const mlTensor_t b, const mlTensor_t running_stats, float beta_dx, mlTensor_t dx, float beta_dw, mlTensor_t dw, mlTensor_t db, mlActivationType_t act) /* [181] */
	{
		NOT_IMPLEMENTED(context, "cuda_batchnorm_backward");
	}
	void cuda_batchnorm_update(mlContext_t context, const mlTensor_t running_stat, mlTensor_t avg_var) /* [184] */
	{
		NOT_IMPLEMENTED(context, "cuda_batchnorm_update");
	}
	void cuda_layernorm_backward(mlContext_t context, mlShape_t shape, const void *input, void *gradient_prev, void *gradient_next, const void *weights, void *weights_update, void *bias_update) /* [193] */
	{
		NOT_IMPLEMENTED(context, "cuda_layernorm_backward");
	}
	void cuda_rmsnorm_backward(mlContext_t context, mlShape_t shape, const void *input, void *gradient_prev, void *gradient_next, const void *weights, void *weights_update) /* [201] */
	{
		NOT_IMPLEMENTED(context, "cuda_rmsnorm_backward");
	}
	void cuda_multi_head_attention_backward(mlContext_t context, mlShape_t input_shape, mlShape_t weights_shape, mlShape_t bias_shape, const void *input, const void *weights, const void *bias, void *gradient_prev, void *gradient_next, void *weights_update, void *bias_update, void *workspace, void *backward_data, int num_heads, bool symmetric) /* [211] */
	{
		NOT_IMPLEMENTED(context, "cuda_multi_head_attention_backward");
	}
	void cuda_window_partitioning(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t output_shape, const void *input, void *output, mlShape_t offset) /* [218] */
	{
		NOT_IMPLEMENTED(context, "cuda_window_partitioning");
	}
	void cuda_window_merging(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t output_shape, const void *input, void *output, mlShape_t offset) /* [220] */
	{
		NOT_IMPLEMENTED(context, "cuda_window_merging");
	}
	void cuda_softmax_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t y, float beta, mlTensor_t dx) /* [231] */
	{
		NOT_IMPLEMENTED(context, "cuda_softmax_backward");
	}
	void cuda_channel_shuffle(mlContext_t context, const mlTensor_t x, float beta, mlTensor_t y, int groups, bool invert) /* [238] */
	{
		NOT_IMPLEMENTED(context, "cuda_channel_shuffle");
	}
	void cuda_group_gemm(mlContext_t context, char opA, char opB, float alpha, const mlTensor_t A, const mlTensor_t B, float beta, mlTensor_t C, int groups) /* [239] */
	{
		NOT_IMPLEMENTED(context, "cuda_group_gemm");
	}
	void cuda_hash_routing(mlContext_t context, const mlTensor_t x, mlTensor_t indices_and_values) /* [245] */
	{
		NOT_IMPLEMENTED(context, "cuda_hash_routing");
	}
	void cuda_token_choice_routing_forward(mlContext_t context, const mlTensor_t x, const mlTensor_t bias, mlTensor_t indices_and_values) /* [246] */
	{
		NOT_IMPLEMENTED(context, "cuda_token_choice_routing_forward");
	}
	void cuda_token_choice_routing_backward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, const mlTensor_t dy, float beta, mlTensor_t dx, float alpha, mlTensor_t bias, mlTensor_t workspace) /* [248] */
	{
		NOT_IMPLEMENTED(context, "cuda_token_choice_routing_backward");
	}
	void cuda_expert_choice_routing_forward(mlContext_t context, const mlTensor_t x, mlTensor_t indices_and_values) /* [250] */
	{
		NOT_IMPLEMENTED(context, "cuda_expert_choice_routing_forward");
	}
	void cuda_expert_choice_routing_backward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, const mlTensor_t dy, float beta, mlTensor_t dx) /* [251] */
	{
		NOT_IMPLEMENTED(context, "cuda_expert_choice_routing_backward");
	}
	void cuda_select_top_k(mlContext_t context, const mlTensor_t x, mlTensor_t indices, mlTensor_t values) /* [253] */
	{
		NOT_IMPLEMENTED(context, "cuda_select_top_k");
	}
	void cuda_gather_tokens_forward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, float beta, mlTensor_t y) /* [254] */
	{
		NOT_IMPLEMENTED(context, "cuda_gather_tokens_forward");
	}
	void cuda_gather_tokens_backward(mlContext_t context, const mlTensor_t dy, const mlTensor_t indices_and_values, float beta, mlTensor_t dx) /* [256] */
	{
		NOT_IMPLEMENTED(context, "cuda_gather_tokens_backward");
	}
	void cuda_scatter_tokens_forward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, float beta, mlTensor_t y) /* [258] */
	{
		NOT_IMPLEMENTED(context, "cuda_scatter_tokens_forward");
	}
	void cuda_scatter_tokens_backward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, const mlTensor_t dy, float beta1, mlTensor_t dx, float beta2, mlTensor_t dscales) /* [260] */
	{
		NOT_IMPLEMENTED(context, "cuda_scatter_tokens_backward");
	}
	void cuda_moe_forward(mlContext_t context, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b, float beta, mlTensor_t y, mlActivationType_t act) /* [262] */
	{
		NOT_IMPLEMENTED(context, "cuda_moe_forward");
	}
	void cuda_moe_backward(mlContext_t context, const mlTensor_t x, const mlTensor_t y, const mlTensor_t w, mlTensor_t dy, float beta_dx, mlTensor_t dx, float beta_dw, mlTensor_t dw, float beta_db, mlTensor_t db, mlActivationType_t act) /* [264] */
	{
		NOT_IMPLEMENTED(context, "cuda_moe_backward");
	}
	void cuda_learnable_scaling_forward(mlContext_t context, float alpha, const mlTensor_t x, mlActivationType_t act, const mlTensor_t w, float beta, mlTensor_t y) /* [270] */
	{
		NOT_IMPLEMENTED(context, "cuda_learnable_scaling_forward");
	}
	void cuda_learnable_scaling_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t x, mlActivationType_t act, const mlTensor_t w, float beta_dx, mlTensor_t dx, float beta_dw, mlTensor_t dw) /* [272] */
	{
		NOT_IMPLEMENTED(context, "cuda_learnable_scaling_backward");
	}
	void cuda_emulate_low_precision(mlContext_t context, mlShape_t shape, mlDataType_t dtype, void *dst, const void *src, mlQuantizationData_t qd) /* [278] */
	{
		NOT_IMPLEMENTED(context, "cuda_emulate_low_precision");
	}
	void cuda_sum_over_first_dim(mlContext_t context, float alpha, const mlTensor_t src, float beta, mlTensor_t dst) /* [287] */
	{
		NOT_IMPLEMENTED(context, "cuda_sum_over_first_dim");
	}
	float cuda_l2_norm(mlContext_t context, const mlTensor_t tensor) /* [292] */
	{
		NOT_IMPLEMENTED(context, "cuda_l2_norm");
		return 0.0f;
	}
	float cuda_mean_squared_loss(mlContext_t context, const mlTensor_t output, const mlTensor_t target, const mlTensor_t mask) /* [293] */
	{
		NOT_IMPLEMENTED(context, "cuda_mean_squared_loss");
		return 0.0f;
	}
	float cuda_cross_entropy_loss(mlContext_t context, const mlTensor_t output, const mlTensor_t target, const mlTensor_t mask) /* [294] */
	{
		NOT_IMPLEMENTED(context, "cuda_cross_entropy_loss");
		return 0.0f;
	}
	void cuda_mean_squared_gradient(mlContext_t context, float alpha, const mlTensor_t output, const mlTensor_t target, const mlTensor_t mask, float beta, mlTensor_t gradient) /* [295] */
	{
		NOT_IMPLEMENTED(context, "cuda_mean_squared_gradient");
	}
	void cuda_cross_entropy_gradient(mlContext_t context, float alpha, const mlTensor_t output, const mlTensor_t target, const mlTensor_t mask, float beta, mlTensor_t gradient) /* [297] */
	{
		NOT_IMPLEMENTED(context, "cuda_cross_entropy_gradient");
	}
	void cuda_fused_radam_optimize(mlContext_t context, float scale, const mlTensor_t *gradients, mlTensor_t *weights, mlTensor_t *momentums, mlTensor_t *variances, mlTensor_t *weights_copy, float learning_rate, float beta1, float beta2, int step, int num_tensors, float weight_decay) /* [300] */
	{
		NOT_IMPLEMENTED(context, "cuda_fused_radam_optimize");
	}
	void cuda_fused_lion_optimize(mlContext_t context, float scale, const mlTensor_t *gradients, mlTensor_t *weights, mlTensor_t *momentums, mlTensor_t *weights_copy, float learning_rate, float beta1, float beta2, int step, int num_tensors, float weight_decay) /* [303] */
	{
		NOT_IMPLEMENTED(context, "cuda_fused_lion_optimize");
	}
	void cuda_fused_is_nan_or_inf(mlContext_t context, const mlTensor_t *tensors, int *result, int num_tensors) /* [306] */
	{
		NOT_IMPLEMENTED(context, "cuda_fused_is_nan_or_inf");
	}
	void cuda_fused_l2_regularization(mlContext_t context, mlTensor_t *gradients, const mlTensor_t *params, float scale, int num_tensors) /* [307] */
	{
		NOT_IMPLEMENTED(context, "cuda_fused_l2_regularization");
	}
	void cuda_combined_loss(mlContext_t context, float *result, const mlTensor_t *outputs, const mlTensor_t *targets, const mlTensor_t *masks, const float *weights) /* [310] */
	{
		NOT_IMPLEMENTED(context, "cuda_combined_loss");
	}
	void cuda_transpose(mlContext_t context, mlDataType_t dtype, mlShape_t output_shape, mlShape_t input_shape, void *output, const void *input, const int *ordering) /* [326] */
	{
		NOT_IMPLEMENTED(context, "cuda_transpose");
	}
}
