/*
 * minml_b200.h -- C ABI of libminml_b200.so
 *
 * The library is a drop-in for the CUDA backend of MaciejKozarzewski/minml: it exports, unmangled, every
 * `cuda_*` symbol that minml's host code (src/core/math.cpp, Context.cpp, Event.cpp, ml_memory.cpp, Device.cpp)
 * binds through include/minml/backend/cuda_backend.h, with identical argument lists and the same POD descriptor
 * types as include/minml/backend/backend_types.h:30-75.  Each group below names the reference file it replaces;
 * the number in brackets after a declaration is its line in the reference's cuda_backend.h.
 *
 * Status tags:
 *   [hot]    implemented with hand-written sm_100a kernels (the convolution / matrix-multiply inference path)
 *   [next]   implemented: the layers adjacent to that path in minml's current architectures (batch-norm inference and
 *            folding, depthwise convolution fp / int8, squeeze-and-excitation channel scaling, RMS normalisation, space-to-depth
 *            and depth-to-space, the elementwise product of the Multiply layer, and the backward-pass Winograd transforms with the fused activation / bias-gradient step)
 *   [infra]  thin native wrapper over the CUDA runtime
 *   [stub]   exported so that minml links; records the sticky error "not implemented" on the context and
 *            launches nothing (training, MoE, pooling variants, ...)
 *
 * Conventions (same as the reference): descriptors are passed by value; pointers inside descriptors and all
 * `void *` tensor arguments are DEVICE pointers; `const int *`, `const mlTensor_t *` and `const void *padding`
 * arguments are HOST pointers; alpha defaults to 1 and beta to 0, both fp32; tensors are dense, row-major, NHWC.
 * No entry point aborts the process: arguments are validated on the host, a failed check records a sticky error
 * on the context (mb200_get_last_error) and the launch is skipped.  There is no CPU fallback.
 */
#ifndef MINML_B200_H_
#define MINML_B200_H_

#include <stddef.h>
#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- descriptor types: layout-identical to include/minml/backend/backend_types.h:30-75 ---- */
typedef struct { int rank; int dim[6]; } mlShape_t;
typedef struct { float scale; float shift; } mlQuantizationData_t;
typedef enum {
	DTYPE_UNKNOWN, DTYPE_FLOAT8, DTYPE_FLOAT16, DTYPE_FLOAT32, DTYPE_FLOAT64,
	DTYPE_UINT8, DTYPE_INT8, DTYPE_INT16, DTYPE_INT32
} mlDataType_t;
typedef enum {
	ACTIVATION_LINEAR, ACTIVATION_SIGMOID, ACTIVATION_TANH, ACTIVATION_RELU, ACTIVATION_LEAKY_RELU, ACTIVATION_EXP
} mlActivationType_t;
typedef struct { void *data; mlDataType_t dtype; int rank; int dim[6]; } mlTensor_t;
typedef void *mlContext_t;
typedef void *mlEvent_t;

/* ---- Device properties
 *      replaces src/backend/cuda/cuda_properties.cpp:213-262 ---- */
int cuda_get_number_of_devices(void); /* [infra] [49] */
void cuda_enable_tf32(mlContext_t context, bool b); /* [infra] [50] */
int cuda_get_memory(int index); /* [infra] [54] */
bool cuda_supports_type(int index, mlDataType_t dtype); /* [infra] [55] */
const char* cuda_get_device_info(int index); /* [infra] [56] */
const char* cuda_get_device_features(int index); /* [infra] [57] */

/* ---- Context: one in-order stream per context
 *      replaces src/backend/cuda/cuda_context.cpp:16-35, src/backend/cuda/utils.cpp:29-199 ---- */
mlContext_t cuda_create_context(int device_index); /* [infra] [60] */
void cuda_synchronize_with_context(mlContext_t context); /* [infra] [61] */
bool cuda_is_context_ready(mlContext_t context); /* [infra] [62] */
void cuda_destroy_context(mlContext_t context); /* [infra] [63] */

/* ---- Events
 *      replaces src/backend/cuda/cuda_event.cpp:16-53 ---- */
mlEvent_t cuda_create_event(mlContext_t context); /* [infra] [66] */
double cuda_get_time_between_events(mlEvent_t start, mlEvent_t end); /* [infra] [67] */
void cuda_wait_for_event(mlEvent_t event); /* [infra] [68] */
bool cuda_is_event_ready(mlEvent_t event); /* [infra] [69] */
void cuda_destroy_event(mlEvent_t event); /* [infra] [70] */

/* ---- Device memory
 *      replaces src/backend/cuda/cuda_memory.cu:133-274 ---- */
void* cuda_malloc(int device_index, size_t count); /* [infra] [73] */
void cuda_page_lock(void *ptr, size_t count); /* [infra] [74] */
void cuda_page_unlock(void *ptr); /* [infra] [75] */
void cuda_free(void *ptr); /* [infra] [76] */
void* cuda_create_view(void *src, size_t offset, size_t count); /* [infra] [77] */
void cuda_destroy_view(void *ptr); /* [infra] [78] */
void cuda_memset(mlContext_t context, void *dst, size_t dst_offset, size_t dst_count, const void *src, size_t src_count); /* [infra] [79] */
void cuda_memcpy_within_device(mlContext_t context, void *dst, size_t dst_offset, const void *src, size_t src_offset, size_t count); /* [infra] [80] */
void cuda_memcpy_from_host(mlContext_t context, void *dst, size_t dst_offset, const void *src, size_t count); /* [infra] [82] */
void cuda_memcpy_to_host(mlContext_t context, void *dst, const void *src, size_t src_offset, size_t count); /* [infra] [83] */

/* ---- Layout and dtype conversion
 *      replaces src/backend/cuda/kernels/conversion.cu:35-54,196-330 ---- */
void cuda_unpack_input(mlContext_t context, mlShape_t shape, mlDataType_t dst_dtype, void *dst, const void *src); /* [hot] [86] */
void cuda_convert_type(mlContext_t context, void *dst, mlDataType_t dst_dtype, const void *src, mlDataType_t src_dtype, int elements); /* [hot] [87] */
void cuda_transpose_021(mlContext_t context, mlDataType_t dtype, mlShape_t shape, const void *input, void *output); /* [hot] [89] */
void cuda_space_to_depth(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, const void *input, mlShape_t output_shape, void *output); /* [next] [90] */
void cuda_depth_to_space(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, const void *input, mlShape_t output_shape, void *output); /* [next] [92] */

/* ---- Winograd transforms
 *      replaces src/backend/cuda/kernels/winograd_nonfused.cu:417-520 ---- */
void cuda_winograd_weight_transform(mlContext_t context, int tile_size, const mlTensor_t w, mlTensor_t matrices, bool invert); /* [hot] [96] */
void cuda_winograd_input_transform(mlContext_t context, int tile_size, const mlTensor_t x, mlTensor_t matrices); /* [hot] [97] */
void cuda_winograd_output_transform(mlContext_t context, int tile_size, const mlTensor_t matrices, const mlTensor_t bias, const mlTensor_t ext, mlTensor_t y, mlActivationType_t act); /* [hot] [98] */
void cuda_winograd_gradient_transform(mlContext_t context, int tile_size, const mlTensor_t dy, mlTensor_t matrices); /* [next] [100] */
void cuda_winograd_update_transform(mlContext_t context, int tile_size, const mlTensor_t matrices, mlTensor_t dw); /* [next] [101] */

/* ---- Fused convolution: y = act(conv(x, w) + bias + add)
 *      replaces src/backend/cuda/cudnn_math.cpp:374-476,691-694 ---- */
void cuda_convolution_implicit_gemm_forward(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape, const void *input, const void *weights, void *output, const void *bias, const void *add, mlActivationType_t act); /* [hot] [104] */

/* ---- Depthwise convolution
 *      replaces src/backend/cuda/kernels/depthwise_conv.cu ---- */
void cuda_depthwise_conv_forward(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b, float beta, mlTensor_t y); /* [next] [111] */
void cuda_depthwise_conv_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t w, float beta, mlTensor_t dx); /* [stub] [113] */
void cuda_depthwise_conv_update(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t dy, float beta, mlTensor_t dw); /* [stub] [115] */

/* ---- Pooling and scaling
 *      replaces src/backend/cuda/kernels/global_pooling.cu:269-314, src/backend/cuda/kernels/pooling.cu ---- */
void cuda_average_pooling_forward(mlContext_t context, float alpha, const mlTensor_t x, float beta, mlTensor_t y, int size); /* [stub] [121] */
void cuda_average_pooling_backward(mlContext_t context, float alpha, const mlTensor_t dy, float beta, mlTensor_t dx, int size); /* [stub] [122] */
void cuda_global_average_pooling_forward(mlContext_t context, float alpha, const mlTensor_t x, float beta, mlTensor_t y); /* [hot] [127] */
void cuda_global_average_pooling_backward(mlContext_t context, float alpha, const mlTensor_t dy, float beta, mlTensor_t dx); /* [stub] [128] */
void cuda_channel_scaling_forward(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t scales, float beta, mlTensor_t y); /* [next] [129] */
void cuda_channel_scaling_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t x, const mlTensor_t scales, float beta_dx, mlTensor_t dx, float beta_scales, mlTensor_t dscales); /* [stub] [131] */
void cuda_channel_average_pooling_forward(mlContext_t context, float alpha, const mlTensor_t x, float beta, mlTensor_t y); /* [stub] [137] */
void cuda_channel_average_pooling_backward(mlContext_t context, float alpha, const mlTensor_t dy, float beta, mlTensor_t dx); /* [stub] [138] */
void cuda_spatial_scaling_forward(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t scales, float beta, mlTensor_t y); /* [stub] [139] */
void cuda_spatial_scaling_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t x, const mlTensor_t scales, float beta_dx, mlTensor_t dx, float beta_scales, mlTensor_t dscales); /* [stub] [141] */

/* ---- Matrix multiplication (row-major)
 *      replaces src/backend/cuda/gemms.cpp:99-407 ---- */
void cuda_gemm_v2(mlContext_t context, char opA, char opB, float alpha, const mlTensor_t A, const mlTensor_t B, float beta, mlTensor_t C); /* [hot] [147] */
void cuda_gemm_batched_v2(mlContext_t context, char opA, char opB, float alpha, const mlTensor_t A, const mlTensor_t B, float beta, mlTensor_t C); /* [hot] [149] */
void cuda_gemm(mlContext_t context, mlDataType_t dtype, mlShape_t shape_C, void *C, mlShape_t shape_A, const void *A, mlShape_t shape_B, const void *B, char opA, char opB, float alpha, float beta); /* [hot] [151] */
void cuda_gemm_batched(mlContext_t context, mlDataType_t dtype, mlShape_t shape_C, void *C, mlShape_t shape_A, const void *A, mlShape_t shape_B, const void *B, char opA, char opB, float alpha, float beta); /* [hot] [153] */

/* ---- GEMM with fused epilogue, cuDNN-era depthwise entries
 *      replaces src/backend/cuda/cudnn_math.cpp:478-549,696-730 ---- */
void cuda_gemm_ex(mlContext_t context, mlDataType_t dtype, mlShape_t shape_D, void *D, float alpha, char opA, mlShape_t shape_A, const void *A, char opB, mlShape_t shape_B, const void *B, float beta, mlShape_t shape_C, const void *C, const void *bias, mlActivationType_t act); /* [hot] [160] */
void cudnn_depthwise_conv_forward(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape, const void *input, const void *weights, const void *bias, void *output); /* [stub] [163] */
void cudnn_depthwise_conv_backward(mlContext_t context, mlShape_t input_shape, mlShape_t weights_shape, const void *gradient_next, const void *weights, void *gradient_prev); /* [stub] [165] */
void cudnn_depthwise_conv_update(mlContext_t context, mlShape_t input_shape, mlShape_t weights_shape, const void *input, const void *gradient_next, void *weights_update); /* [stub] [167] */

/* ---- Bias + activation
 *      replaces src/backend/cuda/kernels/activations.cu:258-284 ---- */
void cuda_add_bias_act(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t b, float beta, mlTensor_t y, mlActivationType_t act); /* [hot] [171] */

/* ---- Batch normalisation
 *      replaces src/backend/cuda/kernels/batchnorm.cu ---- */
void cuda_batchnorm_inference(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b, const mlTensor_t avg_var, float beta, mlTensor_t y, mlActivationType_t act); /* [next] [177] */
void cuda_batchnorm_forward(mlContext_t context, float alpha, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b, float beta, mlTensor_t y, mlTensor_t running_stats, mlActivationType_t act); /* [stub] [179] */
void cuda_batchnorm_backward(mlContext_t context, float alpha, const mlTensor_t x, mlTensor_t dy, const mlTensor_t w, const mlTensor_t b, const mlTensor_t running_stats, float beta_dx, mlTensor_t dx, float beta_dw, mlTensor_t dw, mlTensor_t db, mlActivationType_t act); /* [stub] [181] */
void cuda_batchnorm_update(mlContext_t context, const mlTensor_t running_stat, mlTensor_t avg_var); /* [stub] [184] */
void cuda_fold_batchnorm(mlContext_t context, mlTensor_t layer_weights, mlTensor_t layer_bias, const mlTensor_t bn_weights, const mlTensor_t bn_bias, const mlTensor_t bn_avg_var); /* [next] [185] */

/* ---- Layer / RMS normalisation
 *      replaces src/backend/cuda/kernels/layernorm.cu:480-527, src/backend/cuda/kernels/rmsnorm.cu ---- */
void cuda_layernorm_forward(mlContext_t context, mlShape_t shape, mlDataType_t dtype, const void *input, void *output, const void *weights, const void *bias, const void *ext); /* [hot] [191] */
void cuda_layernorm_backward(mlContext_t context, mlShape_t shape, const void *input, void *gradient_prev, void *gradient_next, const void *weights, void *weights_update, void *bias_update); /* [stub] [193] */
void cuda_rmsnorm_forward(mlContext_t context, mlShape_t shape, mlDataType_t dtype, const void *input, void *output, const void *weights); /* [next] [199] */
void cuda_rmsnorm_backward(mlContext_t context, mlShape_t shape, const void *input, void *gradient_prev, void *gradient_next, const void *weights, void *weights_update); /* [stub] [201] */

/* ---- Multi-head attention
 *      replaces src/backend/cuda/kernels/attention.cu:494-568 ---- */
int cuda_multi_head_attention_get_workspace_size(mlShape_t input_shape, mlShape_t weights_shape, int num_heads, bool training); /* [hot] [207] */
void cuda_multi_head_attention_forward(mlContext_t context, mlShape_t input_shape, mlShape_t weights_shape, mlShape_t bias_shape, mlDataType_t dtype, const void *input, void *output, const void *weights, const void *bias, void *workspace, void *backward_data, int num_heads, bool symmetric); /* [hot] [208] */
void cuda_multi_head_attention_backward(mlContext_t context, mlShape_t input_shape, mlShape_t weights_shape, mlShape_t bias_shape, const void *input, const void *weights, const void *bias, void *gradient_prev, void *gradient_next, void *weights_update, void *bias_update, void *workspace, void *backward_data, int num_heads, bool symmetric); /* [stub] [211] */

/* ---- Window partitioning
 *      replaces src/backend/cuda/kernels/tensor_op.cu:101-151 ---- */
void cuda_window_partitioning(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t output_shape, const void *input, void *output, mlShape_t offset); /* [stub] [218] */
void cuda_window_merging(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t output_shape, const void *input, void *output, mlShape_t offset); /* [stub] [220] */

/* ---- Activations and softmax
 *      replaces src/backend/cuda/kernels/activations.cu:190-257, src/backend/cuda/kernels/softmax.cu ---- */
void cuda_activation_forward(mlContext_t context, float alpha, const mlTensor_t x, float beta, mlTensor_t y, mlActivationType_t act); /* [hot] [226] */
void cuda_activation_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t y, float beta, mlTensor_t dx, mlActivationType_t act); /* [next] [228] */
void cuda_softmax_forward(mlContext_t context, mlDataType_t dtype, mlShape_t shape, void *output, const void *input); /* [hot] [230] */
void cuda_softmax_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t y, float beta, mlTensor_t dx); /* [stub] [231] */
void cuda_fused_act_bias_copy_backward(mlContext_t context, mlTensor_t dy, const mlTensor_t y, float beta_dx, mlTensor_t dx, float beta_dw, mlTensor_t dw, mlActivationType_t act); /* [next] [232] */

/* ---- Channel shuffle and grouped GEMM
 *      replaces src/backend/cuda/kernels/group_conv.cu ---- */
void cuda_channel_shuffle(mlContext_t context, const mlTensor_t x, float beta, mlTensor_t y, int groups, bool invert); /* [stub] [238] */
void cuda_group_gemm(mlContext_t context, char opA, char opB, float alpha, const mlTensor_t A, const mlTensor_t B, float beta, mlTensor_t C, int groups); /* [stub] [239] */

/* ---- Mixture of experts
 *      replaces src/backend/cuda/kernels/moe.cu ---- */
void cuda_hash_routing(mlContext_t context, const mlTensor_t x, mlTensor_t indices_and_values); /* [stub] [245] */
void cuda_token_choice_routing_forward(mlContext_t context, const mlTensor_t x, const mlTensor_t bias, mlTensor_t indices_and_values); /* [stub] [246] */
void cuda_token_choice_routing_backward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, const mlTensor_t dy, float beta, mlTensor_t dx, float alpha, mlTensor_t bias, mlTensor_t workspace); /* [stub] [248] */
void cuda_expert_choice_routing_forward(mlContext_t context, const mlTensor_t x, mlTensor_t indices_and_values); /* [stub] [250] */
void cuda_expert_choice_routing_backward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, const mlTensor_t dy, float beta, mlTensor_t dx); /* [stub] [251] */
void cuda_select_top_k(mlContext_t context, const mlTensor_t x, mlTensor_t indices, mlTensor_t values); /* [stub] [253] */
void cuda_gather_tokens_forward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, float beta, mlTensor_t y); /* [stub] [254] */
void cuda_gather_tokens_backward(mlContext_t context, const mlTensor_t dy, const mlTensor_t indices_and_values, float beta, mlTensor_t dx); /* [stub] [256] */
void cuda_scatter_tokens_forward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, float beta, mlTensor_t y); /* [stub] [258] */
void cuda_scatter_tokens_backward(mlContext_t context, const mlTensor_t x, const mlTensor_t indices_and_values, const mlTensor_t dy, float beta1, mlTensor_t dx, float beta2, mlTensor_t dscales); /* [stub] [260] */
void cuda_moe_forward(mlContext_t context, const mlTensor_t x, const mlTensor_t w, const mlTensor_t b, float beta, mlTensor_t y, mlActivationType_t act); /* [stub] [262] */
void cuda_moe_backward(mlContext_t context, const mlTensor_t x, const mlTensor_t y, const mlTensor_t w, mlTensor_t dy, float beta_dx, mlTensor_t dx, float beta_dw, mlTensor_t dw, float beta_db, mlTensor_t db, mlActivationType_t act); /* [stub] [264] */

/* ---- Learnable scaling
 *      replaces src/backend/cuda/kernels/learnable_scaling.cu ---- */
void cuda_learnable_scaling_forward(mlContext_t context, float alpha, const mlTensor_t x, mlActivationType_t act, const mlTensor_t w, float beta, mlTensor_t y); /* [stub] [270] */
void cuda_learnable_scaling_backward(mlContext_t context, float alpha, const mlTensor_t dy, const mlTensor_t x, mlActivationType_t act, const mlTensor_t w, float beta_dx, mlTensor_t dx, float beta_dw, mlTensor_t dw); /* [stub] [272] */

/* ---- Tensor arithmetic
 *      replaces src/backend/cuda/kernels/tensor_op.cu:290-400 ---- */
void cuda_emulate_low_precision(mlContext_t context, mlShape_t shape, mlDataType_t dtype, void *dst, const void *src, mlQuantizationData_t qd); /* [stub] [278] */
void cuda_scale_tensor(mlContext_t context, float alpha, mlTensor_t x); /* [hot] [281] */
void cuda_add_tensors(mlContext_t context, float alpha1, const mlTensor_t x1, float alpha2, const mlTensor_t x2, float alpha3, const mlTensor_t x3, float beta, mlTensor_t y); /* [hot] [283] */
void cuda_multiply_tensors(mlContext_t context, mlDataType_t dtype, mlShape_t shape, void *dst, const void *src1, const void *src2); /* [next] [285] */
void cuda_sum_over_first_dim(mlContext_t context, float alpha, const mlTensor_t src, float beta, mlTensor_t dst); /* [stub] [287] */

/* ---- Training: losses and optimisers
 *      replaces src/backend/cuda/kernels/training.cu ---- */
float cuda_l2_norm(mlContext_t context, const mlTensor_t tensor); /* [stub] [292] */
float cuda_mean_squared_loss(mlContext_t context, const mlTensor_t output, const mlTensor_t target, const mlTensor_t mask); /* [stub] [293] */
float cuda_cross_entropy_loss(mlContext_t context, const mlTensor_t output, const mlTensor_t target, const mlTensor_t mask); /* [stub] [294] */
void cuda_mean_squared_gradient(mlContext_t context, float alpha, const mlTensor_t output, const mlTensor_t target, const mlTensor_t mask, float beta, mlTensor_t gradient); /* [stub] [295] */
void cuda_cross_entropy_gradient(mlContext_t context, float alpha, const mlTensor_t output, const mlTensor_t target, const mlTensor_t mask, float beta, mlTensor_t gradient); /* [stub] [297] */
void cuda_fused_radam_optimize(mlContext_t context, float scale, const mlTensor_t *gradients, mlTensor_t *weights, mlTensor_t *momentums, mlTensor_t *variances, mlTensor_t *weights_copy, float learning_rate, float beta1, float beta2, int step, int num_tensors, float weight_decay); /* [stub] [300] */
void cuda_fused_lion_optimize(mlContext_t context, float scale, const mlTensor_t *gradients, mlTensor_t *weights, mlTensor_t *momentums, mlTensor_t *weights_copy, float learning_rate, float beta1, float beta2, int step, int num_tensors, float weight_decay); /* [stub] [303] */
void cuda_fused_is_nan_or_inf(mlContext_t context, const mlTensor_t *tensors, int *result, int num_tensors); /* [stub] [306] */
void cuda_fused_l2_regularization(mlContext_t context, mlTensor_t *gradients, const mlTensor_t *params, float scale, int num_tensors); /* [stub] [307] */
void cuda_combined_loss(mlContext_t context, float *result, const mlTensor_t *outputs, const mlTensor_t *targets, const mlTensor_t *masks, const float *weights); /* [stub] [310] */

/* ---- Quantisation
 *      replaces src/backend/cuda/kernels/quantized.cu:515-645 ---- */
void cuda_dequantize(mlContext_t context, mlDataType_t dtype, const void *input, void *output, int elements, float scale, float shift); /* [hot] [316] */
void cuda_quantized_depthwise_conv_forward(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape, const void *input, const void *weights, const void *scales, const void *bias, void *output, mlQuantizationData_t output_qd, int padding_value); /* [next] [318] */
void cuda_quantized_scale_shift_act(mlContext_t context, mlDataType_t dtype, mlShape_t shape, void *output, mlQuantizationData_t output_qd, const void *input, const void *scales, const void *bias, mlActivationType_t act, const void *ext, mlQuantizationData_t ext_qd); /* [hot] [321] */
void cuda_im2row(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, void *output, const void *input, int kernel_size, bool invert, const void *padding); /* [hot] [324] */
void cuda_transpose(mlContext_t context, mlDataType_t dtype, mlShape_t output_shape, mlShape_t input_shape, void *output, const void *input, const int *ordering); /* [stub] [326] */
/* ---- Extensions.  None of these has a counterpart in the reference; minml's host code never calls them. ---- */

/* Text of the first error recorded on the context since the last clear, or NULL.  A NULL context queries the
 * process-wide slot used by calls that arrive without a context. */
const char *mb200_get_last_error(mlContext_t context);
void mb200_clear_last_error(mlContext_t context);
/* Number of kernels this library has launched in this process (all contexts). */
unsigned long long mb200_get_launch_count(void);
/* The cudaStream_t of a context, as an opaque pointer, so a caller can order its own work against it. */
void *mb200_get_stream(mlContext_t context);
/* 0: the three-call Winograd sequence (input transform -> batched GEMM -> output transform) runs as three
 *    kernels through the caller's workspace, as in the reference.
 * 1: the sequence is recognised on the context and replaced by the fused kernel; the workspace is not written.
 * Default 1; the environment variable MINML_B200_EAGER=1 selects 0 at context creation. */
void mb200_set_fusion(mlContext_t context, int enabled);
/* Which kernel cuda_multi_head_attention_forward uses for fp16 inputs with a head dimension of 32:
 * 0: by shape (default) -- the persistent warp-specialised tcgen05 kernel (scores and probabilities in tensor memory) for boards of
 *    up to 256 tokens whose relative offsets stay inside the bias table, the warp-level tensor-core kernel (mma.sync, scores in
 *    registers) for everything else.  Measured on 256 x 225 tokens x 8 heads: 0.083 ms against 0.123 ms;
 * 1: tcgen05 wherever a tcgen05 kernel takes the shape (adds the one-CTA-per-head kernel for 257 .. 462 tokens and clamped offsets,
 *    which measured slower than the warp-level kernel: 2.18 against 1.32 ms on 1024 x 400 tokens);
 * 2: the one-CTA-per-head tcgen05 kernel wherever it takes the shape (up to 462 tokens);
 * 3: never a tcgen05 kernel.
 * Process-wide; the environment variable MINML_B200_MHA_KERNEL=0..3 selects at start. */
void mb200_set_attention_kernel(int kernel);
/* Tells the library that device memory in [ptr, ptr + bytes) has been given new contents (or a new owner) by something other than
 * this ABI: what the library derived from weights lying there -- the snapshot of a layer's raw weights behind its transformed
 * matrices, the border-correction table of an asymmetric int8 layer -- is dropped and made again on the next use.  cuda_free,
 * cuda_memset and the cuda_memcpy_* entries do this themselves; only a host that allocates with an allocator of its own and
 * overwrites weights in place with its own kernels needs to call it. */
void mb200_forget_range(const void *ptr, size_t bytes);
/* Library build identification: "minml_b200 <version> sm_100a". */
const char *mb200_version(void);
/* Failure-path self test: launches one small kernel that waits, with a limit of `polls` polls (1 .. 2^20), on a barrier that
 * nothing completes.  The wait gives up, the kernel writes the context's status word and retires; the next
 * cuda_synchronize_with_context records the same sticky error a tensor-core kernel whose wait ran out would produce.  The
 * context stays usable.  Nothing in the call can hang. */
void mb200_selftest_bounded_wait(mlContext_t context, int polls);
/* Measurement: cycles per tcgen05.mma (kind::f16, M = 128, K = 16, N = n in {16, 32, 64, 128, 256}) when one thread issues 2 000 of
 * them back to back on one SM from a loop with nothing else in it, A from shared memory (0) or tensor memory (1).  Synchronous;
 * returns a negative number on error.  What it reads is the slower of the tensor core and the issuing thread: at N = 128 and 256
 * the figures (64, 128 on a B200) are the tensor core's peak rate; the 46 - 50 cycles at N <= 64 are an upper bound of the
 * instruction's cost, possibly the issue loop's own. */
double mb200_probe_mma_cycles(mlContext_t context, int n, int a_in_tensor_memory);

/* No counterpart in the reference.
 * y = act(conv3x3(x, w) + bias + add) by F(4x4,3x3) Winograd, for callers that must never allocate device memory: a
 * program that gave the whole GPU to its own arena at start-up, or one that cannot take the device-wide synchronisation
 * of cudaMalloc / cudaFree in its serving loop.  Same arguments and result as cuda_convolution_implicit_gemm_forward
 * (fp16 or fp32, 3x3 weights [cout, 3, 3, cin]); the transformed weights, transformed input and products live in a fixed
 * MB200_NOALLOC_SCRATCH_BYTES array inside the library image (held by every GPU that loads the library until the process
 * exits) instead of the context workspace.  A problem needing more than that (36 * elem * (cout*cin + tiles*cin + tiles*cout),
 * tiles = b * ceil(h/4) * ceil(w/4)) is refused with an error on the context.  The call performs no cudaMalloc / cudaFree;
 * the CUDA runtime itself loads each kernel's code on its first launch, so warm up once per data type and shape class (or
 * set CUDA_MODULE_LOADING=EAGER) before the phase in which nothing may be allocated.
 * All calls on a device share the array: calls on one context are ordered by its stream, calls that overlap on the GPU
 * (different contexts) race.  The first call on each device resolves the array's device address; issue it before any
 * stream capture begins. */
#define MB200_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
void mb200_convolution_forward_noalloc(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape, const void *input, const void *weights, void *output, const void *bias, const void *add, mlActivationType_t act);

#ifdef __cplusplus
}
#endif

#endif /* MINML_B200_H_ */
