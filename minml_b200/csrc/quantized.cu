/*
 * quantized.cu -- eager entry points of the int8 path: requantisation of int32 accumulators, im2row, dequantise.
 *
 * Replaces src/backend/cuda/kernels/quantized.cu:219-262,563-645 of the reference.
 *
 *   scale_shift_act:  x = acc[i, c] * scales[c] + bias[c] (+ ext[i, c] * ext_qd.scale + ext_qd.shift);
 *                     activation in {linear, sigmoid, tanh, relu} (anything else is left linear, as in the reference);
 *                     output fp16 / fp32 / fp64, or int8 = clamp(round(x * (1 / s_o) + (-z_o / s_o)), -128, 127) with
 *                     round-half-away-from-zero: the formula and rounding order of the reference's CPU layer
 *                     (src/layers/Conv2D.cpp:283-304), shared with the fused kernels through epilogue.cuh.  The reference's
 *                     CUDA kernel divides, round((x - z_o) / s_o), which can differ from its own CPU layer by one step.
 *   im2row:           [b, h, w, c] -> [b*h*w, k*k*c], columns ordered (kh, kw, c), taps outside the image filled with
 *                     *padding (zero when the pointer is null).  Unlike the reference's active code path this one
 *                     handles int8 and honours `padding`, which the host's int8 3x3 convolution needs
 *                     (src/layers/Conv2D.cpp:227-232).
 */
#include "common.cuh"
#include "conv.cuh"
#include "epilogue.cuh"

#include <algorithm>
#include <cstring>

namespace mb200
{
	namespace
	{
		template<typename T> __device__ __forceinline__ void store_value(T *p, float x, float inv_unused, float scale, float shift);
		template<> __device__ __forceinline__ void store_value<float>(float *p, float x, float, float, float) { *p = x; }
		template<> __device__ __forceinline__ void store_value<double>(double *p, float x, float, float, float) { *p = x; }
		template<> __device__ __forceinline__ void store_value<__half>(__half *p, float x, float, float, float) { *p = __float2half_rn(x); }
		template<> __device__ __forceinline__ void store_value<int8_t>(int8_t *p, float x, float, float inv_scale, float inv_shift)
		{
			*p = static_cast<int8_t>(epi::requant_clamp(epi::requant_round(x, inv_scale, inv_shift)));
		}

		/* One thread requantises VEC consecutive channels of one row (VEC = 4: 16-byte accumulator and scale loads).  With the
		 * cheap rounding the kernel waits on its loads (8.8 stalled warps per issued instruction); a version that kept four items
		 * in flight per thread measured slower (0.223 against 0.180 ms: its 92 registers cost more occupancy than the extra loads
		 * in flight gained), so the loop stays one item per pass. */
		template<typename T, int VEC>
		__global__ void __launch_bounds__(256) kernel_scale_shift_act(T *__restrict__ output, const int *__restrict__ input,
				const float *__restrict__ scales, const float *__restrict__ bias, const int8_t *__restrict__ ext, long long rows, int channels,
				int act, float inv_out_scale, float inv_out_shift, float ext_scale, float ext_shift)
		{
			const long long total = rows * channels / VEC;
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			const bool act_on = (act == ACTIVATION_SIGMOID || act == ACTIVATION_TANH || act == ACTIVATION_RELU);
			const int groups = channels / VEC;
			const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
			int g = static_cast<int>(first % groups); // channel group of the thread's item, advanced without a division
			const int g_step = static_cast<int>(stride % groups);
			for (long long i = first; i < total; i += stride, g = (g + g_step >= groups) ? g + g_step - groups : g + g_step)
			{
				const long long e = i * VEC;
				const int c = g * VEC;
				int acc[VEC];
				float sc[VEC], sh[VEC];
				int ex[VEC];
				if (VEC == 4)
				{
					const int4 a = *reinterpret_cast<const int4*>(input + e);
					acc[0] = a.x; acc[1 % VEC] = a.y; acc[2 % VEC] = a.z; acc[3 % VEC] = a.w;
					const float4 s4 = *reinterpret_cast<const float4*>(scales + c), b4 = *reinterpret_cast<const float4*>(bias + c);
					sc[0] = s4.x; sc[1 % VEC] = s4.y; sc[2 % VEC] = s4.z; sc[3 % VEC] = s4.w;
					sh[0] = b4.x; sh[1 % VEC] = b4.y; sh[2 % VEC] = b4.z; sh[3 % VEC] = b4.w;
					if (ext != nullptr)
					{
						const uint32_t w4 = *reinterpret_cast<const uint32_t*>(ext + e);
#pragma unroll
						for (int k = 0; k < VEC; k++)
							ex[k] = static_cast<int>(static_cast<int8_t>((w4 >> (8 * k)) & 0xFFu));
					}
				}
				else
				{
					acc[0] = input[e];
					sc[0] = scales[c];
					sh[0] = bias[c];
					if (ext != nullptr)
						ex[0] = ext[e];
				}
				float x[VEC];
#pragma unroll
				for (int k = 0; k < VEC; k++)
				{
					x[k] = epi::requant_real(acc[k], sc[k], sh[k]);
					if (ext != nullptr)
						x[k] = epi::requant_add_ext(x[k], ex[k], ext_scale, ext_shift);
					if (act_on)
						x[k] = apply_activation(x[k], act);
				}
				if (VEC == 4 && sizeof(T) == 1)
				{
					int q[VEC];
					#pragma unroll
					for (int k = 0; k < VEC; k++)
						q[k] = epi::requant_round(x[k], inv_out_scale, inv_out_shift);
					*reinterpret_cast<uint32_t*>(output + e) = epi::pack_sat_s8x4(q[0], q[1 % VEC], q[2 % VEC], q[3 % VEC]);
				}
				else
				{
#pragma unroll
					for (int k = 0; k < VEC; k++)
						store_value<T>(output + e + k, x[k], 0.0f, inv_out_scale, inv_out_shift);
				}
			}
		}

		template<typename T>
		__global__ void __launch_bounds__(256) kernel_dequantize(T *__restrict__ output, const int8_t *__restrict__ input, long long elements,
				float scale, float shift)
		{
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += stride)
				store_value<T>(output + i, static_cast<float>(input[i]) * scale + shift, 0.0f, 1.0f, 0.0f);
		}

		/* One thread moves one packet of VB bytes of one tap of one output position. */
		template<int VB> struct PacketOf;
		template<> struct PacketOf<1> { using type = uint8_t; };
		template<> struct PacketOf<2> { using type = uint16_t; };
		template<> struct PacketOf<4> { using type = uint32_t; };
		template<> struct PacketOf<8> { using type = uint2; };
		template<> struct PacketOf<16> { using type = uint4; };

		template<int VB>
		__global__ void __launch_bounds__(256) kernel_im2row(void *__restrict__ output, const void *__restrict__ input, int batch, int height,
				int width, int row_bytes, int kernel, bool invert, typename PacketOf<VB>::type pad)
		{
			using P = typename PacketOf<VB>::type;
			const int packets = row_bytes / VB; // per (position, tap)
			const int pad_hw = (kernel - 1) / 2;
			const long long total = static_cast<long long>(batch) * height * width * kernel * kernel * packets;
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			const P *src = reinterpret_cast<const P*>(input);
			P *dst = reinterpret_cast<P*>(output);
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride)
			{
				const int pk = static_cast<int>(i % packets);
				long long t = i / packets;
				const int kw = static_cast<int>(t % kernel);
				t /= kernel;
				const int kh = static_cast<int>(t % kernel);
				t /= kernel;
				const int w = static_cast<int>(t % width);
				t /= width;
				const int h = static_cast<int>(t % height);
				const int b = static_cast<int>(t / height);
				const int ih = h - pad_hw + (invert ? (kernel - 1 - kh) : kh);
				const int iw = w - pad_hw + (invert ? (kernel - 1 - kw) : kw);
				P v = pad;
				if (ih >= 0 && ih < height && iw >= 0 && iw < width)
					v = src[((static_cast<long long>(b) * height + ih) * width + iw) * packets + pk];
				dst[i] = v;
			}
		}
		/* The same copy with one warp per output position: the position is decomposed once per warp (multiply-high divisions),
		 * the lanes walk over its kernel x kernel x packets pieces, which are contiguous in the output. */
		template<int VB>
		__global__ void __launch_bounds__(256) kernel_im2row_positions(void *__restrict__ output, const void *__restrict__ input, int positions,
				int height, int width, int packets, int kernel, bool invert, typename PacketOf<VB>::type pad, FastDiv by_hw, FastDiv by_w,
				FastDiv by_packets, FastDiv by_kernel)
		{
			using P = typename PacketOf<VB>::type;
			const int pad_hw = (kernel - 1) / 2;
			const uint32_t per_position = static_cast<uint32_t>(kernel) * kernel * packets;
			const P *src = reinterpret_cast<const P*>(input);
			P *dst = reinterpret_cast<P*>(output);
			const int lane = threadIdx.x % 32;
			const int warps = gridDim.x * (blockDim.x / 32);
			for (int pos = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32; pos < positions; pos += warps)
			{
				uint32_t b, rem, h, w;
				by_hw.divmod(static_cast<uint32_t>(pos), b, rem);
				by_w.divmod(rem, h, w);
				P *dst_row = dst + static_cast<long long>(pos) * per_position;
				const P *src_image = src + static_cast<long long>(b) * height * width * packets;
#pragma unroll 4
				for (uint32_t t = lane; t < per_position; t += 32)
				{
					uint32_t tap, pk, kh, kw;
					by_packets.divmod(t, tap, pk);
					by_kernel.divmod(tap, kh, kw);
					const int ih = static_cast<int>(h) - pad_hw + static_cast<int>(invert ? (kernel - 1 - kh) : kh);
					const int iw = static_cast<int>(w) - pad_hw + static_cast<int>(invert ? (kernel - 1 - kw) : kw);
					P v = pad;
					if (ih >= 0 && ih < height && iw >= 0 && iw < width)
						v = src_image[(static_cast<long long>(ih) * width + iw) * packets + pk];
					dst_row[t] = v;
				}
			}
		}
		template<int VB>
		void launch_im2row(cudaStream_t stream, int grid, void *output, const void *input, int batch, int height, int width, int row_bytes,
				int kernel, bool invert, const uint8_t (&pattern)[16])
		{
			typename PacketOf<VB>::type pad;
			std::memcpy(&pad, pattern, VB);
			const long long positions = static_cast<long long>(batch) * height * width;
			const long long per_position = static_cast<long long>(kernel) * kernel * (row_bytes / VB);
			if (positions < (1ll << 31) && per_position < (1ll << 31))
			{
				const int warp_grid = static_cast<int>(std::max<long long>(1, std::min<long long>((positions + 7) / 8, static_cast<long long>(grid))));
				kernel_im2row_positions<VB> <<<warp_grid, 256, 0, stream>>>(output, input, static_cast<int>(positions), height, width, row_bytes / VB,
						kernel, invert, pad, FastDiv(static_cast<uint32_t>(height) * width), FastDiv(static_cast<uint32_t>(width)),
						FastDiv(static_cast<uint32_t>(row_bytes / VB)), FastDiv(static_cast<uint32_t>(kernel)));
			}
			else
				kernel_im2row<VB> <<<grid, 256, 0, stream>>>(output, input, batch, height, width, row_bytes, kernel, invert, pad);
			MB200_COUNT_LAUNCH();
		}
	}
} /* namespace mb200 */

using namespace mb200;

extern "C"
{
	void cuda_quantized_scale_shift_act(mlContext_t context, mlDataType_t dtype, mlShape_t shape, void *output, mlQuantizationData_t output_qd,
			const void *input, const void *scales, const void *bias, mlActivationType_t act, const void *ext, mlQuantizationData_t ext_qd)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_quantized_scale_shift_act: null context");
		if (volume(shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, output != nullptr && input != nullptr && scales != nullptr && bias != nullptr,
				"cuda_quantized_scale_shift_act: null pointer");
		if (requant_complete_fused(context, dtype, shape, output, output_qd, input, scales, bias, act, ext, ext_qd))
			return;
		flush_pending(context);
		const long long rows = volume_without_last_dim(shape);
		const int channels = last_dim(shape);
		if (rows == 0 || channels == 0)
			return;
		cudaStream_t stream = use_stream(context);
		const bool vec4 = channels % 4 == 0 && aligned_to(input, 16) && aligned_to(scales, 16) && aligned_to(bias, 16) && aligned_to(output, 16)
				&& (ext == nullptr || aligned_to(ext, 4));
		const int grid = static_cast<int>(std::min<long long>((rows * channels / (vec4 ? 4 : 1) + 255) / 256,
				static_cast<long long>(get(context)->sm_count) * 16));
#define LAUNCH_SSA(T) do { if (vec4) kernel_scale_shift_act<T, 4> <<<grid, 256, 0, stream>>>(ARGS(T)); \
		else kernel_scale_shift_act<T, 1> <<<grid, 256, 0, stream>>>(ARGS(T)); } while (0)
#define ARGS(T) reinterpret_cast<T*>(output), reinterpret_cast<const int*>(input), reinterpret_cast<const float*>(scales), \
		reinterpret_cast<const float*>(bias), reinterpret_cast<const int8_t*>(ext), rows, channels, static_cast<int>(act), \
		1.0f / output_qd.scale, -output_qd.shift / output_qd.scale, ext_qd.scale, ext_qd.shift
		switch (dtype)
		{
			case DTYPE_FLOAT16:
				LAUNCH_SSA(__half);
				break;
			case DTYPE_FLOAT32:
				LAUNCH_SSA(float);
				break;
			case DTYPE_FLOAT64:
				LAUNCH_SSA(double);
				break;
			case DTYPE_INT8:
				LAUNCH_SSA(int8_t);
				break;
			default:
				record_error(context, "cuda_quantized_scale_shift_act: output dtype %d not supported", static_cast<int>(dtype));
				return;
		}
#undef ARGS
#undef LAUNCH_SSA
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_quantized_scale_shift_act");
	}
	void cuda_dequantize(mlContext_t context, mlDataType_t dtype, const void *input, void *output, int elements, float scale, float shift)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_dequantize: null context");
		if (elements == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		if (elements <= 0)
			return;
		MB200_REQUIRE(context, input != nullptr && output != nullptr, "cuda_dequantize: null pointer");
		flush_pending(context);
		cudaStream_t stream = use_stream(context);
		const int grid = static_cast<int>(std::min<long long>((elements + 255) / 256, static_cast<long long>(get(context)->sm_count) * 16));
		switch (dtype)
		{
			case DTYPE_FLOAT16:
				kernel_dequantize<__half> <<<grid, 256, 0, stream>>>(reinterpret_cast<__half*>(output), reinterpret_cast<const int8_t*>(input),
						elements, scale, shift);
				break;
			case DTYPE_FLOAT32:
				kernel_dequantize<float> <<<grid, 256, 0, stream>>>(reinterpret_cast<float*>(output), reinterpret_cast<const int8_t*>(input),
						elements, scale, shift);
				break;
			case DTYPE_FLOAT64:
				kernel_dequantize<double> <<<grid, 256, 0, stream>>>(reinterpret_cast<double*>(output), reinterpret_cast<const int8_t*>(input),
						elements, scale, shift);
				break;
			default:
				record_error(context, "cuda_dequantize: output dtype %d not supported", static_cast<int>(dtype));
				return;
		}
		MB200_COUNT_LAUNCH();
		check_cuda(context, cudaGetLastError(), "cuda_dequantize");
	}
	void cuda_im2row(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, void *output, const void *input, int kernel_size, bool invert,
			const void *padding)
	{
		MB200_REQUIRE(context, context != nullptr, "cuda_im2row: null context");
		if (volume(input_shape) == 0)
			return; // an empty problem: nothing to validate or launch (its tensors may have null data)
		MB200_REQUIRE(context, input_shape.rank == 4 && output != nullptr && input != nullptr, "cuda_im2row: needs a rank-4 input and buffers");
		MB200_REQUIRE(context, kernel_size >= 1 && kernel_size % 2 == 1, "cuda_im2row: kernel size %d must be odd", kernel_size);
		const int elem = size_of(dtype);
		MB200_REQUIRE(context, elem > 0, "cuda_im2row: dtype %d not supported", static_cast<int>(dtype));
		const int batch = input_shape.dim[0], height = input_shape.dim[1], width = input_shape.dim[2], channels = input_shape.dim[3];
		if (batch == 0 || height == 0 || width == 0 || channels == 0)
			return;
		if (im2row_defer(context, dtype, input_shape, output, input, kernel_size, invert, padding))
			return;
		flush_pending(context);
		const int row_bytes = channels * elem;
		uint8_t pattern[16];
		for (int i = 0; i < 16; i++)
			pattern[i] = (padding == nullptr) ? 0 : reinterpret_cast<const uint8_t*>(padding)[i % elem];
		int vb = 16;
		while (vb > elem && (row_bytes % vb != 0 || !aligned_to(input, vb) || !aligned_to(output, vb)))
			vb /= 2;
		cudaStream_t stream = use_stream(context);
		const long long total = static_cast<long long>(batch) * height * width * kernel_size * kernel_size * (row_bytes / vb);
		const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, static_cast<long long>(get(context)->sm_count) * 32));
		switch (vb)
		{
			case 16:
				launch_im2row<16>(stream, grid, output, input, batch, height, width, row_bytes, kernel_size, invert, pattern);
				break;
			case 8:
				launch_im2row<8>(stream, grid, output, input, batch, height, width, row_bytes, kernel_size, invert, pattern);
				break;
			case 4:
				launch_im2row<4>(stream, grid, output, input, batch, height, width, row_bytes, kernel_size, invert, pattern);
				break;
			case 2:
				launch_im2row<2>(stream, grid, output, input, batch, height, width, row_bytes, kernel_size, invert, pattern);
				break;
			default:
				launch_im2row<1>(stream, grid, output, input, batch, height, width, row_bytes, kernel_size, invert, pattern);
				break;
		}
		check_cuda(context, cudaGetLastError(), "cuda_im2row");
	}
}
