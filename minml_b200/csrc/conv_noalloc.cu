/*
 * conv_noalloc.cu -- mb200_convolution_forward_noalloc: the 3x3 Winograd convolution for callers that are not allowed
 * to allocate device memory.
 *
 * Who needs this.  Some programs hand the whole GPU to an arena of their own at start-up and forbid any later cudaMalloc:
 * an inference server that has sized its pools so that nothing is left over, a game-tree search that runs the network from
 * many host threads and cannot afford the device-wide synchronisation cudaMalloc and cudaFree imply, or a component that is
 * only ever given input and output buffers by its host.  cuda_convolution_implicit_gemm_forward is no use to them on its
 * Winograd route (fp32 data, or fp16 shapes the fused kernel does not take), because that route keeps the transformed
 * weights U, the transformed input V and the products M in the context's scratch workspace, which grows with cudaMalloc.
 *
 * This entry point computes the same thing -- y = act(conv3x3(x, w) + bias + add), F(4x4,3x3), same kernels, same order of
 * operations -- but keeps U, V and M in a fixed array that is part of the library image:
 *
 *     static __device__ g_scratch[MB200_NOALLOC_SCRATCH_BYTES]      (16 MiB, on every GPU that loads the library, until exit)
 *
 * Rules that follow from that:
 *   - a problem whose U + V + M does not fit is refused with an error on the context; nothing is launched;
 *   - the call itself never calls cudaMalloc, cudaFree or any routine that allocates device memory.  One thing outside its
 *     control: the CUDA runtime loads a kernel's code onto the device the first time that kernel is launched (lazy module
 *     loading), and which kernels run depends on the data type and on the shape class (fp16 with even / odd channel counts,
 *     fp32, tensor-core or generic product).  So run one warm-up call per data type and shape class you will use, on every
 *     device, before the phase in which nothing may be allocated -- or start the process with CUDA_MODULE_LOADING=EAGER;
 *   - the array is shared by every call on the device and keeps whatever the last call left in it.  Nothing in it has to
 *     start at zero: U, V and M are each written completely before they are read;
 *   - two calls that are in flight on the same GPU at the same time (two contexts, two processes' worth of streams) use
 *     the same bytes and race.  Calls on one context are ordered by its stream and are safe;
 *   - the first call on each device looks up the device address of the array (cudaGetSymbolAddress, with that device
 *     current).  Make that first call before starting any stream capture.
 */
#include "common.cuh"
#include "winograd.cuh"

#include <mutex>

#ifndef MB200_NOALLOC_SCRATCH_BYTES /* also defined in include/minml_b200.h */
#define MB200_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
#endif

namespace
{
	/* In host code this name is only a handle for cudaGetSymbolAddress; it is not a pointer a kernel could use. */
	static __device__ __align__(256) unsigned char g_scratch[MB200_NOALLOC_SCRATCH_BYTES];

	constexpr int MAX_DEVICES = 64;
	std::mutex g_setup_mutex;
	unsigned char *g_scratch_address[MAX_DEVICES] = { };

	/* Device address of the array on `device`, resolved once per device with that device current. */
	unsigned char* scratch_on(mlContext_t ctx, int device)
	{
		if (device < 0 || device >= MAX_DEVICES)
		{
			mb200::record_error(ctx, "mb200_convolution_forward_noalloc: device index %d out of range", device);
			return nullptr;
		}
		std::lock_guard<std::mutex> lock(g_setup_mutex);
		if (g_scratch_address[device] == nullptr)
		{
			if (!mb200::check_cuda(ctx, cudaSetDevice(device), "mb200_convolution_forward_noalloc: set device"))
				return nullptr;
			void *ptr = nullptr;
			if (!mb200::check_cuda(ctx, cudaGetSymbolAddress(&ptr, g_scratch), "mb200_convolution_forward_noalloc: cudaGetSymbolAddress"))
				return nullptr;
			g_scratch_address[device] = reinterpret_cast<unsigned char*>(ptr);
		}
		return g_scratch_address[device];
	}
	size_t round_up_256(size_t bytes)
	{
		return (bytes + 255) / 256 * 256;
	}
}

using namespace mb200;

extern "C"
{
	void mb200_convolution_forward_noalloc(mlContext_t context, mlDataType_t dtype, mlShape_t input_shape, mlShape_t weights_shape,
			const void *input, const void *weights, void *output, const void *bias, const void *add, mlActivationType_t act)
	{
		MB200_REQUIRE(context, context != nullptr, "mb200_convolution_forward_noalloc: null context");
		MB200_REQUIRE(context, input_shape.rank == 4 && weights_shape.rank == 4, "mb200_convolution_forward_noalloc: rank-4 shapes expected");
		MB200_REQUIRE(context, input != nullptr && weights != nullptr && output != nullptr, "mb200_convolution_forward_noalloc: null pointer");
		MB200_REQUIRE(context, dtype == DTYPE_FLOAT16 || dtype == DTYPE_FLOAT32, "mb200_convolution_forward_noalloc: dtype %d not supported",
				static_cast<int>(dtype));
		const int batch = input_shape.dim[0], height = input_shape.dim[1], width = input_shape.dim[2], cin = input_shape.dim[3];
		const int cout = weights_shape.dim[0];
		MB200_REQUIRE(context, weights_shape.dim[1] == 3 && weights_shape.dim[2] == 3 && weights_shape.dim[3] == cin,
				"mb200_convolution_forward_noalloc: weights must be [cout, 3, 3, %d]", cin);
		if (batch == 0 || height == 0 || width == 0)
			return;

		const size_t elem = size_of(dtype);
		const size_t tiles = static_cast<size_t>(batch) * ((height + 3) / 4) * ((width + 3) / 4);
		const size_t u_bytes = round_up_256(36 * static_cast<size_t>(cout) * cin * elem);
		const size_t v_bytes = round_up_256(36 * tiles * cin * elem);
		const size_t m_bytes = round_up_256(36 * tiles * cout * elem);
		MB200_REQUIRE(context, u_bytes + v_bytes + m_bytes <= MB200_NOALLOC_SCRATCH_BYTES,
				"mb200_convolution_forward_noalloc: this problem needs %zu bytes of scratch (U %zu + V %zu + M %zu), the built-in array holds %u",
				u_bytes + v_bytes + m_bytes, u_bytes, v_bytes, m_bytes, MB200_NOALLOC_SCRATCH_BYTES);

		Context *c = get(context);
		unsigned char *scratch = scratch_on(context, c->device);
		if (scratch == nullptr)
			return;
		flush_pending(context);

		const mlShape_t out_shape = make_shape( { batch, height, width, cout });
		const mlTensor_t x = make_tensor(input, dtype, input_shape);
		const mlTensor_t w = make_tensor(weights, dtype, weights_shape);
		const mlTensor_t y = make_tensor(output, dtype, out_shape);
		const mlTensor_t u = make_tensor(scratch, dtype, make_shape( { 36, cout, cin }));
		const mlTensor_t v = make_tensor(scratch + u_bytes, dtype, make_shape( { 36, static_cast<int>(tiles), cin }));
		const mlTensor_t m = make_tensor(scratch + u_bytes + v_bytes, dtype, make_shape( { 36, static_cast<int>(tiles), cout }));
		const mlTensor_t bias_t = make_tensor(bias, dtype, make_shape( { cout }));
		const mlTensor_t add_t = make_tensor(add, dtype, out_shape);

		std::lock_guard<std::recursive_mutex> lock(c->mutex);
		const bool fusion = c->fusion;
		c->fusion = false; // the four steps run eagerly, in this order, on the context's stream
		winograd_weight_transform_eager(context, 4, w, u, false);
		winograd_input_transform_eager(context, 4, x, v);
		cuda_gemm_batched_v2(context, 'n', 't', 1.0f, v, u, 0.0f, m);
		winograd_output_transform_eager(context, 4, m, bias_t, add_t, y, act);
		c->fusion = fusion;
	}
}
