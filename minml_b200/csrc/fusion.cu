/*
 * fusion.cu -- deferred recognition of the reference's three-call Winograd convolution.
 *
 * minml's Conv2D::forward (src/layers/Conv2D.cpp:365-377) issues
 *     winogradInputTransform(x -> V)   gemmBatched('n','t', V, U -> M)   winogradOutputTransform(M, bias, ext -> y)
 * with V and M as views of the layer workspace.  The single-call fused entry of the ABI
 * (cuda_convolution_implicit_gemm_forward) is never chosen by that host code on this hardware
 * (src/layers/Conv2D.cpp:478-485), so the backend recognises the triple instead:
 *   1. the input transform is recorded, not launched;
 *   2. a batched GEMM whose A operand is the recorded V and whose B operand is a matrix set produced by
 *      cuda_winograd_weight_transform on this device is recorded as well;
 *   3. the output transform on the recorded M launches ONE fused convolution kernel on x and the raw weights.
 * Any other call on the context first replays what was recorded with the eager kernels (flush_pending), so code
 * that inspects V or M -- e.g. the reference's own transform tests -- sees exactly the three-kernel behaviour.
 */
#include "common.cuh"
#include "winograd.cuh"
#include "conv.cuh"

#include <map>
#include <mutex>

namespace mb200
{
	namespace
	{
		struct WeightRecord
		{
				mlTensor_t w;
				int tile_size;
				bool invert;
		};
		std::mutex g_registry_mutex;
		std::map<const void*, WeightRecord> g_registry; // transformed matrices pointer -> raw weights

		bool lookup(const void *matrices, WeightRecord &out)
		{
			std::lock_guard<std::mutex> lock(g_registry_mutex);
			auto it = g_registry.find(matrices);
			if (it == g_registry.end())
				return false;
			out = it->second;
			return true;
		}
	}

	void winograd_register_weights(mlContext_t ctx, const mlTensor_t &w, const mlTensor_t &matrices, int tile_size, bool invert)
	{
		(void) ctx;
		std::lock_guard<std::mutex> lock(g_registry_mutex);
		g_registry[matrices.data] = WeightRecord { w, tile_size, invert };
	}
	void winograd_forget_pointer(const void *ptr)
	{
		std::lock_guard<std::mutex> lock(g_registry_mutex);
		for (auto it = g_registry.begin(); it != g_registry.end();)
		{
			if (it->first == ptr || it->second.w.data == ptr)
				it = g_registry.erase(it);
			else
				++it;
		}
	}

	bool winograd_defer_input(mlContext_t ctx, int tile_size, const mlTensor_t &x, const mlTensor_t &matrices)
	{
		Context *c = get(ctx);
		if (c == nullptr || !c->fusion || tile_size != 4 || matrices.dim[0] != 36)
			return false;
		if (!conv_fused_input_supported(x))
			return false;
		c->pending.stage = 1;
		c->pending.x = x;
		c->pending.v = matrices;
		c->pending.tile_size = tile_size;
		return true;
	}
	bool winograd_defer_gemm(mlContext_t ctx, char opA, char opB, float alpha, const mlTensor_t &A, const mlTensor_t &B, float beta,
			const mlTensor_t &C)
	{
		Context *c = get(ctx);
		if (c == nullptr || c->pending.stage != 1)
			return false;
		if (is_transpose(opA) || !is_transpose(opB) || alpha != 1.0f || beta != 0.0f)
			return false;
		if (A.data != c->pending.v.data || A.rank != 3 || B.rank != 3 || C.rank != 3 || A.dtype != B.dtype || A.dtype != C.dtype)
			return false;
		WeightRecord rec;
		if (!lookup(B.data, rec) || rec.tile_size != c->pending.tile_size || rec.invert)
			return false;
		if (rec.w.dim[0] != B.dim[1] || rec.w.dim[3] != B.dim[2] || rec.w.dtype != A.dtype)
			return false;
		c->pending.stage = 2;
		c->pending.u = B;
		c->pending.m = C;
		return true;
	}
	bool winograd_complete_fused(mlContext_t ctx, int tile_size, const mlTensor_t &matrices, const mlTensor_t &bias, const mlTensor_t &ext,
			const mlTensor_t &y, mlActivationType_t act)
	{
		Context *c = get(ctx);
		if (c == nullptr || c->pending.stage != 2)
			return false;
		if (matrices.data != c->pending.m.data || tile_size != c->pending.tile_size)
			return false;
		WeightRecord rec;
		if (!lookup(c->pending.u.data, rec))
			return false;
		const mlTensor_t x = c->pending.x;
		if (y.dim[0] != x.dim[0] || y.dim[1] != x.dim[1] || y.dim[2] != x.dim[2] || y.dim[3] != rec.w.dim[0])
			return false;
		if (!conv_fused_supported(x, rec.w, y, act))
			return false;
		c->pending.stage = 0;
		return conv_fused_run(ctx, x, rec.w, bias.data, ext.data, y, act);
	}
	void flush_pending(mlContext_t ctx)
	{
		Context *c = get(ctx);
		if (c == nullptr)
			return;
		if (c->pending_i8.stage != 0)
			flush_pending_int8(ctx);
		if (c->pending.stage == 0)
			return;
		const PendingWinograd p = c->pending;
		c->pending.stage = 0; // the eager entry points below call flush_pending again
		winograd_input_transform_eager(ctx, p.tile_size, p.x, p.v);
		if (p.stage == 2)
		{
			const bool fusion = c->fusion;
			c->fusion = false;
			cuda_gemm_batched_v2(ctx, 'n', 't', 1.0f, p.v, p.u, 0.0f, p.m);
			c->fusion = fusion;
		}
	}
} /* namespace mb200 */
