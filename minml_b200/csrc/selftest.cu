/*
 * selftest.cu -- exercises the bounded-wait path of the tensor-core kernels without any kernel of the library misbehaving:
 * one CTA waits on an mbarrier that nothing will ever complete, with a small poll limit, gives up, raises the CTA's abort flag
 * and writes the context's status word -- exactly what kernel_gemm_tc / kernel_conv3x3_igemm do when a wait runs out.  The
 * next cuda_synchronize_with_context then reports the sticky error and the context stays usable.  Nothing here can hang: the
 * only wait is the bounded one.
 *
 * Also here: a measurement of what one tcgen05.mma costs, so that the tile shapes of the kernels can be checked against the
 * hardware instead of against a formula (mb200_probe_mma_cycles).
 */
#include "common.cuh"
#include "tc.cuh"

using namespace mb200;

namespace
{
	__global__ void kernel_wait_that_runs_out(int *status, unsigned polls)
	{
		__shared__ uint64_t barrier_nothing_completes;
		__shared__ int abort_flag;
		if (threadIdx.x == 0)
		{
			tc::mbar_init(tc::smem_u32(&barrier_nothing_completes), 1);
			abort_flag = 0;
			tc::fence_mbar_init();
		}
		__syncthreads();
		bool ok = true;
		if (threadIdx.x == 32) // one waiter, as in the kernels (a single elected lane per role)
			ok = tc::mbar_wait_limited(tc::smem_u32(&barrier_nothing_completes), 0, &abort_flag, polls);
		__syncthreads();
		// every other role sees the flag and drains; the CTA reports through the status word and retires normally
		if (threadIdx.x == 0 && abort_flag != 0 && status != nullptr)
			atomicExch(status, 3);
		(void) ok;
	}
}

namespace
{
	/* `iters` tcgen05.mma (kind::f16, M = 128, K = 16, N) issued back to back by one thread into the same accumulator, A from shared
	 * memory or from tensor memory, B from shared memory; operands are zeros (the cost does not depend on the values).  N and the
	 * source of A are template parameters and the loop issues four instructions with ready-made descriptors per trip: with
	 * anything to compute between two instructions the single issuing thread, not the tensor core, sets the pace (a version with
	 * run-time N and a branch in the loop read 95 cycles where this one reads 46).
	 * out[0] = cycles until the last one is issued, out[1] = cycles until the last one has completed. */
	template<int N, bool A_TMEM>
	__global__ void kernel_probe_mma(long long *out, int *status, int iters)
	{
		extern __shared__ uint8_t smem_raw[];
		__shared__ uint64_t done;
		__shared__ uint32_t tmem_slot;
		__shared__ int abort_flag;
		const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
		uint32_t *words = reinterpret_cast<uint32_t*>(smem_raw + (base - tc::smem_u32(smem_raw)));
		for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x)
			words[i] = 0u; // A tile (16 KB) and B tile (up to 32 KB), 128-byte swizzle
		if (threadIdx.x == 0)
		{
			tc::mbar_init(tc::smem_u32(&done), 1);
			abort_flag = 0;
			tc::fence_mbar_init();
		}
		if (threadIdx.x < 32)
		{
			tc::tmem_alloc(tc::smem_u32(&tmem_slot), 512);
			tc::tmem_relinquish();
		}
		tc::fence_proxy_async_smem();
		tc::tcgen05_fence_before();
		__syncthreads();
		tc::tcgen05_fence_after();
		const uint32_t tmem = tmem_slot;
		if (threadIdx.x == 0)
		{
			constexpr uint32_t idesc = tc::make_idesc_f16(N);
			const uint64_t desc_a = tc::make_desc_k_sw128(base), desc_b = tc::make_desc_k_sw128(base + 16384);
			const uint64_t a0 = desc_a, a1 = desc_a + 2, a2 = desc_a + 4, a3 = desc_a + 6;
			const uint64_t b0 = desc_b, b1 = desc_b + 2, b2 = desc_b + 4, b3 = desc_b + 6;
			const uint32_t t0a = tmem + 256, t1a = tmem + 264, t2a = tmem + 272, t3a = tmem + 280;
			const long long t0 = clock64();
#pragma unroll 1
			for (int i = 0; i < iters; i += 4)
			{
				if (A_TMEM)
				{
					tc::mma_ts_f16(tmem, t0a, b0, idesc, 1u);
					tc::mma_ts_f16(tmem, t1a, b1, idesc, 1u);
					tc::mma_ts_f16(tmem, t2a, b2, idesc, 1u);
					tc::mma_ts_f16(tmem, t3a, b3, idesc, 1u);
				}
				else
				{
					tc::mma_ss<0>(tmem, a0, b0, idesc, 1u);
					tc::mma_ss<0>(tmem, a1, b1, idesc, 1u);
					tc::mma_ss<0>(tmem, a2, b2, idesc, 1u);
					tc::mma_ss<0>(tmem, a3, b3, idesc, 1u);
				}
			}
			const long long t1 = clock64();
			tc::mma_commit(tc::smem_u32(&done));
			const bool ok = tc::mbar_wait(tc::smem_u32(&done), 0, &abort_flag);
			const long long t2 = clock64();
			out[0] = t1 - t0;
			out[1] = t2 - t0;
			if (!ok && status != nullptr)
				atomicExch(status, 3);
		}
		__syncthreads();
		if (threadIdx.x < 32)
		{
			tc::tcgen05_fence_after();
			tc::tmem_dealloc(tmem, 512);
		}
	}
}

extern "C"
{
	double mb200_probe_mma_cycles(mlContext_t context, int n, int a_in_tensor_memory)
	{
		if (context == nullptr || (n != 16 && n != 32 && n != 64 && n != 128 && n != 256))
		{
			record_error(context, "mb200_probe_mma_cycles: needs a context and N = 16, 32, 64, 128 or 256");
			return -1.0;
		}
		flush_pending(context);
		Context *c = get(context);
		cudaStream_t stream = use_stream(context);
		constexpr int ITERS = 2000, SMEM = 50 * 1024;
		long long *out = reinterpret_cast<long long*>(get_workspace(context, 2 * sizeof(long long)));
		if (out == nullptr)
			return -1.0;
		auto run = [&](auto kernel) -> bool
		{
			if (!check_cuda(context, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM), "mb200_probe_mma_cycles"))
				return false;
			for (int rep = 0; rep < 2; rep++) // the second run is the one read
			{
				kernel<<<1, 128, SMEM, stream>>>(out, c->dev_status, ITERS);
				MB200_COUNT_LAUNCH();
			}
			return true;
		};
		bool launched = false;
		const bool t = a_in_tensor_memory != 0;
		switch (n)
		{
			case 16: launched = t ? run(kernel_probe_mma<16, true>) : run(kernel_probe_mma<16, false>); break;
			case 32: launched = t ? run(kernel_probe_mma<32, true>) : run(kernel_probe_mma<32, false>); break;
			case 64: launched = t ? run(kernel_probe_mma<64, true>) : run(kernel_probe_mma<64, false>); break;
			case 128: launched = t ? run(kernel_probe_mma<128, true>) : run(kernel_probe_mma<128, false>); break;
			case 256: launched = t ? run(kernel_probe_mma<256, true>) : run(kernel_probe_mma<256, false>); break;
			default: break;
		}
		if (!launched)
			return -1.0;
		c->kernels_with_waits = true;
		long long host[2] = { 0, 0 };
		if (!check_cuda(context, cudaGetLastError(), "mb200_probe_mma_cycles launch")
				|| !check_cuda(context, cudaMemcpyAsync(host, out, sizeof(host), cudaMemcpyDeviceToHost, stream), "mb200_probe_mma_cycles read")
				|| !check_cuda(context, cudaStreamSynchronize(stream), "mb200_probe_mma_cycles sync"))
			return -1.0;
		return static_cast<double>(host[1]) / ITERS;
	}

	void mb200_selftest_bounded_wait(mlContext_t context, int polls)
	{
		MB200_REQUIRE(context, context != nullptr, "mb200_selftest_bounded_wait: null context");
		MB200_REQUIRE(context, polls > 0 && polls <= (1 << 20), "mb200_selftest_bounded_wait: polls must be in [1, 2^20]");
		flush_pending(context);
		Context *c = get(context);
		kernel_wait_that_runs_out <<<1, 64, 0, use_stream(context)>>>(c->dev_status, static_cast<unsigned>(polls));
		MB200_COUNT_LAUNCH();
		c->kernels_with_waits = true;
		check_cuda(context, cudaGetLastError(), "mb200_selftest_bounded_wait");
	}
}
