/*
 * selftest.cu -- exercises the bounded-wait path of the tensor-core kernels without any kernel of the library misbehaving:
 * one CTA waits on an mbarrier that nothing will ever complete, with a small poll limit, gives up, raises the CTA's abort flag
 * and writes the context's status word -- exactly what kernel_gemm_tc / kernel_conv3x3_igemm do when a wait runs out.  The
 * next cuda_synchronize_with_context then reports the sticky error and the context stays usable.  Nothing here can hang: the
 * only wait is the bounded one.
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

extern "C"
{
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
