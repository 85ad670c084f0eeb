/*
 * common.cuh -- shared host/device helpers of libminml_b200.
 *
 * The backend context replaces ml::cuda_backend::Context (reference: src/backend/cuda/utils.hpp:28-66,
 * src/backend/cuda/utils.cpp:29-199): one device index, one in-order stream, a scratch workspace that
 * grows on demand, and -- new here -- a sticky error slot instead of assert().
 */
#pragma once

#include "../../include/minml_b200.h"

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>

namespace mb200
{
	/* Upper bound on device indices for per-device caches (kernel attributes are set per device, and one process may hold
	 * contexts on several devices, as minml's multi-GPU host code does). */
	constexpr int MAX_DEVICES = 64;

	struct PendingWinograd
	{
			// state of the deferred three-call Winograd sequence (see fusion.cu)
			int stage = 0; // 0 nothing pending, 1 input transform recorded, 2 batched GEMM recorded
			mlTensor_t x {};
			mlTensor_t v {}; // matrices written by the input transform
			mlTensor_t u {}; // transformed weights
			mlTensor_t m {}; // matrices written by the GEMM
			int tile_size = 0;
	};

	struct PendingInt8
	{
			// state of the deferred int8 sequence im2row -> int8 GEMM -> scale_shift_act (see conv_igemm.cu)
			int stage = 0; // 0 nothing pending, 1 im2row recorded, 2 GEMM recorded
			mlTensor_t x {};
			void *rows = nullptr; // im2row destination
			mlTensor_t w {}; // [cout, 9 * cin] int8
			mlTensor_t acc {}; // [b*h*w, cout] int32
			int pad = 0;
	};

	struct Context
	{
			int device = 0;
			cudaStream_t stream = nullptr;
			void *workspace = nullptr;
			size_t workspace_size = 0;
			bool allow_tf32 = false;
			bool fusion = true;
			bool has_error = false;
			std::string error;
			PendingWinograd pending;
			PendingInt8 pending_i8;
			std::recursive_mutex mutex; // guards `pending`, `pending_i8` and `fusion` (recursive: a flush re-enters the eager entry points)
			int sm_count = 148;
			bool kernels_with_waits = false; // a kernel that polls mbarriers ran since the last synchronize
			int *dev_status = nullptr; // device word set to non-zero by a kernel whose bounded wait ran out
	};

	extern std::atomic<unsigned long long> g_launch_count;

	/* Records the first error on the context (or in the process-wide slot when ctx == nullptr). */
	void record_error(mlContext_t ctx, const char *fmt, ...);
	/* Checks cudaGetLastError()/a status after a launch and records it; returns true when fine. */
	bool check_cuda(mlContext_t ctx, cudaError_t status, const char *what);

	inline Context* get(mlContext_t ctx)
	{
		return reinterpret_cast<Context*>(ctx);
	}
	/* Makes the context's device current and returns its stream; a null context means the default stream
	 * of the current device (reference: Context::getStream, src/backend/cuda/utils.cpp:110-124). */
	cudaStream_t use_stream(mlContext_t ctx);
	/* Returns a device scratch buffer of at least `bytes` bytes owned by the context (grows by reallocating;
	 * reference: Context::getWorkspace, src/backend/cuda/utils.cpp:66-96). */
	void* get_workspace(mlContext_t ctx, size_t bytes);

	/* Runs any deferred Winograd sequence of this context with the three-kernel path (fusion.cu). */
	void flush_pending(mlContext_t ctx);
	void flush_all_pending();

#define MB200_COUNT_LAUNCH() (::mb200::g_launch_count.fetch_add(1, std::memory_order_relaxed))
#define MB200_REQUIRE(ctx, cond, ...) \
	do { if (!(cond)) { ::mb200::record_error((ctx), __VA_ARGS__); return; } } while (0)

	__host__ __device__ inline int size_of(mlDataType_t dtype)
	{
		switch (dtype)
		{
			case DTYPE_FLOAT8:
			case DTYPE_UINT8:
			case DTYPE_INT8:
				return 1;
			case DTYPE_FLOAT16:
			case DTYPE_INT16:
				return 2;
			case DTYPE_FLOAT32:
			case DTYPE_INT32:
				return 4;
			case DTYPE_FLOAT64:
				return 8;
			default:
				return 0;
		}
	}
	inline long long volume(const mlShape_t &s)
	{
		if (s.rank == 0)
			return 0;
		long long r = 1;
		for (int i = 0; i < s.rank; i++)
			r *= s.dim[i];
		return r;
	}
	inline long long volume(const mlTensor_t &t)
	{
		if (t.rank == 0)
			return 0;
		long long r = 1;
		for (int i = 0; i < t.rank; i++)
			r *= t.dim[i];
		return r;
	}
	inline int last_dim(const mlShape_t &s)
	{
		return s.rank == 0 ? 0 : s.dim[s.rank - 1];
	}
	inline int last_dim(const mlTensor_t &t)
	{
		return t.rank == 0 ? 0 : t.dim[t.rank - 1];
	}
	inline long long volume_without_last_dim(const mlShape_t &s)
	{
		return s.rank == 0 ? 0 : volume(s) / last_dim(s);
	}
	inline long long volume_without_last_dim(const mlTensor_t &t)
	{
		return t.rank == 0 ? 0 : volume(t) / last_dim(t);
	}
	inline mlTensor_t make_tensor(const void *data, mlDataType_t dtype, const mlShape_t &shape)
	{
		mlTensor_t t;
		t.data = const_cast<void*>(data);
		t.dtype = dtype;
		t.rank = shape.rank;
		for (int i = 0; i < 6; i++)
			t.dim[i] = (i < shape.rank) ? shape.dim[i] : 0;
		return t;
	}
	inline mlShape_t make_shape(std::initializer_list<int> dims)
	{
		mlShape_t s;
		s.rank = static_cast<int>(dims.size());
		int i = 0;
		for (int d : dims)
			s.dim[i++] = d;
		for (; i < 6; i++)
			s.dim[i] = 0;
		return s;
	}
	inline mlShape_t shape_of(const mlTensor_t &t)
	{
		mlShape_t s;
		s.rank = t.rank;
		for (int i = 0; i < 6; i++)
			s.dim[i] = t.dim[i];
		return s;
	}
	inline bool is_transpose(char op)
	{
		return op == 't' || op == 'T';
	}
	inline bool aligned_to(const void *ptr, size_t bytes)
	{
		return (reinterpret_cast<uintptr_t>(ptr) % bytes) == 0;
	}
	inline bool ranges_overlap(const void *a, long long a_bytes, const void *b, long long b_bytes)
	{
		const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
		return a0 < b0 + static_cast<uintptr_t>(b_bytes) && b0 < a0 + static_cast<uintptr_t>(a_bytes);
	}
	inline int ceil_div(long long a, long long b)
	{
		return static_cast<int>((a + b - 1) / b);
	}

	/* ---- device-side scalar helpers shared by the kernels ---- */
	template<typename T> __device__ __forceinline__ float to_float(T x);
	template<> __device__ __forceinline__ float to_float<float>(float x) { return x; }
	template<> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
	template<> __device__ __forceinline__ float to_float<double>(double x) { return static_cast<float>(x); }
	template<typename T> __device__ __forceinline__ T from_float(float x);
	template<> __device__ __forceinline__ float from_float<float>(float x) { return x; }
	template<> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
	template<> __device__ __forceinline__ double from_float<double>(float x) { return static_cast<double>(x); }

	/* Division of a 31-bit number by a run-time constant as a multiply-high and a shift (the divisor's magic number is found
	 * once on the host): copy kernels would otherwise spend more instructions on index arithmetic than on copying. */
	struct FastDiv
	{
			uint32_t divisor = 1, multiplier = 0, shift = 0;
			FastDiv() = default;
			explicit FastDiv(uint32_t d) :
					divisor(d)
			{
				if (d > 1)
				{
					uint32_t log2_ceil = 0;
					while ((1ull << log2_ceil) < d)
						log2_ceil++;
					const uint32_t p = 31 + log2_ceil;
					multiplier = static_cast<uint32_t>(((1ull << p) + d - 1) / d);
					shift = p - 32;
				}
			}
			__device__ __forceinline__ uint32_t div(uint32_t n) const
			{
				return (divisor == 1) ? n : (__umulhi(n, multiplier) >> shift);
			}
			__device__ __forceinline__ void divmod(uint32_t n, uint32_t &q, uint32_t &r) const
			{
				q = div(n);
				r = n - q * divisor;
			}
	};

	/* Activation set of the reference (src/backend/cuda/vec/vector_math.cuh:40-80): leaky slope 0.1. */
	__device__ __forceinline__ float apply_activation(float x, int act)
	{
		switch (act)
		{
			case ACTIVATION_SIGMOID:
				return 1.0f / (1.0f + expf(-x));
			case ACTIVATION_TANH:
				return tanhf(x);
			case ACTIVATION_RELU:
				return fmaxf(x, 0.0f);
			case ACTIVATION_LEAKY_RELU:
				return x > 0.0f ? x : 0.1f * x;
			case ACTIVATION_EXP:
				return expf(x);
			default:
				return x;
		}
	}
} /* namespace mb200 */
