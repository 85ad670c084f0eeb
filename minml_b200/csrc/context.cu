/*
 * context.cu -- device properties, contexts, events and memory entry points of the C ABI.
 *
 * Replaces src/backend/cuda/{cuda_properties.cpp, cuda_context.cpp, cuda_event.cpp, cuda_memory.cu, utils.cpp}
 * of the reference.  Differences that are deliberate:
 *   - no assert(): a failed runtime call records a sticky error on the context and the entry point returns;
 *   - the stream is created together with the context (non-blocking flag off, so the null-context default
 *     stream paths of the reference still order against it);
 *   - every entry that can observe memory written by a deferred Winograd sequence flushes it first.
 */
#include "common.cuh"
#include "winograd.cuh"
#include "conv.cuh"

#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace mb200
{
	std::atomic<unsigned long long> g_launch_count { 0 };

	namespace
	{
		std::mutex g_mutex; // error slots
		std::string g_global_error;
		bool g_global_has_error = false;
		std::mutex g_contexts_mutex; // the list of live contexts; held while flush_all_pending walks it, so that none is destroyed under it
		std::vector<Context*> g_contexts;

		/* Size in bytes of the device allocation that starts at (or contains) ptr; 1 when the driver cannot tell. */
		size_t allocation_size(const void *ptr)
		{
			typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
			static const range_fn fn = []() -> range_fn
			{
				void *entry = nullptr;
				cudaDriverEntryPointQueryResult result;
				if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &entry, cudaEnableDefault, &result) != cudaSuccess || entry == nullptr)
				{
					cudaGetLastError();
					return nullptr;
				}
				return reinterpret_cast<range_fn>(entry);
			}();
			unsigned long long base = 0;
			size_t size = 0;
			if (fn == nullptr || fn(&base, &size, static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(ptr))) != 0 || size == 0)
				return 1;
			return size;
		}

		int device_count()
		{
			static const int number = []()
			{
				int result = 0;
				if (cudaGetDeviceCount(&result) != cudaSuccess)
				{
					cudaGetLastError();
					return 0;
				}
				return result;
			}();
			return number;
		}
		const std::vector<cudaDeviceProp>& device_properties()
		{
			static const std::vector<cudaDeviceProp> props = []()
			{
				std::vector<cudaDeviceProp> result;
				for (int i = 0; i < device_count(); i++)
				{
					cudaDeviceProp p;
					std::memset(&p, 0, sizeof(p));
					if (cudaGetDeviceProperties(&p, i) != cudaSuccess)
						cudaGetLastError();
					result.push_back(p);
				}
				return result;
			}();
			return props;
		}

		template<typename T>
		__global__ void kernel_fill(T *dst, long long elements, T value)
		{
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += stride)
				dst[i] = value;
		}
		template<typename T>
		void launch_fill(mlContext_t ctx, cudaStream_t stream, void *dst, size_t bytes, const void *pattern)
		{
			T value;
			std::memcpy(&value, pattern, sizeof(T));
			const long long elements = static_cast<long long>(bytes / sizeof(T));
			if (elements == 0)
				return;
			const int blocks = static_cast<int>(std::min<long long>((elements + 255) / 256, 148 * 8));
			kernel_fill<T> <<<blocks, 256, 0, stream>>>(reinterpret_cast<T*>(dst), elements, value);
			MB200_COUNT_LAUNCH();
			check_cuda(ctx, cudaGetLastError(), "cuda_memset fill");
		}
	}

	void record_error(mlContext_t ctx, const char *fmt, ...)
	{
		char buffer[512];
		va_list args;
		va_start(args, fmt);
		vsnprintf(buffer, sizeof(buffer), fmt, args);
		va_end(args);
		std::lock_guard<std::mutex> lock(g_mutex);
		if (ctx == nullptr)
		{
			if (!g_global_has_error)
			{
				g_global_has_error = true;
				g_global_error = buffer;
			}
		}
		else
		{
			Context *c = get(ctx);
			if (!c->has_error)
			{
				c->has_error = true;
				c->error = buffer;
			}
		}
		if (std::getenv("MINML_B200_VERBOSE") != nullptr)
			fprintf(stderr, "[minml_b200] error: %s\n", buffer);
	}
	bool check_cuda(mlContext_t ctx, cudaError_t status, const char *what)
	{
		if (status == cudaSuccess)
			return true;
		record_error(ctx, "%s: %s", what, cudaGetErrorString(status));
		return false;
	}
	cudaStream_t use_stream(mlContext_t ctx)
	{
		if (ctx == nullptr)
			return nullptr;
		Context *c = get(ctx);
		cudaSetDevice(c->device);
		return c->stream;
	}
	void* get_workspace(mlContext_t ctx, size_t bytes)
	{
		if (ctx == nullptr)
			return nullptr;
		Context *c = get(ctx);
		if (bytes > c->workspace_size)
		{
			cudaSetDevice(c->device);
			cudaStreamSynchronize(c->stream);
			if (c->workspace != nullptr)
				cudaFree(c->workspace);
			c->workspace = nullptr;
			c->workspace_size = 0;
			const size_t wanted = std::max<size_t>(bytes, size_t(32) << 20);
			if (!check_cuda(ctx, cudaMalloc(&c->workspace, wanted), "workspace allocation"))
				return nullptr;
			c->workspace_size = wanted;
		}
		return c->workspace;
	}
	/* Replays the recorded calls of EVERY context (a freed buffer or a null-context copy may concern any of them).  Each
	 * context is flushed under its own mutex, so the thread that owns it either has not recorded its next call yet or finds
	 * nothing pending and runs that call eagerly on results that exist. */
	void flush_all_pending()
	{
		std::lock_guard<std::mutex> lock(g_contexts_mutex);
		for (Context *c : g_contexts)
			flush_pending(c);
	}
} /* namespace mb200 */

using namespace mb200;

extern "C"
{
	/* ------------------------------------------------------------------ properties */
	int cuda_get_number_of_devices()
	{
		return device_count();
	}
	void cuda_enable_tf32(mlContext_t context, bool b)
	{
		if (context != nullptr)
			get(context)->allow_tf32 = b;
	}
	int cuda_get_memory(int index)
	{
		if (index < 0 || index >= device_count())
			return 0;
		return static_cast<int>(device_properties()[index].totalGlobalMem >> 20);
	}
	bool cuda_supports_type(int index, mlDataType_t dtype)
	{
		if (index < 0 || index >= device_count())
			return false;
		switch (dtype)
		{
			case DTYPE_FLOAT16:
			case DTYPE_FLOAT32:
			case DTYPE_FLOAT64:
			case DTYPE_INT32:
			case DTYPE_INT8:
				return true; // every sm_100 part has all of them
			default:
				return false;
		}
	}
	const char* cuda_get_device_info(int index)
	{
		static const std::vector<std::string> infos = []()
		{
			std::vector<std::string> result;
			for (const cudaDeviceProp &p : device_properties())
				result.push_back(std::string(p.name) + " : " + std::to_string(p.multiProcessorCount) + " x SM " + std::to_string(p.major) + "."
						+ std::to_string(p.minor) + " with " + std::to_string(p.totalGlobalMem >> 20) + "MB of memory");
			return result;
		}();
		if (index < 0 || index >= device_count())
			return nullptr;
		return infos[index].c_str();
	}
	const char* cuda_get_device_features(int index)
	{
		static const std::vector<std::string> features = []()
		{
			std::vector<std::string> result;
			for (const cudaDeviceProp &p : device_properties())
			{
				std::string s;
				s += "name : " + std::string(p.name) + "\n";
				s += "compute capability : " + std::to_string(p.major) + "." + std::to_string(p.minor) + "\n";
				s += "multiProcessorCount : " + std::to_string(p.multiProcessorCount) + "\n";
				s += "totalGlobalMem : " + std::to_string(p.totalGlobalMem) + "\n";
				s += "sharedMemPerBlockOptin : " + std::to_string(p.sharedMemPerBlockOptin) + "\n";
				s += "sharedMemPerMultiprocessor : " + std::to_string(p.sharedMemPerMultiprocessor) + "\n";
				s += "regsPerMultiprocessor : " + std::to_string(p.regsPerMultiprocessor) + "\n";
				s += "l2CacheSize : " + std::to_string(p.l2CacheSize) + "\n";
				s += "memoryBusWidth : " + std::to_string(p.memoryBusWidth) + "\n";
				s += "tensor path : tcgen05 (TMEM accumulators), TMA\n";
				result.push_back(s);
			}
			return result;
		}();
		if (index < 0 || index >= device_count())
			return nullptr;
		return features[index].c_str();
	}

	/* ------------------------------------------------------------------ contexts */
	mlContext_t cuda_create_context(int device_index)
	{
		if (device_index < 0 || device_index >= device_count())
		{
			record_error(nullptr, "cuda_create_context: device %d out of range (%d devices)", device_index, device_count());
			return nullptr;
		}
		Context *c = new Context();
		c->device = device_index;
		c->sm_count = device_properties()[device_index].multiProcessorCount;
		const char *eager = std::getenv("MINML_B200_EAGER");
		c->fusion = !(eager != nullptr && eager[0] == '1');
		cudaSetDevice(device_index);
		if (!check_cuda(nullptr, cudaStreamCreate(&c->stream), "cuda_create_context: stream"))
		{
			delete c;
			return nullptr;
		}
		if (check_cuda(nullptr, cudaMalloc(reinterpret_cast<void**>(&c->dev_status), sizeof(int)), "cuda_create_context: status word"))
			cudaMemset(c->dev_status, 0, sizeof(int));
		std::lock_guard<std::mutex> lock(g_contexts_mutex);
		g_contexts.push_back(c);
		return c;
	}
	void cuda_synchronize_with_context(mlContext_t context)
	{
		if (context == nullptr)
		{
			flush_all_pending();
			check_cuda(nullptr, cudaDeviceSynchronize(), "cuda_synchronize_with_context");
			return;
		}
		flush_pending(context);
		check_cuda(context, cudaStreamSynchronize(use_stream(context)), "cuda_synchronize_with_context");
		Context *c = get(context);
		if (c->dev_status != nullptr && c->kernels_with_waits)
		{
			int status = 0;
			if (check_cuda(context, cudaMemcpy(&status, c->dev_status, sizeof(int), cudaMemcpyDeviceToHost), "status word read") && status != 0)
			{
				record_error(context, "a tensor-core kernel gave up on a bounded wait (status %d); its output is incomplete", status);
				cudaMemset(c->dev_status, 0, sizeof(int));
			}
			c->kernels_with_waits = false;
		}
	}
	bool cuda_is_context_ready(mlContext_t context)
	{
		if (context == nullptr)
			return true;
		flush_pending(context);
		const cudaError_t status = cudaStreamQuery(use_stream(context));
		if (status == cudaErrorNotReady)
			return false;
		return check_cuda(context, status, "cuda_is_context_ready");
	}
	void cuda_destroy_context(mlContext_t context)
	{
		if (context == nullptr)
			return;
		Context *c = get(context);
		flush_pending(context);
		{ // out of the list first: from here on no other thread's flush can reach this context
			std::lock_guard<std::mutex> lock(g_contexts_mutex);
			for (size_t i = 0; i < g_contexts.size(); i++)
				if (g_contexts[i] == c)
				{
					g_contexts.erase(g_contexts.begin() + i);
					break;
				}
		}
		cudaSetDevice(c->device);
		cudaStreamSynchronize(c->stream);
		cudaStreamDestroy(c->stream);
		if (c->workspace != nullptr)
			cudaFree(c->workspace);
		if (c->dev_status != nullptr)
			cudaFree(c->dev_status);
		delete c;
	}

	/* ------------------------------------------------------------------ events */
	mlEvent_t cuda_create_event(mlContext_t context)
	{
		flush_pending(context);
		cudaStream_t stream = use_stream(context);
		cudaEvent_t *result = new cudaEvent_t();
		if (!check_cuda(context, cudaEventCreate(result), "cuda_create_event"))
		{
			delete result;
			return nullptr;
		}
		check_cuda(context, cudaEventRecord(*result, stream), "cuda_create_event: record");
		return reinterpret_cast<mlEvent_t>(result);
	}
	double cuda_get_time_between_events(mlEvent_t start, mlEvent_t end)
	{
		if (start == nullptr || end == nullptr)
			return 0.0;
		float ms = 0.0f;
		if (!check_cuda(nullptr, cudaEventElapsedTime(&ms, *reinterpret_cast<cudaEvent_t*>(start), *reinterpret_cast<cudaEvent_t*>(end)),
				"cuda_get_time_between_events"))
			return 0.0;
		return ms * 1.0e-3; // seconds, as in the reference
	}
	void cuda_wait_for_event(mlEvent_t event)
	{
		if (event != nullptr)
			check_cuda(nullptr, cudaEventSynchronize(*reinterpret_cast<cudaEvent_t*>(event)), "cuda_wait_for_event");
	}
	bool cuda_is_event_ready(mlEvent_t event)
	{
		if (event == nullptr)
			return true;
		const cudaError_t status = cudaEventQuery(*reinterpret_cast<cudaEvent_t*>(event));
		if (status == cudaErrorNotReady)
			return false;
		return check_cuda(nullptr, status, "cuda_is_event_ready");
	}
	void cuda_destroy_event(mlEvent_t event)
	{
		if (event != nullptr)
		{
			cudaEventDestroy(*reinterpret_cast<cudaEvent_t*>(event));
			delete reinterpret_cast<cudaEvent_t*>(event);
		}
	}

	/* ------------------------------------------------------------------ memory */
	void* cuda_malloc(int device_index, size_t count)
	{
		void *result = nullptr;
		if (count > 0)
		{
			if (!check_cuda(nullptr, cudaSetDevice(device_index), "cuda_malloc: set device"))
				return nullptr;
			if (!check_cuda(nullptr, cudaMalloc(&result, count), "cuda_malloc"))
				return nullptr;
		}
		return result;
	}
	void cuda_page_lock(void *ptr, size_t count)
	{
		if (ptr != nullptr)
			check_cuda(nullptr, cudaHostRegister(ptr, count, 0), "cuda_page_lock");
	}
	void cuda_page_unlock(void *ptr)
	{
		if (ptr != nullptr)
			check_cuda(nullptr, cudaHostUnregister(ptr), "cuda_page_unlock");
	}
	void cuda_free(void *ptr)
	{
		if (ptr != nullptr)
		{
			flush_all_pending(); // a deferred sequence may still reference this buffer
			winograd_forget_range(ptr, allocation_size(ptr)); // a recycled address must never alias a stale weight record
			conv_forget_range(ptr, allocation_size(ptr));
			check_cuda(nullptr, cudaFree(ptr), "cuda_free");
		}
	}
	void* cuda_create_view(void *src, size_t offset, size_t count)
	{
		(void) count;
		if (src == nullptr)
			return nullptr;
		return reinterpret_cast<uint8_t*>(src) + offset;
	}
	void cuda_destroy_view(void *ptr)
	{
		(void) ptr;
	}
	void cuda_memset(mlContext_t context, void *dst, size_t dst_offset, size_t dst_count, const void *src, size_t src_count)
	{
		MB200_REQUIRE(context, dst != nullptr, "cuda_memset: null destination");
		if (context == nullptr)
			flush_all_pending();
		else
			flush_pending(context);
		void *tmp_dst = reinterpret_cast<uint8_t*>(dst) + dst_offset;
		winograd_forget_range(tmp_dst, dst_count); // transformed weights written to directly are no longer described by their snapshot
		conv_forget_range(tmp_dst, dst_count);
		cudaStream_t stream = use_stream(context);
		if (src == nullptr)
		{
			if (context == nullptr)
			{ // default stream: must be complete when the call returns
				check_cuda(nullptr, cudaMemset(tmp_dst, 0, dst_count), "cuda_memset");
				check_cuda(nullptr, cudaDeviceSynchronize(), "cuda_memset: synchronize");
			}
			else
				check_cuda(context, cudaMemsetAsync(tmp_dst, 0, dst_count, stream), "cuda_memset");
			return;
		}
		MB200_REQUIRE(context, src_count == 1 || src_count == 2 || src_count == 4 || src_count == 8,
				"cuda_memset: pattern of %zu bytes (1, 2, 4 or 8 supported)", src_count);
		MB200_REQUIRE(context, dst_count % src_count == 0, "cuda_memset: %zu bytes is not a multiple of the %zu-byte pattern", dst_count,
				src_count);
		MB200_REQUIRE(context, aligned_to(tmp_dst, src_count), "cuda_memset: destination not aligned to the %zu-byte pattern", src_count);
		switch (src_count)
		{
			case 1:
				launch_fill<uint8_t>(context, stream, tmp_dst, dst_count, src);
				break;
			case 2:
				launch_fill<uint16_t>(context, stream, tmp_dst, dst_count, src);
				break;
			case 4:
				launch_fill<uint32_t>(context, stream, tmp_dst, dst_count, src);
				break;
			case 8:
				launch_fill<uint64_t>(context, stream, tmp_dst, dst_count, src);
				break;
		}
		if (context == nullptr)
			check_cuda(nullptr, cudaDeviceSynchronize(), "cuda_memset: synchronize");
	}
	void cuda_memcpy_within_device(mlContext_t context, void *dst, size_t dst_offset, const void *src, size_t src_offset, size_t count)
	{
		MB200_REQUIRE(context, dst != nullptr && src != nullptr, "cuda_memcpy_within_device: null pointer");
		if (count == 0)
			return;
		void *d = reinterpret_cast<uint8_t*>(dst) + dst_offset;
		const void *s = reinterpret_cast<const uint8_t*>(src) + src_offset;
		winograd_forget_range(d, count);
		conv_forget_range(d, count);
		if (context == nullptr)
		{
			flush_all_pending();
			check_cuda(nullptr, cudaMemcpy(d, s, count, cudaMemcpyDeviceToDevice), "cuda_memcpy_within_device");
		}
		else
		{
			flush_pending(context);
			check_cuda(context, cudaMemcpyAsync(d, s, count, cudaMemcpyDeviceToDevice, use_stream(context)), "cuda_memcpy_within_device");
		}
	}
	void cuda_memcpy_from_host(mlContext_t context, void *dst, size_t dst_offset, const void *src, size_t count)
	{
		MB200_REQUIRE(context, dst != nullptr && src != nullptr, "cuda_memcpy_from_host: null pointer");
		if (count == 0)
			return;
		void *d = reinterpret_cast<uint8_t*>(dst) + dst_offset;
		winograd_forget_range(d, count);
		conv_forget_range(d, count);
		if (context == nullptr)
		{
			flush_all_pending();
			check_cuda(nullptr, cudaMemcpy(d, src, count, cudaMemcpyHostToDevice), "cuda_memcpy_from_host");
		}
		else
		{
			flush_pending(context);
			check_cuda(context, cudaMemcpyAsync(d, src, count, cudaMemcpyHostToDevice, use_stream(context)), "cuda_memcpy_from_host");
		}
	}
	void cuda_memcpy_to_host(mlContext_t context, void *dst, const void *src, size_t src_offset, size_t count)
	{
		MB200_REQUIRE(context, dst != nullptr && src != nullptr, "cuda_memcpy_to_host: null pointer");
		if (count == 0)
			return;
		const void *s = reinterpret_cast<const uint8_t*>(src) + src_offset;
		if (context == nullptr)
		{
			flush_all_pending();
			check_cuda(nullptr, cudaMemcpy(dst, s, count, cudaMemcpyDeviceToHost), "cuda_memcpy_to_host");
		}
		else
		{
			flush_pending(context);
			check_cuda(context, cudaMemcpyAsync(dst, s, count, cudaMemcpyDeviceToHost, use_stream(context)), "cuda_memcpy_to_host");
		}
	}

	/* ------------------------------------------------------------------ extensions */
	const char* mb200_get_last_error(mlContext_t context)
	{
		std::lock_guard<std::mutex> lock(g_mutex);
		if (context == nullptr)
			return g_global_has_error ? g_global_error.c_str() : nullptr;
		Context *c = get(context);
		return c->has_error ? c->error.c_str() : nullptr;
	}
	void mb200_clear_last_error(mlContext_t context)
	{
		std::lock_guard<std::mutex> lock(g_mutex);
		if (context == nullptr)
		{
			g_global_has_error = false;
			g_global_error.clear();
		}
		else
		{
			get(context)->has_error = false;
			get(context)->error.clear();
		}
	}
	unsigned long long mb200_get_launch_count(void)
	{
		return g_launch_count.load();
	}
	void* mb200_get_stream(mlContext_t context)
	{
		return context == nullptr ? nullptr : reinterpret_cast<void*>(get(context)->stream);
	}
	void mb200_set_fusion(mlContext_t context, int enabled)
	{
		if (context != nullptr)
		{
			std::lock_guard<std::recursive_mutex> lock(get(context)->mutex);
			flush_pending(context);
			get(context)->fusion = (enabled != 0);
		}
	}
	void mb200_forget_range(const void *ptr, size_t bytes)
	{
		if (ptr == nullptr)
			return;
		flush_all_pending();
		winograd_forget_range(ptr, bytes);
		conv_forget_range(ptr, bytes);
	}
	const char* mb200_version(void)
	{
		return "minml_b200 0.1 sm_100a";
	}
}
