/*
 * conv_slab.cu -- fused fp16 3x3 convolution for layers of up to 128 channels: the input of a band of image rows is copied into
 * shared memory ONCE, with its halo, and the nine filter taps read it through shifted operand descriptors.
 *
 *      y = act(conv3x3(x, w) + bias + ext),  stride 1, "same" padding, NHWC fp16, w [cout, 3, 3, cin], fp32 accumulation
 *
 * Why.  The general kernel (conv_igemm.cu) fetches the A operand once per filter tap (im2col-mode TMA); with 128 output channels a
 * 128 x 128 tile then pulls 128 bytes per tensor-core cycle from L2, about twice what the L2 -> SM path delivers, and the tensor
 * pipe idles half of the time.  Here a work unit is a band of R image rows of one batch item:
 *   - the band plus one halo row above and below and one halo column left and right, (R + 2) x (W + 2) positions x 64 channels per
 *     128-byte slice, arrives by ONE tiled TMA copy per slice (zeros outside the image: the copy engine fills what lies outside);
 *   - output position (h, w) of the band is row m = h (W + 2) + w of the GEMM, and its operand for tap (kh, kw) is shared-memory row
 *     m + kh (W + 2) + kw: the same tile, read from a start address shifted by whole 128-byte rows (the 128-byte swizzle is a
 *     function of the absolute shared-memory address, so a shifted start reads what the copy engine wrote);
 *   - rows m whose w falls on the two halo columns compute garbage that is never stored: W / (W + 2) of the tensor work is useful;
 *   - two 128-row tiles per unit share every weight slice (R is the largest band with (R - 1) (W + 2) + W <= 256).
 * Per multiply-add the kernel fetches less than half of the bytes of the general kernel.
 *
 * MEASURED, and not the default: on a B200 the general kernel is faster on the layers this one was built for -- 256 x 15 x 15 x 128
 * -> 128: 23.2 us against 27.1 us here; 512 x 20 x 20 x 128 -> 128: 58.7 us against 76.2 us.  What this kernel saves in operand
 * bytes it loses elsewhere: 12 - 22 % of its tensor work goes to halo columns and to the padding of a band to 256 rows, the
 * 288 KB weight stream per unit is fetched through a ring of only three 16 KB slices (shared memory is taken by the two bands),
 * and a variant in which every weight slice fed four tiles instead of two (two bands per CTA at a time, accumulators in all 512
 * columns) was slower still (30.7 / 114 us) because the epilogue and the band copies then no longer overlap the products.
 * Rounding the shifts to whole 8-row groups (wrong results, timing only) changed nothing, so the shifted descriptors themselves
 * cost nothing.  The kernel stays selectable (MINML_B200_CONV_SLAB=1) and is held to the same parity tests.
 *
 * One CTA per SM, persistent over units, shared memory = two input bands (the next unit's copy runs under this unit's products),
 * a ring of weight slices and the epilogue's staging rows; tensor memory = two accumulator buffers of two tiles:
 *   warp 0      TMA: the band (per unit) and the weight slices (per tap and 64-channel slice)
 *   warp 1      tcgen05.mma issue (one elected lane); owns the tensor-memory allocation
 *   warps 2-9   epilogue: tcgen05.ld, bias / residual / activation, rows staged through shared memory so that global accesses cover
 *               whole 64-byte row segments
 * Every wait is bounded (tc.cuh); on a timeout the kernel sets the context's status word and drains.
 */
#include "common.cuh"
#include "conv.cuh"
#include "tc.cuh"
#include "epilogue.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace mb200
{
	namespace
	{
		using namespace tc;
		using namespace epi;

		constexpr int BM = 128, BN = 128;
		constexpr int TILES = 2; // 128-row tiles per unit
		constexpr int B_STAGES = 3;
		constexpr int B_STAGE_BYTES = BN * 128;
		constexpr int EPI_WARPS = 8;
		constexpr int THREADS = (2 + EPI_WARPS) * 32;

		struct SlabParams
		{
				const __half *x;
				__half *y;
				const __half *bias;
				const __half *ext;
				int batch, height, width, cin, cout;
				int padded_width; // W + 2
				int band_rows, bands_per_image; // R and ceil(H / R)
				int slices; // 64-channel slices of the input: cin / 64
				int slab_bytes; // per slice, rounded up to 1024
				int act;
				FastDiv by_padded_width;
				int *status;
		};
		struct SlabBarriers
		{
				uint64_t slab_full[2], slab_empty[2];
				uint64_t b_full[B_STAGES], b_empty[B_STAGES];
				uint64_t tmem_full[2], tmem_empty[2];
				uint32_t tmem_base;
				int abort_flag;
		};

		__device__ __forceinline__ void tma_load_4d_tiled(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
		{
			asm volatile(
					"cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
					:: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
		}

		__global__ void __launch_bounds__(THREADS, 1) kernel_conv3x3_slab(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
				const SlabParams p)
		{
			extern __shared__ uint8_t smem_raw[];
			__shared__ SlabBarriers bars;
			const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
			const int band_bytes = p.slices * p.slab_bytes; // one input band: all its 64-channel slices
			const uint32_t b_base = smem_base + 2 * band_bytes;
			const uint32_t epi_base = b_base + B_STAGES * B_STAGE_BYTES;
			const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
			const int total_units = p.batch * p.bands_per_image;
			const int k_slices = 9 * p.slices; // weight slices of 128 bytes of K, ordered (kh, kw, 64-channel slice)
			const uint32_t copy_bytes = static_cast<uint32_t>(p.slices) * (p.band_rows + 2) * p.padded_width * 128u; // what the copies of a band deliver

			if (threadIdx.x == 0)
			{
				for (int i = 0; i < 2; i++)
				{
					mbar_init(smem_u32(&bars.slab_full[i]), 1);
					mbar_init(smem_u32(&bars.slab_empty[i]), 1);
					mbar_init(smem_u32(&bars.tmem_full[i]), 1);
					mbar_init(smem_u32(&bars.tmem_empty[i]), EPI_WARPS);
				}
				for (int s = 0; s < B_STAGES; s++)
				{
					mbar_init(smem_u32(&bars.b_full[s]), 1);
					mbar_init(smem_u32(&bars.b_empty[s]), 1);
				}
				bars.abort_flag = 0;
				fence_mbar_init();
			}
			if (warp == 1)
			{
				tmem_alloc(smem_u32(&bars.tmem_base), 2 * TILES * BN);
				tmem_relinquish();
			}
			tcgen05_fence_before();
			__syncthreads();
			tcgen05_fence_after();
			const uint32_t tmem_base = bars.tmem_base;
			volatile int *abort_flag = &bars.abort_flag;

			if (warp == 0)
			{ /* ------------------------------------------------ copies */
				if (elect_one())
				{
					prefetch_tensormap(&map_w);
					prefetch_tensormap(&map_x);
					uint32_t it = 0, local = 0;
					bool ok = true;
					for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, local++)
					{
						const int image = unit / p.bands_per_image, band = unit % p.bands_per_image;
						const uint32_t buf = local & 1u;
						if (!mbar_wait(smem_u32(&bars.slab_empty[buf]), ((local >> 1) & 1u) ^ 1u, abort_flag))
							break;
						const uint32_t full = smem_u32(&bars.slab_full[buf]);
						mbar_arrive_expect_tx(full, copy_bytes);
						for (int s = 0; s < p.slices; s++) // halo: one position before the band in both directions, zeros outside the image
							tma_load_4d_tiled(smem_base + buf * band_bytes + s * p.slab_bytes, &map_x, full, s * 64, -1, band * p.band_rows - 1, image);
						for (int kb = 0; kb < k_slices; kb++, it++)
						{
							const int s = it % B_STAGES;
							if (!mbar_wait(smem_u32(&bars.b_empty[s]), ((it / B_STAGES) & 1u) ^ 1u, abort_flag))
							{
								ok = false;
								break;
							}
							mbar_arrive_expect_tx(smem_u32(&bars.b_full[s]), B_STAGE_BYTES);
							tma_load_3d(b_base + s * B_STAGE_BYTES, &map_w, smem_u32(&bars.b_full[s]), kb * 64, 0, 0);
						}
					}
				}
				__syncwarp();
			}
			else if (warp == 1)
			{ /* ------------------------------------------- MMA issue */
				if (elect_one())
				{
					const uint32_t idesc = make_idesc_f16(BN);
					uint32_t it = 0, local = 0;
					bool ok = true;
					for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, local++)
					{
						const uint32_t buf = local & 1u;
						if (!mbar_wait(smem_u32(&bars.tmem_empty[buf]), ((local >> 1) & 1u) ^ 1u, abort_flag)
								|| !mbar_wait(smem_u32(&bars.slab_full[buf]), (local >> 1) & 1u, abort_flag))
							break;
						tcgen05_fence_after();
						const uint32_t band_addr = smem_base + buf * band_bytes;
						for (int kb = 0; kb < k_slices; kb++, it++)
						{
							const int s = it % B_STAGES;
							if (!mbar_wait(smem_u32(&bars.b_full[s]), (it / B_STAGES) & 1u, abort_flag))
							{
								ok = false;
								break;
							}
							tcgen05_fence_after();
							const int tap = kb / p.slices, slice = kb - tap * p.slices;
							const int shift_rows = (tap / 3) * p.padded_width + (tap % 3); // where this tap's operand of output row 0 lies in the band
							const uint64_t desc_b = make_desc_k_sw128(b_base + s * B_STAGE_BYTES);
#pragma unroll
							for (int t = 0; t < TILES; t++)
							{
								const uint64_t desc_a = make_desc_k_sw128(band_addr + slice * p.slab_bytes + (t * BM + shift_rows) * 128);
#pragma unroll
								for (int k = 0; k < 4; k++)
									mma_ss<0>(tmem_base + (buf * TILES + t) * BN, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
							}
							mma_commit(smem_u32(&bars.b_empty[s]));
						}
						if (ok)
						{
							mma_commit(smem_u32(&bars.slab_empty[buf])); // the band may be overwritten once these products are done
							mma_commit(smem_u32(&bars.tmem_full[buf]));
						}
					}
				}
				__syncwarp();
			}
			else
			{ /* ------------------------------------------------------------ epilogue */
				const int q = warp % 4; // tensor-memory lane quarter
				const int col_part = (warp - 2) / 4; // which half of the columns
				const uint32_t sbuf = epi_base + (warp - 2) * WARP_BYTES;
				const int rr = lane / 4, seg = lane % 4; // cooperative access: 8 rows x 4 segments of 16 bytes per instruction
				const bool vectorisable = (p.cout % 8 == 0) && aligned_to_16(p.y) && (p.ext == nullptr || aligned_to_16(p.ext));
				uint32_t local = 0;
				for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x, local++)
				{
					const int image = unit / p.bands_per_image, band = unit % p.bands_per_image;
					const uint32_t buf = local & 1u;
					if (!mbar_wait_all_lanes(smem_u32(&bars.tmem_full[buf]), (local >> 1) & 1u, abort_flag))
						break;
					tcgen05_fence_after();
					const int h0 = band * p.band_rows;
					const int rows_here = min(p.band_rows, p.height - h0);
					const long long image_row0 = (static_cast<long long>(image) * p.height + h0) * p.width; // output row of position (h0, 0)
					for (int t = 0; t < TILES; t++)
					{
						// output row (in y) of GEMM row m of this tile, or -1 when m is a halo column or lies beyond the band
						auto output_row = [&](int m) -> long long
						{
							uint32_t hh, w;
							p.by_padded_width.divmod(static_cast<uint32_t>(m), hh, w);
							return (static_cast<int>(w) < p.width && static_cast<int>(hh) < rows_here) ? image_row0 + static_cast<long long>(hh) * p.width + w : -1;
						};
						const int m0 = t * BM + q * 32;
						const long long my_row = output_row(m0 + lane);
						for (int cc = 0; cc < BN / 64; cc++)
						{
							const int c = col_part * (BN / 64) + cc;
							const int n0 = c * 32;
							if (n0 >= p.cout)
								continue; // warp-uniform
							const int n_valid = min(32, p.cout - n0);
							const bool fast = vectorisable && n_valid == 32;
							long long coop_row[4];
							uint4 res[4];
							if (fast)
							{
#pragma unroll
								for (int i = 0; i < 4; i++)
								{
									coop_row[i] = output_row(m0 + rr + 8 * i);
									res[i] = (p.ext != nullptr && coop_row[i] >= 0) ? *reinterpret_cast<const uint4*>(p.ext + coop_row[i] * p.cout + n0 + seg * 8) : make_uint4(0,
											0, 0, 0);
								}
							}
							uint32_t r[32];
							tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + (buf * TILES + t) * BN + c * 32, r);
							tmem_wait_ld();
							float v[32];
#pragma unroll
							for (int j = 0; j < 32; j++)
								v[j] = __uint_as_float(r[j]);
							if (fast)
							{
								if (p.bias != nullptr)
								{
									const __half *bs = p.bias + n0;
									if (aligned_to_16(p.bias))
									{
#pragma unroll
										for (int k = 0; k < 4; k++)
											add_half8(v + 8 * k, reinterpret_cast<const uint4*>(bs)[k]);
									}
									else
									{
#pragma unroll
										for (int j = 0; j < 32; j++)
											v[j] += __half2float(bs[j]);
									}
								}
								if (p.ext != nullptr)
								{ // through shared memory: cooperative layout -> one row per lane
#pragma unroll
									for (int i = 0; i < 4; i++)
										st_shared_v4(sbuf + (rr + 8 * i) * PITCH + seg * 16, res[i]);
									__syncwarp();
#pragma unroll
									for (int k = 0; k < 4; k++)
										add_half8(v + 8 * k, ld_shared_v4(sbuf + lane * PITCH + k * 16));
									__syncwarp();
								}
								activate32(v, p.act);
#pragma unroll
								for (int k = 0; k < 4; k++)
									st_shared_v4(sbuf + lane * PITCH + k * 16, pack_half8(v + 8 * k));
								__syncwarp();
#pragma unroll
								for (int i = 0; i < 4; i++)
								{
									const uint4 val = ld_shared_v4(sbuf + (rr + 8 * i) * PITCH + seg * 16);
									if (coop_row[i] >= 0)
										*reinterpret_cast<uint4*>(p.y + coop_row[i] * p.cout + n0 + seg * 8) = val;
								}
								__syncwarp();
								continue;
							}
							/* general path: one row per lane, any alignment, column tails */
							if (my_row < 0)
								continue;
#pragma unroll
							for (int j = 0; j < 32; j++)
								if (j < n_valid)
									v[j] += (p.bias != nullptr ? __half2float(p.bias[n0 + j]) : 0.0f)
											+ (p.ext != nullptr ? __half2float(p.ext[my_row * p.cout + n0 + j]) : 0.0f);
							activate32(v, p.act);
#pragma unroll
							for (int j = 0; j < 32; j++)
								if (j < n_valid)
									p.y[my_row * p.cout + n0 + j] = __float2half_rn(v[j]);
						}
					}
					tcgen05_fence_before();
					__syncwarp();
					if (lane == 0)
						mbar_arrive(smem_u32(&bars.tmem_empty[buf]));
				}
			}

			/* ---------------------------------------------------------------- teardown */
			tcgen05_fence_before();
			__syncthreads();
			if (bars.abort_flag != 0)
			{
				if (threadIdx.x == 0 && p.status != nullptr)
					atomicExch(p.status, 4);
				__nanosleep(1000000); // give copies that are still in flight time to land before the CTA retires
			}
			if (warp == 1)
			{
				tcgen05_fence_after();
				tmem_dealloc(tmem_base, 2 * TILES * BN);
			}
		}

		bool slab_enabled()
		{
			static const bool on = []
			{
				const char *e = std::getenv("MINML_B200_CONV_SLAB"); // 1 = use this kernel for the layers it takes (default: the general kernel, which measured faster)
				return e != nullptr && e[0] == '1';
			}();
			return on;
		}
	}

	/* True when conv_slab_run takes the layer: fp16, 64 or 128 input channels, up to 128 output channels, a board whose bands fit. */
	bool conv_slab_supported(const mlTensor_t &x, const mlTensor_t &w, const mlTensor_t &y)
	{
		if (!slab_enabled() || x.dtype != DTYPE_FLOAT16 || w.dtype != DTYPE_FLOAT16 || y.dtype != DTYPE_FLOAT16 || x.rank != 4 || w.rank != 4)
			return false;
		const int height = x.dim[1], width = x.dim[2], cin = x.dim[3], cout = w.dim[0];
		if ((cin != 64 && cin != 128) || cout > BN || cout < 1 || w.dim[1] != 3 || w.dim[2] != 3 || w.dim[3] != cin)
			return false;
		if (width + 2 > 256 || width < 1 || height < 1 || (width + 2) + width > TILES * BM) // at least one image row per unit
			return false;
		if (!aligned_to(x.data, 16) || !aligned_to(w.data, 16) || !aligned_to(y.data, 2))
			return false;
		const long long positions = static_cast<long long>(x.dim[0]) * height * width;
		return positions > 0 && positions * std::max(cin, cout) < (1LL << 31);
	}

	bool conv_slab_run(mlContext_t ctx, const mlTensor_t &x, const mlTensor_t &w, const void *bias, const void *ext, const mlTensor_t &y,
			mlActivationType_t act)
	{
		Context *c = get(ctx);
		SlabParams p;
		std::memset(&p, 0, sizeof(p));
		p.x = reinterpret_cast<const __half*>(x.data);
		p.y = reinterpret_cast<__half*>(y.data);
		p.bias = reinterpret_cast<const __half*>(bias);
		p.ext = reinterpret_cast<const __half*>(ext);
		p.batch = x.dim[0];
		p.height = x.dim[1];
		p.width = x.dim[2];
		p.cin = x.dim[3];
		p.cout = w.dim[0];
		p.padded_width = p.width + 2;
		const int most_rows = std::min(p.height, (TILES * BM - p.width) / p.padded_width + 1); // (R - 1) (W + 2) + W <= 256
		p.bands_per_image = (p.height + most_rows - 1) / most_rows;
		p.band_rows = (p.height + p.bands_per_image - 1) / p.bands_per_image; // bands of equal height
		p.slices = p.cin / 64;
		// rows the products may touch: TILES * BM output rows plus the largest tap shift; the copy itself delivers (R + 2) (W + 2) rows
		const int slab_rows = std::max(TILES * BM + 2 * p.padded_width + 2, (p.band_rows + 2) * p.padded_width);
		p.slab_bytes = (slab_rows * 128 + 1023) / 1024 * 1024;
		p.act = act;
		p.by_padded_width = FastDiv(static_cast<uint32_t>(p.padded_width));
		p.status = c->dev_status;
		const size_t smem = 1024 + static_cast<size_t>(2) * p.slices * p.slab_bytes + B_STAGES * B_STAGE_BYTES + EPI_WARPS * WARP_BYTES;
		if (smem > 226 * 1024 || p.band_rows + 2 > 256)
			return false;

		CUtensorMap map_w, map_x;
		const uint64_t k_total = static_cast<uint64_t>(9) * p.cin;
		const uint64_t wdims[3] = { k_total, static_cast<uint64_t>(p.cout), 1 };
		const uint64_t wstrides[2] = { k_total * 2, k_total * 2 * p.cout };
		const uint32_t wbox[3] = { 64, BN, 1 };
		if (!encode_tensor_map(ctx, &map_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, w.data, wdims, wstrides, wbox, CU_TENSOR_MAP_SWIZZLE_128B))
			return false;
		const uint64_t xdims[4] = { static_cast<uint64_t>(p.cin), static_cast<uint64_t>(p.width), static_cast<uint64_t>(p.height), static_cast<uint64_t>(p.batch) };
		const uint64_t xstrides[3] = { static_cast<uint64_t>(p.cin) * 2, static_cast<uint64_t>(p.cin) * 2 * p.width,
				static_cast<uint64_t>(p.cin) * 2 * p.width * p.height };
		const uint32_t xbox[4] = { 64, static_cast<uint32_t>(p.padded_width), static_cast<uint32_t>(p.band_rows + 2), 1 };
		if (!encode_tensor_map(ctx, &map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, x.data, xdims, xstrides, xbox, CU_TENSOR_MAP_SWIZZLE_128B))
			return false;

		static std::mutex configured_mutex;
		static bool configured_on[MAX_DEVICES] = { false };
		{
			std::lock_guard<std::mutex> lock(configured_mutex);
			if (c->device < 0 || c->device >= MAX_DEVICES)
				return false;
			if (!configured_on[c->device])
			{
				if (!check_cuda(ctx, cudaFuncSetAttribute(kernel_conv3x3_slab, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024),
						"conv_slab: shared memory opt-in"))
					return false;
				configured_on[c->device] = true;
			}
		}
		const int units = p.batch * p.bands_per_image;
		const int grid = std::min(units, c->sm_count);
		kernel_conv3x3_slab<<<grid, THREADS, smem, use_stream(ctx)>>>(map_w, map_x, p);
		MB200_COUNT_LAUNCH();
		c->kernels_with_waits = true;
		return check_cuda(ctx, cudaGetLastError(), "conv_slab launch");
	}
} /* namespace mb200 */
