/*
 * conv_igemm.cu -- fused 3x3 convolution as an implicit GEMM on the tcgen05 tensor cores:
 *
 *      y = epilogue( conv3x3(x, w) ),  stride 1, "same" padding, NHWC, w [cout, 3, 3, cin]
 *      fp16:  epilogue = act(acc + bias + ext)                       fp32 accumulation, fp16 out
 *      int8:  epilogue = requantise(act(acc * scale[c] + shift[c] + dequant(ext)))   exact int32 accumulation
 *      fp32:  epilogue = act(acc + bias + ext)                       fp32 in and out; the products run on the TF32 tensor cores, either
 *             as one TF32 product (when the host allowed TF32 on the context, cuda_enable_tf32) or, by default, at fp32 accuracy
 *             as three TF32 products of split operands, x * w ~ xh * wh + xh * wl + xl * wh (error analysis in gemm_tc.cu): the
 *             weights arrive already split into two planes [2, cout, 9 cin] (made once per layer, at weight-transform time); of the
 *             activations the tensor core itself takes the upper 19 bits (xh = x truncated to TF32), so the split warps only have
 *             to write xl = x - xh next to the landed tile
 *
 * It is the single-kernel replacement for the two three-call sequences minml's Conv2D::forward issues
 * (Winograd: src/layers/Conv2D.cpp:365-377; int8: src/layers/Conv2D.cpp:214-239) and the body of
 * cuda_convolution_implicit_gemm_forward (empty in the reference without cuDNN, src/backend/cuda/cudnn_math.cpp:691-694).
 * Nothing but x, w, bias, ext and y crosses HBM: there is no transformed-input, im2row or accumulator tensor.
 *
 * GEMM view: M = b*h*w output positions, N = cout, K = 9*cin ordered (kh, kw, cin) -- the weight tensor as stored is
 * the K-major B operand [N, K].  The A operand is never materialised: for every 128-byte slice of K, producer warps
 * gather the 16-byte channel chunks of 128 positions straight from x into the 128B-swizzled shared-memory tile that
 * tcgen05.mma reads (cp.async with zero fill outside the image; a non-zero int8 padding value is stored directly).
 *
 * One CTA per SM, persistent over 128 x BN output tiles, two accumulator buffers in tensor memory so that the
 * epilogue of tile i overlaps the main loop of tile i + 1:
 *   warp 0        TMA loads of the weight tile (BN rows x 128 bytes of K) and, in the TMA_A variant, of the A slice
 *   warp 1        tcgen05.mma issue (one elected lane); owns the tensor-memory allocation
 *   warps 2-9     epilogue: tcgen05.ld, bias / residual / activation / requantisation; residual reads and output
 *                 writes of the fp16 path are staged through shared memory so that every global access of a warp
 *                 covers whole 64-byte row segments
 *   warps 10, 11, 14, 15   A-operand gather (cp.async variant only)
 *
 * The int8 TMA variant runs sixteen epilogue warps (its requantisation is the expensive part).  Tile shapes on top of that:
 *   256 output channels, TMA operands: clusters of two CTAs, tcgen05.mma.cta_group::2 (M = 256, each CTA fetches half of every
 *       weight slice) -- the single-CTA kernel was limited by the operand fetch from L2;
 *   up to 128 output channels, TMA operands, enough rows: two 128-row tiles per CTA and work unit sharing every weight slice.
 *
 * Two variants of the A operand path:
 *   TMA_A = true   im2col-mode TMA: one request per K slice delivers 128 output positions x 128 bytes of channels of one
 *                  filter tap, zero-filled outside the image.  Needs cin * element size to be a multiple of 128 bytes.  A non-zero
 *                  int8 padding value z (the quantised zero of an asymmetric input) is made up for in the epilogue: positions on
 *                  the border get z * (sum of the weights of the taps that fell outside) from a 9 x cout table computed once per weight
 *                  tensor (kernel_border_table, cached_border_table), which keeps the int32 accumulators exact.  This is the fast path (256 -> 256 fp16:
 *                  1.23 PFLOP/s against 0.92 for the gather).
 *   TMA_A = false  cp.async gather of 16-byte channel chunks: any cin that is a multiple of 8 (fp16) / 16 (int8), any
 *                  int8 padding value.
 * Every wait is bounded (tc.cuh); on a timeout the kernel sets its status word and drains.
 */
#include "common.cuh"
#include "conv.cuh"
#include "tc.cuh"
#include "epilogue.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

namespace mb200
{
	namespace
	{
		using namespace tc;
		using namespace epi;

		constexpr int BM = 128;
		/* Warp roles.  Warp 0: TMA, warp 1: MMA issue, then the epilogue warps, then (gather variant) the A-operand producers on
		 * warps 10, 11, 14, 15.  The int8 epilogue costs about 22 instructions per output element against 4 for fp16 and its
		 * tiles take half as many tensor cycles, so the int8 TMA variant runs 16 epilogue warps (four per tensor-memory lane
		 * quarter) instead of 8. */
		template<int KIND, bool TMA_A>
		struct Roles
		{
				static constexpr int epi_warps = (KIND == 1 && TMA_A) ? 16 : 8;
				static constexpr int split_warps = (KIND == 3) ? 4 : 0; // fp32 at full accuracy: warps that write the lo part of the landed A tile
				static constexpr int threads = (TMA_A ? (2 + epi_warps + split_warps) : 16) * 32;
				static constexpr int staging_bytes = (KIND == 0) ? 8 * 32 * 80 : 0; // only the fp16 epilogue stages rows in shared memory
		};
		constexpr int NUM_PRODUCERS = 128;
		constexpr int A_STAGE_BYTES = BM * 128;
		constexpr int EPI_PITCH = epi::PITCH;
		constexpr int EPI_WARP_BYTES = epi::WARP_BYTES;
		constexpr int MAX_STAGES = 8;

		/* TMA_A: the A operand is fetched by im2col-mode TMA (one request per K slice) instead of the cp.async gather.
		 * Possible when every 128-byte K slice lies inside one filter tap and the padding value is zero. */
		/* CTAS: 1 = every CTA computes 128 x BN tiles on its own; 2 = the two CTAs of a cluster compute a 256 x BN tile with
		 * tcgen05 cta_group::2: each holds its own 128 rows of A and HALF of the weight slice, so the weight bytes a CTA pulls
		 * from L2 per tile are halved (the operand fetch from L2, not the tensor pipe, is what limits the single-CTA kernel). */
		/* MT: 128-row tiles per CTA and work unit (1 or 2).  With 128 output channels a 128 x 128 tile does only 128 multiply-adds per
		 * operand byte fetched and the L2 -> SM path caps the tensor pipe near half its rate; two row tiles that share every weight
		 * slice fetch a quarter less per multiply-add and keep each stage busy twice as long (deeper effective prefetch). */
		template<int KIND, int BN, bool TMA_A, int CTAS = 1, int MT = 1>
		struct Cfg
		{
				static constexpr int a_stage_bytes = A_STAGE_BYTES * MT;
				static constexpr int b_planes = (KIND == 3) ? 2 : 1; // KIND 3: the hi and the lo plane of the weight slice, one after the other
				static constexpr int b_stage_bytes = BN / CTAS * 128 * b_planes;
				// The two operand rings are sized separately: the gathered A slices (cp.async, many small requests) need more
				// slices in flight to cover their latency than the weight slices that one TMA request fetches.
				static constexpr bool split = (KIND == 3);
				static constexpr int a_stages = split ? 3 : (MT == 2) ? 4 : (CTAS == 2) ? ((BN == 256) ? 6 : 8) : (TMA_A ? ((BN == 256) ? 4 : 6) : 6);
				static constexpr int b_stages = TMA_A ? a_stages : ((BN == 256) ? 3 : 6);
				// KIND 3: the lo part of a slice's A tile lives in a short ring of its own, from the split to the end of that slice's products
				static constexpr int lo_stages = split ? 2 : 0;
				static constexpr int lo_ring = (lo_stages > 0) ? lo_stages : 1; // divisor that is never zero
				static constexpr int lo_bytes = a_stage_bytes;
				static_assert(!split || BN == 128, "the split-fp32 variant is built for 128-column tiles");
				static constexpr int smem_bytes = a_stages * a_stage_bytes + b_stages * b_stage_bytes + lo_stages * lo_bytes + Roles<KIND, TMA_A>::staging_bytes + 1024;
				static constexpr int tmem_columns = 2 * BN * MT;
				static_assert(tmem_columns <= 512 && smem_bytes <= 227 * 1024, "tile configuration exceeds the SM");
		};

		struct ConvParams
		{
				const void *x;
				void *y;
				const void *bias; // fp16 / fp32 [cout] (floating-point kinds)
				const void *ext; // fp16, fp32 or int8 [b, h, w, cout]
				int batch, height, width, cin, cout;
				int M, K;
				int act;
				int out_dtype;
				const float *scales; // int8 kind
				const float *shifts;
				float ext_scale, ext_shift;
				float inv_out_scale, inv_out_shift; // 1 / out_scale and -out_shift / out_scale, rounded like AffineTransform::get_inverse
				int pad_byte;
				// int8, non-zero padding value on the TMA path (which can only fill with zeros): [9][cout] corrections, already
				// multiplied by the padding value, for the nine kinds of position (3 x 3: first / inner / last row and column)
				const int *border;
				FastDiv by_board, by_width; // position -> (row, column) of the board without divisions (border table only)
				int *status;
		};

		struct ConvBarriers
		{
				uint64_t full_a[MAX_STAGES];
				uint64_t empty_a[MAX_STAGES];
				uint64_t full_b[MAX_STAGES];
				uint64_t empty_b[MAX_STAGES];
				uint64_t split[MAX_STAGES]; // KIND 3: the stage's hi and lo tiles are written
				uint64_t lo_empty[2]; // KIND 3: the products that read this lo tile are done
				uint64_t tmem_full[2];
				uint64_t tmem_empty[2];
				uint32_t tmem_base;
				int abort_flag;
		};

		/* Weight planes of the split-fp32 kernel: planes[0] = w rounded to the nearest TF32 number (13 low mantissa bits clear),
		 * planes[1] = w - planes[0], exact in fp32 (gemm_tc.cu has the error analysis). */
		__global__ void __launch_bounds__(256) kernel_split_weight_planes(float *__restrict__ planes, const float *__restrict__ w, long long elements)
		{
			const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
			for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += stride)
			{
				const uint32_t x = __float_as_uint(w[i]);
				const uint32_t hi = (x + 0x1000u) & 0xFFFFE000u;
				planes[i] = __uint_as_float(hi);
				planes[elements + i] = __uint_as_float(x) - __uint_as_float(hi);
			}
		}
		__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, uint32_t src_bytes)
		{
			asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes) : "memory");
		}
		__device__ __forceinline__ void cp_async_wait_all()
		{
			asm volatile("cp.async.wait_all;" ::: "memory");
		}
		/* One arrival on the mbarrier, delivered when all cp.async issued so far by this thread have completed. */
		__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar)
		{
			asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" :: "r"(bar) : "memory");
		}
		__device__ __forceinline__ void st_shared_16(uint32_t dst, uint32_t v)
		{
			asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" :: "r"(dst), "r"(v) : "memory");
		}
		__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c, int w, int h, int n,
				uint16_t off_w, uint16_t off_h)
		{
			asm volatile(
					"cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
					:: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h) : "memory");
		}

		template<int KIND, int BN, bool TMA_A, int CTAS, int MT>
		__global__ void __launch_bounds__((Roles<KIND, TMA_A>::threads), 1) kernel_conv3x3_igemm(const __grid_constant__ CUtensorMap map_w,
				const __grid_constant__ CUtensorMap map_x, const ConvParams p)
		{
			static_assert(CTAS == 1 || TMA_A, "the paired kernel fetches both operands by TMA");
			static_assert(MT == 1 || (TMA_A && CTAS == 1), "two row tiles per CTA: TMA operands, single CTAs");
			static_assert(KIND < 2 || (TMA_A && CTAS == 1 && MT == 1), "fp32: TMA operands, single CTAs, one row tile");
			using C = Cfg<KIND, BN, TMA_A, CTAS, MT>;
			constexpr int EPI_WARPS = Roles<KIND, TMA_A>::epi_warps;
			constexpr int COLS_PER_WARP = BN / (EPI_WARPS / 4);
			constexpr int ES = (KIND == 0) ? 2 : (KIND == 1) ? 1 : 4; // operand element size
			constexpr int SPLIT_WARPS = Roles<KIND, TMA_A>::split_warps;
			constexpr int CHUNK_ELEMS = 16 / ES;
			extern __shared__ uint8_t smem_raw[];
			__shared__ ConvBarriers bars;

			const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
			const uint32_t b_base = smem_base + C::a_stages * C::a_stage_bytes;
			const uint32_t lo_base = b_base + C::b_stages * C::b_stage_bytes;
			const uint32_t epi_base = lo_base + C::lo_stages * C::lo_bytes;
			const int warp = threadIdx.x / 32;
			const int lane = threadIdx.x % 32;

			const int m_tiles = (p.M + BM - 1) / BM;
			const int n_tiles = (p.cout + BN - 1) / BN;
			const int k_blocks = (p.K * ES + 127) / 128;
			// A work unit is CTAS vertically adjacent 128-row tiles of one column block; CTA `cta_rank` of the cluster owns tile
			// unit_m * CTAS + cta_rank (which may lie wholly beyond M for the last unit: it then computes on rows it never stores).
			const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
			const bool leader = cta_rank == 0;
			const int first_unit = blockIdx.x / CTAS, unit_step = gridDim.x / CTAS;
			const int total_units = ((m_tiles + CTAS * MT - 1) / (CTAS * MT)) * n_tiles;

			if (threadIdx.x == 0)
			{
				for (int s = 0; s < C::a_stages; s++)
				{
					mbar_init(smem_u32(&bars.full_a[s]), NUM_PRODUCERS);
					mbar_init(smem_u32(&bars.empty_a[s]), 1);
				}
				for (int s = 0; s < C::b_stages; s++)
				{
					mbar_init(smem_u32(&bars.full_b[s]), 1);
					mbar_init(smem_u32(&bars.empty_b[s]), 1);
					mbar_init(smem_u32(&bars.split[s]), SPLIT_WARPS > 0 ? SPLIT_WARPS : 1);
				}
				for (int a = 0; a < 2; a++)
				{
					mbar_init(smem_u32(&bars.lo_empty[a]), 1);
					mbar_init(smem_u32(&bars.tmem_full[a]), 1);
					mbar_init(smem_u32(&bars.tmem_empty[a]), EPI_WARPS * CTAS);
				}
				bars.abort_flag = 0;
				fence_mbar_init();
			}
			if (warp == 1)
			{
				tmem_alloc(smem_u32(&bars.tmem_base), C::tmem_columns);
				tmem_relinquish();
			}
			// int8: per-channel scales and shifts in shared memory for the life of the CTA instead of sixteen 16-byte global reads per lane and
			// 32-column chunk (measured 1.5 - 3.5 %: 0.0461 -> 0.0445 ms on 512 x 20 x 20 x 128, 0.195 -> 0.192 ms on 1024 x 20 x 20 x 256)
			__shared__ __align__(16) float qs_s[KIND == 1 ? 512 : 4], qh_s[KIND == 1 ? 512 : 4];
			const bool q_staged = KIND == 1 && p.scales != nullptr && p.shifts != nullptr && p.cout <= 512;
			if (q_staged)
				for (int i = threadIdx.x; i < p.cout; i += blockDim.x)
				{
					qs_s[i] = p.scales[i];
					qh_s[i] = p.shifts[i];
				}
			tcgen05_fence_before();
			if (CTAS == 2)
				cluster_sync(); // the peer's barriers exist before anything signals them
			else
				__syncthreads();
			tcgen05_fence_after();
			const uint32_t tmem_base = bars.tmem_base;
			volatile int *abort_flag = &bars.abort_flag;

			if (warp == 0)
			{ /* ------------------------------------------------ weight tiles by TMA */
				if (elect_one())
				{
					prefetch_tensormap(&map_w);
					if (TMA_A)
						prefetch_tensormap(&map_x);
					uint32_t it = 0;
					bool ok = true;
					for (int unit = first_unit; unit < total_units && ok; unit += unit_step)
					{
						const int nt = unit % n_tiles;
						// first output position of the tile -> (image, row, column); im2col TMA walks on from there
						int m0 = ((unit / n_tiles) * CTAS + static_cast<int>(cta_rank)) * MT * BM;
						if (CTAS == 2 && m0 >= p.M)
							m0 = 0; // a tile wholly beyond M: fetch rows that exist, the epilogue stores none of them
						const int img0 = m0 / (p.height * p.width);
						const int h0 = (m0 - img0 * p.height * p.width) / p.width;
						const int w0 = m0 - img0 * p.height * p.width - h0 * p.width;
						int m1 = m0 + BM; // second row tile of the unit (MT == 2)
						if (m1 >= p.M)
							m1 = 0;
						const int img1 = m1 / (p.height * p.width);
						const int h1 = (m1 - img1 * p.height * p.width) / p.width;
						const int w1 = m1 - img1 * p.height * p.width - h1 * p.width;
						for (int kb = 0; kb < k_blocks; kb++, it++)
						{
							const int s = it % C::b_stages;
							if (!mbar_wait(smem_u32(&bars.empty_b[s]), ((it / C::b_stages) & 1u) ^ 1u, abort_flag))
							{
								ok = false;
								break;
							}
							const uint32_t full = smem_u32(&bars.full_b[s]);
							if (CTAS == 2)
							{ // both CTAs' slices are counted on the leader's barrier, which expects the bytes of both
								if (leader)
									mbar_arrive_expect_tx(full, 2 * (C::b_stage_bytes + A_STAGE_BYTES));
								const uint32_t full_leader = map_to_cta(full, 0);
								const int k0 = kb * (128 / ES);
								const int tap = k0 / p.cin;
								tma_load_im2col_4d_pair(smem_base + s * A_STAGE_BYTES, &map_x, full_leader, k0 - tap * p.cin, w0 - 1, h0 - 1, img0,
										static_cast<uint16_t>(tap % 3), static_cast<uint16_t>(tap / 3));
								tma_load_3d_pair(b_base + s * C::b_stage_bytes, &map_w, full_leader, k0, nt * BN + static_cast<int>(cta_rank) * (BN / 2), 0);
								continue;
							}
							mbar_arrive_expect_tx(full, C::b_stage_bytes + (TMA_A ? C::a_stage_bytes : 0));
							if (TMA_A)
							{
								const int k0 = kb * (128 / ES);
								const int tap = k0 / p.cin;
								tma_load_im2col_4d(smem_base + s * C::a_stage_bytes, &map_x, full, k0 - tap * p.cin, w0 - 1, h0 - 1, img0,
										static_cast<uint16_t>(tap % 3), static_cast<uint16_t>(tap / 3));
								if (MT == 2)
									tma_load_im2col_4d(smem_base + s * C::a_stage_bytes + A_STAGE_BYTES, &map_x, full, k0 - tap * p.cin, w1 - 1, h1 - 1, img1,
											static_cast<uint16_t>(tap % 3), static_cast<uint16_t>(tap / 3));
							}
							tma_load_3d(b_base + s * C::b_stage_bytes, &map_w, full, kb * (128 / ES), nt * BN, 0);
							if (C::split) // the lo plane of the same weight slice
								tma_load_3d(b_base + s * C::b_stage_bytes + BN * 128, &map_w, full, kb * (128 / ES), nt * BN, 1);
						}
					}
				}
				__syncwarp();
			}
			else if (warp == 1)
			{ /* ------------------------------------------- MMA issue */
				if (leader && elect_one())
				{ // in a pair only the even CTA issues; its instructions drive the tensor cores of both SMs
					const uint32_t idesc = (CTAS == 2) ? ((KIND == 0) ? make_idesc_f16_pair(BN) : make_idesc_i8_pair(BN))
							: ((KIND == 0) ? make_idesc_f16(BN) : (KIND == 1) ? make_idesc_i8(BN) : make_idesc_tf32(BN));
					uint64_t *const ready_b = C::split ? bars.split : bars.full_b; // what the tensor core may read
					uint32_t it = 0, local_tile = 0;
					bool ok = true;
					for (int unit = first_unit; unit < total_units && ok; unit += unit_step, local_tile++)
					{
						const uint32_t buf = local_tile & 1u;
						const uint32_t empty_bar = smem_u32(&bars.tmem_empty[buf]), empty_parity = ((local_tile >> 1) & 1u) ^ 1u;
						if (!((CTAS == 2) ? mbar_wait_cluster(empty_bar, empty_parity, abort_flag) : mbar_wait(empty_bar, empty_parity, abort_flag)))
							break;
						tcgen05_fence_after();
						const uint32_t tmem_d = tmem_base + buf * (BN * MT);
						for (int kb = 0; kb < k_blocks; kb++, it++)
						{
							const int sa = it % C::a_stages, sb = it % C::b_stages;
							if (!mbar_wait(smem_u32(&ready_b[sb]), (it / C::b_stages) & 1u, abort_flag)
									|| (!TMA_A && !mbar_wait(smem_u32(&bars.full_a[sa]), (it / C::a_stages) & 1u, abort_flag)))
							{
								ok = false;
								break;
							}
							tcgen05_fence_after();
							if (!TMA_A || C::split)
								fence_proxy_async_smem(); // the slice was written through the generic proxy by other threads
							const uint64_t desc_a = make_desc_k_sw128(smem_base + sa * C::a_stage_bytes);
							const uint64_t desc_b = make_desc_k_sw128(b_base + sb * C::b_stage_bytes);
							if (CTAS == 2)
							{
#pragma unroll
								for (int k = 0; k < 4; k++)
									mma_ss_pair<KIND>(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
								mma_commit_pair(smem_u32(&bars.empty_b[sb])); // frees the stage in both CTAs
							}
							else
							{
#pragma unroll
								for (int k = 0; k < 4; k++)
									mma_ss<KIND>(tmem_d, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
								if (MT == 2)
								{ // the second row tile: next 16 KB of the stage, next BN columns of tensor memory, same weight slice
									const uint64_t desc_a1 = make_desc_k_sw128(smem_base + sa * C::a_stage_bytes + A_STAGE_BYTES);
#pragma unroll
									for (int k = 0; k < 4; k++)
										mma_ss<KIND>(tmem_d + BN, desc_a1 + 2 * k, desc_b + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
								}
								if (C::split)
								{ // x * w = (xh + xl) * (wh + wl) ~ xh * wh + xh * wl + xl * wh  (desc_a names the raw tile: the tensor core reads xh from it)
									const uint64_t lo_a = make_desc_k_sw128(lo_base + (it % C::lo_ring) * C::lo_bytes);
									const uint64_t lo_b = make_desc_k_sw128(b_base + sb * C::b_stage_bytes + BN * 128);
#pragma unroll
									for (int k = 0; k < 4; k++)
										mma_ss<KIND>(tmem_d, desc_a + 2 * k, lo_b + 2 * k, idesc, 1u);
#pragma unroll
									for (int k = 0; k < 4; k++)
										mma_ss<KIND>(tmem_d, lo_a + 2 * k, desc_b + 2 * k, idesc, 1u);
									mma_commit(smem_u32(&bars.lo_empty[it % C::lo_ring]));
								}
								if (!TMA_A)
									mma_commit(smem_u32(&bars.empty_a[sa]));
								mma_commit(smem_u32(&bars.empty_b[sb]));
							}
						}
						if (ok)
						{
							if (CTAS == 2)
								mma_commit_pair(smem_u32(&bars.tmem_full[buf]));
							else
								mma_commit(smem_u32(&bars.tmem_full[buf]));
						}
					}
				}
				__syncwarp();
			}
			else if (warp < 2 + EPI_WARPS)
			{ /* ------------------------------------------------------------ epilogue */
				const int q = warp % 4; // tensor-memory lane quarter
				const int col_part = (warp - 2) / 4; // which share of the BN columns this warp handles
				const uint32_t sbuf = epi_base + (warp - 2) * EPI_WARP_BYTES;
				const int rr = lane / 4, seg = lane % 4; // cooperative access: 8 rows x 4 segments of 16 bytes per instruction
				const bool rows_vectorisable = (p.cout % 8 == 0) && aligned_to_16(p.y) && (p.ext == nullptr || aligned_to_16(p.ext));
				const bool i8_rows_vectorisable = p.out_dtype == DTYPE_INT8 && (p.cout % 16) == 0 && aligned_to_16(p.y) && aligned_to_16(p.scales)
						&& aligned_to_16(p.shifts) && (p.ext == nullptr || aligned_to_16(p.ext));
				uint32_t local_tile = 0;
				for (int unit = first_unit; unit < total_units; unit += unit_step, local_tile++)
				{
					const int nt = unit % n_tiles;
					const uint32_t buf = local_tile & 1u;
					if (!mbar_wait_all_lanes(smem_u32(&bars.tmem_full[buf]), (local_tile >> 1) & 1u, abort_flag))
						break;
					tcgen05_fence_after();
					const int col_begin = col_part * COLS_PER_WARP;
					const int n_valid_tile = min(BN, p.cout - nt * BN);
					constexpr int CHUNKS_PER_WARP = COLS_PER_WARP / 32;
					for (int cc = 0; cc < MT * CHUNKS_PER_WARP; cc++)
					{
						const int sub = cc / CHUNKS_PER_WARP; // which of the unit's row tiles
						const int c = col_begin / 32 + cc % CHUNKS_PER_WARP;
						const int mt = ((unit / n_tiles) * CTAS + static_cast<int>(cta_rank)) * MT + sub;
						const int row0 = mt * BM + q * 32; // first row of this warp
						const int row = row0 + lane;
						const bool row_ok = row < p.M;
						const long long off = static_cast<long long>(row) * p.cout;
						const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * (BN * MT) + sub * BN;
						if (c * 32 >= n_valid_tile)
							continue; // warp-uniform
						const int n0 = nt * BN + c * 32;
						const int n_valid = min(32, p.cout - n0);
						const bool fast = (KIND == 0) && rows_vectorisable && n_valid == 32;

						uint4 res[4];
						if (fast && p.ext != nullptr)
						{ // issue the residual reads before waiting on tensor memory
							const __half *ep = reinterpret_cast<const __half*>(p.ext);
#pragma unroll
							for (int i = 0; i < 4; i++)
							{
								const int r = row0 + rr + 8 * i;
								res[i] = (r < p.M) ? *reinterpret_cast<const uint4*>(ep + static_cast<long long>(r) * p.cout + n0 + seg * 8) : make_uint4(0,
										0, 0, 0);
							}
						}
						const bool fast_i8 = (KIND == 1) && i8_rows_vectorisable && n_valid == 32;
						uint32_t ext_words[8];
						if (fast_i8 && p.ext != nullptr && row_ok)
						{ // likewise: the int8 residual row segment of this lane
							const uint4 *ep = reinterpret_cast<const uint4*>(reinterpret_cast<const int8_t*>(p.ext) + off + n0);
							const uint4 e0 = ep[0], e1 = ep[1];
							ext_words[0] = e0.x; ext_words[1] = e0.y; ext_words[2] = e0.z; ext_words[3] = e0.w;
							ext_words[4] = e1.x; ext_words[5] = e1.y; ext_words[6] = e1.z; ext_words[7] = e1.w;
						}
						uint32_t r[32];
						tmem_ld_32x32(taddr + c * 32, r);
						tmem_wait_ld();
						if (KIND == 1 && p.border != nullptr && row_ok)
						{ /* The copy engine filled positions outside the image with zeros where the host asked for the quantised zero z:
						   * add z * (sum of the weights of the taps that fell outside), which depends only on the kind of position. */
							uint32_t image, pos, ph, pw;
							p.by_board.divmod(static_cast<uint32_t>(row), image, pos);
							p.by_width.divmod(pos, ph, pw);
							const int kind_of_position = (ph == 0 ? 1 : (static_cast<int>(ph) == p.height - 1 ? 2 : 0)) * 3
									+ (pw == 0 ? 1 : (static_cast<int>(pw) == p.width - 1 ? 2 : 0));
							if (kind_of_position != 0)
							{
								const int *bt = p.border + kind_of_position * p.cout + n0;
								if (n_valid == 32 && (p.cout % 4) == 0)
								{ // the table starts on a 16-byte boundary (it is the head of the host's accumulator matrix) and n0 is a multiple of 32
#pragma unroll
									for (int j4 = 0; j4 < 8; j4++)
									{
										const int4 t = reinterpret_cast<const int4*>(bt)[j4];
										r[4 * j4] += static_cast<uint32_t>(t.x);
										r[4 * j4 + 1] += static_cast<uint32_t>(t.y);
										r[4 * j4 + 2] += static_cast<uint32_t>(t.z);
										r[4 * j4 + 3] += static_cast<uint32_t>(t.w);
									}
								}
								else
								{
#pragma unroll
									for (int j = 0; j < 32; j++)
										if (j < n_valid)
											r[j] += static_cast<uint32_t>(bt[j]);
								}
							}
						}

						if (fast)
						{
							float v[32];
#pragma unroll
							for (int j = 0; j < 32; j++)
								v[j] = __uint_as_float(r[j]);
							if (p.bias != nullptr)
							{
								const uint4 *bp = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.bias) + n0);
								if (aligned_to_16(p.bias))
								{
#pragma unroll
									for (int k = 0; k < 4; k++)
										add_half8(v + 8 * k, bp[k]);
								}
								else
								{
									const __half *bs = reinterpret_cast<const __half*>(p.bias) + n0;
#pragma unroll
									for (int j = 0; j < 32; j++)
										v[j] += __half2float(bs[j]);
								}
							}
							if (p.ext != nullptr)
							{ // through shared memory: cooperative layout -> one row per lane
#pragma unroll
								for (int i = 0; i < 4; i++)
									st_shared_v4(sbuf + (rr + 8 * i) * EPI_PITCH + seg * 16, res[i]);
								__syncwarp();
#pragma unroll
								for (int k = 0; k < 4; k++)
									add_half8(v + 8 * k, ld_shared_v4(sbuf + lane * EPI_PITCH + k * 16));
								__syncwarp();
							}
							activate32(v, p.act);
#pragma unroll
							for (int k = 0; k < 4; k++)
								st_shared_v4(sbuf + lane * EPI_PITCH + k * 16, pack_half8(v + 8 * k));
							__syncwarp();
							__half *yp = reinterpret_cast<__half*>(p.y);
#pragma unroll
							for (int i = 0; i < 4; i++)
							{
								const int rg = row0 + rr + 8 * i;
								const uint4 val = ld_shared_v4(sbuf + (rr + 8 * i) * EPI_PITCH + seg * 16);
								if (rg < p.M)
									*reinterpret_cast<uint4*>(yp + static_cast<long long>(rg) * p.cout + n0 + seg * 8) = val;
							}
							__syncwarp();
							continue;
						}

						if (fast_i8)
						{ /* int8 -> int8 fast path.  The arithmetic is the scalar loop of the reference's CPU backend, operation for
						   * operation and without fused multiply-adds (epilogue.cuh: requant_real, requant_add_ext, requant_round) */
							if (!row_ok)
								continue;
							const float4 *sp = reinterpret_cast<const float4*>((q_staged ? qs_s : p.scales) + n0);
							const float4 *hp = reinterpret_cast<const float4*>((q_staged ? qh_s : p.shifts) + n0);
							const bool relu = p.act == ACTIVATION_RELU;
							const bool other_act = p.act == ACTIVATION_SIGMOID || p.act == ACTIVATION_TANH;
							uint32_t packed[8];
#pragma unroll
							for (int g4 = 0; g4 < 8; g4++)
							{
								const float4 sc = sp[g4], sh = hp[g4];
								const float scs[4] = { sc.x, sc.y, sc.z, sc.w }, shs[4] = { sh.x, sh.y, sh.z, sh.w };
								int q4[4];
#pragma unroll
								for (int t = 0; t < 4; t++)
								{
									float x = requant_real(static_cast<int>(r[4 * g4 + t]), scs[t], shs[t]);
									if (p.ext != nullptr)
										x = requant_add_ext(x, static_cast<int>(static_cast<int8_t>((ext_words[g4] >> (8 * t)) & 0xFFu)), p.ext_scale, p.ext_shift);
									if (relu)
										x = fmaxf(x, 0.0f);
									else if (other_act)
										x = activation_out_of_line(x, p.act);
									q4[t] = requant_round(x, p.inv_out_scale, p.inv_out_shift);
								}
								packed[g4] = pack_sat_s8x4(q4[0], q4[1], q4[2], q4[3]);
							}
							int8_t *dp = reinterpret_cast<int8_t*>(p.y) + off + n0;
							*reinterpret_cast<uint4*>(dp) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
							*reinterpret_cast<uint4*>(dp + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
							continue;
						}

						/* general path: one row per lane, any alignment, column tails, and the other int8 output kinds */
						if (!row_ok)
							continue;
						float v[32];
						if (KIND >= 2)
						{ /* fp32 in and out: the lane owns 32 consecutive floats (one 128-byte line) of its row */
#pragma unroll
							for (int j = 0; j < 32; j++)
								v[j] = __uint_as_float(r[j]);
							const float *bp = (p.bias != nullptr) ? reinterpret_cast<const float*>(p.bias) + n0 : nullptr;
							const float *ep = (p.ext != nullptr) ? reinterpret_cast<const float*>(p.ext) + off + n0 : nullptr;
							float *dp = reinterpret_cast<float*>(p.y) + off + n0;
							const bool vec = n_valid == 32 && (p.cout % 4) == 0 && aligned_to_16(p.y) && (bp == nullptr || aligned_to_16(p.bias))
									&& (ep == nullptr || aligned_to_16(p.ext));
							if (vec)
							{
#pragma unroll
								for (int j4 = 0; j4 < 8; j4++)
								{
									float4 t = make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
									if (bp != nullptr)
									{
										const float4 b4 = reinterpret_cast<const float4*>(bp)[j4];
										t.x += b4.x; t.y += b4.y; t.z += b4.z; t.w += b4.w;
									}
									if (ep != nullptr)
									{
										const float4 e4 = reinterpret_cast<const float4*>(ep)[j4];
										t.x += e4.x; t.y += e4.y; t.z += e4.z; t.w += e4.w;
									}
									v[4 * j4] = t.x; v[4 * j4 + 1] = t.y; v[4 * j4 + 2] = t.z; v[4 * j4 + 3] = t.w;
								}
								activate32(v, p.act);
#pragma unroll
								for (int j4 = 0; j4 < 8; j4++)
									reinterpret_cast<float4*>(dp)[j4] = make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
							}
							else
							{
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (j < n_valid)
										v[j] += (bp != nullptr ? bp[j] : 0.0f) + (ep != nullptr ? ep[j] : 0.0f);
								activate32(v, p.act);
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (j < n_valid)
										dp[j] = v[j];
							}
							continue;
						}
						if (KIND == 0)
						{
#pragma unroll
							for (int j = 0; j < 32; j++)
								v[j] = __uint_as_float(r[j]);
							if (p.bias != nullptr)
							{
								const __half *bp = reinterpret_cast<const __half*>(p.bias) + n0;
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (j < n_valid)
										v[j] += __half2float(bp[j]);
							}
							if (p.ext != nullptr)
							{
								const __half *ep = reinterpret_cast<const __half*>(p.ext) + off + n0;
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (j < n_valid)
										v[j] += __half2float(ep[j]);
							}
							activate32(v, p.act);
							__half *dp = reinterpret_cast<__half*>(p.y) + off + n0;
#pragma unroll
							for (int j = 0; j < 32; j++)
								if (j < n_valid)
									dp[j] = __float2half_rn(v[j]);
							continue;
						}
						if (p.out_dtype == DTYPE_INT32)
						{ // raw accumulators
							int *dp = reinterpret_cast<int*>(p.y) + off + n0;
#pragma unroll
							for (int j = 0; j < 32; j++)
								if (j < n_valid)
									dp[j] = static_cast<int>(r[j]);
							continue;
						}
						const int8_t *ep = (p.ext != nullptr) ? reinterpret_cast<const int8_t*>(p.ext) + off + n0 : nullptr;
						const bool act_on = (p.act == ACTIVATION_SIGMOID || p.act == ACTIVATION_TANH || p.act == ACTIVATION_RELU);
						const bool ext_vec = ep != nullptr && n_valid == 32 && (reinterpret_cast<uintptr_t>(ep) % 16) == 0;
						if (ext_vec)
						{
							const uint4 e0 = *reinterpret_cast<const uint4*>(ep), e1 = *reinterpret_cast<const uint4*>(ep + 16);
							ext_words[0] = e0.x; ext_words[1] = e0.y; ext_words[2] = e0.z; ext_words[3] = e0.w;
							ext_words[4] = e1.x; ext_words[5] = e1.y; ext_words[6] = e1.z; ext_words[7] = e1.w;
						}
#pragma unroll
						for (int j = 0; j < 32; j++)
						{
							float x = 0.0f;
							if (j < n_valid)
							{
								x = requant_real(static_cast<int>(r[j]), p.scales[n0 + j], p.shifts[n0 + j]);
								if (ep != nullptr)
								{
									const int e = ext_vec ? static_cast<int>(static_cast<int8_t>((ext_words[j / 4] >> (8 * (j % 4))) & 0xFFu)) : static_cast<int>(ep[j]);
									x = requant_add_ext(x, e, p.ext_scale, p.ext_shift);
								}
							}
							v[j] = x;
						}
						if (act_on)
							activate32(v, p.act);
						if (p.out_dtype == DTYPE_INT8)
						{
							int8_t *dp = reinterpret_cast<int8_t*>(p.y) + off + n0;
							uint32_t packed[8];
#pragma unroll
							for (int j = 0; j < 32; j += 4)
							{
								uint32_t w4 = 0;
#pragma unroll
								for (int t = 0; t < 4; t++)
								{
									const int qv = requant_clamp(requant_round(v[j + t], p.inv_out_scale, p.inv_out_shift));
									w4 |= (static_cast<uint32_t>(qv) & 0xFFu) << (8 * t);
								}
								packed[j / 4] = w4;
							}
							if (n_valid == 32 && (reinterpret_cast<uintptr_t>(dp) % 16) == 0)
							{
								*reinterpret_cast<uint4*>(dp) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
								*reinterpret_cast<uint4*>(dp + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
							}
							else
							{
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (j < n_valid)
										dp[j] = static_cast<int8_t>((packed[j / 4] >> (8 * (j % 4))) & 0xFFu);
							}
						}
						else if (p.out_dtype == DTYPE_FLOAT16)
						{
							__half *dp = reinterpret_cast<__half*>(p.y) + off + n0;
#pragma unroll
							for (int j = 0; j < 32; j++)
								if (j < n_valid)
									dp[j] = __float2half_rn(v[j]);
						}
						else
						{
							float *dp = reinterpret_cast<float*>(p.y) + off + n0;
							if (n_valid == 32 && (reinterpret_cast<uintptr_t>(dp) % 16) == 0)
							{
#pragma unroll
								for (int j = 0; j < 32; j += 4)
									*reinterpret_cast<float4*>(dp + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
							}
							else
							{
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (j < n_valid)
										dp[j] = v[j];
							}
						}
					}
					tcgen05_fence_before();
					__syncwarp();
					if (lane == 0)
					{
						if (CTAS == 2) // the issuing CTA waits for the epilogue warps of both
							mbar_arrive_cluster(map_to_cta(smem_u32(&bars.tmem_empty[buf]), 0));
						else
							mbar_arrive(smem_u32(&bars.tmem_empty[buf]));
					}
				}
			}
			else if (C::split && warp >= 2 + EPI_WARPS)
			{ /* ------------------------------------------------------------ split warps (fp32 at full accuracy): x -> hi (in place) and lo */
				const int t = threadIdx.x - (2 + EPI_WARPS) * 32;
				constexpr int SPLIT_THREADS = (SPLIT_WARPS > 0 ? SPLIT_WARPS : 1) * 32;
				uint32_t it = 0;
				bool ok = true;
				for (int unit = first_unit; unit < total_units && ok; unit += unit_step)
					for (int kb = 0; kb < k_blocks; kb++, it++)
					{
						const int s = it % C::b_stages;
						if (!mbar_wait(smem_u32(&bars.lo_empty[it % C::lo_ring]), ((it / C::lo_ring) & 1u) ^ 1u, abort_flag)
								|| !mbar_wait(smem_u32(&bars.full_b[s]), (it / C::b_stages) & 1u, abort_flag))
						{
							ok = false;
							break;
						}
						// elementwise, so it keeps whatever swizzled layout the copy engine wrote: xl = x - (x truncated to TF32), exact in fp32
						const uint32_t raw_tile = smem_base + s * C::a_stage_bytes;
						const uint32_t lo_tile = lo_base + (it % C::lo_ring) * C::lo_bytes;
						constexpr int PER_THREAD = C::a_stage_bytes / 16 / SPLIT_THREADS;
						uint4 x[PER_THREAD];
#pragma unroll
						for (int u = 0; u < PER_THREAD; u++)
							x[u] = ld_shared_v4(raw_tile + (t + u * SPLIT_THREADS) * 16);
#pragma unroll
						for (int u = 0; u < PER_THREAD; u++)
						{
							uint4 l;
							l.x = __float_as_uint(__uint_as_float(x[u].x) - __uint_as_float(x[u].x & 0xFFFFE000u));
							l.y = __float_as_uint(__uint_as_float(x[u].y) - __uint_as_float(x[u].y & 0xFFFFE000u));
							l.z = __float_as_uint(__uint_as_float(x[u].z) - __uint_as_float(x[u].z & 0xFFFFE000u));
							l.w = __float_as_uint(__uint_as_float(x[u].w) - __uint_as_float(x[u].w & 0xFFFFE000u));
							st_shared_v4(lo_tile + (t + u * SPLIT_THREADS) * 16, l);
						}
						fence_proxy_async_smem(); // plain stores -> visible to the tensor core's reads
						__syncwarp();
						if (lane == 0)
							mbar_arrive(smem_u32(&bars.split[s]));
					}
			}
			else if (!TMA_A && (warp == 10 || warp == 11 || warp == 14 || warp == 15))
			{ /* ------------------------------------------------------------ A-operand gather */
				// The gather warps sit on the two scheduler partitions (warp % 4 = 2, 3) that do not host the MMA-issuing
				// warp, so their address arithmetic never delays a tcgen05.mma issue slot; warps 12 and 13 stay idle.
				const int pt = ((warp < 12) ? (warp - 10) : (warp - 12)) * 32 + lane; // 0..127
				const int j = pt % 8; // 16-byte chunk of the 128-byte K slice
				const int g = pt / 8; // rows g, g + 16, g + 32, ...
				const uint32_t row_byte = static_cast<uint32_t>(g) * 128 + static_cast<uint32_t>((j ^ (g & 7)) * 16);
				const uint8_t *xb = reinterpret_cast<const uint8_t*>(p.x);
				const uint32_t pad_word = static_cast<uint32_t>(p.pad_byte & 0xFF) * 0x01010101u;
				const bool store_pad = (KIND == 1) && (p.pad_byte != 0);
				const int hw = p.height * p.width;
				constexpr int ROWS = BM / 16; // rows per producer thread
				uint32_t it = 0;
				bool ok = true;
				for (int unit = first_unit; unit < total_units && ok; unit += unit_step)
				{
					const int mt = unit / n_tiles;
					uint32_t tap_mask[ROWS]; // bit t set: tap t of this row lies inside the image (0 for a row beyond M)
					int pos_off[ROWS]; // element offset of the position's channel 0
#pragma unroll
					for (int i = 0; i < ROWS; i++)
					{
						const int m = mt * BM + g + 16 * i;
						tap_mask[i] = 0;
						pos_off[i] = 0;
						if (m < p.M)
						{
							const int rem = m % hw;
							const int h = rem / p.width;
							const int w = rem - h * p.width;
							const uint32_t rows_ok = (h > 0 ? 1u : 0u) | 2u | (h + 1 < p.height ? 4u : 0u);
							const uint32_t cols_ok = (w > 0 ? 1u : 0u) | 2u | (w + 1 < p.width ? 4u : 0u);
							tap_mask[i] = ((rows_ok & 1u) ? cols_ok : 0u) | ((rows_ok & 2u) ? (cols_ok << 3) : 0u) | ((rows_ok & 4u) ? (cols_ok << 6) : 0u)
									| (1u << 9); // bit 9: the row exists
							pos_off[i] = m * p.cin;
						}
					}
					for (int kb = 0; kb < k_blocks; kb++, it++)
					{
						const int s = it % C::a_stages;
						if (!mbar_wait(smem_u32(&bars.empty_a[s]), ((it / C::a_stages) & 1u) ^ 1u, abort_flag))
						{
							ok = false;
							break;
						}
						const uint32_t dst0 = smem_base + s * A_STAGE_BYTES + row_byte;
						const int k0 = kb * (128 / ES) + j * CHUNK_ELEMS;
						const bool k_ok = k0 < p.K;
						const int tap = k_ok ? k0 / p.cin : 0;
						const int c0 = k0 - tap * p.cin;
						const int dh = tap / 3 - 1, dw = tap % 3 - 1;
						const int delta = (dh * p.width + dw) * p.cin + c0;
#pragma unroll
						for (int i = 0; i < ROWS; i++)
						{
							const bool inside = k_ok && ((tap_mask[i] >> tap) & 1u);
							const uint32_t dst = dst0 + i * 16 * 128;
							if (store_pad && !inside && k_ok && (tap_mask[i] >> 9))
								st_shared_16(dst, pad_word);
							else // src-size 0 writes 16 zero bytes: padding outside the image, rows beyond M, K tail
								cp_async_16(dst, inside ? xb + static_cast<long long>(pos_off[i] + delta) * ES : xb, inside ? 16u : 0u);
						}
						if (store_pad)
							fence_proxy_async_smem(); // the padding values were plain stores
						// the barrier receives this thread's arrival when its copies above have landed; the thread itself
						// moves on and fills the next free stage
						cp_async_arrive_noinc(smem_u32(&bars.full_a[s]));
					}
				}
				cp_async_wait_all(); // nothing of this thread may still be in flight when the CTA retires
			}

			/* ---------------------------------------------------------------- teardown */
			tcgen05_fence_before();
			if (CTAS == 2)
				cluster_sync(); // neither CTA retires while the other may still signal its barriers or read its operands
			else
				__syncthreads();
			if (bars.abort_flag != 0)
			{
				if (threadIdx.x == 0 && p.status != nullptr)
					atomicExch(p.status, 2);
				__nanosleep(1000000);
			}
			if (warp == 1)
			{
				tcgen05_fence_after();
				tmem_dealloc(tmem_base, C::tmem_columns);
			}
		}

		template<int KIND, int BN, bool TMA_A, int MT = 1>
		bool launch(mlContext_t ctx, const CUtensorMap &map_w, const CUtensorMap &map_x, const ConvParams &p)
		{
			using C = Cfg<KIND, BN, TMA_A, 1, MT>;
			static bool configured_on[MAX_DEVICES] = { false }; // the opt-in is a per-device attribute of the kernel
			static std::mutex configured_mutex; // contexts on several threads may reach a kernel for the first time together
			const int device = get(ctx)->device;
			if (device < 0 || device >= MAX_DEVICES)
				return false;
			std::unique_lock<std::mutex> configured_lock(configured_mutex);
			bool &configured = configured_on[device];
			if (!configured)
			{
				if (!check_cuda(ctx, cudaFuncSetAttribute(kernel_conv3x3_igemm<KIND, BN, TMA_A, 1, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_bytes),
						"conv_igemm: shared memory opt-in"))
					return false;
				configured = true;
			}
			configured_lock.unlock();
			const int tiles = (((p.M + BM - 1) / BM + MT - 1) / MT) * ((p.cout + BN - 1) / BN);
			const int grid = std::min(tiles, get(ctx)->sm_count);
			kernel_conv3x3_igemm<KIND, BN, TMA_A, 1, MT> <<<grid, Roles<KIND, TMA_A>::threads, C::smem_bytes, use_stream(ctx)>>>(map_w, map_x, p);
			MB200_COUNT_LAUNCH();
			get(ctx)->kernels_with_waits = true;
			return check_cuda(ctx, cudaGetLastError(), "conv_igemm launch");
		}

		/* Paired kernel: clusters of two CTAs, as many clusters as the device can hold at once (queried once per device). */
		template<int KIND, int BN>
		bool launch_pair(mlContext_t ctx, const CUtensorMap &map_w, const CUtensorMap &map_x, const ConvParams &p)
		{
			using C = Cfg<KIND, BN, true, 2>;
			static int max_clusters[MAX_DEVICES] = { 0 }; // per device; 0 = not queried yet, -1 = clusters of this size cannot be placed
			static std::mutex max_clusters_mutex;
			std::lock_guard<std::mutex> max_clusters_lock(max_clusters_mutex);
			const int device = get(ctx)->device;
			cudaLaunchConfig_t config;
			std::memset(&config, 0, sizeof(config));
			cudaLaunchAttribute attribute;
			attribute.id = cudaLaunchAttributeClusterDimension;
			attribute.val.clusterDim.x = 2;
			attribute.val.clusterDim.y = 1;
			attribute.val.clusterDim.z = 1;
			config.blockDim = dim3(Roles<KIND, true>::threads, 1, 1);
			config.dynamicSmemBytes = C::smem_bytes;
			config.stream = use_stream(ctx);
			config.attrs = &attribute;
			config.numAttrs = 1;
			if (device < 0 || device >= MAX_DEVICES)
				return false;
			if (max_clusters[device] == 0)
			{
				if (!check_cuda(ctx, cudaFuncSetAttribute(kernel_conv3x3_igemm<KIND, BN, true, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_bytes),
						"conv_igemm pair: shared memory opt-in"))
					return false;
				config.gridDim = dim3(2 * (get(ctx)->sm_count / 2), 1, 1);
				int n = 0;
				if (cudaOccupancyMaxActiveClusters(&n, kernel_conv3x3_igemm<KIND, BN, true, 2, 1>, &config) != cudaSuccess || n <= 0)
				{
					cudaGetLastError();
					n = -1;
				}
				max_clusters[device] = n;
			}
			if (max_clusters[device] < 0)
				return false;
			const int units = (((p.M + BM - 1) / BM + 1) / 2) * ((p.cout + BN - 1) / BN);
			config.gridDim = dim3(2 * std::min(units, max_clusters[device]), 1, 1);
			const cudaError_t status = cudaLaunchKernelEx(&config, kernel_conv3x3_igemm<KIND, BN, true, 2, 1>, map_w, map_x, p);
			MB200_COUNT_LAUNCH();
			get(ctx)->kernels_with_waits = true;
			return check_cuda(ctx, status, "conv_igemm pair launch") && check_cuda(ctx, cudaGetLastError(), "conv_igemm pair launch");
		}

		bool env_flag(const char *name)
		{
			const char *v = std::getenv(name);
			return v != nullptr && v[0] == '1';
		}

		bool shape_ok(int kind, const mlTensor_t &x, int cout, const void *w)
		{
			const int chunk = (kind == 0) ? 8 : (kind == 1) ? 16 : 32; // fp32: copy-engine operand path only, 128 bytes of channels per slice
			if (x.rank != 4 || x.dim[3] % chunk != 0)
				return false;
			if (!aligned_to(x.data, 16) || !aligned_to(w, 16))
				return false;
			const long long m = static_cast<long long>(x.dim[0]) * x.dim[1] * x.dim[2];
			if (m <= 0 || m * std::max(x.dim[3], cout) >= (1LL << 31))
				return false;
			if (x.dim[1] >= 32768 || x.dim[2] >= 32768)
				return false;
			return true;
		}

		/* im2col-mode tensor map over x [n, h, w, c]: one request delivers 128 consecutive output positions x 128 bytes of
		 * channels for one filter tap, walking w, then h, then n, with zeros outside the image.  For a 3x3 filter with padding 1
		 * the base pixel of output (p, q) is (q - 1, p - 1): lower corner -1, upper corner -1, tap offsets 0..2. */
		bool encode_im2col_map(mlContext_t ctx, CUtensorMap *map, int kind, const mlTensor_t &x)
		{
			typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*,
					const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
					CUtensorMapFloatOOBfill);
			static encode_fn fn = []() -> encode_fn
			{
				void *ptr = nullptr;
				cudaDriverEntryPointQueryResult result;
				if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &ptr, cudaEnableDefault, &result) != cudaSuccess || ptr == nullptr)
				{
					cudaGetLastError();
					return nullptr;
				}
				return reinterpret_cast<encode_fn>(ptr);
			}();
			if (fn == nullptr)
			{
				record_error(ctx, "cuTensorMapEncodeIm2col is not available from the driver");
				return false;
			}
			const int es = (kind == 0) ? 2 : (kind == 1) ? 1 : 4;
			const cuuint64_t dims[4] = { static_cast<cuuint64_t>(x.dim[3]), static_cast<cuuint64_t>(x.dim[2]), static_cast<cuuint64_t>(x.dim[1]),
					static_cast<cuuint64_t>(x.dim[0]) };
			const cuuint64_t strides[3] = { static_cast<cuuint64_t>(x.dim[3]) * es, static_cast<cuuint64_t>(x.dim[3]) * es * x.dim[2],
					static_cast<cuuint64_t>(x.dim[3]) * es * x.dim[2] * x.dim[1] };
			const int lower[2] = { -1, -1 };
			const int upper[2] = { -1, -1 };
			const cuuint32_t traversal[4] = { 1, 1, 1, 1 };
			const CUresult status = fn(map, kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : (kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32), 4, x.data, dims, strides,
					lower, upper, static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(BM), traversal, CU_TENSOR_MAP_INTERLEAVE_NONE,
					CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
			if (status != CUDA_SUCCESS)
			{
				record_error(ctx, "cuTensorMapEncodeIm2col failed with code %d", static_cast<int>(status));
				return false;
			}
			// Drivers up to CUDA 13.1 encode im2col maps of tensors smaller than 128 KiB with a flag (bit 21 of the second
			// descriptor word) that must be cleared -- the same adjustment CUTLASS applies after this call.
			int driver_version = 0;
			if (cudaDriverGetVersion(&driver_version) == cudaSuccess && driver_version <= 13010
					&& volume(x) * es < 131072)
				reinterpret_cast<uint64_t*>(map)[1] &= ~(1ull << 21);
			return true;
		}

		/* table[kind][co] = pad * sum over the taps outside the image for that kind of position of sum_ci w[co][tap][ci];
		 * one CTA per output channel, one warp per tap. */
		__global__ void __launch_bounds__(9 * 32) kernel_border_table(int *__restrict__ table, const int8_t *__restrict__ w, int cin, int cout, int pad)
		{
			__shared__ int tap_sum[9];
			const int co = blockIdx.x, tap = threadIdx.x / 32, lane = threadIdx.x % 32;
			const int8_t *src = w + (static_cast<long long>(co) * 9 + tap) * cin;
			int s = 0;
			for (int i = lane; i < cin; i += 32)
				s += src[i];
			for (int k = 16; k >= 1; k /= 2)
				s += __shfl_xor_sync(0xffffffffu, s, k);
			if (lane == 0)
				tap_sum[tap] = s;
			__syncthreads();
			if (threadIdx.x < 9)
			{
				const int hk = threadIdx.x / 3, wk = threadIdx.x % 3; // 0 inner, 1 first, 2 last row / column
				int total = 0;
				for (int kh = 0; kh < 3; kh++)
					for (int kw = 0; kw < 3; kw++)
					{
						const bool outside = (hk == 1 && kh == 0) || (hk == 2 && kh == 2) || (wk == 1 && kw == 0) || (wk == 2 && kw == 2);
						if (outside)
							total += tap_sum[kh * 3 + kw];
					}
				table[threadIdx.x * cout + co] = total * pad;
			}
		}

		/* kind 3 expects `w` to be the two planes [2, cout, 9 cin] written by kernel_split_weight_planes */
		/* Border corrections of asymmetric int8 layers, kept per weight tensor: the table depends only on the weights and on the
		 * padding value, so it is computed once (the first call of a layer) into memory the library owns and reused by every later
		 * call; conv_forget_range drops an entry when the weights are freed or written to through the ABI.  A first call that
		 * arrives while its stream is being captured into a CUDA graph may not allocate: it computes the table into the caller's
		 * accumulator scratch, as every call did before the cache existed. */
		struct BorderRecord
		{
				int *table;
				size_t weight_bytes;
				int pad, cin, cout, device;
		};
		std::mutex g_border_mutex;
		std::map<const void*, BorderRecord> g_border_tables;

		const int* cached_border_table(mlContext_t ctx, const void *w, int cin, int cout, int pad)
		{
			Context *c = get(ctx);
			std::lock_guard<std::mutex> lock(g_border_mutex);
			auto it = g_border_tables.find(w);
			if (it != g_border_tables.end())
			{
				const BorderRecord &rec = it->second;
				if (rec.pad == pad && rec.cin == cin && rec.cout == cout && rec.device == c->device)
					return rec.table;
				cudaFree(rec.table); // the same address now holds other weights, or the layer is used with another zero point
				g_border_tables.erase(it);
			}
			cudaStream_t stream = use_stream(ctx);
			cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
			if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone)
			{
				cudaGetLastError();
				return nullptr;
			}
			int *table = nullptr;
			if (cudaMalloc(reinterpret_cast<void**>(&table), static_cast<size_t>(9) * cout * sizeof(int)) != cudaSuccess)
			{
				cudaGetLastError();
				return nullptr;
			}
			kernel_border_table<<<cout, 9 * 32, 0, stream>>>(table, reinterpret_cast<const int8_t*>(w), cin, cout, pad);
			MB200_COUNT_LAUNCH();
			g_border_tables[w] = BorderRecord { table, static_cast<size_t>(9) * cin * cout, pad, cin, cout, c->device };
			return table;
		}

		bool run(mlContext_t ctx, int kind, const mlTensor_t &x, const void *w, int cout, ConvParams p)
		{
			const int es = (kind == 0) ? 2 : (kind == 1) ? 1 : 4;
			p.x = x.data;
			p.batch = x.dim[0];
			p.height = x.dim[1];
			p.width = x.dim[2];
			p.cin = x.dim[3];
			p.cout = cout;
			p.M = x.dim[0] * x.dim[1] * x.dim[2];
			p.K = 9 * x.dim[3];
			p.status = get(ctx)->dev_status;
			p.by_board = FastDiv(static_cast<uint32_t>(p.height) * p.width);
			p.by_width = FastDiv(static_cast<uint32_t>(p.width));
			const int bn = (cout > 128 && kind != 3) ? 256 : 128;
			/* A operand by im2col TMA when each 128-byte K slice stays inside one tap and the padding value is zero */
			static const bool force_gather = env_flag("MINML_B200_CONV_GATHER"); // measurement switches: each forces the slower variant
			static const bool force_single = env_flag("MINML_B200_CONV_SINGLE_CTA");
			// (int8 with a non-zero padding value: still by TMA when the caller supplied room for the border corrections)
			const bool zero_fill_ok = p.pad_byte == 0 || (kind == 1 && p.border != nullptr && p.height >= 2 && p.width >= 2);
			const bool tma_a = (p.cin * es) % 128 == 0 && zero_fill_ok && (!force_gather || kind >= 2); // (fp32 has the copy-engine path only)
			if (tma_a && p.pad_byte != 0)
			{
				const int *cached = cached_border_table(ctx, w, p.cin, cout, p.pad_byte);
				if (cached != nullptr)
					p.border = cached;
				else
				{ // no cached table could be made (the stream is being captured, or no memory): this call's own, in the host's scratch
					kernel_border_table<<<cout, 9 * 32, 0, use_stream(ctx)>>>(const_cast<int*>(p.border), reinterpret_cast<const int8_t*>(w), p.cin, cout,
							p.pad_byte);
					MB200_COUNT_LAUNCH();
				}
			}
			else
				p.border = nullptr; // the gather variant stores the padding value itself
			// Pairs pay off where the operand fetch is the limit (256-column tiles: 0.383 -> 0.353 ms on the 256 -> 256 layer); with
			// 128-column tiles the epilogue is, and coupling two CTAs' accumulator hand-offs costs more than it saves (measured).
			static const bool force_pair = env_flag("MINML_B200_CONV_PAIR");
			const bool pair = kind < 2 && tma_a && !force_single && (bn == 256 || force_pair) && p.M > BM && get(ctx)->sm_count >= 2;
			CUtensorMap map_w;
			const uint64_t dims[3] = { static_cast<uint64_t>(p.K), static_cast<uint64_t>(cout), static_cast<uint64_t>(kind == 3 ? 2 : 1) };
			const uint64_t strides[2] = { static_cast<uint64_t>(p.K) * es, static_cast<uint64_t>(p.K) * es * cout };
			const uint32_t box[3] = { static_cast<uint32_t>(128 / es), static_cast<uint32_t>(pair ? bn / 2 : bn), 1 };
			if (!encode_tensor_map(ctx, &map_w, kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : (kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32),
					3, w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
				return false;
			CUtensorMap map_x;
			std::memset(&map_x, 0, sizeof(map_x));
			if (tma_a && !encode_im2col_map(ctx, &map_x, kind, x))
				return false;
			if (kind >= 2)
			{ // fp32: one TF32 product when the host allowed it on this context, three products of split operands otherwise
				if (!tma_a)
					return false;
				if (kind == 2)
					return bn == 256 ? launch<2, 256, true>(ctx, map_w, map_x, p) : launch<2, 128, true>(ctx, map_w, map_x, p);
				return launch<3, 128, true>(ctx, map_w, map_x, p);
			}
			if (pair)
			{
				if (kind == 0)
					return bn == 256 ? launch_pair<0, 256>(ctx, map_w, map_x, p) : launch_pair<0, 128>(ctx, map_w, map_x, p);
				return bn == 256 ? launch_pair<1, 256>(ctx, map_w, map_x, p) : launch_pair<1, 128>(ctx, map_w, map_x, p);
			}
			static const bool force_narrow = env_flag("MINML_B200_CONV_ONE_ROW_TILE");
			const bool wide = tma_a && bn == 128 && !force_narrow && p.M > 2 * BM * get(ctx)->sm_count; // enough work for 256-row units on every SM
			if (wide)
				return kind == 0 ? launch<0, 128, true, 2>(ctx, map_w, map_x, p) : launch<1, 128, true, 2>(ctx, map_w, map_x, p);
			if (kind == 0)
			{
				if (tma_a)
					return bn == 256 ? launch<0, 256, true>(ctx, map_w, map_x, p) : launch<0, 128, true>(ctx, map_w, map_x, p);
				return bn == 256 ? launch<0, 256, false>(ctx, map_w, map_x, p) : launch<0, 128, false>(ctx, map_w, map_x, p);
			}
			if (tma_a)
				return bn == 256 ? launch<1, 256, true>(ctx, map_w, map_x, p) : launch<1, 128, true>(ctx, map_w, map_x, p);
			return bn == 256 ? launch<1, 256, false>(ctx, map_w, map_x, p) : launch<1, 128, false>(ctx, map_w, map_x, p);
		}
	}

	namespace
	{
		/* fp32 convolutions by the fused kernel: always with TF32 permission (one product per slice: 0.70 ms against the Winograd
		 * path's 1.50 ms on a 1024 x 20 x 20 x 256 -> 256 layer).  At full fp32 accuracy (three products per slice, fp32 operands
		 * streamed from L2 at twice the bytes of fp16) only for layers of up to 128 channels, where one launch measured 3 - 17 %
		 * faster than the Winograd path's three (64 x 15 x 15: 31.8 against 38.2 us; 512 x 20 x 20: 0.288 against 0.315 ms); at 256
		 * channels F(4x4,3x3), which does a quarter of the multiply-adds, wins (0.40 against 0.53 ms).
		 * MINML_B200_FP32_FUSED=always|never overrides the rule (measurement switch). */
		bool fp32_fused_wanted(mlContext_t ctx, const mlTensor_t &x, int cout)
		{
			static const char *mode = std::getenv("MINML_B200_FP32_FUSED");
			if (mode != nullptr && mode[0] == 'n')
				return false;
			if (get(ctx)->allow_tf32 || (mode != nullptr && mode[0] == 'a'))
				return true;
			return x.dim[3] <= 128 && cout <= 128;
		}
	}
	void conv_forget_range(const void *ptr, size_t bytes)
	{
		std::lock_guard<std::mutex> lock(g_border_mutex);
		if (g_border_tables.empty())
			return;
		const uint8_t *lo = reinterpret_cast<const uint8_t*>(ptr);
		const uint8_t *hi = lo + std::max<size_t>(bytes, 1);
		for (auto it = g_border_tables.begin(); it != g_border_tables.end();)
		{
			const uint8_t *w = reinterpret_cast<const uint8_t*>(it->first);
			if (w < hi && lo < w + it->second.weight_bytes)
			{
				int current = 0;
				cudaGetDevice(&current);
				cudaSetDevice(it->second.device);
				cudaFree(it->second.table);
				cudaSetDevice(current);
				it = g_border_tables.erase(it);
			}
			else
				++it;
		}
	}
	bool conv_fused_input_supported(mlContext_t ctx, const mlTensor_t &x)
	{
		if (x.dtype == DTYPE_FLOAT32)
			return shape_ok(2, x, 1, x.data) && fp32_fused_wanted(ctx, x, 1);
		return x.dtype == DTYPE_FLOAT16 && shape_ok(0, x, 1, x.data);
	}
	bool conv_fused_weights_supported(const mlTensor_t &w)
	{
		if (w.dtype == DTYPE_FLOAT32)
			return w.rank == 4 && w.dim[3] % 32 == 0;
		return w.dtype == DTYPE_FLOAT16 && w.rank == 4 && w.dim[3] % 8 == 0;
	}
	bool conv_fused_supported(mlContext_t ctx, const mlTensor_t &x, const mlTensor_t &w, const mlTensor_t &y, mlActivationType_t act)
	{
		(void) act;
		if ((x.dtype != DTYPE_FLOAT16 && x.dtype != DTYPE_FLOAT32) || w.dtype != x.dtype || y.dtype != x.dtype)
			return false;
		if (w.rank != 4 || w.dim[1] != 3 || w.dim[2] != 3 || w.dim[3] != x.dim[3])
			return false;
		if (x.dtype == DTYPE_FLOAT32)
			return shape_ok(2, x, w.dim[0], w.data) && aligned_to(y.data, 4) && fp32_fused_wanted(ctx, x, w.dim[0]);
		return shape_ok(0, x, w.dim[0], w.data) && aligned_to(y.data, 2);
	}
	size_t conv_fused_weight_bytes(const mlTensor_t &w)
	{
		return static_cast<size_t>(volume(w)) * size_of(w.dtype) * (w.dtype == DTYPE_FLOAT32 ? 2 : 1);
	}
	bool conv_fused_prepare_weights(mlContext_t ctx, const mlTensor_t &w, void *prepared)
	{
		cudaStream_t stream = use_stream(ctx);
		if (w.dtype != DTYPE_FLOAT32)
			return check_cuda(ctx, cudaMemcpyAsync(prepared, w.data, conv_fused_weight_bytes(w), cudaMemcpyDeviceToDevice, stream), "weight snapshot");
		const long long elements = volume(w);
		const int grid = static_cast<int>(std::min<long long>((elements + 255) / 256, static_cast<long long>(get(ctx)->sm_count) * 8));
		kernel_split_weight_planes<<<grid, 256, 0, stream>>>(reinterpret_cast<float*>(prepared), reinterpret_cast<const float*>(w.data), elements);
		MB200_COUNT_LAUNCH();
		return check_cuda(ctx, cudaGetLastError(), "weight planes");
	}
	bool conv_fused_run(mlContext_t ctx, const mlTensor_t &x, const mlTensor_t &w, const void *bias, const void *ext, const mlTensor_t &y,
			mlActivationType_t act, bool prepared)
	{
		if (conv_slab_supported(x, w, y)) // MINML_B200_CONV_SLAB=1 only: the variant with the input band resident in shared memory (conv_slab.cu)
			return conv_slab_run(ctx, x, w, bias, ext, y, act);
		ConvParams p;
		std::memset(&p, 0, sizeof(p));
		p.y = y.data;
		p.bias = bias;
		p.ext = ext;
		p.act = act;
		p.out_dtype = x.dtype;
		const int kind = (x.dtype == DTYPE_FLOAT16) ? 0 : (get(ctx)->allow_tf32 ? 2 : 3);
		const void *weights = w.data;
		if (kind == 3 && !prepared)
		{ // raw fp32 weights handed over per call (the single-call entry): their two planes go to the context's scratch first
			void *planes = get_workspace(ctx, conv_fused_weight_bytes(w));
			if (planes == nullptr || !conv_fused_prepare_weights(ctx, w, planes))
				return false;
			weights = planes;
		}
		return run(ctx, kind, x, weights, w.dim[0], p); // (kind 2 on prepared weights reads plane 0: the properly rounded TF32 values)
	}

	/* ------------------------------------------------------------------------------------------------------------
	 * Deferred int8 sequence: im2row (recorded) -> int8 GEMM (recorded) -> scale_shift_act (launches the fused kernel).
	 * ---------------------------------------------------------------------------------------------------------- */
	bool im2row_defer(mlContext_t ctx, mlDataType_t dtype, const mlShape_t &input_shape, void *output, const void *input, int kernel_size,
			bool invert, const void *padding)
	{
		Context *c = get(ctx);
		if (c == nullptr || !c->fusion || dtype != DTYPE_INT8 || kernel_size != 3 || invert)
			return false;
		const mlTensor_t x = make_tensor(input, DTYPE_INT8, input_shape);
		if (!shape_ok(1, x, 1, input))
			return false;
		std::lock_guard<std::recursive_mutex> lock(c->mutex);
		flush_pending(ctx);
		c->pending_i8.stage = 1;
		c->pending_i8.x = x;
		c->pending_i8.rows = output;
		c->pending_i8.pad = (padding == nullptr) ? 0 : *reinterpret_cast<const int8_t*>(padding);
		return true;
	}
	bool int8_gemm_defer(mlContext_t ctx, char opA, char opB, const mlTensor_t &A, const mlTensor_t &B, const mlTensor_t &C)
	{
		Context *c = get(ctx);
		if (c == nullptr)
			return false;
		std::lock_guard<std::recursive_mutex> lock(c->mutex);
		if (c->pending_i8.stage != 1)
			return false;
		if (is_transpose(opA) || !is_transpose(opB) || A.data != c->pending_i8.rows || A.dtype != DTYPE_INT8 || B.dtype != DTYPE_INT8
				|| C.dtype != DTYPE_INT32 || A.rank != 2 || B.rank != 2 || C.rank != 2)
			return false;
		const mlTensor_t &x = c->pending_i8.x;
		if (B.dim[1] != 9 * x.dim[3] || A.dim[1] != B.dim[1] || C.dim[1] != B.dim[0] || !aligned_to(B.data, 16))
			return false;
		c->pending_i8.stage = 2;
		c->pending_i8.w = B;
		c->pending_i8.acc = C;
		return true;
	}
	bool requant_complete_fused(mlContext_t ctx, mlDataType_t dtype, const mlShape_t &shape, void *output, mlQuantizationData_t output_qd,
			const void *input, const void *scales, const void *bias, mlActivationType_t act, const void *ext, mlQuantizationData_t ext_qd)
	{
		Context *c = get(ctx);
		if (c == nullptr)
			return false;
		std::lock_guard<std::recursive_mutex> lock(c->mutex);
		if (c->pending_i8.stage != 2 || input != c->pending_i8.acc.data)
			return false;
		if (dtype != DTYPE_INT8 && dtype != DTYPE_FLOAT16 && dtype != DTYPE_FLOAT32)
			return false;
		const mlTensor_t x = c->pending_i8.x;
		const int cout = c->pending_i8.w.dim[0];
		if (volume(shape) != static_cast<long long>(x.dim[0]) * x.dim[1] * x.dim[2] * cout || last_dim(shape) != cout)
			return false;
		ConvParams p;
		std::memset(&p, 0, sizeof(p));
		p.y = output;
		p.ext = ext;
		p.act = act;
		p.out_dtype = dtype;
		p.scales = reinterpret_cast<const float*>(scales);
		p.shifts = reinterpret_cast<const float*>(bias);
		p.ext_scale = ext_qd.scale;
		p.ext_shift = ext_qd.shift;
		// (the output transform reaches the kernel as its inverse, below)
		p.inv_out_scale = 1.0f / output_qd.scale;
		p.inv_out_shift = -output_qd.shift / output_qd.scale;
		p.pad_byte = c->pending_i8.pad;
		// the int32 matrix the host set aside for the accumulators is not written by the fused kernel: its first 9 x cout words
		// hold the border corrections when the padding value is not zero
		if (p.pad_byte != 0 && volume(c->pending_i8.acc) >= 9LL * cout && aligned_to(c->pending_i8.acc.data, 16))
			p.border = reinterpret_cast<const int*>(c->pending_i8.acc.data);
		c->pending_i8.stage = 0;
		return run(ctx, 1, x, c->pending_i8.w.data, cout, p);
	}
	void flush_pending_int8(mlContext_t ctx)
	{
		Context *c = get(ctx);
		if (c == nullptr)
			return;
		std::lock_guard<std::recursive_mutex> lock(c->mutex);
		if (c->pending_i8.stage == 0)
			return;
		const PendingInt8 pend = c->pending_i8;
		c->pending_i8.stage = 0;
		const bool fusion = c->fusion;
		c->fusion = false;
		const int8_t pad = static_cast<int8_t>(pend.pad);
		cuda_im2row(ctx, DTYPE_INT8, shape_of(pend.x), pend.rows, pend.x.data, 3, false, &pad);
		if (pend.stage == 2)
		{
			mlTensor_t a = make_tensor(pend.rows, DTYPE_INT8, make_shape( { pend.acc.dim[0], pend.w.dim[1] }));
			cuda_gemm_v2(ctx, 'n', 't', 1.0f, a, pend.w, 0.0f, pend.acc);
		}
		c->fusion = fusion;
	}
} /* namespace mb200 */
