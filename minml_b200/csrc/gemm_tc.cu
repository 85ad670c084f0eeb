/*
 * gemm_tc.cu -- the tensor-core GEMM of the backend: D[b] = epilogue(alpha * op(A[b]) * op(B[b]) + beta * C[b]).
 *
 * Serves every 'n','t' matrix product of the inference path (reference call sites: the 36 batched Winograd
 * products of Conv2D::forward, src/layers/Conv2D.cpp:371; 1x1 convolutions and dense layers through gemm_ex,
 * src/core/math.cpp:682-702; the int8 -> int32 product of the quantised path, src/layers/Conv2D.cpp:232) and,
 * for fp16 and fp32 operands, the other transpositions (the 'n','n' and 't','n' products of Conv2D::backward,
 * src/layers/Conv2D.cpp:383-448), which the reference sends to cuBLAS (src/backend/cuda/gemms.cpp:99-259).
 *
 * Design (one CTA per SM, persistent over output tiles of 128 x BN):
 *   warp 0      TMA producer: A and B tiles (128 bytes of K per row, 128B swizzle) into a ring of shared-memory stages
 *   warp 1      issues tcgen05.mma (one elected lane); owns the tensor-memory allocation
 *   warps 2-9   epilogue (two warps per tensor-memory lane quarter, each half of the tile's columns): tcgen05.ld of the
 *               fp32 / s32 accumulators, alpha/beta/bias/activation or requantisation.  fp16 results (and the fp16 C operand)
 *               are staged through shared memory so that one global access covers 8 rows x 64 contiguous bytes.  Two
 *               accumulator buffers in tensor memory let the epilogue of tile i overlap the main loop of tile i+1.
 * An operand stored [rows, K] ('n' on A, 't' on B) is K-major for the tensor core; one stored [K, rows] ('t' on A, 'n' on B) is
 * fetched in boxes of [K slice x 128 bytes of rows] and read as an MN-major operand (descriptor strides and, for 32-bit
 * elements, the swizzle in 32-byte pieces: make_desc_mn_sw128 in tc.cuh).  8-bit operands are K-major only.  K tails and M/N
 * tails are zero-filled by TMA.  Measured on the 36 batched products of a 256-channel layer over 25 600 tiles, fp16:
 * 'n','t' 0.159 ms, 'n','n' 0.166 ms, 't','n' 0.168 ms (0.87 - 0.92 of the copy bandwidth; the CUDA-core engine that served the
 * transposed forms before reached 41 TFLOP/s against 720 here).
 */
#include "common.cuh"
#include "tc.cuh"
#include "gemm.cuh"
#include "epilogue.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace mb200
{
	bool encode_tensor_map(void *ctx, CUtensorMap *map, CUtensorMapDataType dtype, int rank, const void *base, const uint64_t *dims,
			const uint64_t *strides_bytes, const uint32_t *box, CUtensorMapSwizzle swizzle)
	{
		typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
				const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
				CUtensorMapFloatOOBfill);
		static encode_fn fn = []() -> encode_fn
		{
			void *ptr = nullptr;
			cudaDriverEntryPointQueryResult result;
			if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess || ptr == nullptr)
			{
				cudaGetLastError();
				return nullptr;
			}
			return reinterpret_cast<encode_fn>(ptr);
		}();
		if (fn == nullptr)
		{
			record_error(ctx, "cuTensorMapEncodeTiled is not available from the driver");
			return false;
		}
		cuuint32_t element_strides[5] = { 1, 1, 1, 1, 1 };
		cuuint64_t gdims[5];
		cuuint64_t gstrides[5];
		cuuint32_t gbox[5];
		for (int i = 0; i < rank; i++)
		{
			gdims[i] = dims[i];
			gbox[i] = box[i];
			if (i + 1 < rank)
				gstrides[i] = strides_bytes[i];
		}
		const CUresult status = fn(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox, element_strides,
				CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
		if (status != CUDA_SUCCESS)
		{
			record_error(ctx, "cuTensorMapEncodeTiled failed with code %d (rank %d, dims %llu x %llu)", static_cast<int>(status), rank,
					static_cast<unsigned long long>(dims[0]), static_cast<unsigned long long>(rank > 1 ? dims[1] : 0));
			return false;
		}
		return true;
	}

	namespace
	{
		using namespace tc;
		using namespace epi;

		constexpr int BM = 128;
		constexpr int BK_BYTES = 128; // one swizzle row: 64 fp16 or 128 int8
		constexpr int EPI_WARPS = 8;
		constexpr int SPLIT_WARPS = 4; // only in the split-fp32 kernel
		constexpr int num_threads(int kind)
		{
			return (2 + EPI_WARPS + (kind == 3 ? SPLIT_WARPS : 0)) * 32;
		}

		/*
		 * KIND 3 multiplies fp32 operands at (nearly) fp32 accuracy on the TF32 tensor cores: every element x is split in shared
		 * memory into hi = x rounded to a TF32 number (low 13 mantissa bits clear) and lo = x - hi (exact in fp32), and
		 * the product is accumulated as hi*hi + hi*lo + lo*hi in fp32. The dropped lo*lo term and the truncation of lo to TF32
		 * are both of relative size 2^-21, a little above the 2^-24 of an fp32 multiply and far below TF32's 2^-11. The landed
		 * tile is overwritten with hi; lo goes to a ring of its own, two deep, which only has to live from the split to the end
		 * of that slice's products, so most of shared memory stays with the copies in flight (the kernel streams fp32 operands
		 * and is short of bytes in flight before it is short of anything else). It has no use for the epilogue staging.
		 */
		/*
		 * RES (weight-resident): for products with a short K -- the 1x1 convolutions and dense layers of a network, K = 256 ... 512 --
		 * a 128 x BN tile is only a few K slices, and fetching the weight tile again for every 128 rows of output made the copies
		 * into shared memory, not HBM, the limit (l1tex 62 % of peak, tensor pipe 30 %).  Here every CTA takes a CONTIGUOUS range of
		 * tiles ordered (batch, column tile, row tile), keeps the whole [BN, K] weight tile in shared memory for as long as
		 * consecutive tiles share it, streams only A through the ring, and moves C and D as 32 x 32 boxes through tensor maps (see the
		 * epilogue below).  What paces these products is still the epilogue of each SM, not a chip-wide limit: the same product on 135,
		 * 74 and 37 CTAs takes 0.040, 0.063 and 0.110 ms, i.e. 3.6, 3.1 and 2.9 us per 128 x 256 tile and CTA -- were the memory system the
		 * limit, half the CTAs would have finished in nearly the same time.  (That a tile's 64 KB of D every 5 000 cycles on 135 SMs
		 * comes to the 3.3 TB/s a write-only kernel reaches on this GPU is a coincidence that was first read as the cause.)  About a
		 * fifth of the tile time at full occupancy is contention; the rest is the chain of a 32-column chunk, 1 100 - 1 200 cycles
		 * against 512 of tensor work.
		 * Measured, 57 600 rows, K = 256 (staged epilogue -> box epilogue -> its chunk loop unrolled by two instead of whole, which took
		 * the kernel's instruction-fetch stalls down: ncu had one stalled warp per issued instruction on `no instruction`): N = 768 0.043 ->
		 * 0.040 -> 0.037 ms, N = 256 with a residual 0.031 -> 0.025 -> 0.023 ms, N = 1024 with ReLU 0.055 -> 0.052 -> 0.049 ms; the 36 Winograd products
		 * of a 256-channel layer 0.167 -> 0.159 ms with the resident weights alone (0.92 of the copy bandwidth).
		 */
		constexpr int RESIDENT_BYTES = 128 * 1024;
		template<int KIND, int BN, bool RES = false, bool BOX = false>
		struct Tiling
		{
				static constexpr bool split = (KIND == 3);
				static constexpr int a_bytes = BM * BK_BYTES, b_bytes = BN * BK_BYTES;
				static constexpr int operand_bytes = a_bytes + b_bytes;
				static constexpr int stage_bytes = RES ? a_bytes : operand_bytes;
				static constexpr int stages = RES ? (BOX ? 3 : 4) : split ? ((BN == 256) ? 3 : 5) : ((BN == 256) ? 4 : 6);
				static constexpr int resident_offset = stages * stage_bytes;
				static constexpr int lo_stages = split ? ((BN == 256) ? 1 : 2) : 0;
				static constexpr int lo_ring = (lo_stages > 0) ? lo_stages : 1; // divisor that is never zero
				static constexpr int lo_offset = resident_offset + (RES ? RESIDENT_BYTES : 0);
				static constexpr int staging_offset = lo_offset + lo_stages * operand_bytes;
				static constexpr int box_bytes = 32 * 64; // RES: a 32-row x 32-column fp16 box of C or D, 64-byte swizzle
				static constexpr int boxes = 3; // per epilogue warp: D of two chunks in flight, C of the next chunk
				static constexpr int staging_bytes = split ? 0 : BOX ? EPI_WARPS * boxes * box_bytes : EPI_WARPS * epi::WARP_BYTES;
				static constexpr int smem_bytes = staging_offset + staging_bytes + 1024;
				static constexpr int tmem_columns = 2 * BN; // two accumulator buffers
		};

		struct Barriers
		{
				uint64_t full[6];
				uint64_t empty[6];
				uint64_t split[6]; // KIND 3: the stage's hi and lo tiles are written
				uint64_t lo_empty[2]; // KIND 3: the products that read this lo tile are done
				uint64_t resident_full, resident_empty; // RES: the weight tile has landed / every product that reads it is done
				uint64_t tmem_full[2];
				uint64_t tmem_empty[2];
				uint64_t c_full[EPI_WARPS][3]; // RES: the box of C has landed (one ring of three per epilogue warp)
				uint32_t tmem_base;
				int abort_flag;
		};

		/* hi = x rounded to the nearest TF32 number (13 low mantissa bits clear); lo = x - hi (exact, either sign, so the
		 * truncation of lo by the tensor core does not bias the sum). An infinite x turns into NaN in the product (inf * 0 in
		 * the cross terms) where fp32 arithmetic would give an infinity. */
		__device__ __forceinline__ void split_tf32(uint32_t x, uint32_t &hi, uint32_t &lo)
		{
			hi = (x + 0x1000u) & 0xFFFFE000u;
			lo = __float_as_uint(__uint_as_float(x) - __uint_as_float(hi));
		}

		// (requantisation arithmetic: epilogue.cuh)

		template<int KIND, int BN, bool RES = false, bool BOX = false>
		__global__ void __launch_bounds__(num_threads(KIND), 1) kernel_gemm_tc(const __grid_constant__ CUtensorMap map_a,
				const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_d,
				const GemmTcParams p)
		{
			static_assert(!RES || KIND == 0, "the weight-resident variant is built for fp16");
			static_assert(!BOX || RES, "the box epilogue belongs to the weight-resident variant");
			using T = Tiling<KIND, BN, RES, BOX>;
			extern __shared__ uint8_t smem_raw[];
			__shared__ Barriers bars;

			const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
			const int warp = threadIdx.x / 32;
			const int lane = threadIdx.x % 32;

			const int m_tiles = (p.M + BM - 1) / BM;
			const int n_tiles = (p.N + BN - 1) / BN;
			const long long total_tiles = static_cast<long long>(m_tiles) * n_tiles * p.batch;
			constexpr int ES = (KIND == 0) ? 2 : (KIND == 1 ? 1 : 4); // operand element size
			const int elems_per_kblock = 128 / ES; // 128 bytes of K per row (or, MN-major, 128 bytes of rows per K index)
			const int k_blocks = (p.K + elems_per_kblock - 1) / elems_per_kblock;
			// Which tiles this CTA computes: every gridDim-th one, or (RES) a contiguous range, so that consecutive tiles share weights.
			const long long per_cta = (total_tiles + gridDim.x - 1) / gridDim.x;
			const long long tile_first = RES ? blockIdx.x * per_cta : blockIdx.x;
			const long long tile_last = RES ? min(total_tiles, tile_first + per_cta) : total_tiles;
			const long long tile_step = RES ? 1 : gridDim.x;
			// Position of a tile -- column tile, row tile, batch item -- kept by increments: every role walks the same sequence, and a
			// 64-bit division per tile and role was a tenth of a short-K tile's time.
			struct Walk
			{
					int nt, mt, b;
			};
			const long long per_item = static_cast<long long>(n_tiles) * m_tiles;
			const int step_b = static_cast<int>(tile_step / per_item), step_rest = static_cast<int>(tile_step % per_item);
			const int step_mt = RES ? 0 : step_rest / n_tiles, step_nt = RES ? 0 : step_rest % n_tiles;
			auto start = [&]() -> Walk
			{
				Walk w;
				const long long rest = tile_first % per_item;
				w.b = static_cast<int>(tile_first / per_item);
				if (RES)
				{ // row tiles fastest: a column tile's weights stay while the rows go by
					w.mt = static_cast<int>(rest % m_tiles);
					w.nt = static_cast<int>(rest / m_tiles);
				}
				else
				{
					w.nt = static_cast<int>(rest % n_tiles);
					w.mt = static_cast<int>(rest / n_tiles);
				}
				return w;
			};
			auto advance = [&](Walk &w)
			{
				if (RES)
				{ // one tile on
					if (++w.mt == m_tiles)
					{
						w.mt = 0;
						if (++w.nt == n_tiles)
						{
							w.nt = 0;
							w.b++;
						}
					}
				}
				else
				{ // gridDim.x tiles on
					w.nt += step_nt;
					if (w.nt >= n_tiles)
					{
						w.nt -= n_tiles;
						w.mt++;
					}
					w.mt += step_mt;
					if (w.mt >= m_tiles)
					{
						w.mt -= m_tiles;
						w.b++;
					}
					w.b += step_b;
				}
			};

			if (threadIdx.x == 0)
			{
				for (int s = 0; s < T::stages; s++)
				{
					mbar_init(smem_u32(&bars.full[s]), 1);
					mbar_init(smem_u32(&bars.empty[s]), 1);
					mbar_init(smem_u32(&bars.split[s]), SPLIT_WARPS);
				}
				for (int a = 0; a < 2; a++)
				{
					mbar_init(smem_u32(&bars.lo_empty[a]), 1);
					mbar_init(smem_u32(&bars.tmem_full[a]), 1);
					mbar_init(smem_u32(&bars.tmem_empty[a]), EPI_WARPS);
				}
				mbar_init(smem_u32(&bars.resident_full), 1);
				mbar_init(smem_u32(&bars.resident_empty), 1);
				for (int e = 0; e < EPI_WARPS; e++)
					for (int k = 0; k < 3; k++)
						mbar_init(smem_u32(&bars.c_full[e][k]), 1);
				bars.abort_flag = 0;
				fence_mbar_init();
			}
			if (warp == 1)
			{
				tmem_alloc(smem_u32(&bars.tmem_base), T::tmem_columns);
				tmem_relinquish();
			}
			tcgen05_fence_before();
			__syncthreads();
			tcgen05_fence_after();
			const uint32_t tmem_base = bars.tmem_base;
			volatile int *abort_flag = &bars.abort_flag;

			if (warp == 0)
			{ /* ------------------------------------------------ TMA producer */
				if (elect_one())
				{
					prefetch_tensormap(&map_a);
					prefetch_tensormap(&map_b);
					uint32_t it = 0;
					bool ok = true;
					long long weights_loaded = -1; // RES: which weight tile shared memory holds
					uint32_t weight_loads = 0;
					Walk w = start();
					for (long long tile = tile_first; tile < tile_last && ok; tile += tile_step, advance(w))
					{
						const int nt = w.nt, mt = w.mt, b = w.b;
						const long long weights = static_cast<long long>(p.b_broadcast ? 0 : b) * n_tiles + nt;
						if (RES && weights != weights_loaded)
						{ // a new weight tile: once every product on the old one is done, all its K slices in one go
							if (!mbar_wait(smem_u32(&bars.resident_empty), (weight_loads & 1u) ^ 1u, abort_flag))
								break;
							const uint32_t full = smem_u32(&bars.resident_full);
							mbar_arrive_expect_tx(full, static_cast<uint32_t>(k_blocks) * T::b_bytes);
							for (int kb = 0; kb < k_blocks; kb++)
								tma_load_3d(smem_base + T::resident_offset + kb * T::b_bytes, &map_b, full, kb * elems_per_kblock, nt * BN, p.b_broadcast ? 0 : b);
							weights_loaded = weights;
							weight_loads++;
						}
						for (int kb = 0; kb < k_blocks; kb++, it++)
						{
							const int s = it % T::stages;
							const uint32_t parity = ((it / T::stages) & 1u) ^ 1u;
							if (!mbar_wait(smem_u32(&bars.empty[s]), parity, abort_flag))
							{
								ok = false;
								break;
							}
							const uint32_t full = smem_u32(&bars.full[s]);
							mbar_arrive_expect_tx(full, T::stage_bytes);
							const uint32_t dst_a = smem_base + s * T::stage_bytes;
							// K-major operand: one box of [rows x 128 bytes of K]; MN-major operand (stored [K, rows]): one box of
							// [K slice x 128 bytes of rows] per 128 bytes of rows, one after the other
							if (!RES && p.a_mn)
							{
#pragma unroll
								for (int j = 0; j < BM * ES / 128; j++)
									tma_load_3d(dst_a + j * (T::a_bytes / (BM * ES / 128)), &map_a, full, mt * BM + j * elems_per_kblock, kb * elems_per_kblock,
											p.a_broadcast ? 0 : b);
							}
							else
								tma_load_3d(dst_a, &map_a, full, kb * elems_per_kblock, mt * BM, p.a_broadcast ? 0 : b);
							if (!RES && p.b_mn)
							{
#pragma unroll
								for (int j = 0; j < BN * ES / 128; j++)
									tma_load_3d(dst_a + T::a_bytes + j * (T::b_bytes / (BN * ES / 128)), &map_b, full, nt * BN + j * elems_per_kblock,
											kb * elems_per_kblock, p.b_broadcast ? 0 : b);
							}
							else if (!RES)
								tma_load_3d(dst_a + T::a_bytes, &map_b, full, kb * elems_per_kblock, nt * BN, p.b_broadcast ? 0 : b);
						}
					}
				}
				__syncwarp();
			}
			else if (warp == 1)
			{ /* ------------------------------------------- MMA issuer */
				if (elect_one())
				{
					const uint32_t idesc = ((KIND == 0) ? make_idesc_f16(BN) : (KIND == 1 ? make_idesc_i8(BN) : make_idesc_tf32(BN)))
							| (p.a_mn ? (1u << 15) : 0u) | (p.b_mn ? (1u << 16) : 0u);
					// descriptor step per instruction (in 16-byte units): 32 bytes along K for a K-major operand, one instruction's K indices
					// (16 fp16 or 8 fp32) times 128 bytes for an MN-major one
					const uint32_t step_a = p.a_mn ? (32 / ES) * 128 / 16 : 2, step_b = p.b_mn ? (32 / ES) * 128 / 16 : 2;
					const uint32_t block_a = T::a_bytes / (BM * ES / 128), block_b = T::b_bytes / (BN * ES / 128);
					uint64_t *const ready = T::split ? bars.split : bars.full; // what the tensor core may read
					uint32_t it = 0;
					uint32_t local_tile = 0;
					bool ok = true;
					long long weights_loaded = -1;
					uint32_t weight_loads = 0;
					Walk w = start();
					for (long long tile = tile_first; tile < tile_last && ok; tile += tile_step, local_tile++, advance(w))
					{
						if (RES)
						{
							const int nt = w.nt, b = w.b;
							const long long weights = static_cast<long long>(p.b_broadcast ? 0 : b) * n_tiles + nt;
							if (weights != weights_loaded)
							{
								if (weight_loads > 0)
									mma_commit(smem_u32(&bars.resident_empty)); // arrives when every product issued so far, all on the old tile, is done
								if (!mbar_wait(smem_u32(&bars.resident_full), (weight_loads & 1u), abort_flag))
									break;
								weights_loaded = weights;
								weight_loads++;
							}
						}
						const uint32_t acc = local_tile & 1u;
						const uint32_t acc_parity = ((local_tile >> 1) & 1u) ^ 1u;
						if (!mbar_wait(smem_u32(&bars.tmem_empty[acc]), acc_parity, abort_flag))
							break;
						tcgen05_fence_after();
						const uint32_t tmem_d = tmem_base + acc * BN;
						for (int kb = 0; kb < k_blocks; kb++, it++)
						{
							const int s = it % T::stages;
							const uint32_t parity = (it / T::stages) & 1u;
							if (!mbar_wait(smem_u32(&ready[s]), parity, abort_flag))
							{
								ok = false;
								break;
							}
							tcgen05_fence_after();
							if (T::split)
								fence_proxy_async_smem(); // the hi and lo tiles were plain stores of the split warps
							const uint32_t addr_a = smem_base + s * T::stage_bytes;
							const uint32_t addr_b = RES ? smem_base + T::resident_offset + kb * T::b_bytes : addr_a + T::a_bytes;
							const uint64_t desc_a = p.a_mn ? make_desc_mn_sw128(addr_a, block_a, KIND >= 2) : make_desc_k_sw128(addr_a);
							const uint64_t desc_b = p.b_mn ? make_desc_mn_sw128(addr_b, block_b, KIND >= 2) : make_desc_k_sw128(addr_b);
#pragma unroll
							for (int k = 0; k < 4; k++) // 4 instructions per stage: 32 bytes of K each
								mma_ss<KIND>(tmem_d, desc_a + step_a * k, desc_b + step_b * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
							if (T::split)
							{
								const uint32_t lo = smem_base + T::lo_offset + (it % T::lo_ring) * T::operand_bytes;
								const uint64_t lo_a = p.a_mn ? make_desc_mn_sw128(lo, block_a, KIND >= 2) : make_desc_k_sw128(lo);
								const uint64_t lo_b = p.b_mn ? make_desc_mn_sw128(lo + BM * BK_BYTES, block_b, KIND >= 2) : make_desc_k_sw128(lo + BM * BK_BYTES);
#pragma unroll
								for (int k = 0; k < 4; k++)
									mma_ss<KIND>(tmem_d, desc_a + step_a * k, lo_b + step_b * k, idesc, 1u);
#pragma unroll
								for (int k = 0; k < 4; k++)
									mma_ss<KIND>(tmem_d, lo_a + step_a * k, desc_b + step_b * k, idesc, 1u);
								mma_commit(smem_u32(&bars.lo_empty[it % T::lo_ring]));
							}
							mma_commit(smem_u32(&bars.empty[s]));
						}
						if (ok)
							mma_commit(smem_u32(&bars.tmem_full[acc]));
					}
				}
				__syncwarp();
			}
			else if (T::split && warp >= 2 + EPI_WARPS)
			{ /* ------------------------------------------- split warps (KIND 3): x -> hi (in place) and lo */
				const int t = threadIdx.x - (2 + EPI_WARPS) * 32;
				uint32_t it = 0;
				bool ok = true;
				for (long long tile = tile_first; tile < tile_last && ok; tile += tile_step)
					for (int kb = 0; kb < k_blocks; kb++, it++)
					{
						const int s = it % T::stages;
						if (!mbar_wait(smem_u32(&bars.lo_empty[it % T::lo_ring]), ((it / T::lo_ring) & 1u) ^ 1u, abort_flag)
								|| !mbar_wait(smem_u32(&bars.full[s]), (it / T::stages) & 1u, abort_flag))
						{
							ok = false;
							break;
						}
						// the split is elementwise, so it keeps whatever swizzled layout the copy engine wrote
						const uint32_t hi = smem_base + s * T::stage_bytes;
						const uint32_t lo = smem_base + T::lo_offset + (it % T::lo_ring) * T::operand_bytes;
						constexpr int PER_THREAD = T::operand_bytes / 16 / (SPLIT_WARPS * 32);
						constexpr int GROUP = 8; // loads issued back to back before the first is used
						static_assert(PER_THREAD % GROUP == 0, "the split loop assumes whole groups");
#pragma unroll 1
						for (int g = 0; g < PER_THREAD; g += GROUP)
						{
							uint4 x[GROUP];
#pragma unroll
							for (int u = 0; u < GROUP; u++)
								x[u] = ld_shared_v4(hi + (t + (g + u) * SPLIT_WARPS * 32) * 16);
#pragma unroll
							for (int u = 0; u < GROUP; u++)
							{
								uint4 h, l;
								split_tf32(x[u].x, h.x, l.x);
								split_tf32(x[u].y, h.y, l.y);
								split_tf32(x[u].z, h.z, l.z);
								split_tf32(x[u].w, h.w, l.w);
								st_shared_v4(hi + (t + (g + u) * SPLIT_WARPS * 32) * 16, h);
								st_shared_v4(lo + (t + (g + u) * SPLIT_WARPS * 32) * 16, l);
							}
						}
						fence_proxy_async_smem(); // plain stores -> visible to the tensor core's reads
						__syncwarp();
						if (lane == 0)
							mbar_arrive(smem_u32(&bars.split[s]));
					}
			}
			else if (BOX)
			{ /* ------------------------------------------------------------ box epilogue of the weight-resident variant
			   * fp16 D (and C) whose rows start on 16-byte boundaries, which the host checks before it picks this epilogue.  A tile of
			   * a short-K product is a few K slices, so the epilogue sets the pace; here it is kept to what only it can do:
			   *   - chunks of 32 columns with the next chunk's tcgen05.ld in flight under the arithmetic of the current one, and the
			   *     accumulator buffer handed back as soon as the tile's last chunk is in registers;
			   *   - C arrives and D leaves as 32 x 32 boxes through TMA (64-byte swizzle, so that a lane's 64-byte row goes in and out
			   *     of shared memory without bank conflicts): no cooperative re-layout, no per-row address arithmetic, tails clipped
			   *     by the tensor map.  Three boxes per warp rotate: chunk n's D leaves from box n % 3 while chunk n + 1's C lands
			   *     in box (n + 1) % 3, which chunk n - 2's store has finished reading (cp.async.bulk.wait_group.read 1). */
				const int e = warp - 2; // epilogue warp
				const int q = warp % 4; // tensor-memory lane quarter this warp may read
				const int col_part = e / 4; // which half of the tile's columns
				constexpr int NCH = BN / 64; // chunks of 32 columns per warp and tile
				const uint32_t boxes = smem_base + T::staging_offset + e * T::boxes * T::box_bytes;
				const bool use_c = p.beta != 0.0f && p.C != nullptr;
				// a lane's row inside a box: four 16-byte pieces, piece k at (k ^ ((lane >> 1) & 3))
				uint32_t piece[4];
#pragma unroll
				for (int k = 0; k < 4; k++)
					piece[k] = lane * 64 + ((k ^ ((lane >> 1) & 3)) * 16);
				auto active_chunks = [&](const Walk &w) -> int
				{ // of this warp in tile w: chunks whose first column exists
					const int n_valid_tile = min(BN, p.N - w.nt * BN);
					return max(0, min(NCH, (n_valid_tile - col_part * (BN / 2) + 31) / 32));
				};
				auto issue_c = [&](const Walk &w, int i, uint32_t n)
				{ // lane 0: chunk i of tile w is this warp's n-th chunk
					const uint32_t bar = smem_u32(&bars.c_full[e][n % 3]);
					mbar_arrive_expect_tx(bar, T::box_bytes);
					tma_load_3d(boxes + (n % 3) * T::box_bytes, &map_c, bar, w.nt * BN + col_part * (BN / 2) + i * 32, w.mt * BM + q * 32, w.b);
				};
				uint32_t local_tile = 0, n = 0, c_issued = 0; // chunks done, boxes of C asked for (both warp-uniform)
				Walk w = start();
				for (long long tile = tile_first; tile < tile_last; tile += tile_step, local_tile++, advance(w))
				{
					Walk next = w;
					advance(next);
					const bool has_next = tile + tile_step < tile_last;
					const int chunks = active_chunks(w);
					if (use_c && chunks > 0 && c_issued == n)
					{ // nothing asked for this tile's first chunk yet (the first tile, or a tile after one without chunks for this warp)
						if (lane == 0)
						{
							bulk_wait_group_read<1>();
							issue_c(w, 0, n);
						}
						c_issued++;
					}
					const uint32_t acc = local_tile & 1u;
					const uint32_t acc_parity = (local_tile >> 1) & 1u;
					if (!mbar_wait_warp(smem_u32(&bars.tmem_full[acc]), acc_parity, abort_flag, 20u))
						break;
					tcgen05_fence_after();
					const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + col_part * (BN / 2);
					uint32_t r[2][32];
					if (chunks > 0)
						tmem_ld_32x32(taddr, r[0]);
					bool ok = true;
					// two chunks per trip of the loop (one per register buffer): the four-chunk body unrolled whole was twice the code, and ncu had the
					// kernel's warps stalled on instruction fetch (`no instruction`) once per issued instruction
#pragma unroll 1
					for (int ip = 0; ip < NCH && ok; ip += 2)
#pragma unroll
					for (int j = 0; j < 2; j++)
					{
						const int i = ip + j;
						if (i >= chunks)
							break; // warp-uniform
						tmem_wait_ld();
						if (i + 1 < chunks)
							tmem_ld_32x32(taddr + (i + 1) * 32, r[(j + 1) & 1]);
						else
						{ // the tile's accumulators are all in registers: the issue warp may have the buffer back
							tcgen05_fence_before();
							__syncwarp();
							if (lane == 0)
								mbar_arrive(smem_u32(&bars.tmem_empty[acc]));
						}
						// the box after this chunk's is free once chunk n - 2's store has read it; C of the next chunk goes there
						const bool more_here = i + 1 < chunks;
						const bool more_next = !more_here && has_next && active_chunks(next) > 0;
						if (lane == 0)
						{
							bulk_wait_group_read<1>();
							if (use_c && c_issued == n + 1 && (more_here || more_next))
								issue_c(more_here ? w : next, more_here ? i + 1 : 0, n + 1);
						}
						if (use_c && c_issued == n + 1 && (more_here || more_next))
							c_issued++;
						__syncwarp();

						const int n0 = w.nt * BN + col_part * (BN / 2) + i * 32;
						const uint32_t box = boxes + (n % 3) * T::box_bytes;
						float v[32];
						const uint32_t (&ri)[32] = r[j];
#pragma unroll
						for (int j = 0; j < 32; j++)
							v[j] = __uint_as_float(ri[j]) * p.alpha;
						if (use_c)
						{
							if (!mbar_wait_warp(smem_u32(&bars.c_full[e][n % 3]), (n / 3) & 1u, abort_flag, 20u))
							{
								ok = false;
								break;
							}
#pragma unroll
							for (int k = 0; k < 4; k++)
								add_half8(v + 8 * k, ld_shared_v4(box + piece[k]), p.beta);
							__syncwarp(); // every lane has read its row of C before D goes into the same box
						}
						if (p.bias != nullptr)
						{
							const __half *bs = reinterpret_cast<const __half*>(p.bias) + n0;
							if (n0 + 32 <= p.N && aligned_to_16(bs))
							{
#pragma unroll
								for (int k = 0; k < 4; k++)
									add_half8(v + 8 * k, reinterpret_cast<const uint4*>(bs)[k]);
							}
							else
							{
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (n0 + j < p.N)
										v[j] += __half2float(bs[j]);
							}
						}
						activate32(v, p.act);
#pragma unroll
						for (int k = 0; k < 4; k++)
							st_shared_v4(box + piece[k], pack_half8(v + 8 * k));
						fence_proxy_async_smem(); // plain stores, read by the copy engine
						__syncwarp();
						if (lane == 0)
						{
							tma_store_3d(&map_d, box, n0, w.mt * BM + q * 32, w.b);
							bulk_commit_group();
						}
						n++;
					}
					if (!ok)
						break;
					if (chunks == 0)
					{ // nothing of this tile is this warp's: hand the buffer back
						tcgen05_fence_before();
						__syncwarp();
						if (lane == 0)
							mbar_arrive(smem_u32(&bars.tmem_empty[acc]));
					}
				}
				if (lane == 0)
					bulk_wait_group_read<0>(); // shared memory stays until the last store has read it
				__syncwarp();
			}
			else
			{ /* ------------------------------------------------------------ epilogue */
				const int q = warp % 4; // tensor-memory lane quarter this warp may read
				const int col_part = (warp - 2) / 4; // which half of the tile's columns
				const uint32_t sbuf = smem_base + T::staging_offset + (warp - 2) * epi::WARP_BYTES; // fp16 fast path only
				const int rr = lane / 4, seg = lane % 4; // cooperative access: 8 rows x 4 segments of 16 bytes per instruction
				const bool use_c = p.beta != 0.0f && p.C != nullptr;
				// fp16 rows can be moved in 16-byte pieces when every row (of every batch item) starts on a 16-byte boundary
				const bool rows_vectorisable = (KIND == 0) && p.out_dtype == DTYPE_FLOAT16 && aligned_to_16(p.D) && (p.ldd % 8) == 0
						&& (p.stride_d % 8) == 0 && (!use_c || (aligned_to_16(p.C) && (p.ldc % 8) == 0 && (p.stride_c % 8) == 0));
				uint32_t local_tile = 0;
				Walk w = start();
				for (long long tile = tile_first; tile < tile_last; tile += tile_step, local_tile++, advance(w))
				{
					const int nt = w.nt, mt = w.mt, b = w.b;
					const uint32_t acc = local_tile & 1u;
					const uint32_t acc_parity = (local_tile >> 1) & 1u;
					if (!mbar_wait_all_lanes(smem_u32(&bars.tmem_full[acc]), acc_parity, abort_flag))
						break;
					tcgen05_fence_after();

					const int row0 = mt * BM + q * 32;
					const int row = row0 + lane;
					const bool row_ok = row < p.M;
					const long long d_off = static_cast<long long>(b) * p.stride_d + static_cast<long long>(row) * p.ldd;
					const long long c_off = static_cast<long long>(b) * p.stride_c + static_cast<long long>(row) * p.ldc;
					const int n_valid_tile = min(BN, p.N - nt * BN);

					for (int c = col_part * (BN / 64); c < (col_part + 1) * (BN / 64); c++)
					{
						if (c * 32 >= n_valid_tile)
							break; // warp-uniform
						const int n0 = nt * BN + c * 32;
						const int n_valid = min(32, p.N - n0);
						const bool fast = rows_vectorisable && n_valid == 32;
						uint4 res[4];
						if (fast && use_c)
						{ // issue the reads of C before waiting on tensor memory
							const __half *cp = reinterpret_cast<const __half*>(p.C) + static_cast<long long>(b) * p.stride_c;
#pragma unroll
							for (int i = 0; i < 4; i++)
							{
								const int rg = row0 + rr + 8 * i;
								res[i] = (rg < p.M) ? *reinterpret_cast<const uint4*>(cp + static_cast<long long>(rg) * p.ldc + n0 + seg * 8) : make_uint4(0, 0,
										0, 0);
							}
						}
						uint32_t r[32];
						tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32, r);
						tmem_wait_ld();
						float v[32];
						if (fast)
						{
#pragma unroll
							for (int j = 0; j < 32; j++)
								v[j] = __uint_as_float(r[j]) * p.alpha;
							if (use_c)
							{ // through shared memory: cooperative layout -> one row per lane
#pragma unroll
								for (int i = 0; i < 4; i++)
									st_shared_v4(sbuf + (rr + 8 * i) * epi::PITCH + seg * 16, res[i]);
								__syncwarp();
#pragma unroll
								for (int k = 0; k < 4; k++)
									add_half8(v + 8 * k, ld_shared_v4(sbuf + lane * epi::PITCH + k * 16), p.beta);
								__syncwarp();
							}
							if (p.bias != nullptr)
							{
								const __half *bs = reinterpret_cast<const __half*>(p.bias) + n0;
								if (aligned_to_16(bs))
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
							activate32(v, p.act);
#pragma unroll
							for (int k = 0; k < 4; k++)
								st_shared_v4(sbuf + lane * epi::PITCH + k * 16, pack_half8(v + 8 * k));
							__syncwarp();
							__half *dp = reinterpret_cast<__half*>(p.D) + static_cast<long long>(b) * p.stride_d;
#pragma unroll
							for (int i = 0; i < 4; i++)
							{
								const int rg = row0 + rr + 8 * i;
								const uint4 val = ld_shared_v4(sbuf + (rr + 8 * i) * epi::PITCH + seg * 16);
								if (rg < p.M)
									*reinterpret_cast<uint4*>(dp + static_cast<long long>(rg) * p.ldd + n0 + seg * 8) = val;
							}
							__syncwarp();
							continue;
						}
						if (!row_ok)
							continue;
						if (KIND == 0 || KIND >= 2)
						{
#pragma unroll
							for (int j = 0; j < 32; j++)
								v[j] = __uint_as_float(r[j]) * p.alpha;
							if (p.beta != 0.0f && p.C != nullptr)
							{
								if (p.out_dtype == DTYPE_FLOAT16)
								{
									const __half *cp = reinterpret_cast<const __half*>(p.C) + c_off + n0;
#pragma unroll
									for (int j = 0; j < 32; j++)
										if (j < n_valid)
											v[j] += p.beta * __half2float(cp[j]);
								}
								else
								{
									const float *cp = reinterpret_cast<const float*>(p.C) + c_off + n0;
#pragma unroll
									for (int j = 0; j < 32; j++)
										if (j < n_valid)
											v[j] += p.beta * cp[j];
								}
							}
							if (p.bias != nullptr)
							{
								if (p.out_dtype == DTYPE_FLOAT16)
								{
									const __half *bp = reinterpret_cast<const __half*>(p.bias) + n0;
#pragma unroll
									for (int j = 0; j < 32; j++)
										if (j < n_valid)
											v[j] += __half2float(bp[j]);
								}
								else
								{
									const float *bp = reinterpret_cast<const float*>(p.bias) + n0;
#pragma unroll
									for (int j = 0; j < 32; j++)
										if (j < n_valid)
											v[j] += bp[j];
								}
							}
							activate32(v, p.act);
						}
						else if (p.out_dtype != DTYPE_INT32)
						{ // fused requantisation: x = acc * scale[n] + shift[n] (+ dequantised ext), activation
							const int8_t *ep = (p.ext != nullptr) ? p.ext + c_off + n0 : nullptr;
#pragma unroll
							for (int j = 0; j < 32; j++)
								if (j < n_valid)
								{
									float x = requant_real(static_cast<int>(r[j]), p.scales[n0 + j], p.shifts[n0 + j]);
									if (ep != nullptr)
										x = requant_add_ext(x, static_cast<int>(ep[j]), p.ext_scale, p.ext_shift);
									v[j] = x;
								}
							if (p.act == ACTIVATION_SIGMOID || p.act == ACTIVATION_TANH || p.act == ACTIVATION_RELU)
								activate32(v, p.act);
						}

						if (p.out_dtype == DTYPE_FLOAT16)
						{
							__half *dp = reinterpret_cast<__half*>(p.D) + d_off + n0;
							if (n_valid == 32 && (reinterpret_cast<uintptr_t>(dp) % 16) == 0)
							{
#pragma unroll
								for (int j = 0; j < 32; j += 8)
								{
									uint4 pk;
									__half2 h0 = __floats2half2_rn(v[j + 0], v[j + 1]);
									__half2 h1 = __floats2half2_rn(v[j + 2], v[j + 3]);
									__half2 h2 = __floats2half2_rn(v[j + 4], v[j + 5]);
									__half2 h3 = __floats2half2_rn(v[j + 6], v[j + 7]);
									pk.x = *reinterpret_cast<uint32_t*>(&h0);
									pk.y = *reinterpret_cast<uint32_t*>(&h1);
									pk.z = *reinterpret_cast<uint32_t*>(&h2);
									pk.w = *reinterpret_cast<uint32_t*>(&h3);
									*reinterpret_cast<uint4*>(dp + j) = pk;
								}
							}
							else
							{
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (j < n_valid)
										dp[j] = __float2half_rn(v[j]);
							}
						}
						else if (p.out_dtype == DTYPE_FLOAT32)
						{
							float *dp = reinterpret_cast<float*>(p.D) + d_off + n0;
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
						else if (p.out_dtype == DTYPE_INT32)
						{
							int *dp = reinterpret_cast<int*>(p.D) + d_off + n0;
							if (n_valid == 32 && (reinterpret_cast<uintptr_t>(dp) % 16) == 0)
							{
#pragma unroll
								for (int j = 0; j < 32; j += 4)
									*reinterpret_cast<uint4*>(dp + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
							}
							else
							{
#pragma unroll
								for (int j = 0; j < 32; j++)
									if (j < n_valid)
										dp[j] = static_cast<int>(r[j]);
							}
						}
						else if (p.out_dtype == DTYPE_INT8)
						{
							int8_t *dp = reinterpret_cast<int8_t*>(p.D) + d_off + n0;
#pragma unroll
							for (int j = 0; j < 32; j++)
								if (j < n_valid)
									dp[j] = static_cast<int8_t>(requant_clamp(requant_round(v[j], p.inv_out_scale, p.inv_out_shift)));
						}
					}
					tcgen05_fence_before();
					__syncwarp();
					if (lane == 0)
						mbar_arrive(smem_u32(&bars.tmem_empty[acc]));
				}
			}

			/* ---------------------------------------------------------------- teardown */
			tcgen05_fence_before();
			__syncthreads();
			if (bars.abort_flag != 0)
			{
				if (threadIdx.x == 0 && p.status != nullptr)
					atomicExch(p.status, 1);
				__nanosleep(1000000); // give copies that are still in flight time to land before the CTA retires
			}
			if (warp == 1)
			{
				tcgen05_fence_after();
				tmem_dealloc(tmem_base, T::tmem_columns);
			}
		}

		template<int KIND, int BN, bool RES = false, bool BOX = false>
		bool launch(mlContext_t ctx, cudaStream_t stream, const CUtensorMap &map_a, const CUtensorMap &map_b, const CUtensorMap &map_c,
				const CUtensorMap &map_d, const GemmTcParams &p, int sm_count)
		{
			using T = Tiling<KIND, BN, RES, BOX>;
			static bool configured_on[MAX_DEVICES] = { false }; // the opt-in is a per-device attribute of the kernel
			const int device = get(ctx)->device;
			if (device < 0 || device >= MAX_DEVICES)
				return false;
			bool &configured = configured_on[device];
			if (!configured)
			{
				if (!check_cuda(ctx,
						cudaFuncSetAttribute(kernel_gemm_tc<KIND, BN, RES, BOX>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::smem_bytes),
						"gemm_tc: shared memory opt-in"))
					return false;
				configured = true;
			}
			const long long tiles = static_cast<long long>((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch;
			const int grid = static_cast<int>(std::min<long long>(tiles, sm_count));
			kernel_gemm_tc<KIND, BN, RES, BOX> <<<grid, num_threads(KIND), T::smem_bytes, stream>>>(map_a, map_b, map_c, map_d, p);
			MB200_COUNT_LAUNCH();
			return check_cuda(ctx, cudaGetLastError(), "gemm_tc launch");
		}
	}

	bool gemm_tc_supported(const GemmTcProblem &g)
	{
		if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.batch <= 0)
			return false;
		if (g.kind == 1 && (g.a_mn || g.b_mn))
			return false; // 8-bit operands are K-major only
		const int elem = (g.kind == 0) ? 2 : (g.kind == 1 ? 1 : 4);
		// TMA: 16-byte aligned bases and row strides
		if (!aligned_to(g.A, 16) || !aligned_to(g.B, 16))
			return false;
		if ((static_cast<long long>(g.lda) * elem) % 16 != 0 || (static_cast<long long>(g.ldb) * elem) % 16 != 0)
			return false;
		if (g.batch > 1)
		{
			if (g.stride_a != 0 && (g.stride_a * elem) % 16 != 0)
				return false;
			if (g.stride_b != 0 && (g.stride_b * elem) % 16 != 0)
				return false;
		}
		if (g.kind == 0 && g.out_dtype != DTYPE_FLOAT16 && g.out_dtype != DTYPE_FLOAT32)
			return false;
		if (g.kind >= 2 && g.out_dtype != DTYPE_FLOAT32)
			return false;
		if (g.kind == 1 && g.out_dtype != DTYPE_INT32 && g.out_dtype != DTYPE_INT8 && g.out_dtype != DTYPE_FLOAT16
				&& g.out_dtype != DTYPE_FLOAT32)
			return false;
		return true;
	}

	bool gemm_tc_run(mlContext_t ctx, const GemmTcProblem &g)
	{
		Context *c = get(ctx);
		cudaStream_t stream = use_stream(ctx);
		const int elem = (g.kind == 0) ? 2 : (g.kind == 1 ? 1 : 4);
		const CUtensorMapDataType dt = (g.kind == 0) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
				: (g.kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
		// the split-fp32 kernel is bound by shared-memory bandwidth either way; 256-wide tiles (three landing stages, one lo
		// buffer) measured no faster than 128-wide ones (five and two)
		const int bn = (g.N > 128 && g.kind != 3) ? 256 : 128;
		const uint32_t box_k = 128 / elem;

		const bool a_bcast = (g.batch > 1 && g.stride_a == 0);
		const bool b_bcast = (g.batch > 1 && g.stride_b == 0);
		CUtensorMap map_a, map_b;
		// an operand stored [rows, K] is fetched in boxes of [rows of the tile x 128 bytes of K]; one stored [K, rows] (MN-major for the
		// tensor core) in boxes of [one K slice x 128 bytes of rows]
		auto encode_operand = [&](CUtensorMap *map, const void *base, bool mn, int rows, int tile_rows, int ld, long long stride, bool bcast) -> bool
		{
			const uint64_t inner = static_cast<uint64_t>(mn ? rows : g.K), outer = static_cast<uint64_t>(mn ? g.K : rows);
			const uint64_t dims[3] = { inner, outer, static_cast<uint64_t>((bcast || g.batch == 1) ? 1 : g.batch) };
			const uint64_t strides[2] = { static_cast<uint64_t>(ld) * elem, (bcast || g.batch == 1) ? static_cast<uint64_t>(ld) * elem * outer
					: static_cast<uint64_t>(stride) * elem };
			const uint32_t box[3] = { box_k, mn ? box_k : static_cast<uint32_t>(tile_rows), 1 };
			// 32-bit elements in this order need the swizzle in 32-byte pieces
			return encode_tensor_map(ctx, map, dt, 3, base, dims, strides, box, (mn && elem == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B);
		};
		if (!encode_operand(&map_a, g.A, g.a_mn, g.M, BM, g.lda, g.stride_a, a_bcast) || !encode_operand(&map_b, g.B, g.b_mn, g.N, bn, g.ldb, g.stride_b, b_bcast))
			return false;
		GemmTcParams p;
		std::memset(&p, 0, sizeof(p));
		p.M = g.M;
		p.N = g.N;
		p.K = g.K;
		p.batch = g.batch;
		p.a_mn = g.a_mn ? 1 : 0;
		p.b_mn = g.b_mn ? 1 : 0;
		p.a_broadcast = a_bcast ? 1 : 0;
		p.b_broadcast = b_bcast ? 1 : 0;
		p.D = g.D;
		p.ldd = g.ldd;
		p.stride_d = g.stride_d;
		p.C = g.C;
		p.ldc = g.ldc;
		p.stride_c = g.stride_c;
		p.bias = g.bias;
		p.alpha = g.alpha;
		p.beta = g.beta;
		p.act = g.act;
		p.out_dtype = g.out_dtype;
		p.scales = g.scales;
		p.shifts = g.shifts;
		p.ext = g.ext;
		p.ext_scale = g.ext_scale;
		p.ext_shift = g.ext_shift;
		p.inv_out_scale = 1.0f / g.out_scale; // AffineTransform::get_inverse of the reference's host code
		p.inv_out_shift = -g.out_shift / g.out_scale;
		p.status = c->dev_status;
		c->kernels_with_waits = true;

		if (g.kind == 3)
			return launch<3, 128>(ctx, stream, map_a, map_b, map_a, map_a, p, c->sm_count);
		if (g.kind == 2)
			return (bn == 256) ? launch<2, 256>(ctx, stream, map_a, map_b, map_a, map_a, p, c->sm_count) : launch<2, 128>(ctx, stream, map_a, map_b, map_a, map_a, p,
							c->sm_count);
		CUtensorMap map_c = map_a, map_d = map_a; // read only by the weight-resident variant
		if (g.kind == 0)
		{
			// weight-resident variant: the whole [bn, K] weight tile fits its 128 KB, and a CTA's contiguous range of tiles stays on one
			// weight tile for long enough to pay for the reload (MINML_B200_GEMM_RESIDENT=0: measurement switch); with the box epilogue
			// when D (and C) are fp16 with 16-byte aligned rows
			static const bool resident_allowed = []
			{
				const char *e = std::getenv("MINML_B200_GEMM_RESIDENT");
				return !(e != nullptr && e[0] == '0');
			}();
			const int k_blocks = (g.K + 63) / 64;
			const long long m_tiles = (g.M + BM - 1) / BM;
			const bool use_c = g.beta != 0.0f && g.C != nullptr;
			const bool boxes_ok = g.out_dtype == DTYPE_FLOAT16 && aligned_to(g.D, 16) && g.ldd % 8 == 0 && (g.batch == 1 || g.stride_d % 8 == 0)
					&& (!use_c || (aligned_to(g.C, 16) && g.ldc % 8 == 0 && (g.batch == 1 || g.stride_c % 8 == 0)));
			const bool resident = resident_allowed && !g.a_mn && !g.b_mn && static_cast<long long>(k_blocks) * bn * BK_BYTES <= RESIDENT_BYTES && m_tiles >= 8;
			if (resident && !boxes_ok)
				return (bn == 256) ? launch<0, 256, true>(ctx, stream, map_a, map_b, map_c, map_d, p, c->sm_count) : launch<0, 128, true>(ctx, stream,
								map_a, map_b, map_c, map_d, p, c->sm_count);
			if (resident)
			{
				const uint64_t dims[3] = { static_cast<uint64_t>(g.N), static_cast<uint64_t>(g.M), static_cast<uint64_t>(g.batch) };
				const uint32_t box[3] = { 32, 32, 1 };
				const uint64_t strides_d[2] = { static_cast<uint64_t>(g.ldd) * 2, g.batch == 1 ? static_cast<uint64_t>(g.ldd) * 2 * g.M
						: static_cast<uint64_t>(g.stride_d) * 2 };
				if (!encode_tensor_map(ctx, &map_d, dt, 3, g.D, dims, strides_d, box, CU_TENSOR_MAP_SWIZZLE_64B))
					return false;
				if (use_c)
				{
					const uint64_t strides_c[2] = { static_cast<uint64_t>(g.ldc) * 2, g.batch == 1 ? static_cast<uint64_t>(g.ldc) * 2 * g.M
							: static_cast<uint64_t>(g.stride_c) * 2 };
					if (!encode_tensor_map(ctx, &map_c, dt, 3, g.C, dims, strides_c, box, CU_TENSOR_MAP_SWIZZLE_64B))
						return false;
				}
				return (bn == 256) ? launch<0, 256, true, true>(ctx, stream, map_a, map_b, map_c, map_d, p, c->sm_count) : launch<0, 128, true, true>(ctx,
								stream, map_a, map_b, map_c, map_d, p, c->sm_count);
			}
			return (bn == 256) ? launch<0, 256>(ctx, stream, map_a, map_b, map_c, map_d, p, c->sm_count) : launch<0, 128>(ctx, stream, map_a, map_b,
							map_c, map_d, p, c->sm_count);
		}
		else
			return (bn == 256) ? launch<1, 256>(ctx, stream, map_a, map_b, map_c, map_d, p, c->sm_count) : launch<1, 128>(ctx, stream, map_a, map_b, map_c, map_d, p,
							c->sm_count);
	}
} /* namespace mb200 */
