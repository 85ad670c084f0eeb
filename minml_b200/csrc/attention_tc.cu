/*
 * attention_tc.cu -- fp16 multi-head attention forward on the tcgen05 tensor cores with the scores in tensor memory.
 *
 *   input  [b, h, w, parts * heads * 32]   packed [q | k | v] (parts = 3) or [q = k | v] (parts = 2), head dimension 32
 *   S = Q K^T / sqrt(d);  S[i, j] += table[head, r + clamp(hj - hi, -r, r), r + clamp(wj - wi, -r, r)];  P = softmax(S);  O = P V
 *
 * Replaces the batched GEMM -> softmax kernel -> batched GEMM sequence of the reference
 * (src/backend/cuda/kernels/attention.cu:494-568), whose [b, heads, T, T] score tensor never exists here.
 *
 * One CTA of 256 threads per (head, batch item); two CTAs share an SM when the board has up to 256 tokens.  This is the simple form of
 * the tcgen05 path: boards of up to 256 tokens go to the persistent warp-specialised kernel (attention_ws.cu) by default, and this
 * kernel runs only when selected (mb200_set_attention_kernel 1 or 2), where it also takes 257 .. 462 tokens and tables whose
 * offsets need clamping.  Per tile of 128 queries:
 *   1. Q (128 x 64 bytes), K and V (N x 64 bytes each, N = tokens rounded up to 16) arrive by TMA in the 64-byte-swizzled layout;
 *      V stays as it landed: [key][d] is the MN-major B operand of the second product;
 *   2. S = Q K^T: one tcgen05.mma (two for more than 256 keys) of M = 128 into N columns of tensor memory;
 *   3. softmax straight from tensor memory, two threads per query row, each with half of the key columns (a tensor-memory lane is
 *      a row, so row maxima and sums need one exchange through shared memory and no shuffles): pass 1 adds scale and
 *      relative-position bias, writes the biased scores back to tensor memory and keeps the maximum; pass 2 exponentiates, sums,
 *      and writes P as fp16 into shared memory in the 128-byte-swizzled K-major layout the tensor core reads;
 *   4. O = P V: tcgen05.mma of M = 128, N = 32 over the keys, into the first 32 columns (the scores are dead by then);
 *   5. each thread reads its half of its row of O, divides by the row sum and stores 32 bytes.
 * Measured against the warp-level kernel (attention_mma.cu) on a B200: 256 x 225 tokens x 8 heads 0.128 ms against 0.123 ms, 1024 x 400
 * tokens 2.18 ms against 1.32 ms: its phases -- copy, product, softmax, product, store -- run one after the other inside a CTA with
 * at most two CTAs per SM to overlap them, where the warp-level kernel has sixteen independent warps per SM.  The persistent kernel
 * removes that serialisation (0.083 ms on the first shape).
 * All tcgen05.mma are issued by thread 0; every wait is bounded (tc.cuh) and a timeout sets the context's status word.
 * Keys beyond the last token (the TMA box runs into the next batch item, or past the end of the tensor where it is filled
 * with zeros) get P = 0 and their rows of V are cleared; query rows beyond it are computed and never stored.
 */
#include "common.cuh"
#include "tc.cuh"
#include "epilogue.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace mb200
{
	namespace
	{
		using namespace tc;
		using epi::st_shared_v4;

		constexpr int D = 32; // head dimension
		constexpr int QM = 128; // queries per tile = tensor-memory lanes
		constexpr int NT = 256; // threads: two per query row, each with half of the key columns (a warp reaches the lanes 32 * (warp % 4) ...)

		struct MhaTcParams
		{
				__half *output;
				const __half *input;
				const __half *table;
				int height, width, heads, parts, table_n, table_pad;
				int tokens, keys; // keys = N: tokens rounded up (16, or 32 when two boxes are needed)
				int boxes, box_rows; // K arrives in `boxes` TMA boxes of `box_rows` rows
				int tmem_columns;
				int *status;
		};
		struct MhaBarriers
		{
				uint64_t tma_k, tma_q, mma;
				uint32_t tmem_base;
				int abort_flag;
				float row_max[2][QM], row_sum[2][QM]; // the two column halves of a row exchange their maximum and their sum here
		};

		__global__ void __launch_bounds__(NT) kernel_mha_tc(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
				const MhaTcParams p)
		{
			extern __shared__ uint8_t smem_raw[];
			__shared__ MhaBarriers bars;
			const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
			const int head = blockIdx.x, b = blockIdx.y;
			const int tokens = p.tokens, keys = p.keys;
			const int key_tiles = (keys + 63) / 64; // 64 keys = one 128-byte K slice of P and V^T

			const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
			const uint32_t s_q = smem_base; // 128 x 64 B
			const uint32_t s_k = s_q + QM * 64; // keys x 64 B
			const uint32_t s_vt = (s_k + keys * 64 + 1023u) & ~1023u; // key_tiles x (32 x 128 B)
			const uint32_t s_p = s_vt + key_tiles * 4096; // key_tiles x (128 x 128 B)
			uint8_t *generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
			float *st = reinterpret_cast<float*>(generic_base + (s_p + key_tiles * 16384 - smem_base)); // table, log2 domain
			int *spos = reinterpret_cast<int*>(st + p.table_n * p.table_pad); // position code of every key slot

			if (tid == 0)
			{
				mbar_init(smem_u32(&bars.tma_k), 1);
				mbar_init(smem_u32(&bars.tma_q), 1);
				mbar_init(smem_u32(&bars.mma), 1);
				bars.abort_flag = 0;
				fence_mbar_init();
			}
			if (warp == 0)
			{
				tmem_alloc(smem_u32(&bars.tmem_base), p.tmem_columns);
				tmem_relinquish();
			}
			tcgen05_fence_before();
			__syncthreads();
			tcgen05_fence_after();
			const uint32_t tmem_base = bars.tmem_base;
			volatile int *abort_flag = &bars.abort_flag;

			const int stride = p.parts * p.heads * D; // channels per token
			const long long row0 = static_cast<long long>(b) * tokens; // first token of this batch item in the [b * tokens, channels] view
			const int q_col = head * D;
			const int k_col = (p.parts == 3 ? 1 : 0) * p.heads * D + head * D;
			const int v_col = (p.parts - 1) * p.heads * D + head * D;

			if (tid == 0)
			{ // K (all boxes) and the first Q tile
				prefetch_tensormap(&map_q);
				prefetch_tensormap(&map_k);
				mbar_arrive_expect_tx(smem_u32(&bars.tma_k), static_cast<uint32_t>(keys) * 128u);
				for (int i = 0; i < p.boxes; i++)
				{
					tma_load_3d(s_k + i * p.box_rows * 64, &map_k, smem_u32(&bars.tma_k), k_col, static_cast<int>(row0) + i * p.box_rows, 0);
					tma_load_3d(s_vt + i * p.box_rows * 64, &map_k, smem_u32(&bars.tma_k), v_col, static_cast<int>(row0) + i * p.box_rows, 0);
				}
				mbar_arrive_expect_tx(smem_u32(&bars.tma_q), QM * 64u);
				tma_load_3d(s_q, &map_q, smem_u32(&bars.tma_q), q_col, static_cast<int>(row0), 0);
			}

			/* ---- while the copies fly: the bias table, the key positions, and V^T */
			for (int i = tid; i < p.table_n * p.table_pad; i += NT)
				st[i] = __half2float(p.table[static_cast<long long>(head) * p.table_n * p.table_pad + i]) * LOG2E;
			// Relative offsets never leave the table when the board is no larger than the table's range + 1 (the usual case: the table
			// is built for the board).  The index is then linear in the two positions and needs no clamping:
			// (jh - qh + range) * pad + (jw - qw + range) = lin(j) - lin(q) + range * (pad + 1), lin(t) = th * pad + tw.
			const int range = (p.table_n - 1) / 2;
			const bool linear_bias = p.table != nullptr && (p.height - 1 <= range) && (p.width - 1 <= range);
			for (int i = tid; i < keys; i += NT)
			{ // slots beyond the last token repeat the last token's position, so that every index formed from them stays in the table
				const int t = min(i, tokens - 1);
				spos[i] = linear_bias ? (t / p.width) * p.table_pad + (t % p.width) : (((t / p.width) << 16) | (t % p.width));
			}
			// V arrives beside K; its rows beyond the last token belong to the next batch item (or are the copy's zero fill): cleared, so
			// that nothing of them reaches this item's output even if they hold infinities
			bool v_ok = mbar_wait(smem_u32(&bars.tma_k), 0, abort_flag);
			for (int i = tid; i < (keys - tokens) * 4; i += NT)
				st_shared_v4(s_vt + (tokens + i / 4) * 64 + (i % 4) * 16, make_uint4(0, 0, 0, 0));
			fence_proxy_async_smem(); // plain stores; the tensor core reads V through the async proxy
			v_ok = __syncthreads_and(v_ok ? 1 : 0) != 0;

			const float scale = rsqrtf(static_cast<float>(D)) * LOG2E; // exp(x) = 2^(x log2 e)
			const int q_tiles = (tokens + QM - 1) / QM;
			const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>((warp % 4) * 32) << 16); // this warp's 32 lanes
			const int row_in_tile = tid % QM, half = tid / QM;
			// chunks of 32 key columns; the first `split` belong to the threads of half 0, the rest (and the zero fill up to a whole
			// 64-key slice) to half 1
			const int n_chunks = (keys + 31) / 32, all_chunks = key_tiles * 2, split = (n_chunks + 1) / 2;
			const int chunk_begin = half == 0 ? 0 : split, chunk_end = half == 0 ? split : all_chunks;
			uint32_t mma_phase = 0;
			bool ok = v_ok;

			for (int qt = 0; qt < (ok ? q_tiles : 0); qt++)
			{
				/* ---- S = Q K^T */
				if (tid == 0 && ok)
				{
					ok = (qt > 0 || mbar_wait(smem_u32(&bars.tma_k), 0, abort_flag)) && mbar_wait(smem_u32(&bars.tma_q), qt & 1u, abort_flag);
					if (ok)
					{
						tcgen05_fence_after();
						const uint32_t idesc = make_idesc_f16(p.box_rows);
						for (int i = 0; i < p.boxes; i++)
						{
							const uint64_t desc_a = make_desc_k_sw64(s_q);
							const uint64_t desc_b = make_desc_k_sw64(s_k + i * p.box_rows * 64);
#pragma unroll
							for (int k = 0; k < D / 16; k++) // 32 bytes of the head dimension per instruction
								mma_ss<0>(tmem_base + i * p.box_rows, desc_a + 2 * k, desc_b + 2 * k, idesc, k > 0 ? 1u : 0u);
						}
						mma_commit(smem_u32(&bars.mma));
					}
				}
				ok = mbar_wait(smem_u32(&bars.mma), mma_phase, abort_flag) && ok;
				mma_phase ^= 1u;
				ok = __syncthreads_and(ok ? 1 : 0) != 0;
				if (!ok)
					break;
				tcgen05_fence_after();
				if (tid == 0 && qt + 1 < q_tiles)
				{ // the Q tile is free again: fetch the next one under the softmax
					mbar_arrive_expect_tx(smem_u32(&bars.tma_q), QM * 64u);
					tma_load_3d(s_q, &map_q, smem_u32(&bars.tma_q), q_col, static_cast<int>(row0) + (qt + 1) * QM, 0);
				}

				/* ---- softmax: this thread's half of its row */
				const int q = min(qt * QM + row_in_tile, tokens - 1); // rows beyond the last token repeat it (computed, never stored)
				const int pq = linear_bias ? (q / p.width) * p.table_pad + (q % p.width) : 0;
				const int qh = q / p.width, qw = q % p.width;
				const float *bias_row = st + (range * (p.table_pad + 1) - pq); // linear form: bias of key slot j = bias_row[spos[j]]
				float my_max = -1.0e30f;
				for (int c = chunk_begin; c < min(chunk_end, n_chunks); c++)
				{ // pass 1: s = acc * scale + bias, written back; running maximum over the real keys
					const int j0 = c * 32;
					const bool wide = j0 + 32 <= keys;
					uint32_t r[32];
					tmem_ld_chunk(lane_taddr + j0, r, wide);
					if (linear_bias && j0 + 32 <= tokens)
					{ // the common chunk: 32 real keys, table index linear in the two positions
#pragma unroll
						for (int j4 = 0; j4 < 8; j4++)
						{
							const int4 pj = *reinterpret_cast<const int4*>(spos + j0 + 4 * j4);
							const float s0 = fmaf(__uint_as_float(r[4 * j4]), scale, bias_row[pj.x]);
							const float s1 = fmaf(__uint_as_float(r[4 * j4 + 1]), scale, bias_row[pj.y]);
							const float s2 = fmaf(__uint_as_float(r[4 * j4 + 2]), scale, bias_row[pj.z]);
							const float s3 = fmaf(__uint_as_float(r[4 * j4 + 3]), scale, bias_row[pj.w]);
							my_max = fmaxf(fmaxf(my_max, fmaxf(s0, s1)), fmaxf(s2, s3));
							r[4 * j4] = __float_as_uint(s0);
							r[4 * j4 + 1] = __float_as_uint(s1);
							r[4 * j4 + 2] = __float_as_uint(s2);
							r[4 * j4 + 3] = __float_as_uint(s3);
						}
					}
					else
					{
#pragma unroll
						for (int j = 0; j < 32; j++)
						{
							if (!wide && j >= 16)
								break;
							float v = __uint_as_float(r[j]) * scale;
							if (p.table != nullptr)
							{
								const int pj = spos[j0 + j];
								if (linear_bias)
									v += bias_row[pj];
								else
								{
									const int jh = pj >> 16, jw = pj & 0xFFFF;
									v += st[(min(max(jh - qh, -range), range) + range) * p.table_pad + min(max(jw - qw, -range), range) + range];
								}
							}
							if (j0 + j < tokens)
								my_max = fmaxf(my_max, v);
							r[j] = __float_as_uint(v);
						}
					}
					if (wide)
						tmem_st_32x32(lane_taddr + j0, r);
					else
						tmem_st_32x16(lane_taddr + j0, r);
				}
				tmem_wait_st();
				bars.row_max[half][row_in_tile] = my_max;
				__syncthreads();
				const float row_max = fmaxf(bars.row_max[0][row_in_tile], bars.row_max[1][row_in_tile]);
				float my_sum = 0.0f;
				for (int c = chunk_begin; c < chunk_end; c++)
				{ // pass 2: p = 2^(s - max), summed in fp32, stored as fp16 in the operand layout of the second product
					const int j0 = c * 32;
					uint32_t packed[16];
					if (j0 < tokens)
					{
						const bool wide = j0 + 32 <= keys;
						uint32_t r[32];
						tmem_ld_chunk(lane_taddr + j0, r, wide);
						if (j0 + 32 <= tokens)
						{
#pragma unroll
							for (int j = 0; j < 32; j += 2)
							{
								const float e0 = exp2_approx(__uint_as_float(r[j]) - row_max), e1 = exp2_approx(__uint_as_float(r[j + 1]) - row_max);
								my_sum += e0 + e1;
								packed[j / 2] = pack_half2(e0, e1);
							}
						}
						else
						{
#pragma unroll
							for (int j = 0; j < 32; j += 2)
							{
								float e0 = 0.0f, e1 = 0.0f;
								if (wide || j < 16)
								{
									e0 = (j0 + j < tokens) ? exp2_approx(__uint_as_float(r[j]) - row_max) : 0.0f;
									e1 = (j0 + j + 1 < tokens) ? exp2_approx(__uint_as_float(r[j + 1]) - row_max) : 0.0f;
								}
								my_sum += e0 + e1;
								packed[j / 2] = pack_half2(e0, e1);
							}
						}
					}
					else
					{
#pragma unroll
						for (int j = 0; j < 16; j++)
							packed[j] = 0u;
					}
					const uint32_t tile = s_p + (j0 / 64) * 16384 + row_in_tile * 128;
					const int chunk0 = (j0 % 64) / 8;
#pragma unroll
					for (int k = 0; k < 4; k++)
						st_shared_v4(tile + (((chunk0 + k) ^ (row_in_tile & 7)) * 16), make_uint4(packed[4 * k], packed[4 * k + 1], packed[4 * k + 2], packed[4 * k + 3]));
				}
				bars.row_sum[half][row_in_tile] = my_sum;
				fence_proxy_async_smem(); // P was written with plain stores
				tcgen05_fence_before();
				__syncthreads(); // every row of P is in place, and nobody reads the scores any more

				/* ---- O = P V (into the first 32 columns) */
				if (tid == 0)
				{
					tcgen05_fence_after();
					const uint32_t idesc = make_idesc_f16(D) | (1u << 16); // B = V as stored: [key][d], MN-major
					const int k_steps = keys / 16;
					for (int ks = 0; ks < k_steps; ks++)
					{ // 16 keys = 32 bytes of the 128-byte slice per instruction
						const uint64_t desc_a = make_desc_k_sw128(s_p + (ks / 4) * 16384) + 2 * (ks % 4);
						const uint64_t desc_b = make_desc_mn_sw64(s_vt + ks * 1024);
						mma_ss<0>(tmem_base, desc_a, desc_b, idesc, ks > 0 ? 1u : 0u);
					}
					mma_commit(smem_u32(&bars.mma));
				}
				ok = mbar_wait(smem_u32(&bars.mma), mma_phase, abort_flag);
				mma_phase ^= 1u;
				ok = __syncthreads_and(ok ? 1 : 0) != 0;
				if (!ok)
					break;
				tcgen05_fence_after();
				{ // each thread of a row's pair takes 16 of the 32 output columns
					uint32_t r[16];
					tmem_ld_32x16(lane_taddr + half * 16, r);
					tmem_wait_ld();
					const int row = qt * QM + row_in_tile;
					if (row < tokens)
					{
						const float inv = 1.0f / (bars.row_sum[0][row_in_tile] + bars.row_sum[1][row_in_tile]);
						__half *out = p.output + (row0 + row) * (static_cast<long long>(p.heads) * D) + head * D + half * 16;
#pragma unroll
						for (int c = 0; c < 2; c++)
						{
							uint4 v;
							v.x = pack_half2(__uint_as_float(r[8 * c]) * inv, __uint_as_float(r[8 * c + 1]) * inv);
							v.y = pack_half2(__uint_as_float(r[8 * c + 2]) * inv, __uint_as_float(r[8 * c + 3]) * inv);
							v.z = pack_half2(__uint_as_float(r[8 * c + 4]) * inv, __uint_as_float(r[8 * c + 5]) * inv);
							v.w = pack_half2(__uint_as_float(r[8 * c + 6]) * inv, __uint_as_float(r[8 * c + 7]) * inv);
							*reinterpret_cast<uint4*>(out + c * 8) = v;
						}
					}
				}
				tcgen05_fence_before();
				__syncthreads(); // O is read: the next tile's scores may overwrite it
			}

			/* ---- teardown */
			tcgen05_fence_before();
			__syncthreads();
			if (bars.abort_flag != 0)
			{
				if (tid == 0 && p.status != nullptr)
					atomicExch(p.status, 3);
				__nanosleep(1000000); // give copies that are still in flight time to land before the CTA retires
			}
			if (warp == 0)
			{
				tcgen05_fence_after();
				tmem_dealloc(tmem_base, p.tmem_columns);
			}
		}

		/* 0 = by shape (the persistent tcgen05 kernel where it applies, else the warp-level kernel), 1 = tcgen05 wherever one of the two
		 * tcgen05 kernels takes the shape, 2 = this kernel wherever it takes the shape, 3 = never tcgen05; MINML_B200_MHA_KERNEL=0..3 at
		 * start, mb200_set_attention_kernel at run time */
		std::atomic<int> g_attention_kernel { []
		{
			const char *e = std::getenv("MINML_B200_MHA_KERNEL");
			return (e != nullptr && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 0;
		}() };
	}

	void g_attention_kernel_store(int kernel)
	{
		g_attention_kernel.store((kernel >= 0 && kernel <= 3) ? kernel : 0);
	}
	bool mha_forward_ws(mlContext_t ctx, void *output, const void *input, const void *table, int batch, int height, int width, int heads,
			int head_dim, int parts, int table_n, int table_pad);
	/* The tcgen05 kernels, as selected.  Returns false when neither is to run (the caller then uses the warp-level kernel). */
	bool mha_forward_tc(mlContext_t ctx, void *output, const void *input, const void *table, int batch, int height, int width, int heads,
			int head_dim, int parts, int table_n, int table_pad)
	{
		const int selected = g_attention_kernel.load();
		if (selected <= 1 && mha_forward_ws(ctx, output, input, table, batch, height, width, heads, head_dim, parts, table_n, table_pad))
			return true;
		if (selected == 0 || selected == 3 || head_dim != D || height >= 32768 || width >= 32768 || batch > 65535 || heads > 65535)
			return false;
		const int channels = parts * heads * D;
		const long long rows = static_cast<long long>(batch) * height * width;
		if (!aligned_to(input, 16) || !aligned_to(output, 16) || rows >= (1LL << 31))
			return false;
		const int tokens = height * width;
		const int boxes = (tokens > 256) ? 2 : 1;
		const int keys = (tokens + 16 * boxes - 1) / (16 * boxes) * (16 * boxes);
		if (keys > 480 || keys / boxes > 256)
			return false; // the scores of a 128-query tile must fit the 512 columns of tensor memory
		int tmem_columns = 32;
		while (tmem_columns < keys)
			tmem_columns *= 2;
		const int key_tiles = (keys + 63) / 64;
		const size_t smem = 1024 + QM * 64 + (static_cast<size_t>(keys) * 64 + 1023) / 1024 * 1024 + static_cast<size_t>(key_tiles) * (4096 + 16384)
				+ static_cast<size_t>(table_n) * table_pad * sizeof(float) + static_cast<size_t>(keys) * sizeof(int) + 64;
		constexpr size_t SMEM_LIMIT = 223 * 1024; // the opt-in limit of 227 KB per CTA includes the kernel's static shared memory
		if (smem > SMEM_LIMIT)
			return false;
		Context *c = get(ctx);
		cudaStream_t stream = use_stream(ctx);
		{
			static std::mutex configured_mutex;
			static size_t configured_bytes[MAX_DEVICES] = { 0 };
			std::lock_guard<std::mutex> lock(configured_mutex);
			if (c->device < 0 || c->device >= MAX_DEVICES)
				return false;
			if (configured_bytes[c->device] < smem)
			{
				if (!check_cuda(ctx, cudaFuncSetAttribute(kernel_mha_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_LIMIT)),
						"attention: shared memory opt-in"))
					return false;
				configured_bytes[c->device] = SMEM_LIMIT;
			}
		}
		CUtensorMap map_q, map_k;
		const uint64_t dims[3] = { static_cast<uint64_t>(channels), static_cast<uint64_t>(rows), 1 };
		const uint64_t strides[2] = { static_cast<uint64_t>(channels) * 2, static_cast<uint64_t>(channels) * 2 * static_cast<uint64_t>(rows) };
		const uint32_t box_q[3] = { D, QM, 1 };
		const uint32_t box_k[3] = { D, static_cast<uint32_t>(keys / boxes), 1 };
		if (!encode_tensor_map(ctx, &map_q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, input, dims, strides, box_q, CU_TENSOR_MAP_SWIZZLE_64B)
				|| !encode_tensor_map(ctx, &map_k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, input, dims, strides, box_k, CU_TENSOR_MAP_SWIZZLE_64B))
			return false;
		MhaTcParams p;
		std::memset(&p, 0, sizeof(p));
		p.output = reinterpret_cast<__half*>(output);
		p.input = reinterpret_cast<const __half*>(input);
		p.table = reinterpret_cast<const __half*>(table);
		p.height = height;
		p.width = width;
		p.heads = heads;
		p.parts = parts;
		p.table_n = (table != nullptr) ? table_n : 0;
		p.table_pad = (table != nullptr) ? table_pad : 0;
		p.tokens = tokens;
		p.keys = keys;
		p.boxes = boxes;
		p.box_rows = keys / boxes;
		p.tmem_columns = tmem_columns;
		p.status = c->dev_status;
		kernel_mha_tc<<<dim3(heads, batch), NT, smem, stream>>>(map_q, map_k, p);
		MB200_COUNT_LAUNCH();
		c->kernels_with_waits = true;
		return check_cuda(ctx, cudaGetLastError(), "cuda_multi_head_attention_forward (tcgen05)");
	}
} /* namespace mb200 */

extern "C" void mb200_set_attention_kernel(int kernel)
{
	mb200::g_attention_kernel_store(kernel);
}
