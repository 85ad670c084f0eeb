/*
 * attention_ws.cu -- persistent, warp-specialised fp16 multi-head attention forward on the tcgen05 tensor cores.
 *
 *   input  [b, h, w, parts * heads * 32]   packed [q | k | v] (parts = 3) or [q = k | v] (parts = 2), head dimension 32
 *   S = Q K^T / sqrt(d);  S[i, j] += table[head, r + (hj - hi), r + (wj - wi)];  P = softmax(S);  O = P V
 *
 * Replaces the batched GEMM -> softmax kernel -> batched GEMM sequence of the reference
 * (src/backend/cuda/kernels/attention.cu:494-568) for boards of up to 256 tokens whose relative offsets stay inside the
 * bias table (or that have no table); other shapes go to kernel_mha_tc (attention_tc.cu) or the warp-level kernel.
 *
 * One CTA per SM walks a contiguous range of (head, batch item) pairs, head-major, so that the bias table in shared memory
 * changes once or twice per CTA.  Inside the CTA two independent pipelines ("groups") take alternate pairs; each has its own
 * Q, K and V buffers in shared memory, its own half of tensor memory, and four roles:
 *   - a copy warp: K, V (whole item) and Q (128 queries at a time) by TMA in the 64-byte-swizzled layout, as soon as the
 *     tensor core has released the buffer (tcgen05.commit on the "empty" barriers), which is one item ahead of the softmax;
 *   - an issue warp: S = Q K^T (M = 128, N = keys) into the group's tensor-memory columns and, once P is there, O = P V with
 *     P as the tensor-memory A operand and V as the MN-major B operand exactly as the copy left it;
 *   - SPLIT x 128 softmax threads, SPLIT per query row (a tensor-memory lane is a row: no shuffles), in units of 16 key
 *     columns with the next unit's tcgen05.ld in flight under the arithmetic of the current one: pass 1 scales, adds the bias,
 *     writes the biased scores back and keeps the maximum; pass 2 exponentiates, sums, and writes P as fp16 pairs over the
 *     scores the thread has already consumed; then they read O (last 32 columns of the group), divide by the row sum and store.
 * The groups take turns at pass 2, so that one group's exponentials run beside the other group's table lookups and products.
 * The bias table sits in shared memory as the window of offsets the board can produce, with a row pitch congruent to the board
 * width modulo 32: the 32 rows of a warp then read 32 different banks for every key.  For the 15 x 15 board every table offset
 * is a compile-time constant of the unrolled loops (template parameters H, W); other boards read the offsets from a list.
 * Every wait is an mbarrier wait with a poll limit (tc.cuh); a timeout raises the CTA's abort flag, every role leaves its
 * loop, and the context's status word is set.  No role waits at a CTA-wide barrier inside the loops.
 */
#include "common.cuh"
#include "tc.cuh"
#include "epilogue.cuh"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#ifndef MB200_MHA_TRACE
#define MB200_MHA_TRACE 0 // 1: cycle stamps of one CTA's phases (MINML_B200_MHA_TRACE=1 prints them), for tuning
#endif

namespace mb200
{
	namespace
	{
		using namespace tc;
		using epi::st_shared_v4;

		constexpr int D = 32; // head dimension
		constexpr int QM = 128; // queries per tile = tensor-memory lanes
		constexpr int GROUPS = 2;

		/* pitch of the table window in shared memory: at least 2w - 1 words, congruent to w modulo 32 */
		__host__ __device__ constexpr int smem_pitch(int w)
		{
			return (2 * w - 1) + (((w - (2 * w - 1)) % 32) + 32) % 32;
		}

		struct WsParams
		{
				__half *output;
				const __half *input;
				const __half *table; // [heads][table_n][table_pad]
				int height, width, heads, batch, parts;
				int table_n, table_pad;
				int table_floats; // per group, in shared memory: (2 height - 1) rows of smem_pitch(width) words
				int tokens, keys, q_tiles;
				int group_columns; // tensor-memory columns per group
				int o_column; // where O goes within them (beyond P, over consumed scores)
				int items; // batch * heads
				int take_turns;
				int *status;
				long long *trace;
		};
		struct WsGroupBarriers
		{
				uint64_t q_full, k_full, v_full; // copies landed
				uint64_t q_empty, k_empty, v_empty; // the products that read the buffer are complete
				uint64_t s_full, o_full; // products complete
				uint64_t p_full, s_empty; // every softmax thread of the group: P is in tensor memory / O has been read
				uint64_t exchange, table_ready; // every softmax thread: partial maxima are in shared memory / the bias table is
				uint64_t pass2_done; // every softmax thread: the exponentials of a tile are done (the other group's turn)
		};
		template<int SPLIT>
		struct WsShared
		{
				WsGroupBarriers bar[GROUPS];
				uint32_t tmem_base;
				int abort_flag;
				float row_max[GROUPS][SPLIT][QM], row_sum[GROUPS][SPLIT][QM];
		};

		/* 8 columns of this thread's lane */
		__device__ __forceinline__ void tmem_st_8(uint32_t taddr, const uint32_t (&r)[8])
		{
			asm volatile(
					"tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
					:: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
		}

		/* ---- the two passes over a thread's units of 16 key columns [U0, U0 + NU) for a board known at compile time: every key's
		 * position, table offset and validity is a constant of the unrolled code. */
		template<int H, int W, int U0, int NU, bool TABLE>
		__device__ __forceinline__ float pass1_fixed(uint32_t lane_taddr, const float *bias_q, float scale)
		{
			constexpr int TOKENS = H * W, PITCH = smem_pitch(W);
			uint32_t buf[2][16];
			float mx0 = -1.0e30f, mx1 = -1.0e30f;
			tmem_ld_32x16(lane_taddr + 16 * U0, buf[0]);
			tmem_wait_ld();
#pragma unroll
			for (int i = 0; i < NU; i++)
			{
				if (i + 1 < NU)
					tmem_ld_32x16(lane_taddr + 16 * (U0 + i + 1), buf[(i + 1) & 1]);
				uint32_t (&r)[16] = buf[i & 1];
#pragma unroll
				for (int e = 0; e < 16; e += 2)
				{
					const int j = 16 * (U0 + i) + e;
					float s0 = __uint_as_float(r[e]) * scale, s1 = __uint_as_float(r[e + 1]) * scale;
					if (TABLE && j < TOKENS)
						s0 = fmaf(__uint_as_float(r[e]), scale, bias_q[(j / W) * PITCH + (j % W)]);
					if (TABLE && j + 1 < TOKENS)
						s1 = fmaf(__uint_as_float(r[e + 1]), scale, bias_q[((j + 1) / W) * PITCH + ((j + 1) % W)]);
					float &mx = (e & 2) ? mx1 : mx0;
					if (j + 1 < TOKENS)
						mx = max3(mx, s0, s1);
					else if (j < TOKENS)
						mx = fmaxf(mx, s0);
					r[e] = __float_as_uint(s0);
					r[e + 1] = __float_as_uint(s1);
				}
				tmem_st_32x16(lane_taddr + 16 * (U0 + i), r);
				if (i + 1 < NU)
					tmem_wait_ld();
			}
			return fmaxf(mx0, mx1);
		}
		template<int H, int W, int U0, int NU>
		__device__ __forceinline__ float pass2_fixed(uint32_t lane_taddr, float row_max)
		{
			constexpr int TOKENS = H * W;
			uint32_t buf[2][16];
			float sum0 = 0.0f, sum1 = 0.0f;
			tmem_ld_32x16(lane_taddr + 16 * U0, buf[0]);
			tmem_wait_ld();
#pragma unroll
			for (int i = 0; i < NU; i++)
			{
				if (i + 1 < NU)
					tmem_ld_32x16(lane_taddr + 16 * (U0 + i + 1), buf[(i + 1) & 1]);
				const uint32_t (&r)[16] = buf[i & 1];
				uint32_t packed[8];
#pragma unroll
				for (int e = 0; e < 16; e += 2)
				{
					const int j = 16 * (U0 + i) + e;
					const float e0 = (j < TOKENS) ? exp2_approx(__uint_as_float(r[e]) - row_max) : 0.0f;
					const float e1 = (j + 1 < TOKENS) ? exp2_approx(__uint_as_float(r[e + 1]) - row_max) : 0.0f;
					float &sum = (e & 2) ? sum1 : sum0;
					sum += e0 + e1;
					packed[e / 2] = pack_half2(e0, e1);
				}
				// P replaces scores this thread has consumed: two fp16 per column, from the first column of the thread's own range
				tmem_st_8(lane_taddr + 16 * U0 + 8 * i, packed);
				if (i + 1 < NU)
					tmem_wait_ld();
			}
			return sum0 + sum1;
		}
		/* ---- the same for any board: units [u_begin, u_end), table offsets from the list `spos` */
		__device__ __forceinline__ float pass1_any(uint32_t lane_taddr, int u_begin, int u_end, int tokens, const float *bias_q, const int *spos,
				float scale, bool has_table)
		{
			float mx = -1.0e30f;
			for (int u = u_begin; u < u_end; u++)
			{
				uint32_t r[16];
				tmem_ld_32x16(lane_taddr + 16 * u, r);
				tmem_wait_ld();
				const int j0 = 16 * u;
				if (j0 + 16 <= tokens)
				{
#pragma unroll
					for (int e = 0; e < 16; e += 4)
					{
						float s[4];
						if (has_table)
						{
							const int4 pj = *reinterpret_cast<const int4*>(spos + j0 + e);
							s[0] = fmaf(__uint_as_float(r[e]), scale, bias_q[pj.x]);
							s[1] = fmaf(__uint_as_float(r[e + 1]), scale, bias_q[pj.y]);
							s[2] = fmaf(__uint_as_float(r[e + 2]), scale, bias_q[pj.z]);
							s[3] = fmaf(__uint_as_float(r[e + 3]), scale, bias_q[pj.w]);
						}
						else
						{
#pragma unroll
							for (int k = 0; k < 4; k++)
								s[k] = __uint_as_float(r[e + k]) * scale;
						}
						mx = max3(max3(mx, s[0], s[1]), s[2], s[3]);
#pragma unroll
						for (int k = 0; k < 4; k++)
							r[e + k] = __float_as_uint(s[k]);
					}
				}
				else
				{
#pragma unroll
					for (int e = 0; e < 16; e++)
					{
						float v = __uint_as_float(r[e]) * scale;
						if (has_table)
							v += bias_q[spos[j0 + e]];
						if (j0 + e < tokens)
							mx = fmaxf(mx, v);
						r[e] = __float_as_uint(v);
					}
				}
				tmem_st_32x16(lane_taddr + 16 * u, r);
			}
			return mx;
		}
		__device__ __forceinline__ float pass2_any(uint32_t lane_taddr, int u_begin, int u_end, int tokens, float row_max)
		{
			float sum = 0.0f;
			for (int u = u_begin; u < u_end; u++)
			{
				uint32_t r[16], packed[8];
				tmem_ld_32x16(lane_taddr + 16 * u, r);
				tmem_wait_ld();
				const int j0 = 16 * u;
#pragma unroll
				for (int e = 0; e < 16; e += 2)
				{
					const float e0 = (j0 + e < tokens) ? exp2_approx(__uint_as_float(r[e]) - row_max) : 0.0f;
					const float e1 = (j0 + e + 1 < tokens) ? exp2_approx(__uint_as_float(r[e + 1]) - row_max) : 0.0f;
					sum += e0 + e1;
					packed[e / 2] = pack_half2(e0, e1);
				}
				tmem_st_8(lane_taddr + 16 * u_begin + 8 * (u - u_begin), packed);
			}
			return sum;
		}

#if MB200_MHA_TRACE
#define WS_TRACE(i) do { if (p.trace != nullptr && blockIdx.x == 1 && gt == 0 && tile_count < 32) p.trace[(g * 32 + tile_count) * 8 + (i)] = clock64(); } while (0)
#define WS_TRACE_ISSUE(i) do { if (p.trace != nullptr && blockIdx.x == 1 && tile_count < 32) p.trace[512 + (g * 32 + tile_count) * 4 + (i)] = clock64(); } while (0)
#else
#define WS_TRACE(i) do { } while (0)
#define WS_TRACE_ISSUE(i) do { } while (0)
#endif

		/* H, W: the board, or 0, 0 for any board (sizes then come from the parameters) */
		template<int SPLIT, int H, int W>
		__global__ void __launch_bounds__(GROUPS * QM * SPLIT + 128, 1) kernel_mha_ws(const __grid_constant__ CUtensorMap map_q,
				const __grid_constant__ CUtensorMap map_kv, const WsParams p)
		{
			constexpr bool FIXED = H > 0;
			constexpr int GT = QM * SPLIT; // softmax threads of a group
			constexpr int SOFTMAX_WARPS = GROUPS * GT / 32;
			extern __shared__ uint8_t smem_raw[];
			__shared__ WsShared<SPLIT> sh;
			const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
			const int height = FIXED ? H : p.height, width = FIXED ? W : p.width;
			const int tokens = FIXED ? H * W : p.tokens, keys = FIXED ? (H * W + 15) / 16 * 16 : p.keys;
			const int q_tiles = FIXED ? (H * W + QM - 1) / QM : p.q_tiles;
			const int units = keys / 16; // of 16 key columns
			const int per_thread = (units + SPLIT - 1) / SPLIT; // units of each of the SPLIT threads of a row
			const int pitch = smem_pitch(width);

			const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
			const uint32_t kv_bytes = (static_cast<uint32_t>(keys) * 64u + 1023u) & ~1023u;
			const uint32_t group_bytes = QM * 64u + 2u * kv_bytes;
			uint8_t *generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
			float *tables = reinterpret_cast<float*>(generic_base + GROUPS * group_bytes); // GROUPS x table_floats, log2 domain
			int *spos = reinterpret_cast<int*>(tables + GROUPS * p.table_floats); // table offset of every key slot (boards not known at compile time)

			if (tid == 0)
			{
				for (int g = 0; g < GROUPS; g++)
				{
					WsGroupBarriers &b = sh.bar[g];
					mbar_init(smem_u32(&b.q_full), 1);
					mbar_init(smem_u32(&b.k_full), 1);
					mbar_init(smem_u32(&b.v_full), 1);
					mbar_init(smem_u32(&b.q_empty), 1);
					mbar_init(smem_u32(&b.k_empty), 1);
					mbar_init(smem_u32(&b.v_empty), 1);
					mbar_init(smem_u32(&b.s_full), 1);
					mbar_init(smem_u32(&b.o_full), 1);
					mbar_init(smem_u32(&b.p_full), GT);
					mbar_init(smem_u32(&b.s_empty), GT);
					mbar_init(smem_u32(&b.exchange), GT);
					mbar_init(smem_u32(&b.table_ready), GT);
					mbar_init(smem_u32(&b.pass2_done), GT);
				}
				sh.abort_flag = 0;
				fence_mbar_init();
			}
			if (warp == 0)
			{
				tmem_alloc(smem_u32(&sh.tmem_base), GROUPS * p.group_columns);
				tmem_relinquish();
			}
			if (!FIXED)
				for (int i = tid; i < keys; i += blockDim.x)
				{ // slots beyond the last token repeat the last token's position, so that every offset formed from them stays in the table
					const int t = min(i, tokens - 1);
					spos[i] = (t / width) * pitch + (t % width);
				}
			tcgen05_fence_before();
			__syncthreads();
			tcgen05_fence_after();
			const uint32_t tmem_base = sh.tmem_base;
			volatile int *abort_flag = &sh.abort_flag;

			// 32-bit arithmetic from here on: the host has checked that items and rows stay below 2^31
			const int first = static_cast<int>(static_cast<long long>(blockIdx.x) * p.items / gridDim.x);
			const int last = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * p.items / gridDim.x);
			const int k_col0 = (p.parts == 3 ? 1 : 0) * p.heads * D, v_col0 = (p.parts - 1) * p.heads * D;

			if (warp < SOFTMAX_WARPS)
			{ /* ---------------------------------------------------------------- softmax threads */
				const int g = tid / GT, gt = tid % GT;
				const int row_in_tile = gt % QM, half = gt / QM;
				WsGroupBarriers &bar = sh.bar[g];
				const uint32_t s_v = smem_base + g * group_bytes + QM * 64u + kv_bytes;
				float *st = tables + g * p.table_floats;
				const uint32_t lane_taddr = tmem_base + g * p.group_columns + (static_cast<uint32_t>((warp % 4) * 32) << 16);
				const bool has_table = p.table != nullptr;
				const int range = (p.table_n - 1) / 2;
				const float scale = rsqrtf(static_cast<float>(D)) * LOG2E; // exp(x) = 2^(x log2 e)
				const int u_begin = half * per_thread, u_end = min(units, u_begin + per_thread);
				uint32_t tile_count = 0, item_count = 0, table_count = 0;
				// The groups take turns at pass 2 (group 0's n-th tile, group 1's n-th, group 0's (n+1)-th ...): its exponentials keep the
				// special-function units busy and pass 1 the shared-memory loads, so one group's pass 2 runs beside the other's pass 1 and
				// products instead of both groups meeting in the same phase.  A group skips the wait once the other has no tile left.
				const int n_items = last - first;
				const uint32_t other_tiles = p.take_turns ? static_cast<uint32_t>(g == 0 ? n_items / 2 : (n_items + 1) / 2) * q_tiles : 0u;
				WsGroupBarriers &other = sh.bar[g ^ 1];
				int loaded_head = -1;
				bool ok = true;

				int head = (first + g) / p.batch, b = (first + g) - head * p.batch;
				for (int item = first + g; item < last && ok; item += GROUPS, item_count++, b += GROUPS)
				{
					while (b >= p.batch)
					{ // head-major order: the next head's first items
						b -= p.batch;
						head++;
					}
					// this thread's 16 or 32 output columns of the item's first row
					__half *out_item = p.output + (static_cast<long long>(b) * tokens * p.heads + head) * D + half * (D / SPLIT);
					if (has_table && head != loaded_head)
					{ // nobody of this group reads the table any more: all passed the previous tile's o_full, which follows everybody's pass 1.
					  // Window of the offsets this board can produce: row (dh + height - 1), column (dw + width - 1)
						const __half *src = p.table + (static_cast<long long>(head) * p.table_n + (range - (height - 1))) * p.table_pad + (range - (width - 1));
						const int cols = 2 * width - 1;
						for (int i = gt; i < (2 * height - 1) * cols; i += GT)
						{
							const int r = i / cols, c = i % cols;
							st[r * pitch + c] = __half2float(src[r * p.table_pad + c]) * LOG2E;
						}
						loaded_head = head;
						mbar_arrive(smem_u32(&bar.table_ready));
						ok = mbar_wait_warp(smem_u32(&bar.table_ready), table_count & 1u, abort_flag, 20u);
						table_count++;
						if (!ok)
							break;
					}
					for (int qt = 0; qt < q_tiles; qt++, tile_count++)
					{
						WS_TRACE(0);
						ok = mbar_wait_warp(smem_u32(&bar.s_full), tile_count & 1u, abort_flag, 20u);
						if (!ok)
							break;
						tcgen05_fence_after();
						WS_TRACE(1);

						const int q = min(qt * QM + row_in_tile, tokens - 1); // rows beyond the last token repeat it (computed, never stored)
						// bias of the key at (jh, jw) = bias_q[jh * pitch + jw]
						const float *bias_q = st + ((height - 1 - q / width) * pitch + (width - 1 - q % width));
						float my_max;
						if constexpr (FIXED)
						{
							constexpr int UNITS = (H * W + 15) / 16, PT = (UNITS + SPLIT - 1) / SPLIT;
							constexpr int U1 = SPLIT > 1 ? PT : 0, N1 = SPLIT > 1 ? UNITS - PT : PT; // the second thread of a row
							if (half == 0)
								my_max = has_table ? pass1_fixed<H, W, 0, PT, true>(lane_taddr, bias_q, scale) : pass1_fixed<H, W, 0, PT, false>(lane_taddr, bias_q, scale);
							else
								my_max = has_table ? pass1_fixed<H, W, U1, N1, true>(lane_taddr, bias_q, scale) : pass1_fixed<H, W, U1, N1, false>(lane_taddr, bias_q, scale);
						}
						else
							my_max = pass1_any(lane_taddr, u_begin, u_end, tokens, bias_q, spos, scale, has_table);
						tmem_wait_st();
						WS_TRACE(2);
						float row_max = my_max;
						if (SPLIT > 1)
						{
							sh.row_max[g][half][row_in_tile] = my_max;
							mbar_arrive(smem_u32(&bar.exchange));
							ok = mbar_wait_warp(smem_u32(&bar.exchange), tile_count & 1u, abort_flag, 20u);
							if (!ok)
								break;
#pragma unroll
							for (int h = 0; h < SPLIT; h++)
								row_max = fmaxf(row_max, sh.row_max[g][h][row_in_tile]);
						}
						{
							const uint32_t awaited = (g == 0) ? tile_count - 1u : tile_count; // which of the other group's tiles (0 - 1 wraps: none)
							if (awaited < other_tiles)
							{
								ok = mbar_wait_warp(smem_u32(&other.pass2_done), awaited & 1u, abort_flag, 20u);
								if (!ok)
									break;
							}
						}
						WS_TRACE(3);
						float my_sum;
						if constexpr (FIXED)
						{
							constexpr int UNITS = (H * W + 15) / 16, PT = (UNITS + SPLIT - 1) / SPLIT;
							constexpr int U1 = SPLIT > 1 ? PT : 0, N1 = SPLIT > 1 ? UNITS - PT : PT;
							if (half == 0)
								my_sum = pass2_fixed<H, W, 0, PT>(lane_taddr, row_max);
							else
								my_sum = pass2_fixed<H, W, U1, N1>(lane_taddr, row_max);
						}
						else
							my_sum = pass2_any(lane_taddr, u_begin, u_end, tokens, row_max);
						mbar_arrive(smem_u32(&bar.pass2_done));
						tmem_wait_st();
						if (SPLIT > 1)
							sh.row_sum[g][half][row_in_tile] = my_sum;
						if (qt == 0 && keys > tokens)
						{ // V's rows beyond the last token belong to the next batch item (or are the copy's zero fill): cleared, so that
						  // nothing of them reaches this item's output even if they hold infinities
							ok = mbar_wait_warp(smem_u32(&bar.v_full), item_count & 1u, abort_flag, 20u);
							if (!ok)
								break;
							for (int i = gt; i < (keys - tokens) * 4; i += GT)
								st_shared_v4(s_v + (tokens + i / 4) * 64 + (i % 4) * 16, make_uint4(0, 0, 0, 0));
							fence_proxy_async_smem(); // plain stores, read by the tensor core through the async proxy
						}
						tcgen05_fence_before();
						mbar_arrive(smem_u32(&bar.p_full));
						WS_TRACE(4);

						ok = mbar_wait_warp(smem_u32(&bar.o_full), tile_count & 1u, abort_flag, 20u);
						if (!ok)
							break;
						tcgen05_fence_after();
						WS_TRACE(5);
						constexpr int OC = D / SPLIT; // output columns of this thread
						uint32_t o[OC];
						if constexpr (SPLIT == 1)
							tmem_ld_32x32(lane_taddr + p.o_column, o);
						else
							tmem_ld_32x16(lane_taddr + p.o_column + half * OC, o);
						tmem_wait_ld();
						float sum = my_sum;
						if (SPLIT > 1)
						{
							sum = 0.0f;
#pragma unroll
							for (int h = 0; h < SPLIT; h++)
								sum += sh.row_sum[g][h][row_in_tile];
						}
						tcgen05_fence_before();
						mbar_arrive(smem_u32(&bar.s_empty)); // the group's columns may take the next tile's scores
						WS_TRACE(6);
						const int row = qt * QM + row_in_tile;
						if (row < tokens)
						{
							const float inv = 1.0f / sum;
							__half *out = out_item + row * (p.heads * D);
#pragma unroll
							for (int c = 0; c < OC / 8; c++)
							{
								uint4 v;
								v.x = pack_half2(__uint_as_float(o[8 * c]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
								v.y = pack_half2(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
								v.z = pack_half2(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
								v.w = pack_half2(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
								*reinterpret_cast<uint4*>(out + c * 8) = v;
							}
						}
						WS_TRACE(7);
					}
				}
			}
			else if (warp < SOFTMAX_WARPS + GROUPS)
			{ /* ---------------------------------------------------------------- copy warps */
				const int g = warp - SOFTMAX_WARPS;
				if (lane == 0)
				{
					WsGroupBarriers &bar = sh.bar[g];
					const uint32_t s_q = smem_base + g * group_bytes, s_k = s_q + QM * 64u, s_v = s_k + kv_bytes;
					prefetch_tensormap(&map_q);
					prefetch_tensormap(&map_kv);
					uint32_t tile_count = 0, item_count = 0;
					bool ok = true;
					int head = (first + g) / p.batch, b = (first + g) - head * p.batch;
					for (int item = first + g; item < last && ok; item += GROUPS, item_count++, b += GROUPS)
					{
						while (b >= p.batch)
						{
							b -= p.batch;
							head++;
						}
						const int row0 = b * tokens;
						for (int qt = 0; qt < q_tiles && ok; qt++, tile_count++)
						{
							if (qt == 0)
							{
								ok = mbar_wait_sleeping(smem_u32(&bar.k_empty), (item_count & 1u) ^ 1u, abort_flag, 200u);
								if (!ok)
									break;
								mbar_arrive_expect_tx(smem_u32(&bar.k_full), static_cast<uint32_t>(keys) * 64u);
								tma_load_3d(s_k, &map_kv, smem_u32(&bar.k_full), k_col0 + head * D, row0, 0);
							}
							ok = mbar_wait_sleeping(smem_u32(&bar.q_empty), (tile_count & 1u) ^ 1u, abort_flag, 200u);
							if (!ok)
								break;
							mbar_arrive_expect_tx(smem_u32(&bar.q_full), QM * 64u);
							tma_load_3d(s_q, &map_q, smem_u32(&bar.q_full), head * D, row0 + qt * QM, 0);
							if (qt == 0)
							{
								ok = mbar_wait_sleeping(smem_u32(&bar.v_empty), (item_count & 1u) ^ 1u, abort_flag, 200u);
								if (!ok)
									break;
								mbar_arrive_expect_tx(smem_u32(&bar.v_full), static_cast<uint32_t>(keys) * 64u);
								tma_load_3d(s_v, &map_kv, smem_u32(&bar.v_full), v_col0 + head * D, row0, 0);
							}
						}
					}
				}
			}
			else
			{ /* ---------------------------------------------------------------- issue warps */
				const int g = warp - SOFTMAX_WARPS - GROUPS;
				if (lane == 0)
				{
					WsGroupBarriers &bar = sh.bar[g];
					const uint32_t s_q = smem_base + g * group_bytes, s_k = s_q + QM * 64u, s_v = s_k + kv_bytes;
					const uint32_t tmem_s = tmem_base + g * p.group_columns, tmem_o = tmem_s + p.o_column;
					const uint32_t idesc_s = make_idesc_f16(keys);
					const uint32_t idesc_o = make_idesc_f16(D) | (1u << 16); // B = V as stored: [key][d], MN-major
					const uint64_t desc_q = make_desc_k_sw64(s_q), desc_k = make_desc_k_sw64(s_k), desc_v = make_desc_mn_sw64(s_v);
					uint32_t tile_count = 0, item_count = 0;
					bool ok = true;
					for (int item = first + g; item < last && ok; item += GROUPS, item_count++)
					{
						ok = mbar_wait(smem_u32(&bar.k_full), item_count & 1u, abort_flag);
						for (int qt = 0; qt < q_tiles && ok; qt++, tile_count++)
						{
							const bool last_tile = qt + 1 == q_tiles;
							ok = mbar_wait(smem_u32(&bar.q_full), tile_count & 1u, abort_flag)
									&& mbar_wait(smem_u32(&bar.s_empty), (tile_count & 1u) ^ 1u, abort_flag);
							if (!ok)
								break;
							tcgen05_fence_after();
#pragma unroll
							for (int k = 0; k < D / 16; k++) // S = Q K^T, 32 bytes of the head dimension per instruction
								mma_ss<0>(tmem_s, desc_q + 2 * k, desc_k + 2 * k, idesc_s, k > 0 ? 1u : 0u);
							mma_commit(smem_u32(&bar.q_empty));
							if (last_tile)
								mma_commit(smem_u32(&bar.k_empty));
							mma_commit(smem_u32(&bar.s_full));

							WS_TRACE_ISSUE(0);
							ok = (qt > 0 || mbar_wait(smem_u32(&bar.v_full), item_count & 1u, abort_flag))
									&& mbar_wait(smem_u32(&bar.p_full), tile_count & 1u, abort_flag);
							if (!ok)
								break;
							tcgen05_fence_after();
							WS_TRACE_ISSUE(1);
							// O = P V: 16 keys per instruction = 8 columns of P in tensor memory (each softmax thread's P starts at the first
							// column of its own range of scores) and two 8-key groups of V (1024 bytes) in shared memory
#pragma unroll
							for (int h = 0; h < SPLIT; h++)
							{
								const int u0 = h * per_thread, u1 = min(units, u0 + per_thread);
								uint32_t a_addr = tmem_s + 16 * u0;
								uint64_t desc_b = desc_v + static_cast<uint64_t>(u0) * 64u;
#pragma unroll 4
								for (int u = u0; u < u1; u++, a_addr += 8, desc_b += 64)
									mma_ts_f16(tmem_o, a_addr, desc_b, idesc_o, u > 0 ? 1u : 0u);
							}
							if (last_tile)
								mma_commit(smem_u32(&bar.v_empty));
							mma_commit(smem_u32(&bar.o_full));
							WS_TRACE_ISSUE(2);
						}
					}
				}
			}

			/* ---- teardown */
			__syncwarp();
			tcgen05_fence_before();
			__syncthreads();
			if (sh.abort_flag != 0)
			{
				if (tid == 0 && p.status != nullptr)
					atomicExch(p.status, 3);
				__nanosleep(1000000); // give copies that are still in flight time to land before the CTA retires
			}
			if (warp == 0)
			{
				tcgen05_fence_after();
				tmem_dealloc(tmem_base, GROUPS * p.group_columns);
			}
		}

		int env_int(const char *name, int fallback)
		{
			const char *e = std::getenv(name);
			return (e != nullptr && e[0] >= '0' && e[0] <= '9') ? std::atoi(e) : fallback;
		}
		/* threads per query row: MINML_B200_MHA_SPLIT=1|2 */
		int ws_split()
		{
			static const int split = env_int("MINML_B200_MHA_SPLIT", 2) == 1 ? 1 : 2;
			return split;
		}

		template<int SPLIT, int H, int W>
		bool launch(mlContext_t ctx, Context *c, cudaStream_t stream, int grid, size_t smem, size_t smem_limit, const CUtensorMap &map_q,
				const CUtensorMap &map_kv, const WsParams &p)
		{
			static std::mutex configured_mutex;
			static bool configured[MAX_DEVICES] = { false };
			{
				std::lock_guard<std::mutex> lock(configured_mutex);
				if (c->device < 0 || c->device >= MAX_DEVICES)
					return false;
				if (!configured[c->device])
				{
					if (!check_cuda(ctx,
							cudaFuncSetAttribute(kernel_mha_ws<SPLIT, H, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_limit)),
							"attention: shared memory opt-in"))
						return false;
					configured[c->device] = true;
				}
			}
			kernel_mha_ws<SPLIT, H, W> <<<grid, GROUPS * QM * SPLIT + 128, smem, stream>>>(map_q, map_kv, p);
			return true;
		}
	}

	/* Returns false when the shape is outside what this kernel handles (the caller then tries the other kernels). */
	bool mha_forward_ws(mlContext_t ctx, void *output, const void *input, const void *table, int batch, int height, int width, int heads,
			int head_dim, int parts, int table_n, int table_pad)
	{
		if (head_dim != D || height >= 32768 || width >= 32768)
			return false;
		const int channels = parts * heads * D;
		const long long rows = static_cast<long long>(batch) * height * width;
		const long long items = static_cast<long long>(batch) * heads;
		if (!aligned_to(input, 16) || !aligned_to(output, 16) || rows >= (1LL << 31) || items >= (1LL << 31))
			return false;
		const int tokens = height * width;
		const int keys = (tokens + 15) / 16 * 16;
		if (keys > 256)
			return false; // two groups of `keys` columns each must fit the 512 columns of tensor memory
		int table_floats = 0;
		if (table != nullptr)
		{
			const int range = (table_n - 1) / 2;
			if (height - 1 > range || width - 1 > range)
				return false; // offsets would need clamping
			table_floats = ((2 * height - 1) * smem_pitch(width) + 3) / 4 * 4;
		}
		// P (two fp16 per column) overwrites each softmax thread's own consumed scores from the start of its column range; O takes the last
		// 32 columns of the group, beyond all of P
		const int split = ws_split(), units = keys / 16, per_thread = (units + split - 1) / split;
		const int p_extent = 16 * per_thread * (split - 1) + 8 * per_thread;
		int group_columns = 32;
		while (group_columns < std::max(keys, p_extent + 32))
			group_columns *= 2;
		if (GROUPS * group_columns > 512)
			return false;
		const size_t kv_bytes = (static_cast<size_t>(keys) * 64 + 1023) / 1024 * 1024;
		const size_t smem = 1024 + GROUPS * (QM * 64 + 2 * kv_bytes) + GROUPS * static_cast<size_t>(table_floats) * sizeof(float)
				+ static_cast<size_t>(keys) * sizeof(int) + 64;
		constexpr size_t SMEM_LIMIT = 222 * 1024; // the opt-in limit of 227 KB per CTA includes the kernel's static shared memory
		if (smem > SMEM_LIMIT)
			return false;
		Context *c = get(ctx);
		cudaStream_t stream = use_stream(ctx);
		CUtensorMap map_q, map_kv;
		const uint64_t dims[3] = { static_cast<uint64_t>(channels), static_cast<uint64_t>(rows), 1 };
		const uint64_t strides[2] = { static_cast<uint64_t>(channels) * 2, static_cast<uint64_t>(channels) * 2 * static_cast<uint64_t>(rows) };
		const uint32_t box_q[3] = { D, QM, 1 };
		const uint32_t box_kv[3] = { D, static_cast<uint32_t>(keys), 1 };
		if (!encode_tensor_map(ctx, &map_q, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, input, dims, strides, box_q, CU_TENSOR_MAP_SWIZZLE_64B)
				|| !encode_tensor_map(ctx, &map_kv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, input, dims, strides, box_kv, CU_TENSOR_MAP_SWIZZLE_64B))
			return false;
		WsParams p;
		std::memset(&p, 0, sizeof(p));
		p.output = reinterpret_cast<__half*>(output);
		p.input = reinterpret_cast<const __half*>(input);
		p.table = reinterpret_cast<const __half*>(table);
		p.height = height;
		p.width = width;
		p.heads = heads;
		p.batch = batch;
		p.parts = parts;
		p.table_n = (table != nullptr) ? table_n : 0;
		p.table_pad = (table != nullptr) ? table_pad : 0;
		p.table_floats = table_floats;
		p.tokens = tokens;
		p.keys = keys;
		p.q_tiles = (tokens + QM - 1) / QM;
		p.group_columns = group_columns;
		p.o_column = group_columns - 32;
		p.items = static_cast<int>(items);
		static const int take_turns = env_int("MINML_B200_MHA_TURNS", 1);
		p.take_turns = take_turns;
		p.status = c->dev_status;
#if MB200_MHA_TRACE
		static long long *trace = nullptr;
		constexpr int TRACE_WORDS = 512 + 256;
		if (std::getenv("MINML_B200_MHA_TRACE") != nullptr && trace == nullptr)
		{
			cudaMalloc(&trace, TRACE_WORDS * sizeof(long long));
			cudaMemset(trace, 0, TRACE_WORDS * sizeof(long long));
		}
		p.trace = trace;
#endif
		const int grid = static_cast<int>(std::min<long long>(items, c->sm_count));
		static const bool any_board = env_int("MINML_B200_MHA_ANY_BOARD", 0) != 0; // 1: never the code specialised for a board
		bool launched;
		if (height == 15 && width == 15 && !any_board)
			launched = split == 1 ? launch<1, 15, 15>(ctx, c, stream, grid, smem, SMEM_LIMIT, map_q, map_kv, p) :
					launch<2, 15, 15>(ctx, c, stream, grid, smem, SMEM_LIMIT, map_q, map_kv, p);
		else
			launched = split == 1 ? launch<1, 0, 0>(ctx, c, stream, grid, smem, SMEM_LIMIT, map_q, map_kv, p) :
					launch<2, 0, 0>(ctx, c, stream, grid, smem, SMEM_LIMIT, map_q, map_kv, p);
		if (!launched)
			return false;
		MB200_COUNT_LAUNCH();
		c->kernels_with_waits = true;
#if MB200_MHA_TRACE
		if (trace != nullptr)
		{
			static int dumps = 0;
			cudaStreamSynchronize(stream);
			if (dumps++ == 2)
			{
				long long host[TRACE_WORDS];
				cudaMemcpy(host, trace, sizeof(host), cudaMemcpyDeviceToHost);
				for (int g = 0; g < 2; g++)
					for (int t = 0; t < 32; t++)
					{
						printf("TRACE g%d t%02d", g, t);
						for (int i = 0; i < 8; i++)
							printf(" %lld", host[(g * 32 + t) * 8 + i] == 0 ? 0 : host[(g * 32 + t) * 8 + i] - host[0]);
						const long long *m = host + 512 + (g * 32 + t) * 4;
						printf(" | issue warp: saw p_full %lld, issued %lld\n", m[1] == 0 ? 0 : m[1] - host[0], m[2] == 0 ? 0 : m[2] - host[0]);
					}
				fflush(stdout);
			}
		}
#endif
		return check_cuda(ctx, cudaGetLastError(), "cuda_multi_head_attention_forward (tcgen05, warp-specialised)");
	}
} /* namespace mb200 */
