/*
 * attention_mma.cu -- fp16 multi-head attention forward on the warp-level tensor-core path (mma.sync m16n8k16, fp32
 * accumulation), flash-attention style: the [b, heads, T, T] score tensor that the reference materialises in its workspace
 * (src/backend/cuda/kernels/attention.cu:494-568: batched GEMM, softmax kernel, batched GEMM) never exists.
 *
 *   input  [b, h, w, parts * heads * d]   packed [q | k | v] (parts = 3) or [q = k | v] (parts = 2)
 *   S = Q K^T / sqrt(d);  S[i, j] += table[head, r + clamp(hj - hi, -r, r), r + clamp(wj - wi, -r, r)];  P = softmax(S);  O = P V
 *
 * One CTA per (head, batch item) stages K and V of that head in shared memory once; each of its 4 warps owns one or two tiles
 * of 16 queries at a time and walks the keys in blocks of 32 or 64 with a running maximum and sum, keeping S, P and O in
 * registers (head dimensions up to 32: two tiles, 32 keys; larger ones: one tile, 64 keys).
 * Tokens here are at most a few hundred (a 20x20 board has 400) with head dimensions of 16-128.  For head dimension 32 and boards
 * of up to 256 tokens the persistent tcgen05 kernel (attention_ws.cu) is the default: 0.083 ms against this kernel's 0.123 ms on
 * 256 x 225 tokens x 8 heads.  This kernel takes every other fp16 case; on 1024 x 400 tokens it measured 1.32 ms against the
 * 2.18 ms of the one-CTA-per-head tcgen05 kernel (attention_tc.cu).
 */
#include "common.cuh"

#include <cstdlib>

namespace mb200
{
	namespace
	{
		constexpr int WARPS = 4;

		__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
		{
			asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
					: "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
		}
		__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t &r0, uint32_t &r1, uint32_t smem_addr)
		{
			asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_addr));
		}
		__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
		{
			const __half2 h = __floats2half2_rn(lo, hi);
			return *reinterpret_cast<const uint32_t*>(&h);
		}

		constexpr float LOG2E = 1.4426950408889634f;
		__device__ __forceinline__ float exp2_approx(float x)
		{
			float y;
			asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
			return y;
		}

		/* D = head dimension (multiple of 16); QT = query tiles of 16 rows a warp carries at once (every K and V fragment it loads
		 * from shared memory then feeds QT products, and QT independent softmax chains hide each other's latencies); KB = keys per
		 * block of the running softmax. */
		template<int D, int QT, int KB>
		__global__ void __launch_bounds__(WARPS * 32) kernel_mha_mma(__half *__restrict__ output, const __half *__restrict__ input,
				const __half *__restrict__ table, int height, int width, int heads, int parts, int table_n, int table_pad)
		{
			constexpr int LD = D + 8; // row pitch in halves: 16-byte aligned rows, conflict-free fragment loads
			constexpr int KC = D / 16; // k-chunks of the first product
			constexpr int NT = D / 8; // n-tiles of the second product
			extern __shared__ __align__(16) unsigned char smem_raw[];
			const int tokens = height * width;
			const int padded = (tokens + KB - 1) / KB * KB;
			__half *sk = reinterpret_cast<__half*>(smem_raw);
			__half *sv = sk + padded * LD;
			float *st = reinterpret_cast<float*>(sv + padded * LD);
			int *spos = reinterpret_cast<int*>(st + table_n * table_pad); // (h << 16) | w of every token

			const int head = blockIdx.x, b = blockIdx.y;
			const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
			const int g = lane / 4, tig = lane % 4;
			const int stride = parts * heads * D; // channels per token
			const __half *base = input + static_cast<long long>(b) * tokens * stride;
			const int k_off = (parts == 3 ? 1 : 0) * heads * D + head * D;
			const int v_off = (parts - 1) * heads * D + head * D;

			// stage K and V (16 bytes per access), zero rows beyond the last token
			constexpr int CHUNKS = D / 8;
			for (int i = threadIdx.x; i < padded * CHUNKS; i += blockDim.x)
			{
				const int t = i / CHUNKS, ch = i % CHUNKS;
				uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
				if (t < tokens)
				{
					kv = *reinterpret_cast<const uint4*>(base + static_cast<long long>(t) * stride + k_off + ch * 8);
					vv = *reinterpret_cast<const uint4*>(base + static_cast<long long>(t) * stride + v_off + ch * 8);
				}
				*reinterpret_cast<uint4*>(sk + t * LD + ch * 8) = kv;
				*reinterpret_cast<uint4*>(sv + t * LD + ch * 8) = vv;
			}
			for (int i = threadIdx.x; i < table_n * table_pad; i += blockDim.x)
				st[i] = __half2float(table[static_cast<long long>(head) * table_n * table_pad + i]) * LOG2E; // scores live in the log2 domain
			// Relative offsets never leave the table when the board is no larger than the table's range + 1 (the usual case: the
			// table is built for the board).  The index is then linear in the two positions and needs no clamping:
			// (jh - qh + range) * pad + (jw - qw + range) = lin(j) - lin(q) + range * (pad + 1), lin(t) = th * pad + tw.
			const int range = (table_n - 1) / 2;
			const bool linear_bias = (height - 1 <= range) && (width - 1 <= range);
			for (int i = threadIdx.x; i < padded; i += blockDim.x)
			{ // slots beyond the last token repeat the last token's position, so that every index formed from them stays in the table
				const int t = min(i, tokens - 1);
				spos[i] = linear_bias ? (t / width) * table_pad + (t % width) : (((t / width) << 16) | (t % width));
			}
			__syncthreads();

			const float scale = rsqrtf(static_cast<float>(D)) * LOG2E; // exp(x) = 2^(x log2 e): one multiply less per score
			const uint32_t sv_addr = static_cast<uint32_t>(__cvta_generic_to_shared(sv));

			for (int q0 = warp * 16 * QT; q0 < tokens; q0 += WARPS * 16 * QT)
			{
				// per query tile t: Q fragments of rows r[t][0] = q0 + 16 t + g and r[t][1] = r[t][0] + 8
				uint32_t qa[QT][KC][4];
				int r[QT][2], lin[QT][2], qh[QT][2], qw[QT][2];
				float o[QT][NT][4], m[QT][2], l[QT][2];
#pragma unroll
				for (int t = 0; t < QT; t++)
				{
					r[t][0] = q0 + t * 16 + g;
					r[t][1] = r[t][0] + 8;
#pragma unroll
					for (int kc = 0; kc < KC; kc++)
					{
						const int col = head * D + kc * 16 + tig * 2;
#pragma unroll
						for (int half = 0; half < 2; half++)
						{
							const bool ok = r[t][half] < tokens;
							const __half *src = base + static_cast<long long>(r[t][half]) * stride + col;
							qa[t][kc][half] = ok ? *reinterpret_cast<const uint32_t*>(src) : 0u;
							qa[t][kc][2 + half] = ok ? *reinterpret_cast<const uint32_t*>(src + 8) : 0u;
						}
					}
#pragma unroll
					for (int half = 0; half < 2; half++)
					{
						const int pq = spos[min(r[t][half], tokens - 1)];
						qh[t][half] = pq >> 16; // clamped form
						qw[t][half] = pq & 0xFFFF;
						lin[t][half] = range * (table_pad + 1) - pq; // linear form
						m[t][half] = -1.0e30f;
						l[t][half] = 0.0f;
					}
#pragma unroll
					for (int n = 0; n < NT; n++)
#pragma unroll
						for (int k = 0; k < 4; k++)
							o[t][n][k] = 0.0f;
				}

				for (int kb = 0; kb < padded; kb += KB)
				{
					float s[QT][KB / 8][4];
#pragma unroll
					for (int nt = 0; nt < KB / 8; nt++)
					{
#pragma unroll
						for (int t = 0; t < QT; t++)
#pragma unroll
							for (int k = 0; k < 4; k++)
								s[t][nt][k] = 0.0f;
						const __half *krow = sk + (kb + nt * 8 + g) * LD + tig * 2;
#pragma unroll
						for (int kc = 0; kc < KC; kc++)
						{
							const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + kc * 16);
							const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + kc * 16 + 8);
#pragma unroll
							for (int t = 0; t < QT; t++)
								mma_16816(s[t][nt], qa[t][kc], b0, b1);
						}
					}
#pragma unroll
					for (int t = 0; t < QT; t++)
					{
						// scale, relative-position bias, mask keys beyond the last token; block maxima
						float bm0 = -1.0e30f, bm1 = -1.0e30f;
#pragma unroll
						for (int nt = 0; nt < KB / 8; nt++)
#pragma unroll
							for (int e = 0; e < 2; e++)
							{
								const int j = kb + nt * 8 + tig * 2 + e;
								float v0 = s[t][nt][e] * scale, v1 = s[t][nt][2 + e] * scale;
								if (table != nullptr)
								{
									const int pj = spos[j];
									if (linear_bias)
									{
										v0 += st[pj + lin[t][0]];
										v1 += st[pj + lin[t][1]];
									}
									else
									{
										const int jh = pj >> 16, jw = pj & 0xFFFF;
										v0 += st[(min(max(jh - qh[t][0], -range), range) + range) * table_pad + min(max(jw - qw[t][0], -range), range) + range];
										v1 += st[(min(max(jh - qh[t][1], -range), range) + range) * table_pad + min(max(jw - qw[t][1], -range), range) + range];
									}
								}
								if (kb + KB > tokens && j >= tokens)
								{
									v0 = -1.0e30f;
									v1 = -1.0e30f;
								}
								s[t][nt][e] = v0;
								s[t][nt][2 + e] = v1;
								bm0 = fmaxf(bm0, v0);
								bm1 = fmaxf(bm1, v1);
							}
						bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 1));
						bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, 2));
						bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 1));
						bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, 2));
						const float n0 = fmaxf(m[t][0], bm0), n1 = fmaxf(m[t][1], bm1);
						const float c0 = exp2_approx(m[t][0] - n0), c1 = exp2_approx(m[t][1] - n1);
						m[t][0] = n0;
						m[t][1] = n1;
						float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
						for (int nt = 0; nt < KB / 8; nt++)
#pragma unroll
							for (int e = 0; e < 2; e++)
							{
								const float e0 = exp2_approx(s[t][nt][e] - n0), e1 = exp2_approx(s[t][nt][2 + e] - n1);
								s[t][nt][e] = e0;
								s[t][nt][2 + e] = e1;
								sum0 += e0;
								sum1 += e1;
							}
						l[t][0] = l[t][0] * c0 + sum0;
						l[t][1] = l[t][1] * c1 + sum1;
#pragma unroll
						for (int n = 0; n < NT; n++)
						{
							o[t][n][0] *= c0;
							o[t][n][1] *= c0;
							o[t][n][2] *= c1;
							o[t][n][3] *= c1;
						}
					}
					// O += P V: the accumulator layout of two neighbouring score tiles is the A-fragment layout of one k16 step
#pragma unroll
					for (int kc = 0; kc < KB / 16; kc++)
					{
						uint32_t pa[QT][4];
#pragma unroll
						for (int t = 0; t < QT; t++)
						{
							pa[t][0] = pack_half2(s[t][2 * kc][0], s[t][2 * kc][1]);
							pa[t][1] = pack_half2(s[t][2 * kc][2], s[t][2 * kc][3]);
							pa[t][2] = pack_half2(s[t][2 * kc + 1][0], s[t][2 * kc + 1][1]);
							pa[t][3] = pack_half2(s[t][2 * kc + 1][2], s[t][2 * kc + 1][3]);
						}
#pragma unroll
						for (int n = 0; n < NT; n++)
						{
							uint32_t b0, b1;
							// lanes 0-15 name the 16 key rows of this step; the transposing load returns V^T fragments
							ldmatrix_x2_trans(b0, b1, sv_addr + static_cast<uint32_t>(((kb + kc * 16 + (lane & 15)) * LD + n * 8) * 2));
#pragma unroll
							for (int t = 0; t < QT; t++)
								mma_16816(o[t][n], pa[t], b0, b1);
						}
					}
				}
				__half *out = output + static_cast<long long>(b) * tokens * heads * D + head * D;
#pragma unroll
				for (int t = 0; t < QT; t++)
				{
					// the row sums live in the four lanes of a quad
					float l0 = l[t][0], l1 = l[t][1];
					l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
					l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
					l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
					l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
					const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
#pragma unroll
					for (int n = 0; n < NT; n++)
					{
						if (r[t][0] < tokens)
							*reinterpret_cast<uint32_t*>(out + static_cast<long long>(r[t][0]) * heads * D + n * 8 + tig * 2) = pack_half2(o[t][n][0] * inv0,
									o[t][n][1] * inv0);
						if (r[t][1] < tokens)
							*reinterpret_cast<uint32_t*>(out + static_cast<long long>(r[t][1]) * heads * D + n * 8 + tig * 2) = pack_half2(o[t][n][2] * inv1,
									o[t][n][3] * inv1);
					}
				}
			}
		}

		template<int D, int QT, int KB>
		bool launch(mlContext_t ctx, __half *output, const __half *input, const __half *table, int batch, int height, int width, int heads, int parts,
				int table_n, int table_pad)
		{
			const int tokens = height * width;
			const int padded = (tokens + KB - 1) / KB * KB;
			const size_t smem = static_cast<size_t>(2) * padded * (D + 8) * sizeof(__half) + static_cast<size_t>(table_n) * table_pad * sizeof(float)
					+ static_cast<size_t>(padded) * sizeof(int);
			if (smem > 200 * 1024)
				return false;
			if (!check_cuda(ctx, cudaFuncSetAttribute(kernel_mha_mma<D, QT, KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
					"attention: shared memory opt-in"))
				return false;
			kernel_mha_mma<D, QT, KB> <<<dim3(heads, batch), WARPS * 32, smem, use_stream(ctx)>>>(output, input, table, height, width, heads, parts,
					table_n, table_pad);
			MB200_COUNT_LAUNCH();
			check_cuda(ctx, cudaGetLastError(), "cuda_multi_head_attention_forward");
			return true;
		}
		/* Variant by environment for measurements: MINML_B200_MHA_VARIANT = 0 (one query tile, 64 keys), 1 (two tiles, 64 keys),
		 * 2 (two tiles, 32 keys: the default), 3 (one tile, 32 keys). */
		int mha_variant()
		{
			static const int v = []
			{
				const char *e = std::getenv("MINML_B200_MHA_VARIANT");
				return (e != nullptr && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 2;
			}();
			return v;
		}
		template<int D>
		bool launch_small_head(mlContext_t ctx, __half *o, const __half *x, const __half *t, int batch, int height, int width, int heads, int parts,
				int table_n, int table_pad)
		{
			switch (mha_variant())
			{
				case 0:
					return launch<D, 1, 64>(ctx, o, x, t, batch, height, width, heads, parts, table_n, table_pad);
				case 1:
					return launch<D, 2, 64>(ctx, o, x, t, batch, height, width, heads, parts, table_n, table_pad);
				case 3:
					return launch<D, 1, 32>(ctx, o, x, t, batch, height, width, heads, parts, table_n, table_pad);
				default:
					return launch<D, 2, 32>(ctx, o, x, t, batch, height, width, heads, parts, table_n, table_pad);
			}
		}
	}

	/* Returns false when the shape is outside what this kernel handles (the caller then uses the generic kernel). */
	bool mha_forward_mma(mlContext_t ctx, void *output, const void *input, const void *table, int batch, int height, int width, int heads,
			int head_dim, int parts, int table_n, int table_pad)
	{
		if (height >= 32768 || width >= 32768 || batch > 65535)
			return false;
		if (!aligned_to(input, 16) || !aligned_to(output, 4) || (parts * heads * head_dim) % 8 != 0)
			return false;
		__half *o = reinterpret_cast<__half*>(output);
		const __half *x = reinterpret_cast<const __half*>(input);
		const __half *t = reinterpret_cast<const __half*>(table);
		switch (head_dim)
		{
			case 16:
				return launch_small_head<16>(ctx, o, x, t, batch, height, width, heads, parts, table_n, table_pad);
			case 32:
				return launch_small_head<32>(ctx, o, x, t, batch, height, width, heads, parts, table_n, table_pad);
			case 64:
				return launch<64, 1, 64>(ctx, o, x, t, batch, height, width, heads, parts, table_n, table_pad);
			case 128:
				return launch<128, 1, 64>(ctx, o, x, t, batch, height, width, heads, parts, table_n, table_pad);
			default:
				return false;
		}
	}
} /* namespace mb200 */
