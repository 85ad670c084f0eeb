/*
 * tc.cuh -- inline-PTX wrappers for the Blackwell (sm_100a) tensor path: mbarrier, TMA (cp.async.bulk.tensor),
 * tensor memory (tcgen05.alloc / ld / dealloc) and tcgen05.mma with shared-memory operand descriptors.
 *
 * Every wait in here is bounded: after SPIN_LIMIT failed polls the waiter raises the CTA-wide abort flag and
 * returns false, so a kernel built from these pieces always terminates and reports through its status word.
 */
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace mb200
{
	namespace tc
	{
		constexpr uint32_t SPIN_LIMIT = 1u << 22;

		__device__ __forceinline__ uint32_t smem_u32(const void *ptr)
		{
			return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
		}
		__device__ __forceinline__ bool elect_one()
		{
			uint32_t pred = 0;
			asm volatile(
					"{\n\t"
					".reg .pred P;\n\t"
					"elect.sync _|P, 0xffffffff;\n\t"
					"selp.u32 %0, 1, 0, P;\n\t"
					"}\n" : "=r"(pred));
			return pred != 0;
		}

		/* ---------------------------------------------------------------- mbarrier */
		__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
		{
			asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count));
		}
		__device__ __forceinline__ void fence_mbar_init()
		{
			asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
		}
		__device__ __forceinline__ void mbar_arrive(uint32_t bar)
		{
			asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
		}
		__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
		{
			asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
		}
		__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
		{
			uint32_t done;
			asm volatile(
					"{\n\t"
					".reg .pred P;\n\t"
					"mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
					"selp.u32 %0, 1, 0, P;\n\t"
					"}\n" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
			return done != 0;
		}
		/* Bounded wait.  `abort_flag` lives in shared memory and is shared by all roles of the CTA. */
		__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t limit)
		{
			for (uint32_t it = 0; it < limit; ++it)
			{
				if (mbar_try_wait(bar, parity))
					return true;
				if ((it & 255u) == 255u && *abort_flag != 0)
					return false;
			}
			*abort_flag = 1;
			return false;
		}
		__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag)
		{
			return mbar_wait_limited(bar, parity, abort_flag, SPIN_LIMIT);
		}

		/* Wait that leaves most of the issue slots to the other warps: after a few immediate polls the thread sleeps `sleep_ns` between
		 * polls.  The bound is a time, two seconds of the global timer, checked every 256 polls together with the abort flag. */
		__device__ __forceinline__ uint64_t global_timer_ns()
		{
			uint64_t t;
			asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
			return t;
		}
		__device__ __forceinline__ bool mbar_wait_sleeping(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t sleep_ns)
		{
#pragma unroll 1
			for (int it = 0; it < 8; ++it)
				if (mbar_try_wait(bar, parity))
					return true;
			const uint64_t start = global_timer_ns();
#pragma unroll 1
			for (uint32_t it = 1;; ++it)
			{
				__nanosleep(sleep_ns);
				if (mbar_try_wait(bar, parity))
					return true;
				if ((it & 255u) == 0u)
				{
					if (*abort_flag != 0)
						return false;
					if (global_timer_ns() - start > 2000000000ull)
						break;
				}
			}
			*abort_flag = 1;
			return false;
		}

		/* mbar_wait for a whole warp, with an outcome all its lanes share (see mbar_wait_warp below for why) */
		__device__ __forceinline__ bool mbar_wait_all_lanes(uint32_t bar, uint32_t parity, volatile int *abort_flag)
		{
			return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag) ? 1 : 0) != 0;
		}
		/* The same for a whole warp, with an outcome all its lanes share: what follows such a wait are warp-wide tensor-memory
		 * instructions, which a warp split by a timeout on some of its lanes must not reach. */
		__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t sleep_ns)
		{
			return __all_sync(0xFFFFFFFFu, mbar_wait_sleeping(bar, parity, abort_flag, sleep_ns) ? 1 : 0) != 0;
		}

		/* ---------------------------------------------------------------- TMA */
		__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map)
		{
			asm volatile("prefetch.tensormap [%0];" :: "l"(reinterpret_cast<uint64_t>(map)) : "memory");
		}
		__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2)
		{
			asm volatile(
					"cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
					:: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
		}
		__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
		{
			asm volatile(
					"cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
					:: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
		}
		/* Store of a shared-memory box to global memory through a tensor map; completion is tracked by the thread's bulk groups. */
		__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2)
		{
			asm volatile(
					"cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
					:: "l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
		}
		__device__ __forceinline__ void bulk_commit_group()
		{
			asm volatile("cp.async.bulk.commit_group;" ::: "memory");
		}
		/* Returns once all but the newest PENDING bulk groups of this thread have finished READING shared memory. */
		template<int PENDING>
		__device__ __forceinline__ void bulk_wait_group_read()
		{
			asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(PENDING) : "memory");
		}
		/* Makes generic-proxy writes to shared memory visible to the async proxy (TMA / tcgen05.mma operand reads). */
		__device__ __forceinline__ void fence_proxy_async_smem()
		{
			asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
		}

		/* ---------------------------------------------------------------- tensor memory */
		__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns)
		{
			asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_result), "r"(columns) : "memory");
		}
		__device__ __forceinline__ void tmem_relinquish()
		{
			asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
		}
		__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
		{
			asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(columns) : "memory");
		}
		__device__ __forceinline__ void tcgen05_fence_before()
		{
			asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
		}
		__device__ __forceinline__ void tcgen05_fence_after()
		{
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
		}
		__device__ __forceinline__ void tmem_wait_ld()
		{
			asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
		}
		/* 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives row (lane base + t). */
		__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
		{
			asm volatile(
					"tcgen05.ld.sync.aligned.32x32b.x32.b32 "
					"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
					"%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
					: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
					"=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
					"=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
					"=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
					: "r"(taddr) : "memory");
		}
		__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
		{
			asm volatile(
					"tcgen05.ld.sync.aligned.32x32b.x16.b32 "
					"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
					: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
					"=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
					: "r"(taddr) : "memory");
		}
		__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8])
		{
			asm volatile(
					"tcgen05.ld.sync.aligned.32x32b.x8.b32 "
					"{%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
					: "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
					: "r"(taddr) : "memory");
		}

		/* ---------------------------------------------------------------- tcgen05.mma */
		/* Shared-memory operand descriptor for a K-major tile stored with the 128-byte swizzle: rows of 128 bytes,
		 * 8-row groups 1024 bytes apart (stride byte offset), leading byte offset unused (1), descriptor version 1. */
		__device__ __forceinline__ uint64_t make_desc_k_sw128(uint32_t smem_addr)
		{
			uint64_t desc = 0;
			desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
			desc |= static_cast<uint64_t>(1) << 16;
			desc |= static_cast<uint64_t>(1024 >> 4) << 32;
			desc |= static_cast<uint64_t>(1) << 46;
			desc |= static_cast<uint64_t>(2) << 61;
			return desc;
		}
		/* MN-major operand, 128-byte swizzle: rows of 128 bytes along M (or N), one row per K index; 8 K indices form a 1024-byte group
		 * (stride byte offset); `block_bytes` (leading byte offset) separates the blocks of 128 bytes along M (or N).
		 * `atom_32b`: 32-bit elements in this order: the swizzle moves 32-byte pieces and repeats every 4 rows (the copy engine writes it
		 * with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B), so a group is 4 K indices, 512 bytes (found by trying the combinations of layout
		 * code, copy swizzle and stride against an exact integer product: this is the one that gives it). */
		__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr, uint32_t block_bytes, bool atom_32b = false)
		{
			uint64_t desc = 0;
			desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
			desc |= static_cast<uint64_t>(block_bytes >> 4) << 16;
			desc |= static_cast<uint64_t>((atom_32b ? 512 : 1024) >> 4) << 32;
			desc |= static_cast<uint64_t>(1) << 46;
			desc |= static_cast<uint64_t>(atom_32b ? 1 : 2) << 61;
			return desc;
		}
		/* Instruction descriptors: D fp32 <- fp16 x fp16, and D s32 <- s8 x s8; M = 128; operands K-major unless bit 15 (A) / 16 (B) is set. */
		__host__ __device__ constexpr uint32_t make_idesc_f16(int n)
		{
			return (1u << 4) | (0u << 7) | (0u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
		}
		__host__ __device__ constexpr uint32_t make_idesc_i8(int n)
		{
			return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
		}
		/* D fp32 <- tf32 x tf32: fp32 operands in shared memory, of which the tensor core reads the upper 19 bits. */
		__host__ __device__ constexpr uint32_t make_idesc_tf32(int n)
		{
			return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
		}
		template<int KIND> // 0: kind::f16, 1: kind::i8, 2 and above: kind::tf32
		__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
		{
			if (KIND >= 2)
				asm volatile(
						"{\n\t"
						".reg .pred p;\n\t"
						"setp.ne.b32 p, %4, 0;\n\t"
						"tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
						"}\n" :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
			else if (KIND == 0)
				asm volatile(
						"{\n\t"
						".reg .pred p;\n\t"
						"setp.ne.b32 p, %4, 0;\n\t"
						"tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
						"}\n" :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
			else
				asm volatile(
						"{\n\t"
						".reg .pred p;\n\t"
						"setp.ne.b32 p, %4, 0;\n\t"
						"tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
						"}\n" :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
		}
		/* A from tensor memory (128 lanes = rows; a 32-bit column holds two consecutive 16-bit elements along K), B from shared memory */
		__device__ __forceinline__ void mma_ts_f16(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
		{
			asm volatile(
					"{\n\t"
					".reg .pred p;\n\t"
					"setp.ne.b32 p, %4, 0;\n\t"
					"tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
					"}\n" :: "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
		}
		/* The mbarrier receives one arrival once every tcgen05.mma issued so far by this thread has completed. */
		__device__ __forceinline__ void mma_commit(uint32_t bar)
		{
			asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
		}

		/* ---------------------------------------------------------------- CTA pairs (cluster of 2, tcgen05 cta_group::2)
		 * One tcgen05.mma issued by the even CTA of the pair multiplies a 256-row A tile (128 rows in each CTA's shared
		 * memory) by a B tile whose N rows are split in halves between the two CTAs; each CTA's tensor memory receives
		 * the 128 accumulator rows of its own A half.  Both CTAs use the same shared-memory layout, so one descriptor
		 * names the operand in both. */
		__device__ __forceinline__ uint32_t cluster_ctarank()
		{
			uint32_t r;
			asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
			return r;
		}
		/* shared::cluster address of the same shared-memory location in the CTA of rank `cta` */
		__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta)
		{
			uint32_t r;
			asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
			return r;
		}
		/* All threads of all CTAs of the cluster; release / acquire at cluster scope. */
		__device__ __forceinline__ void cluster_sync()
		{
			asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
			asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
		}
		/* `bar` is a shared::cluster address (own or peer CTA). */
		__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar)
		{
			asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(bar) : "memory");
		}
		__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
		{
			uint32_t done;
			asm volatile(
					"{\n\t"
					".reg .pred P;\n\t"
					"mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
					"selp.u32 %0, 1, 0, P;\n\t"
					"}\n" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
			return done != 0;
		}
		/* Bounded wait on an own barrier whose arrivals come from the peer CTA as well. */
		__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag)
		{
			for (uint32_t it = 0; it < SPIN_LIMIT; ++it)
			{
				if (mbar_try_wait_cluster(bar, parity))
					return true;
				if ((it & 255u) == 255u && *abort_flag != 0)
					return false;
			}
			*abort_flag = 1;
			return false;
		}
		/* TMA loads into this CTA's shared memory whose completion is counted on a barrier of either CTA of the pair
		 * (`bar` is a shared::cluster address).  The source is always this GPU's own memory; no multicast. */
		__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2)
		{
			asm volatile(
					"cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
					:: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
		}
		__device__ __forceinline__ void tma_load_im2col_4d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c, int w, int h, int n,
				uint16_t off_w, uint16_t off_h)
		{
			asm volatile(
					"cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
					:: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h) : "memory");
		}
		template<int KIND>
		__device__ __forceinline__ void mma_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
		{
			if (KIND == 0)
				asm volatile(
						"{\n\t"
						".reg .pred p;\n\t"
						"setp.ne.b32 p, %4, 0;\n\t"
						"tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
						"}\n" :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
			else
				asm volatile(
						"{\n\t"
						".reg .pred p;\n\t"
						"setp.ne.b32 p, %4, 0;\n\t"
						"tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
						"}\n" :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
		}
		/* One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair, once every tcgen05.mma issued so
		 * far by this thread has completed.  (A barrier arrival, not a data load.) */
		__device__ __forceinline__ void mma_commit_pair(uint32_t bar)
		{
			asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
					:: "r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
		}
		/* Instruction descriptors with M = 256 (128 rows per CTA). */
		__host__ __device__ constexpr uint32_t make_idesc_f16_pair(int n)
		{
			return (1u << 4) | (0u << 7) | (0u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
		}
		__host__ __device__ constexpr uint32_t make_idesc_i8_pair(int n)
		{
			return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
		}

		/* ---------------------------------------------------------------- pieces of the attention kernels */
		constexpr float LOG2E = 1.4426950408889634f;
		__device__ __forceinline__ float exp2_approx(float x)
		{
			float y;
			asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
			return y;
		}
		/* K-major operand with 64-byte rows and the 64-byte swizzle: 8-row groups 512 bytes apart */
		__device__ __forceinline__ uint64_t make_desc_k_sw64(uint32_t smem_addr)
		{
			uint64_t desc = 0;
			desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
			desc |= static_cast<uint64_t>(1) << 16;
			desc |= static_cast<uint64_t>(512 >> 4) << 32;
			desc |= static_cast<uint64_t>(1) << 46;
			desc |= static_cast<uint64_t>(4) << 61;
			return desc;
		}
		/* MN-major operand of up to 32 fp16 along MN (one 64-byte row per K index, 64-byte swizzle): 8-row groups along K 512 bytes apart */
		__device__ __forceinline__ uint64_t make_desc_mn_sw64(uint32_t smem_addr)
		{
			uint64_t desc = 0;
			desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
			desc |= static_cast<uint64_t>(512 >> 4) << 16;
			desc |= static_cast<uint64_t>(512 >> 4) << 32;
			desc |= static_cast<uint64_t>(1) << 46;
			desc |= static_cast<uint64_t>(4) << 61;
			return desc;
		}
		__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32])
		{
			asm volatile(
					"tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
					"{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
					"%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
					:: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
					"r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
					"r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
					"r"(r[30]), "r"(r[31]) : "memory");
		}
		__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[32])
		{
			asm volatile(
					"tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
					"{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
					:: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
					"r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
		}
		__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16])
		{
			asm volatile(
					"tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
					"{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
					:: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
					"r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
		}
		__device__ __forceinline__ void tmem_wait_st()
		{
			asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
		}
		/* 32 (or, for the last chunk of a row, 16) columns of this thread's lane */
		__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t (&r)[32], bool wide)
		{
			if (wide)
				tmem_ld_32x32(taddr, r);
			else
			{
				uint32_t h[16];
				tmem_ld_32x16(taddr, h);
#pragma unroll
				for (int i = 0; i < 16; i++)
					r[i] = h[i];
			}
			tmem_wait_ld();
		}
		__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
		{
			const __half2 h = __floats2half2_rn(lo, hi);
			return *reinterpret_cast<const uint32_t*>(&h);
		}
		__device__ __forceinline__ float max3(float a, float b, float c)
		{
			float d;
			asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
			return d;
		}
		__device__ __forceinline__ float ld_shared_f32(uint32_t addr)
		{
			float v;
			asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
			return v;
		}
	} /* namespace tc */

	/* Host side: cuTensorMapEncodeTiled fetched through the runtime so the library has no link-time dependency
	 * on libcuda.  Returns false (and records an error on ctx) when the driver entry point is unavailable. */
	bool encode_tensor_map(void *ctx, CUtensorMap *map, CUtensorMapDataType dtype, int rank, const void *base, const uint64_t *dims,
			const uint64_t *strides_bytes, const uint32_t *box, CUtensorMapSwizzle swizzle);
} /* namespace mb200 */
