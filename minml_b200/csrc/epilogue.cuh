/*
 * epilogue.cuh -- pieces shared by the epilogues of the tcgen05 kernels (conv_igemm.cu, gemm_tc.cu): 16-byte shared-memory
 * accesses for staging rows, fp16 <-> fp32 helpers on 8-element groups, the compact activation and saturating int8 packing.
 *
 * Staging: a warp owns 32 accumulator rows (one per lane) of a 32-column chunk.  Global reads of the residual and writes of
 * the result go through a per-warp shared-memory buffer so that one instruction touches 8 rows x 64 contiguous bytes
 * instead of 32 rows x 16 bytes: lane -> (row lane / 4 + 8 i, 16-byte segment lane % 4).
 */
#pragma once

#include "common.cuh"

#include <cuda_fp16.h>
#include <cstdint>

namespace mb200
{
	namespace epi
	{
		constexpr int PITCH = 80; // bytes per staged row: 64 of payload + 16 of padding against bank conflicts
		constexpr int WARP_BYTES = 32 * PITCH;

		__device__ __forceinline__ void st_shared_v4(uint32_t dst, const uint4 &v)
		{
			asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
		}
		__device__ __forceinline__ uint4 ld_shared_v4(uint32_t src)
		{
			uint4 v;
			asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(src) : "memory");
			return v;
		}
		__device__ __forceinline__ bool aligned_to_16(const void *ptr)
		{
			return (reinterpret_cast<uintptr_t>(ptr) % 16) == 0;
		}
		/* v[0..7] += scale * (8 halves in raw) */
		__device__ __forceinline__ void add_half8(float *v, const uint4 &raw, float scale = 1.0f)
		{
			const uint32_t w4[4] = { raw.x, raw.y, raw.z, raw.w };
#pragma unroll
			for (int t = 0; t < 4; t++)
			{
				const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w4[t]));
				v[2 * t] += scale * f.x;
				v[2 * t + 1] += scale * f.y;
			}
		}
		__device__ __forceinline__ uint4 pack_half8(const float *v)
		{
			uint4 pk;
			const __half2 h0 = __floats2half2_rn(v[0], v[1]);
			const __half2 h1 = __floats2half2_rn(v[2], v[3]);
			const __half2 h2 = __floats2half2_rn(v[4], v[5]);
			const __half2 h3 = __floats2half2_rn(v[6], v[7]);
			pk.x = *reinterpret_cast<const uint32_t*>(&h0);
			pk.y = *reinterpret_cast<const uint32_t*>(&h1);
			pk.z = *reinterpret_cast<const uint32_t*>(&h2);
			pk.w = *reinterpret_cast<const uint32_t*>(&h3);
			return pk;
		}

		/* Everything but ReLU goes through one out-of-line call per element: the epilogue code stays small enough for the
		 * instruction cache that the producer, the MMA issue and the epilogue share. */
		static __device__ __noinline__ float activation_out_of_line(float x, int act)
		{
			return apply_activation(x, act);
		}
		__device__ __forceinline__ void activate32(float (&v)[32], int act)
		{
			if (act == ACTIVATION_RELU)
			{
#pragma unroll
				for (int j = 0; j < 32; j++)
					v[j] = fmaxf(v[j], 0.0f);
			}
			else if (act != ACTIVATION_LINEAR)
			{
#pragma unroll
				for (int j = 0; j < 32; j++)
					v[j] = activation_out_of_line(v[j], act);
			}
		}
		/* Requantisation of an int32 accumulator, the one formula of every int8 output path of the library (fused convolution,
		 * tensor-core GEMM epilogue, eager cuda_quantized_scale_shift_act).  It is the arithmetic of the reference's CPU layer
		 * (src/layers/Conv2D.cpp:283-304 with AffineTransform::get_inverse, include/minml/layers/quantization.hpp:47-55), step
		 * for step and with every step rounded on its own -- no fused multiply-add -- so that all paths give the same bits:
		 *     x = acc * scale[c] + shift[c]  (+ (ext * s_e + z_e));   activation;   q = clamp(round(x * (1 / s_o) + (-z_o / s_o)))
		 * with round-half-away-from-zero.  (The reference's CUDA kernel divides instead, round((x - z_o) / s_o),
		 * src/backend/cuda/kernels/quantized.cu:44-47, which can differ from its CPU layer by one step.) */
		__device__ __forceinline__ float requant_real(int acc, float scale, float shift)
		{
			return __fadd_rn(__fmul_rn(static_cast<float>(acc), scale), shift);
		}
		__device__ __forceinline__ float requant_add_ext(float x, int e, float ext_scale, float ext_shift)
		{
			return __fadd_rn(x, __fadd_rn(__fmul_rn(static_cast<float>(e), ext_scale), ext_shift));
		}
		/* Rounded but not yet saturated: the float -> int conversion saturates at the int32 range, pack_sat_s8x4 or
		 * requant_clamp then at the int8 range, which together are the reference's clamp(round(.), -128, 127).
		 * Round half away from zero (std::round) is computed as trunc(y + copysign(0.49999997, y)), 0.49999997 being the
		 * largest float below one half: three instructions instead of the eight of roundf, and the same result for EVERY
		 * float -- checked exhaustively for |y| < 2^23 (tests/test_oracle.py samples it); beyond that y is an integer and the
		 * addition returns it unchanged. */
		__device__ __forceinline__ int requant_round(float x, float inv_out_scale, float inv_out_shift)
		{
			const float y = __fadd_rn(__fmul_rn(x, inv_out_scale), inv_out_shift);
			const float half_towards_y = __uint_as_float((__float_as_uint(y) & 0x80000000u) | 0x3EFFFFFFu);
			return __float2int_rz(__fadd_rn(y, half_towards_y));
		}
		__device__ __forceinline__ int requant_clamp(int q)
		{
			return max(-128, min(127, q));
		}
		/* Four int32 -> four int8 with saturation, byte t of the result = value t. */
		__device__ __forceinline__ uint32_t pack_sat_s8x4(int a, int b, int c, int d)
		{
			uint32_t hi, out;
			asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
			asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
			return out;
		}
	} /* namespace epi */
} /* namespace mb200 */
