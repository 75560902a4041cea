// Device-side pieces of the Q8_0 arithmetic shared by every kernel: the activation quantiser and the
// packed int8 dot.  The quantiser reproduces quantize_row_q8_0 of the reference
// (include/nihilus-incl/cpu/avx_2.hpp:4439-4489) bit for bit: IEEE divide and multiply with no
// contraction, round-half-even to int, fp16 round-to-nearest-even for the stored scale.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace nhb {

	constexpr int QK = 32;

	struct act_scale {
		float id;// 127 / amax (0 when amax == 0)
		float d;// fp16-rounded amax / 127, widened back to f32
	};

	__device__ __forceinline__ act_scale q8_scales(float amax) {
		act_scale s;
		s.d	 = __half2float(__float2half_rn(__fdiv_rn(amax, 127.f)));
		s.id = (amax != 0.0f) ? __fdiv_rn(127.f, amax) : 0.0f;
		return s;
	}

	// one quant; the reference saturates through two pack instructions, NaN handling differs (0 here)
	__device__ __forceinline__ int q8_quant(float x, float id) {
		int q = __float2int_rn(__fmul_rn(x, id));
		return max(-128, min(127, q));
	}

	__device__ __forceinline__ uint32_t q8_pack4(float a, float b, float c, float d, float id) {
		return (static_cast<uint32_t>(q8_quant(a, id)) & 0xffu) | ((static_cast<uint32_t>(q8_quant(b, id)) & 0xffu) << 8) |
			((static_cast<uint32_t>(q8_quant(c, id)) & 0xffu) << 16) | ((static_cast<uint32_t>(q8_quant(d, id)) & 0xffu) << 24);
	}

	__device__ __forceinline__ float absmax4(float4 v, float m) {
		return fmaxf(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))), m);
	}

	// silu(g) * u, the reference's ffn_silu -> ffn_gate_par pair (include/nihilus-incl/infra/core_traits.hpp:982-986; its
	// kernels for them are empty, the traits name the arithmetic): g / (1 + exp(-g)) in f32 with an IEEE divide, then one
	// f32 multiply
	__device__ __forceinline__ float swiglu(float g, float u) {
		return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
	}
	__device__ __forceinline__ float4 swiglu4(float4 g, float4 u) {
		return make_float4(swiglu(g.x, u.x), swiglu(g.y, u.y), swiglu(g.z, u.z), swiglu(g.w, u.w));
	}

	// One lane of the reference's simd_sum_squares (include/nihilus-incl/cpu/avx_2.hpp:758-779): acc = fma(v, v, acc) over
	// r[0], r[8], r[16], ... (`steps` values), strictly in that order.  The fmas depend on each other (4 cycles a step
	// at best), so the only thing to hide is the latency of the shared-memory loads: a 16-entry register window, each
	// slot refilled for step s + 16 right after step s consumed it (5.3 cycles a step measured; loading 16 values and
	// then running 16 fmas takes 7.7, a two-buffer scheme with a copy 11.5).
	__device__ __forceinline__ float sum_squares_lane(const float* r, int steps) {
		float acc = 0.f;
		int s	  = 0;
		if (steps >= 16) {
			float buf[16];
#pragma unroll
			for (int j = 0; j < 16; ++j)
				buf[j] = r[8 * j];
			for (; s + 32 <= steps; s += 16) {
#pragma unroll
				for (int j = 0; j < 16; ++j) {
					acc	   = __fmaf_rn(buf[j], buf[j], acc);
					buf[j] = r[8 * (s + 16 + j)];
				}
			}
#pragma unroll
			for (int j = 0; j < 16; ++j)
				acc = __fmaf_rn(buf[j], buf[j], acc);
			s += 16;
		}
		for (; s < steps; ++s)
			acc = __fmaf_rn(r[8 * s], r[8 * s], acc);
		return acc;
	}

	// exact dot of 16 int8 pairs
	__device__ __forceinline__ int dot16(const uint4& w, const uint4& a) {
		int s = __dp4a(static_cast<int>(w.x), static_cast<int>(a.x), 0);
		s	  = __dp4a(static_cast<int>(w.y), static_cast<int>(a.y), s);
		s	  = __dp4a(static_cast<int>(w.z), static_cast<int>(a.z), s);
		s	  = __dp4a(static_cast<int>(w.w), static_cast<int>(a.w), s);
		return s;
	}

}
