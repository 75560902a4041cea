// Postlude for the in-place build of the reference's Q8_0 helpers -- TEST INFRASTRUCTURE ONLY.
// (see ref_prelude.hpp; the namespace opened there is closed here.)
//
// Exposes the reference's functions through a C ABI so that the Python tests can pin the oracle
// against them, and adds a row-partitioned, multi-threaded mul_mat driver around them so the same
// code can be timed as the CPU baseline.  The driver loop is ours (the reference's eval-time
// dispatcher, cpu/avx_2.hpp:4978-5004, runs every row on thread 0; its prompt-time driver,
// :4968-4975, does not compile); the per-row arithmetic is the reference's.

}// namespace nihilus

#include <cstdlib>
#include <thread>
#include <vector>

namespace {

	using blk = nihilus::block_q8_0<nihilus::half>;

	template<uint64_t n> float fixed_dot(const blk* w, const blk* a) {
		float s;
		nihilus::vec_dot_q8_0_q8_0<n>::impl(&s, w, a);
		return s;
	}

	float fixed_dot_rt(const blk* w, const blk* a, int n) {
		switch (n) {
#define NHB_CASE(v) \
	case v: \
		return fixed_dot<v>(w, a);
			NHB_CASE(1)
			NHB_CASE(2)
			NHB_CASE(3)
			NHB_CASE(4)
			NHB_CASE(5)
			NHB_CASE(6)
			NHB_CASE(7)
			NHB_CASE(8)
			NHB_CASE(9)
			NHB_CASE(10)
			NHB_CASE(11)
			NHB_CASE(12)
			NHB_CASE(13)
			NHB_CASE(14)
			NHB_CASE(15)
			NHB_CASE(16)
#undef NHB_CASE
			default:
				return NAN;
		}
	}

	// The reference's compile-time-n driver for n > 16 (cpu/avx_2.hpp:4715-4747) names an
	// ill-formed specialisation at :4682 and cannot be compiled; this is that loop, re-stated,
	// around the reference's own <16> and <remainder> kernels.
	float chunk16_dot(const blk* w, const blk* a, int64_t nb) {
		if (nb <= 16)
			return fixed_dot_rt(w, a, static_cast<int>(nb));
		const int64_t total_chunks = (nb + 15) / 16;
		const int rem			   = static_cast<int>(nb % 16);
		float total				   = 0.0f;
		for (int64_t c = 0; c + 1 < total_chunks; ++c) {
			total += fixed_dot<16>(w + c * 16, a + c * 16);
		}
		const int64_t last = total_chunks - 1;
		total += fixed_dot_rt(w + last * 16, a + last * 16, rem == 0 ? 16 : rem);
		return total;
	}

#define NHB_EVAL_SIZES(X) X(32) X(64) X(96) X(128) X(256) X(512) X(1024) X(2048) X(3072) X(4096) X(8192) X(11008) X(14336)

	bool eval_supported(int64_t K) {
#define NHB_CASE(v) \
	if (K == v) \
		return true;
		NHB_EVAL_SIZES(NHB_CASE)
#undef NHB_CASE
		return false;
	}

	float eval_dot(const float* x, const blk* w, int64_t K) {
#define NHB_CASE(v) \
	if (K == v) \
		return nihilus::vec_dot_q8_f32<v>::impl(x, w, 0);
		NHB_EVAL_SIZES(NHB_CASE)
#undef NHB_CASE
		return NAN;
	}

	template<typename fn_t> void parallel_rows(int64_t n0, int64_t n1, int threads, fn_t&& fn) {
		if (threads < 1)
			threads = 1;
		const int64_t rows = n1 - n0;
		if (rows <= 0)
			return;
		if (threads > rows)
			threads = static_cast<int>(rows);
		if (threads == 1) {
			fn(n0, n1);
			return;
		}
		const int64_t per = (rows + threads - 1) / threads;
		std::vector<std::thread> pool;
		for (int t = 0; t < threads; ++t) {
			const int64_t a = n0 + t * per;
			const int64_t b = a + per < n1 ? a + per : n1;
			if (a >= b)
				break;
			pool.emplace_back([=, &fn] {
				fn(a, b);
			});
		}
		for (auto& t: pool)
			t.join();
	}
#define NHB_NORM_SIZES(X) X(32) X(64) X(96) X(128) X(160) X(256) X(512) X(1024) X(2048) X(4096) X(14336)

	// one row of the rms_norm_mul kernel (cpu/avx_2.hpp:3907-3915): the reference's sum of squares, its sqrtf_fast and
	// its vec_scale_mul_f32<K>; the row loop around it is ours.  The reference stores with aligned and streaming
	// stores, so the row goes through 64-byte aligned buffers.  false when K has no instantiation here.
	bool norm_row(const float* x, const float* w, float eps, int sqrt_mode, float* y, int64_t K) {
		const float sum	  = nihilus::simd_sum_squares(x, static_cast<uint64_t>(K));
		const float mean  = sum / static_cast<float>(K);
		const float root  = sqrt_mode == 1 ? nihilus::sqrtf_fast(mean + eps) : std::sqrt(mean + eps);// 0: what the NEON build's sqrtf_fast is
		const float scale = 1.0f / root;
		switch (K) {
#define NHB_CASE(v) \
	case v: \
		nihilus::vec_scale_mul_f32<v>::impl(y, x, scale, w); \
		return true;
			NHB_NORM_SIZES(NHB_CASE)
#undef NHB_CASE
			default:
				return false;
		}
	}

	struct aligned_rows {
		float *x, *w, *y;
		explicit aligned_rows(int64_t K) {
			const size_t bytes = (static_cast<size_t>(K) * 4 + 63) & ~size_t(63);
			x				   = static_cast<float*>(std::aligned_alloc(64, bytes));
			w				   = static_cast<float*>(std::aligned_alloc(64, bytes));
			y				   = static_cast<float*>(std::aligned_alloc(64, bytes));
		}
		~aligned_rows() {
			std::free(x);
			std::free(w);
			std::free(y);
		}
	};
}

extern "C" {

uint16_t ref_fp32_to_fp16(float f) {
	return static_cast<uint16_t>(nihilus::fp32_to_fp16(f));
}
uint16_t ref_fp32_to_fp16_bittrick(float f) {
	return static_cast<uint16_t>(nihilus::fp32_to_fp16_f16c(f));
}
float ref_fp16_to_fp32(uint16_t h) {
	return nihilus::fp16_to_fp32(static_cast<nihilus::half>(h));
}

void ref_quantize_row_q8_0(const float* x, void* blocks, int64_t k) {
	nihilus::quantize_row_q8_0(x, static_cast<blk*>(blocks), k);
}

// cpu/avx_2.hpp:4749-4780
float ref_vec_dot_q8_0_q8_0(const void* w, const void* a, int64_t nb) {
	float s;
	nihilus::vec_dot_q8_0_q8_0_impl(nb * 32, &s, static_cast<const blk*>(w), static_cast<const blk*>(a));
	return s;
}

// cpu/avx_2.hpp:4536-4677 (n in 1..16), and the 16-chunk driver for larger n
float ref_vec_dot_q8_0_q8_0_chunk16(const void* w, const void* a, int64_t nb) {
	return chunk16_dot(static_cast<const blk*>(w), static_cast<const blk*>(a), nb);
}

// cpu/avx_2.hpp:4800-4852; NaN when K is not one of the instantiated sizes
float ref_vec_dot_q8_f32_eval(const float* x, const void* w, int64_t K) {
	return eval_dot(x, static_cast<const blk*>(w), K);
}

// cpu/avx_2.hpp:4881-4907
float ref_scalar_dot_product_q8_f32(const float* x, const void* w, int64_t K) {
	return nihilus::scalar_dot_product_q8_f32(x, static_cast<const blk*>(w), K);
}

// mode numbering matches enum orc_mode in q8_oracle.h (0 lanes, 2 chunk16, 3 f32 eval, 4 f32 prompt).
// y[m*ldy + n]; returns 0, -1 on bad arguments, -2 when the mode/K has no reference instantiation.
int ref_mul_mat_q8_0(int mode, const void* w_blocks, int64_t N, int64_t K, const float* x, int64_t ldx, int64_t M, float* y, int64_t ldy,
	int threads) {
	if (!w_blocks || !x || !y || N < 0 || K <= 0 || K % 32 != 0 || M < 0 || ldx < K || ldy < N)
		return -1;
	if (mode != 0 && mode != 2 && mode != 3 && mode != 4)
		return -2;
	const blk* w = static_cast<const blk*>(w_blocks);
	const int64_t nb = K / 32;
	if (mode == 3 && !eval_supported(K))
		return -2;
	std::vector<blk> aq;
	if (mode == 0 || mode == 2) {
		aq.resize(static_cast<size_t>(M * nb));
		for (int64_t m = 0; m < M; ++m)
			nihilus::quantize_row_q8_0(x + m * ldx, aq.data() + m * nb, K);
	}
	parallel_rows(0, N, threads, [&](int64_t a, int64_t b) {
		for (int64_t m = 0; m < M; ++m) {
			for (int64_t n = a; n < b; ++n) {
				const blk* wr = w + n * nb;
				float r;
				if (mode == 0) {
					nihilus::vec_dot_q8_0_q8_0_impl(K, &r, wr, aq.data() + m * nb);
				} else if (mode == 2) {
					r = chunk16_dot(wr, aq.data() + m * nb, nb);
				} else if (mode == 3) {
					r = eval_dot(x + m * ldx, wr, K);
				} else {
					r = nihilus::scalar_dot_product_q8_f32(x + m * ldx, wr, K);
				}
				y[m * ldy + n] = r;
			}
		}
	});
	return 0;
}

// cpu/avx_2.hpp:758-779 and cpu/common.hpp:448-450
float ref_sum_squares(const float* x, int64_t K) {
	return nihilus::simd_sum_squares(x, static_cast<uint64_t>(K));
}
float ref_sqrtf_fast(float x) {
	return nihilus::sqrtf_fast(x);
}

// rms_norm x norm-weight, f32 out; 0, -1 on bad arguments, -2 when K has no instantiation
int ref_rms_norm_mul(const float* x, int64_t ldx, const float* w, float eps, int sqrt_mode, float* y, int64_t ldy, int64_t M, int64_t K) {
	if (!x || !w || !y || M < 0 || K <= 0 || ldx < K || ldy < K)
		return -1;
	aligned_rows r(K);
	std::memcpy(r.w, w, static_cast<size_t>(K) * 4);
	for (int64_t m = 0; m < M; ++m) {
		std::memcpy(r.x, x + m * ldx, static_cast<size_t>(K) * 4);
		if (!norm_row(r.x, r.w, eps, sqrt_mode, r.y, K))
			return -2;
		std::memcpy(y + m * ldy, r.y, static_cast<size_t>(K) * 4);
	}
	return 0;
}

// the same rows through the reference's quantize_row_q8_0_avx2 (cpu/avx_2.hpp:671-721); blocks [M][K/32]
int ref_rms_norm_mul_q8_0(const float* x, int64_t ldx, const float* w, float eps, int sqrt_mode, void* blocks, int64_t M, int64_t K) {
	if (!x || !w || !blocks || M < 0 || K <= 0 || K % 32 != 0 || ldx < K)
		return -1;
	aligned_rows r(K);
	std::memcpy(r.w, w, static_cast<size_t>(K) * 4);
	for (int64_t m = 0; m < M; ++m) {
		std::memcpy(r.x, x + m * ldx, static_cast<size_t>(K) * 4);
		if (!norm_row(r.x, r.w, eps, sqrt_mode, r.y, K))
			return -2;
		nihilus::quantize_row_q8_0_avx2(r.y, static_cast<blk*>(blocks) + m * (K / 32), static_cast<uint64_t>(K));
	}
	return 0;
}
}
