/*
 * CPU oracle for the Q8_0 mul_mat path -- TEST INFRASTRUCTURE ONLY (see q8_oracle.h).
 *
 * Every function restates, in scalar C, one piece of the reference's dead AVX2 code in
 * include/nihilus-incl/cpu/avx_2.hpp; the line ranges are cited at each function.  Build with
 * -ffp-contract=off: a float multiply followed by an add must stay two roundings unless the
 * reference used an explicit fused multiply-add (then fmaf is called here).
 */
#include "q8_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ---- fp16 <-> fp32 ------------------------------------------------------------------------------------------ */

static inline uint32_t f2u(float f) {
	uint32_t u;
	memcpy(&u, &f, 4);
	return u;
}
static inline float u2f(uint32_t u) {
	float f;
	memcpy(&f, &u, 4);
	return f;
}

/* IEEE-754 binary32 -> binary16, round to nearest even: what cpu/common.hpp:215-217 gets from
 * _mm_cvtps_ph(_MM_FROUND_TO_NEAREST_INT). */
uint16_t orc_fp32_to_fp16(float f) {
	const uint32_t u	= f2u(f);
	const uint32_t sign = (u >> 16) & 0x8000u;
	const uint32_t absu = u & 0x7FFFFFFFu;
	if (absu >= 0x7F800000u) { /* inf / nan */
		if (absu == 0x7F800000u)
			return (uint16_t)(sign | 0x7C00u);
		return (uint16_t)(sign | 0x7C00u | 0x0200u | ((absu >> 13) & 0x03FFu)); /* quiet nan, payload kept */
	}
	if (absu >= 0x477FF000u) /* >= 65520 rounds to inf */
		return (uint16_t)(sign | 0x7C00u);
	if (absu < 0x33000001u) /* <= 2^-25 rounds to zero (exactly 2^-25 ties to even = 0) */
		return (uint16_t)sign;
	int32_t e  = (int32_t)(absu >> 23) - 127;
	uint32_t m = (absu & 0x007FFFFFu) | 0x00800000u; /* 24-bit significand */
	uint32_t shift;
	uint32_t base;
	if (e < -14) { /* subnormal half: value = m * 2^(e-23); unit = 2^-24 */
		shift = (uint32_t)(-14 - e) + 13;
		base  = 0;
	} else {
		shift = 13;
		base  = ((uint32_t)(e + 15) << 10) - 0x0400u; /* the implicit bit of m adds 0x400 back */
	}
	uint32_t q	 = m >> shift;
	uint32_t rem = m & ((1u << shift) - 1u);
	uint32_t half = 1u << (shift - 1);
	if (rem > half || (rem == half && (q & 1u)))
		q += 1;
	return (uint16_t)(sign | (base + q));
}

/* the bit-trick converter the reference quantiser actually calls, avx_2.hpp:4418-4437 */
uint16_t orc_fp32_to_fp16_bittrick(float f) {
	const float scale_to_inf  = u2f(0x77800000u);
	const float scale_to_zero = u2f(0x08800000u);
	float base				  = (fabsf(f) * scale_to_inf) * scale_to_zero;
	const uint32_t w		  = f2u(f);
	const uint32_t shl1_w	  = w + w;
	const uint32_t sign		  = w & 0x80000000u;
	uint32_t bias			  = shl1_w & 0xFF000000u;
	if (bias < 0x71000000u)
		bias = 0x71000000u;
	base						 = u2f((bias >> 1) + 0x07800000u) + base;
	const uint32_t bits			 = f2u(base);
	const uint32_t exp_bits		 = (bits >> 13) & 0x00007C00u;
	const uint32_t mantissa_bits = bits & 0x00000FFFu;
	const uint32_t nonsign		 = exp_bits + mantissa_bits;
	return (uint16_t)((sign >> 16) | (shl1_w > 0xFF000000u ? 0x7E00u : nonsign));
}

/* binary16 -> binary32 (exact), cpu/common.hpp:219-221 / :455-473 */
float orc_fp16_to_fp32(uint16_t h) {
	const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
	const uint32_t e	= (h >> 10) & 0x1Fu;
	const uint32_t m	= h & 0x03FFu;
	if (e == 0x1Fu)
		return u2f(sign | 0x7F800000u | (m << 13));
	if (e == 0) {
		if (m == 0)
			return u2f(sign);
		const float v = (float)m * u2f(0x33800000u); /* m * 2^-24, exact */
		return sign ? -v : v;
	}
	return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

/* ---- block access ------------------------------------------------------------------------------------------- */

static inline uint16_t blk_d(const uint8_t* b) {
	return (uint16_t)(b[0] | ((uint16_t)b[1] << 8));
}
static inline const int8_t* blk_q(const uint8_t* b) {
	return (const int8_t*)(b + 2);
}

/* ---- activation quantiser, avx_2.hpp:4439-4489 (twin at :671-721) -------------------------------------------- */

static inline int8_t sat_round_i8(float v) {
	if (!(v == v))
		return -128; /* cvtps_epi32 yields INT_MIN for NaN, the two saturating packs turn that into -128 */
	float r = nearbyintf(v); /* _MM_ROUND_NEAREST = ties to even (default rounding mode) */
	if (r > 127.f)
		return 127;
	if (r < -128.f)
		return -128;
	return (int8_t)(int32_t)r;
}

void orc_quantize_row_q8_0(const float* x, uint8_t* blocks, int64_t k) {
	const int64_t nb = k / ORC_QK;
	for (int64_t i = 0; i < nb; ++i) {
		const float* xb = x + i * ORC_QK;
		float amax		= 0.f;
		for (int j = 0; j < ORC_QK; ++j) {
			const float a = fabsf(xb[j]);
			if (a > amax)
				amax = a;
		}
		const float d	 = amax / 127.f;
		const uint16_t h = orc_fp32_to_fp16(d);
		const float id	 = (amax != 0.0f) ? 127.f / amax : 0.0f;
		uint8_t* b		 = blocks + i * ORC_BLOCK_BYTES;
		b[0]			 = (uint8_t)(h & 0xFF);
		b[1]			 = (uint8_t)(h >> 8);
		for (int j = 0; j < ORC_QK; ++j)
			b[2 + j] = (uint8_t)sat_round_i8(xb[j] * id);
	}
}

void orc_quantize_matrix_q8_0(const float* w, int64_t N, int64_t K, uint8_t* blocks, int threads);

/* ---- int8 block products, avx_2.hpp:4509-4524 ------------------------------------------------------------------ */

/* lane l of mul_sum_i8_pairs_float: products 4l..4l+3, built from maddubs (saturating int16 pair sums of
 * |x| * (y*sign(x))) followed by madd with ones.  Exact whenever no quant is -128. */
static inline int32_t lane_sum4(const int8_t* x, const int8_t* y, int l) {
	int32_t s = 0;
	for (int p = 0; p < 2; ++p) {
		int32_t pair = 0;
		for (int t = 0; t < 2; ++t) {
			const int j		 = 4 * l + 2 * p + t;
			const int32_t ax = x[j] < 0 ? -(int32_t)x[j] : (int32_t)x[j]; /* unsigned 0..128 */
			int8_t sy;
			if (x[j] > 0)
				sy = y[j];
			else if (x[j] == 0)
				sy = 0;
			else
				sy = (int8_t)(uint8_t)(0u - (uint8_t)y[j]); /* psignb wraps -(-128) to -128 */
			pair += ax * (int32_t)sy;
		}
		if (pair > 32767)
			pair = 32767;
		if (pair < -32768)
			pair = -32768;
		s += pair;
	}
	return s;
}

static inline int32_t block_dot_i32(const int8_t* x, const int8_t* y) {
	int32_t s = 0;
	for (int j = 0; j < ORC_QK; ++j)
		s += (int32_t)x[j] * (int32_t)y[j];
	return s;
}

static inline float hsum_float_8(const float* a) { /* avx_2.hpp:4526-4532 */
	float r0 = a[4] + a[0], r1 = a[5] + a[1], r2 = a[6] + a[2], r3 = a[7] + a[3];
	r0 = r0 + r2;
	r1 = r1 + r3;
	return r0 + r1;
}

/* avx_2.hpp:4749-4780 */
static float dot_q8q8_lanes(const uint8_t* w, const uint8_t* a, int64_t nb) {
	float acc[8] = { 0 };
	for (int64_t ib = 0; ib < nb; ++ib) {
		const uint8_t* wb = w + ib * ORC_BLOCK_BYTES;
		const uint8_t* ab = a + ib * ORC_BLOCK_BYTES;
		const float d	  = orc_fp16_to_fp32(blk_d(wb)) * orc_fp16_to_fp32(blk_d(ab));
		for (int l = 0; l < 8; ++l)
			acc[l] = fmaf(d, (float)lane_sum4(blk_q(wb), blk_q(ab), l), acc[l]);
	}
	return hsum_float_8(acc);
}

/* avx_2.hpp:4536-4553 */
static float dot_q8q8_scalar(const uint8_t* w, const uint8_t* a, int64_t nb) {
	float sumf = 0.0f;
	for (int64_t ib = 0; ib < nb; ++ib) {
		const uint8_t* wb  = w + ib * ORC_BLOCK_BYTES;
		const uint8_t* ab  = a + ib * ORC_BLOCK_BYTES;
		const int64_t sumi = block_dot_i32(blk_q(wb), blk_q(ab));
		/* "sumf += sumi * (...)" is one expression: both of the reference's compiler set-ups contract it
		 * (GCC default -ffp-contract=fast; Clang is given -ffp-contract=on, cmake/flags_and_options.cmake:54) */
		sumf = fmaf((float)sumi, orc_fp16_to_fp32(blk_d(wb)) * orc_fp16_to_fp32(blk_d(ab)), sumf);
	}
	return sumf;
}

/* n accumulators (1, 2 or 4) over n_blocks blocks, block ib feeds accumulator ib % n_acc; avx_2.hpp:4555-4677 */
static float dot_q8q8_multiacc(const uint8_t* w, const uint8_t* a, int n_blocks, int n_acc) {
	float acc[4][8];
	memset(acc, 0, sizeof(acc));
	for (int ib = 0; ib < n_blocks; ++ib) {
		const uint8_t* wb = w + (int64_t)ib * ORC_BLOCK_BYTES;
		const uint8_t* ab = a + (int64_t)ib * ORC_BLOCK_BYTES;
		const float d	  = orc_fp16_to_fp32(blk_d(wb)) * orc_fp16_to_fp32(blk_d(ab));
		float* c		  = acc[ib % n_acc];
		for (int l = 0; l < 8; ++l)
			c[l] = fmaf(d, (float)lane_sum4(blk_q(wb), blk_q(ab), l), c[l]);
	}
	float fin[8];
	for (int l = 0; l < 8; ++l) {
		if (n_acc == 1)
			fin[l] = acc[0][l];
		else if (n_acc == 2)
			fin[l] = acc[0][l] + acc[1][l];
		else
			fin[l] = (acc[0][l] + acc[1][l]) + (acc[2][l] + acc[3][l]);
	}
	return hsum_float_8(fin);
}

/* the compile-time-n family for n <= 16, avx_2.hpp:4536-4677 */
static float dot_q8q8_upto16(const uint8_t* w, const uint8_t* a, int n) {
	if (n < 4)
		return dot_q8q8_scalar(w, a, n);
	if (n == 4)
		return dot_q8q8_multiacc(w, a, 4, 1);
	if (n < 8) {
		float s = dot_q8q8_multiacc(w, a, 4, 1);
		return s + dot_q8q8_upto16(w + 4 * ORC_BLOCK_BYTES, a + 4 * ORC_BLOCK_BYTES, n - 4);
	}
	if (n == 8)
		return dot_q8q8_multiacc(w, a, 8, 2);
	if (n < 16) {
		float s = dot_q8q8_multiacc(w, a, 8, 2);
		return s + dot_q8q8_upto16(w + 8 * ORC_BLOCK_BYTES, a + 8 * ORC_BLOCK_BYTES, n - 8);
	}
	return dot_q8q8_multiacc(w, a, 16, 4);
}

/* n > 16: 16-block chunks summed in order, avx_2.hpp:4715-4747 */
static float dot_q8q8_chunk16(const uint8_t* w, const uint8_t* a, int64_t nb) {
	if (nb <= 16)
		return dot_q8q8_upto16(w, a, (int)nb);
	const int64_t total_chunks = (nb + 15) / 16;
	const int rem			   = (int)(nb % 16);
	float total				   = 0.0f;
	for (int64_t c = 0; c + 1 < total_chunks; ++c)
		total = total + dot_q8q8_upto16(w + c * 16 * ORC_BLOCK_BYTES, a + c * 16 * ORC_BLOCK_BYTES, 16);
	const int64_t last = total_chunks - 1;
	total			   = total + dot_q8q8_upto16(w + last * 16 * ORC_BLOCK_BYTES, a + last * 16 * ORC_BLOCK_BYTES, rem == 0 ? 16 : rem);
	return total;
}

static float dot_q8q8_f64(const uint8_t* w, const uint8_t* a, int64_t nb) {
	double s = 0.0;
	for (int64_t ib = 0; ib < nb; ++ib) {
		const uint8_t* wb = w + ib * ORC_BLOCK_BYTES;
		const uint8_t* ab = a + ib * ORC_BLOCK_BYTES;
		s += (double)block_dot_i32(blk_q(wb), blk_q(ab)) * ((double)orc_fp16_to_fp32(blk_d(wb)) * (double)orc_fp16_to_fp32(blk_d(ab)));
	}
	return (float)s;
}

float orc_vec_dot_q8_0_q8_0(int mode, const uint8_t* w, const uint8_t* a, int64_t nb) {
	switch (mode) {
		case ORC_Q8ACT_LANES:
			return dot_q8q8_lanes(w, a, nb);
		case ORC_Q8ACT_SCALAR:
			return dot_q8q8_scalar(w, a, nb);
		case ORC_Q8ACT_CHUNK16:
			return dot_q8q8_chunk16(w, a, nb);
		default:
			return dot_q8q8_f64(w, a, nb);
	}
}

void orc_block_dots(const uint8_t* w, const uint8_t* a, int64_t nb, int32_t* out) {
	for (int64_t ib = 0; ib < nb; ++ib)
		out[ib] = block_dot_i32(blk_q(w + ib * ORC_BLOCK_BYTES), blk_q(a + ib * ORC_BLOCK_BYTES));
}

/* ---- f32-activation dots ------------------------------------------------------------------------------------ */

/* How "sum += x[i] * float(q)" and "sum += block_sum" round in the eval-time variant depends on the compiler:
 * g++ 13 -O3 vectorises the 32 multiplies and then adds them one by one (no contraction), which is the form
 * used here; with it this function is bit-identical to the compiled reference for every K tested except
 * K = 64, where g++ fuses the outer accumulate.  Tests therefore compare this mode at 1e-5, not bit-exactly. */
#define INNER_ACC(a, b, c) ((c) + (a) * (b))
#define OUTER_ACC(s, scale, sum) ((sum) + (s) * (scale))
/* eval-time: vec_dot_q8_f32<Q_SIZE> per block (avx_2.hpp:4800-4815) summed by the >=64 driver (:4830-4852) */
static float dot_q8f32_eval(const uint8_t* w, const float* x, int64_t nb) {
	float sum = 0.0f;
	for (int64_t ib = 0; ib < nb; ++ib) {
		const uint8_t* wb = w + ib * ORC_BLOCK_BYTES;
		const float scale = orc_fp16_to_fp32(blk_d(wb));
		const int8_t* q	  = blk_q(wb);
		float s			  = 0.0f;
		for (int i = 0; i < ORC_QK; ++i)
			s = INNER_ACC(x[ib * ORC_QK + i], (float)q[i], s);
		sum = OUTER_ACC(s, scale, sum);
	}
	return sum;
}

/* prompt-time: scalar_dot_product_q8_f32, avx_2.hpp:4881-4907 */
static float dot_q8f32_prompt(const uint8_t* w, const float* x, int64_t nb) {
	float sum = 0.0f;
	for (int64_t ib = 0; ib < nb; ++ib) {
		const uint8_t* wb = w + ib * ORC_BLOCK_BYTES;
		const float scale = orc_fp16_to_fp32(blk_d(wb));
		const int8_t* q	  = blk_q(wb);
		for (int i = 0; i < ORC_QK; ++i) {
			const float wv = (float)q[i] * scale;
			sum			   = fmaf(x[ib * ORC_QK + i], wv, sum); /* "sum += x * (float(q) * scale)": contracted */
		}
	}
	return sum;
}

static float dot_q8f32_f64(const uint8_t* w, const float* x, int64_t nb) {
	double sum = 0.0;
	for (int64_t ib = 0; ib < nb; ++ib) {
		const uint8_t* wb  = w + ib * ORC_BLOCK_BYTES;
		const double scale = (double)orc_fp16_to_fp32(blk_d(wb));
		const int8_t* q	   = blk_q(wb);
		double s		   = 0.0;
		for (int i = 0; i < ORC_QK; ++i)
			s += (double)x[ib * ORC_QK + i] * (double)q[i];
		sum += s * scale;
	}
	return (float)sum;
}

float orc_vec_dot_q8_f32(int mode, const uint8_t* w, const float* x, int64_t nb) {
	switch (mode) {
		case ORC_F32ACT_EVAL:
			return dot_q8f32_eval(w, x, nb);
		case ORC_F32ACT_PROMPT:
			return dot_q8f32_prompt(w, x, nb);
		default:
			return dot_q8f32_f64(w, x, nb);
	}
}

/* ---- mul_mat drivers ------------------------------------------------------------------------------------------ */

typedef struct {
	int mode;
	const uint8_t* w;
	int64_t K, M, ldx, ldy;
	const float* x;
	const uint8_t* aq; /* quantised activations, M rows of nb blocks (Q8ACT modes) */
	float* y;
	int32_t* dots;
	int64_t N;
	int64_t r0, r1;
} mm_job;

static int is_q8act(int mode) {
	return mode == ORC_Q8ACT_LANES || mode == ORC_Q8ACT_SCALAR || mode == ORC_Q8ACT_CHUNK16 || mode == ORC_Q8ACT_F64;
}

/* loop nest of process_tensor_elements, avx_2.hpp:4926-4963: activation row outer, weight row inner */
static void* mm_worker(void* p) {
	mm_job* j		 = (mm_job*)p;
	const int64_t nb = j->K / ORC_QK;
	for (int64_t m = 0; m < j->M; ++m) {
		for (int64_t n = j->r0; n < j->r1; ++n) {
			const uint8_t* wrow = j->w + n * nb * ORC_BLOCK_BYTES;
			if (j->dots) {
				orc_block_dots(wrow, j->aq + m * nb * ORC_BLOCK_BYTES, nb, j->dots + (m * j->N + n) * nb);
			} else if (is_q8act(j->mode)) {
				j->y[m * j->ldy + n] = orc_vec_dot_q8_0_q8_0(j->mode, wrow, j->aq + m * nb * ORC_BLOCK_BYTES, nb);
			} else {
				j->y[m * j->ldy + n] = orc_vec_dot_q8_f32(j->mode, wrow, j->x + m * j->ldx, nb);
			}
		}
	}
	return NULL;
}

static int run_jobs(mm_job* proto, int64_t n0, int64_t n1, int threads) {
	if (threads < 1)
		threads = 1;
	if (threads > 256)
		threads = 256;
	const int64_t rows = n1 - n0;
	if (rows <= 0)
		return 0;
	if (threads > rows)
		threads = (int)rows;
	mm_job jobs[256];
	pthread_t tids[256];
	const int64_t per = (rows + threads - 1) / threads;
	int started		  = 0;
	for (int t = 0; t < threads; ++t) {
		jobs[t]	   = *proto;
		jobs[t].r0 = n0 + t * per;
		jobs[t].r1 = jobs[t].r0 + per < n1 ? jobs[t].r0 + per : n1;
		if (jobs[t].r0 >= jobs[t].r1)
			break;
		if (threads == 1) {
			mm_worker(&jobs[t]);
		} else {
			if (pthread_create(&tids[t], NULL, mm_worker, &jobs[t]) != 0) {
				mm_worker(&jobs[t]);
				tids[t] = 0;
			}
		}
		++started;
	}
	if (threads > 1)
		for (int t = 0; t < started; ++t)
			if (tids[t])
				pthread_join(tids[t], NULL);
	return 0;
}

int orc_mul_mat_q8_0(int mode, const uint8_t* w, int64_t N, int64_t K, const float* x, int64_t ldx, int64_t M, float* y, int64_t ldy,
	int64_t n0, int64_t n1, int threads) {
	if (!w || !x || !y || N < 0 || K <= 0 || (K % ORC_QK) != 0 || M < 0 || n0 < 0 || n1 > N || n0 > n1 || ldx < K || ldy < N)
		return -1;
	if (mode < ORC_Q8ACT_LANES || mode > ORC_F32ACT_F64)
		return -1;
	if (M == 0 || n0 == n1)
		return 0;
	const int64_t nb = K / ORC_QK;
	uint8_t* aq		 = NULL;
	if (is_q8act(mode)) {
		aq = (uint8_t*)malloc((size_t)(M * nb * ORC_BLOCK_BYTES));
		if (!aq)
			return -1;
		for (int64_t m = 0; m < M; ++m)
			orc_quantize_row_q8_0(x + m * ldx, aq + m * nb * ORC_BLOCK_BYTES, K);
	}
	mm_job j;
	memset(&j, 0, sizeof(j));
	j.mode = mode;
	j.w	   = w;
	j.K	   = K;
	j.M	   = M;
	j.ldx  = ldx;
	j.ldy  = ldy;
	j.x	   = x;
	j.aq   = aq;
	j.y	   = y;
	j.N	   = N;
	run_jobs(&j, n0, n1, threads);
	free(aq);
	return 0;
}

int orc_mul_mat_block_dots(const uint8_t* w, int64_t N, int64_t K, const float* x, int64_t ldx, int64_t M, int32_t* dots, int threads) {
	if (!w || !x || !dots || N < 0 || K <= 0 || (K % ORC_QK) != 0 || M < 0 || ldx < K)
		return -1;
	if (M == 0 || N == 0)
		return 0;
	const int64_t nb = K / ORC_QK;
	uint8_t* aq		 = (uint8_t*)malloc((size_t)(M * nb * ORC_BLOCK_BYTES));
	if (!aq)
		return -1;
	for (int64_t m = 0; m < M; ++m)
		orc_quantize_row_q8_0(x + m * ldx, aq + m * nb * ORC_BLOCK_BYTES, K);
	mm_job j;
	memset(&j, 0, sizeof(j));
	j.mode = ORC_Q8ACT_LANES;
	j.w	   = w;
	j.K	   = K;
	j.M	   = M;
	j.ldx  = ldx;
	j.x	   = x;
	j.aq   = aq;
	j.dots = dots;
	j.N	   = N;
	run_jobs(&j, 0, N, threads);
	free(aq);
	return 0;
}

/* ---- repack ------------------------------------------------------------------------------------------------------ */

void orc_repack_planes(const uint8_t* w, int64_t K, int64_t n0, int64_t n1, int8_t* q_plane, uint16_t* d_plane) {
	const int64_t nb = K / ORC_QK;
	for (int64_t n = n0; n < n1; ++n) {
		for (int64_t b = 0; b < nb; ++b) {
			const uint8_t* blk			= w + (n * nb + b) * ORC_BLOCK_BYTES;
			d_plane[(n - n0) * nb + b] = blk_d(blk);
			memcpy(q_plane + (n - n0) * K + b * ORC_QK, blk + 2, ORC_QK);
		}
	}
}

void orc_unpack_planes(const int8_t* q_plane, const uint16_t* d_plane, int64_t K, int64_t rows, uint8_t* w) {
	const int64_t nb = K / ORC_QK;
	for (int64_t n = 0; n < rows; ++n) {
		for (int64_t b = 0; b < nb; ++b) {
			uint8_t* blk	 = w + (n * nb + b) * ORC_BLOCK_BYTES;
			const uint16_t h = d_plane[n * nb + b];
			blk[0]			 = (uint8_t)(h & 0xFF);
			blk[1]			 = (uint8_t)(h >> 8);
			memcpy(blk + 2, q_plane + n * K + b * ORC_QK, ORC_QK);
		}
	}
}

/* ---- synthetic weight quantisation (rows in parallel) -------------------------------------------------------------- */

typedef struct {
	const float* w;
	uint8_t* blocks;
	int64_t K, r0, r1;
} qm_job;

static void* qm_worker(void* p) {
	qm_job* j		 = (qm_job*)p;
	const int64_t nb = j->K / ORC_QK;
	for (int64_t n = j->r0; n < j->r1; ++n)
		orc_quantize_row_q8_0(j->w + n * j->K, j->blocks + n * nb * ORC_BLOCK_BYTES, j->K);
	return NULL;
}

void orc_quantize_matrix_q8_0(const float* w, int64_t N, int64_t K, uint8_t* blocks, int threads) {
	if (threads < 1)
		threads = 1;
	if (threads > 256)
		threads = 256;
	if (threads > N)
		threads = N > 0 ? (int)N : 1;
	qm_job jobs[256];
	pthread_t tids[256];
	const int64_t per = (N + threads - 1) / threads;
	int started		  = 0;
	for (int t = 0; t < threads; ++t) {
		jobs[t].w	   = w;
		jobs[t].blocks = blocks;
		jobs[t].K	   = K;
		jobs[t].r0	   = t * per;
		jobs[t].r1	   = (t + 1) * per < N ? (t + 1) * per : N;
		if (jobs[t].r0 >= jobs[t].r1)
			break;
		if (threads == 1 || pthread_create(&tids[t], NULL, qm_worker, &jobs[t]) != 0) {
			qm_worker(&jobs[t]);
			tids[t] = 0;
		}
		++started;
	}
	for (int t = 0; t < started; ++t)
		if (threads > 1 && tids[t])
			pthread_join(tids[t], NULL);
}

/* ---- rms_norm x norm-weight (-> Q8_0), the producer of a projection's activations ---------------------------------- */

/* simd_sum_squares, avx_2.hpp:758-779 (again at :3598-3619): lane l of a 256-bit accumulator takes elements
 * 8i + l through one fma each, in ascending i; then (lo + hi) on 4 lanes, (x + movehl) on 2, add_ss on 1. */
float orc_sum_squares(const float* x, int64_t k) {
	float lane[8]	   = { 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f };
	const int64_t full = k & ~(int64_t)7;
	for (int64_t i = 0; i < full; i += 8)
		for (int l = 0; l < 8; ++l)
			lane[l] = fmaf(x[i + l], x[i + l], lane[l]);
	const float q0 = lane[0] + lane[4], q1 = lane[1] + lane[5], q2 = lane[2] + lane[6], q3 = lane[3] + lane[7];
	const float d0 = q0 + q2, d1 = q1 + q3;
	float sum	   = d0 + d1;
	for (int64_t i = full; i < k; ++i)
		sum += x[i] * x[i]; /* scalar tail of the reference; no caller here has k % 8 != 0 */
	return sum;
}

/* sqrtf_fast, cpu/common.hpp:448-450 (the x86 build): an integer approximation of the square root, not sqrtf. */
float orc_sqrtf_fast(float x) {
	uint32_t b;
	memcpy(&b, &x, 4);
	b = ((b + 0x3f800000u) >> 1) + 0x20000000u;
	float r;
	memcpy(&r, &b, 4);
	return r;
}

/* the scale of one row: avx_2.hpp:3907-3909.  sqrt_mode 0: sqrtf_fast is the IEEE square root (the NEON build,
 * cpu/common.hpp:310-312); sqrt_mode 1: the x86 build's integer formula above, which as written returns about
 * 2^64 * sqrt(x), so every scale carries a factor of about 2^-64 -- kept bit for bit because it is what that build
 * computes. */
float orc_rms_norm_scale(const float* x, int64_t k, float eps, int sqrt_mode) {
	const float sum	 = orc_sum_squares(x, k);
	const float mean = sum / (float)k;
	const float root = sqrt_mode == 1 ? orc_sqrtf_fast(mean + eps) : sqrtf(mean + eps);
	return 1.0f / root;
}

/* (x * w) * scale, two roundings -- vec_scale_mul_f32, avx_2.hpp:3621-3850, as called by the rms_norm_mul kernel
 * (:3907-3915).  (The Q8_0-producing helper vec_scale_mul_f32_to_q8_0, :723-756, hands quantize_row_q8_0_avx2 a
 * count of 1 element, i.e. zero blocks, and so produces nothing to compare with; the Q8_0 output below is the
 * reference's quantiser applied to the f32 kernel's row, which is what the rms_norm_mul -> mul_mat chain computes.) */
static inline float norm_elem(float x, float w, float scale) {
	const float t = x * w;
	return t * scale;
}

int orc_rms_norm_mul(const float* x, int64_t ldx, const float* w, float eps, int sqrt_mode, float* y, int64_t ldy, int64_t M, int64_t K) {
	if (!x || !w || !y || M < 0 || K <= 0 || (K % 8) != 0 || ldx < K || ldy < K || sqrt_mode < 0 || sqrt_mode > 1)
		return -1;
	for (int64_t m = 0; m < M; ++m) {
		const float scale = orc_rms_norm_scale(x + m * ldx, K, eps, sqrt_mode);
		for (int64_t i = 0; i < K; ++i)
			y[m * ldy + i] = norm_elem(x[m * ldx + i], w[i], scale);
	}
	return 0;
}

/* the same row, quantised block by block (quantize_row_q8_0_avx2, avx_2.hpp:671-721, has the arithmetic of
 * quantize_row_q8_0). blocks: [M][K/32][34]. */
int orc_rms_norm_mul_q8_0(const float* x, int64_t ldx, const float* w, float eps, int sqrt_mode, uint8_t* blocks, int64_t M, int64_t K) {
	if (!x || !w || !blocks || M < 0 || K <= 0 || (K % ORC_QK) != 0 || ldx < K || sqrt_mode < 0 || sqrt_mode > 1)
		return -1;
	float* row = (float*)malloc((size_t)K * sizeof(float));
	if (!row)
		return -1;
	for (int64_t m = 0; m < M; ++m) {
		const float scale = orc_rms_norm_scale(x + m * ldx, K, eps, sqrt_mode);
		for (int64_t i = 0; i < K; ++i)
			row[i] = norm_elem(x[m * ldx + i], w[i], scale);
		orc_quantize_row_q8_0(row, blocks + m * (K / ORC_QK) * ORC_BLOCK_BYTES, K);
	}
	free(row);
	return 0;
}

/* ---- element-wise neighbours of the mul_mats (infra/core_traits.hpp:771-772, 982-992: trait declarations only) ---- */
void orc_swiglu(const float* g, const float* u, float* h, int64_t n) {
	for (int64_t i = 0; i < n; ++i) {
		const float s = g[i] / (1.0f + expf(-g[i]));
		h[i]		  = s * u[i];
	}
}

void orc_swiglu_f64(const float* g, const float* u, float* h, int64_t n) {
	for (int64_t i = 0; i < n; ++i)
		h[i] = (float)(((double)g[i] / (1.0 + exp(-(double)g[i]))) * (double)u[i]);
}

void orc_add(const float* a, const float* b, float* y, int64_t n) {
	for (int64_t i = 0; i < n; ++i)
		y[i] = a[i] + b[i];
}

/* cuda/cuda_12.hpp:560-601 */
int orc_get_rows_q8_0(const uint8_t* table_blocks, int64_t N, int64_t K, const int32_t* ids, int64_t M, float* y, int64_t ldy) {
	const int64_t nb = K / ORC_QK;
	for (int64_t m = 0; m < M; ++m) {
		if (ids[m] < 0 || ids[m] >= N)
			return -1;
		const uint8_t* row = table_blocks + (int64_t)ids[m] * nb * ORC_BLOCK_BYTES;
		for (int64_t b = 0; b < nb; ++b) {
			uint16_t dbits;
			memcpy(&dbits, row + b * ORC_BLOCK_BYTES, 2);
			const float scale = orc_fp16_to_fp32(dbits);
			const int8_t* q	  = (const int8_t*)(row + b * ORC_BLOCK_BYTES + 2);
			for (int j = 0; j < ORC_QK; ++j)
				y[m * ldy + b * ORC_QK + j] = scale * (float)q[j];
		}
	}
	return 0;
}
