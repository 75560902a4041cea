/*
 * CPU oracle for the Q8_0 mul_mat path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic in the reference's (commented-out) AVX2 kernels,
 * include/nihilus-incl/cpu/avx_2.hpp:4418-5004.  Nothing in the product library links, loads
 * or calls this file; it is the checker used by the tests, the smoke test and the CPU-baseline
 * leg of the benchmark.
 *
 * Pinning: the reference ships no golden vectors for this path.  The oracle is pinned against
 * the reference's own helper functions compiled in place (see build_ref.sh) and against the
 * fixtures generated from them under tests/golden/.
 */
#ifndef NIHILUS_B200_Q8_ORACLE_H
#define NIHILUS_B200_Q8_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_QK 32          /* Q_SIZE, common/data_types.hpp:28 */
#define ORC_BLOCK_BYTES 34 /* sizeof(block_q8_0<half>), common/data_types.hpp:37-44 */

/* arithmetic variants of "Q8_0 mul_mat" that exist in the reference */
enum orc_mode {
	ORC_Q8ACT_LANES   = 0, /* vec_dot_q8_0_q8_0_impl, avx_2.hpp:4749-4780: 8 fma lane accumulators + hsum_float_8 */
	ORC_Q8ACT_SCALAR  = 1, /* vec_dot_q8_0_q8_0<n<4>, avx_2.hpp:4536-4553: sumf += sumi * (dw*da), ascending blocks */
	ORC_Q8ACT_CHUNK16 = 2, /* vec_dot_q8_0_q8_0<n>16>, avx_2.hpp:4634-4677 + 4715-4747: 16-block chunks, 4 accumulators */
	ORC_F32ACT_EVAL   = 3, /* vec_dot_q8_f32<K>, avx_2.hpp:4800-4852: per block (sum_j x*float(q)) * d */
	ORC_F32ACT_PROMPT = 4, /* scalar_dot_product_q8_f32, avx_2.hpp:4881-4907: sum += x * (float(q) * d) */
	ORC_Q8ACT_F64     = 5, /* order-independent truth: same products, double accumulation */
	ORC_F32ACT_F64    = 6
};

uint16_t orc_fp32_to_fp16(float f);
float orc_fp16_to_fp32(uint16_t h);
uint16_t orc_fp32_to_fp16_bittrick(float f);

/* k floats -> k/32 blocks of 34 bytes {fp16 d; int8 qs[32]} */
void orc_quantize_row_q8_0(const float* x, uint8_t* blocks, int64_t k);

/* one output element: dot of one weight row (nb blocks) with one activation row */
float orc_vec_dot_q8_0_q8_0(int mode, const uint8_t* w_blocks, const uint8_t* a_blocks, int64_t nb);
float orc_vec_dot_q8_f32(int mode, const uint8_t* w_blocks, const float* x, int64_t nb);

/* exact per-block integer dots for one (weight row, activation row) pair */
void orc_block_dots(const uint8_t* w_blocks, const uint8_t* a_blocks, int64_t nb, int32_t* out);

/*
 * y[m*ldy + n] = row n of W (N rows, K/32 blocks each)  .  activation row m (x + m*ldx, K floats)
 * Output indexing follows avx_2.hpp:4934,4942,4959 (dst_offset = ir1 * nr0; dst_ptr[ir0]).
 * rows [n0, n1) only; threads > 1 partitions rows over pthreads.  Returns 0, or -1 on bad arguments.
 */
int orc_mul_mat_q8_0(int mode, const uint8_t* w_blocks, int64_t N, int64_t K, const float* x, int64_t ldx, int64_t M,
	float* y, int64_t ldy, int64_t n0, int64_t n1, int threads);

/* dots[((m*N)+n)*nb + b], Q8ACT only; activations are quantised with orc_quantize_row_q8_0 */
int orc_mul_mat_block_dots(const uint8_t* w_blocks, int64_t N, int64_t K, const float* x, int64_t ldx, int64_t M, int32_t* dots,
	int threads);

/* the upload-time repack restated on the host: 34 B blocks -> int8 plane [rows][K] + fp16 plane [rows][K/32] */
void orc_repack_planes(const uint8_t* w_blocks, int64_t K, int64_t n0, int64_t n1, int8_t* q_plane, uint16_t* d_plane);
void orc_unpack_planes(const int8_t* q_plane, const uint16_t* d_plane, int64_t K, int64_t rows, uint8_t* w_blocks);

/* weights for the synthetic workloads: f32 rows -> Q8_0 blocks (row by row, threads-parallel) */
void orc_quantize_matrix_q8_0(const float* w, int64_t N, int64_t K, uint8_t* blocks, int threads);

/* rms_norm x norm-weight, f32 out or Q8_0 blocks out: y = (x*w)*scale, scale = 1 / sqrtf_fast(sum_squares/K + eps)
 * (avx_2.hpp:671-779, 3598-3950).  sqrt_mode 0: IEEE square root (sqrtf_fast of the NEON build, cpu/common.hpp:310-312);
 * 1: the integer formula of the x86 build (cpu/common.hpp:448-450), which is off by a factor of about 2^64. */
float orc_sum_squares(const float* x, int64_t k);
float orc_sqrtf_fast(float x);
float orc_rms_norm_scale(const float* x, int64_t k, float eps, int sqrt_mode);
int orc_rms_norm_mul(const float* x, int64_t ldx, const float* w, float eps, int sqrt_mode, float* y, int64_t ldy, int64_t M, int64_t K);
int orc_rms_norm_mul_q8_0(const float* x, int64_t ldx, const float* w, float eps, int sqrt_mode, uint8_t* blocks, int64_t M, int64_t K);

/* The element-wise ops between the mul_mats of the FFN and attention cores.  The reference declares them as traits only
 * (ffn_silu, ffn_gate_par, residual_add: infra/core_traits.hpp:771-772, 982-992); its kernels for silu and mul are empty
 * (cpu/avx_2.hpp:1946-2075, 5325-5330), so what is restated here is the arithmetic the trait names fix:
 *   h = silu(g) * u with silu(g) = g / (1 + exp(-g)), f32 (orc_swiglu), or fp64 throughout, rounded once (orc_swiglu_f64);
 *   y = a + b in f32. */
void orc_swiglu(const float* g, const float* u, float* h, int64_t n);
void orc_swiglu_f64(const float* g, const float* u, float* h, int64_t n);
void orc_add(const float* a, const float* b, float* y, int64_t n);

/* Token-embedding gather: y[m][k] = fp16_to_fp32(d) * (float)q of row ids[m] of a Q8_0 table, the arithmetic of the
 * reference's live GPU kernel (cuda/cuda_12.hpp:587-598; the eval-time twin at :691-722 computes the same products but
 * reads row 0 whatever the token id, :710).  Returns -1 when an id lies outside [0, N). */
int orc_get_rows_q8_0(const uint8_t* table_blocks, int64_t N, int64_t K, const int32_t* ids, int64_t M, float* y, int64_t ldy);

#ifdef __cplusplus
}
#endif
#endif
