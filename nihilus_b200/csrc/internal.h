// Internal declarations shared by the translation units of libnihilus_b200.so (not part of the ABI).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/nihilus_b200.h"

#define NHB_MAX_BATCH 8
#define NHB_STATUS_WORDS 8
#define NHB_MAX_WORLD 8

namespace nhb {

	// device status word values (written by kernels whose bounded waits ran out, or that met an index outside its table)
	enum : int { DEV_OK = 0, DEV_TIMEOUT_FULL = 1, DEV_TIMEOUT_EMPTY = 2, DEV_TIMEOUT_DRAIN = 3, DEV_TIMEOUT_MMA = 4, DEV_TIMEOUT_PEER = 5, DEV_BAD_INDEX = 6 };

	// one mul_mat as the streaming GEMV sees it: this context's row shard of the two planes
	struct stream_op {
		const int8_t* wq;// [rows][K]
		const __half* wd;// [rows][K/32]
		const float* x;// [M][ldx]
		float* y;// already offset to this shard's first column
		long long ldx, ldy;
		int rows;
		int K;
		int rows_per_tile;
		int tile_begin;// index of this op's first tile in the batch-wide tile list
	};

	struct stream_batch {
		int n_ops;
		int total_tiles;
		int stage_bytes;// ring slot size
		int n_stages;
		stream_op op[NHB_MAX_BATCH];
	};

	// one mul_mat as the warp-per-row GEMV sees it
	struct rows_op {
		const int8_t* wq;
		const __half* wd;
		const float* x;
		float* y;// already offset to this shard's first column
		long long ldx, ldy;
		int rows;
		int K;
		int row_begin;// first row of this op in the batch-wide row list
		int act_off;// byte offset of this op's quantised activations in shared memory
		int preq_off;// byte offset of the same data in the pre-quantised scratch (preq mode)
		int pad;
		// the element-wise neighbours of the reference's FFN and attention cores (infra/core_traits.hpp:768-772, 976-992), fused:
		const float* x2;// not null: the activation is silu(x) * x2 (x = the gate projection's rows, x2 = the up projection's, same ldx)
		const float* res;// not null: res[m * ldr + n] is added to the output (the residual stream; offset like y)
		long long ldr;
	};

	// Fused all-gather of the decode GEMV.  A delivering launch (world > 1) stores its output values straight into all
	// ranks' copies of the output (peer-mapped memory) and counts itself completed.  The next launch of the context
	// (peers > 1) announces that count in a flag array on every rank, and every launch waits, for a bounded time, until the
	// other ranks have announced as much as the host found this launch depends on (wait_world > 1, wait_lag).
	struct push_ctl {
		int world;// > 1: this launch delivers its rows to the other ranks
		int wait_world;// > 1: wait for the other ranks' announcements before reading activations
		int rank;
		int wait_lag;// the wait is for every rank's announcement number (this rank's completed delivering launches - wait_lag)
		int peers;// > 1: the context exchanges rows: announce this rank's completed delivering launches first
		int pad;
		unsigned long long wait_ns;// bound of that wait
		unsigned* done_ctas;// local: CTAs of this grid that have stored everything
		unsigned* epoch;// local: number of delivering launches completed on this rank
		unsigned* announced;// local: the count this rank last announced
		unsigned* flags_local;// [world], written by the peers: their epoch after their matching launch
		unsigned* flags_peer[NHB_MAX_WORLD];// the same array on every rank (this rank's own included)
		int* status;// the context's device status word
	};

	struct rows_batch {
		int n_ops;
		int total_rows;
		int act_bytes;// dynamic shared memory
		int n_slots;// distinct activation inputs
		int slot_op[NHB_MAX_BATCH];// a representative op per slot
		int preq;// 1: activations were quantised by a separate kernel into preq_base
		int f32act;// 1: f32 activations x dequantised weights instead of the Q8 arithmetic
		const unsigned char* preq_base;
		// rms_norm x norm-weight inside the GEMV's prologue (null = off): every CTA normalises the rows for itself,
		// staging them as f32 at byte offset norm_off of the dynamic shared memory
		const float* norm_w;
		float norm_eps;
		int norm_sqrt;
		int norm_off;
		rows_op op[NHB_MAX_BATCH];
		push_ctl push;
		float* y_peer[NHB_MAX_BATCH][NHB_MAX_WORLD];// per op: the output on every rank, offset like rows_op::y
	};

	struct launch_cfg {
		cudaStream_t stream;
		int sm_count;
		bool pdl;// attach the programmatic-serialization attribute
		int* dev_status;
	};

	// gemv.cu
	cudaError_t launch_gemv_stream(const stream_batch& b, int M, const launch_cfg& cfg, int ctas_per_sm, int* launches);
	bool gemv_stream_supports(int64_t K, int64_t M);
	cudaError_t launch_gemv_ldg(const int8_t* wq, const __half* wd, const float* x, long long ldx, float* y, long long ldy, int rows, int K, int M,
		int act_mode, const launch_cfg& cfg, int* launches);
	int gemv_ldg_max_m(int64_t K, int act_mode);
	cudaError_t launch_quantize(const float* x, long long ldx, int M, int K, int8_t* q, float* d, cudaStream_t s, bool pdl = false);

	// gemv_rows.cu
	size_t gemv_rows_act_bytes(int64_t K, int M, bool f32act = false);
	size_t gemv_rows_norm_bytes(int64_t K, int M);// extra shared memory of the in-kernel rms_norm
	size_t gemv_rows_norm_smem_cap(bool fat);
	bool gemv_rows_norm_inside(int total_rows, size_t act_bytes, int64_t K, int M, int sm_count, bool fat_ctas);
	bool gemv_rows_supports(int64_t K, int64_t M, bool f32act = false);
	cudaError_t launch_gemv_rows(const rows_batch& b, int M, const launch_cfg& cfg, int ctas_per_sm, int* launches, bool double_buffer = false, int cluster = 1,
		bool fat_ctas = false, bool split_long_rows = false);
	// the CTA shape launch_gemv_rows takes for this batch: grid size, and whether CTAs get contiguous row ranges (split)
	struct rows_shape {
		int grid, warps;
		bool fat, split;
	};
	rows_shape gemv_rows_shape(const rows_batch& b, int M, int sm_count, int ctas_per_sm, bool double_buffer, int cluster, bool fat_ctas, bool split_long_rows);
	// a one-warp kernel that only waits for the other ranks' announcements (for consumers that are not GEMV launches)
	cudaError_t launch_peer_wait(const push_ctl& pc, const launch_cfg& cfg, int* launches);

	cudaError_t launch_block_dots(const int8_t* wq, const int8_t* qa, int rows, int K, int M, int32_t* dots, cudaStream_t s);

	// rms_norm.cu: any subset of the three outputs (null = not wanted)
	struct norm_out {
		float* y;// [M][ldy] f32 rows
		long long ldy;
		int8_t* q;// [M][K] quants ...
		float* d;// ... with [M][K/32] f32 scales (the layout the decode GEMV stages from)
		unsigned char* blocks;// [M][K/32] 34-byte Q8_0 blocks
	};
	bool rms_norm_supports(long long K);
	cudaError_t launch_rms_norm(const float* x, long long ldx, const float* w, float eps, int sqrt_mode, int M, int K, const norm_out& o, cudaStream_t s,
		bool pdl = false);

	// elementwise.cu: h = silu(gate) * up, and y += res on `cols` columns
	cudaError_t launch_swiglu(const float* gate, const float* up, long long ld, float* h, long long ldh, int M, int K, cudaStream_t s, bool pdl = false);
	cudaError_t launch_add_rows(float* y, long long ldy, const float* res, long long ldr, int M, int cols, cudaStream_t s, bool pdl = false);

	// repack.cu
	cudaError_t launch_repack(const uint8_t* blocks34, int64_t rows, int64_t K, int8_t* q, __half* d, cudaStream_t s);
	cudaError_t launch_unpack(const int8_t* q, const __half* d, int64_t rows, int64_t K, uint8_t* blocks34, cudaStream_t s);

	// gemm_tc.cu
	struct gemm_plan {
		int swapped;// 0: lanes = weight rows, columns = tokens; 1: lanes = tokens, columns = weight rows
		int n_t;// columns per tile
		int lane_tiles, col_tiles;
	};
	gemm_plan gemm_tc_plan(int64_t rows, int64_t M, int sms);
	bool gemm_tc_supports(int64_t rows, int64_t K, int64_t M);
	int gemm_tc_pad(int64_t n);
	size_t gemm_tc_scratch_bytes(int64_t K, int64_t M, int64_t rows, int sms);
	size_t gemm_tc_counter_bytes();
	cudaError_t launch_weight_gemm_planes(const int8_t* q, const __half* d, int64_t rows, int64_t K, __half* w16, float* wdT, cudaStream_t s);
	cudaError_t launch_gemm_tc(const __half* w16, const float* wdT, const float* x, long long ldx, float* y, long long ldy, int rows, int K, int M, void* scratch,
		unsigned* counters, const launch_cfg& cfg, int* launches, std::string* err, bool activations_ready = false);

}
