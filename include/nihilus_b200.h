/*
 * nihilus_b200 -- C ABI of the B200 (sm_100a) Q8_0 mul_mat path.
 *
 * This is the boundary a Nihilus maintainer binds: plain C types, device pointers owned by the
 * caller, no exceptions, no implicit device synchronisation.  Every entry point returns an int
 * status (0 = ok, negative = error, text via nhb_last_error).  Each declaration cites the piece of
 * the reference it stands in for (paths relative to the reference's include/nihilus-incl/).
 *
 * Conventions (same as the reference's tensors, infra/core_traits.hpp:145-182):
 *   weight  W : N rows, each K/32 Q8_0 blocks of 34 bytes {fp16 d; int8 qs[32]}  (ne0 = K contiguous)
 *   input   X : M rows of K floats, row m at x + m*ldx                             (ne0 = K contiguous)
 *   output  Y : M rows of N floats, Y[m*ldy + n] = W[n,:] . X[m,:]                 (ne0 = N contiguous)
 * A context owns one GPU and one row shard [n0, n1) of every weight it uploads; with world > 1 it
 * writes only columns [n0, n1) of Y and nhb_all_gather completes the rows on every rank.
 */
#ifndef NIHILUS_B200_H
#define NIHILUS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NHB_VERSION 100

enum nhb_status {
	NHB_OK				= 0,
	NHB_ERR_ARG			= -1, /* null pointer, K not a multiple of 32, M < 0, bad leading dimension ... */
	NHB_ERR_CUDA		= -2, /* a CUDA runtime call failed (text in nhb_last_error) */
	NHB_ERR_NCCL		= -3,
	NHB_ERR_TIMEOUT		= -4, /* a bounded device-side wait ran out; the context stays usable */
	NHB_ERR_UNSUPPORTED = -5,
	NHB_ERR_NOMEM		= -6
};

/* Which of the reference's two arithmetics to run (both exist in cpu/avx_2.hpp):
 *   NHB_ACT_Q8  activations quantised to Q8_0 (quantize_row_q8_0, :4439-4489), exact int8 block dots, scales
 *               applied per block (vec_dot_q8_0_q8_0, :4534-4780)
 *   NHB_ACT_F32 f32 activations times dequantised weights (vec_dot_q8_f32, :4782-4852) */
enum nhb_act_mode { NHB_ACT_Q8 = 0, NHB_ACT_F32 = 1 };

/* kernel choice; AUTO picks from M (the reference picks by processing_phases, common/kernel_traits.hpp:114-117) */
enum nhb_kernel {
	NHB_KERNEL_AUTO		   = 0,
	NHB_KERNEL_GEMV_LDG	   = 1, /* any K % 32 == 0: coalesced 128-bit loads, dp4a, warp-shuffle reduce */
	NHB_KERNEL_GEMV_STREAM = 2, /* K % 256 == 0, K <= 16384: persistent CTAs fed by a bulk-copy (TMA) ring */
	NHB_KERNEL_GEMM_TC	   = 3, /* tcgen05 / TMEM tensor-core contraction for prefill */
	NHB_KERNEL_GEMV_ROWS   = 4	/* default GEMV: warp per row, batched ops, weight loads issued ahead of the previous kernel's end */
};

typedef struct nhb_ctx nhb_ctx;
typedef struct nhb_weight nhb_weight;
typedef struct nhb_graph nhb_graph;
typedef struct nhb_chain nhb_chain;

typedef struct nhb_weight_info {
	int64_t N, K;	  /* full logical shape */
	int64_t n0, n1;	  /* rows held by this context */
	const void* q;	  /* device: int8 plane  [n1-n0][K], 256-byte aligned */
	const void* d;	  /* device: fp16 plane  [n1-n0][K/32], 256-byte aligned */
	int64_t bytes_q8; /* (n1-n0) * (K/32) * 34: the Q8_0 bytes this shard stands for */
} nhb_weight_info;

/* one independent mul_mat of a batch (no op of a batch may read another op's output) */
typedef struct nhb_mul_mat_op {
	const nhb_weight* w;
	const float* x; /* device */
	int64_t ldx;
	float* y; /* device */
	int64_t ldy;
	int64_t M;
} nhb_mul_mat_op;

/* ---- library ---- */
int nhb_version(void);
/* compute capability the kernels were built for (100); replaces the build-time arch index of
 * infra/monolithic_dispatcher.hpp:30-39, which has no entry for compute capability 10 */
int nhb_arch(void);
/* last error text of this thread (ctx may be NULL for errors raised before a context existed) */
const char* nhb_last_error(const nhb_ctx* ctx);

/* ---- host-only helpers (no GPU needed) ---- */
/* rows [n0, n1) of an N-row weight owned by `rank` of `world`; the remainder goes to the lowest ranks.
 * No counterpart in the reference (device 0 is hard-wired, cuda/common.hpp:36-40). */
int nhb_shard_rows(int64_t N, int world, int rank, int64_t* n0, int64_t* n1);
/* the rows nhb_weight_upload_q8_0 gives `rank`: the shard above, or all N rows when the weight's Q8_0 size,
 * N * (K/32) * 34 bytes, is below `replicate_below_bytes` (the "replicate_below_mb" option of a context) */
int nhb_place_rows(int64_t N, int64_t K, int world, int rank, int64_t replicate_below_bytes, int64_t* n0, int64_t* n1);
/* 34-byte blocks -> int8 plane + fp16 plane for rows [n0, n1); the layout nhb_weight_upload_q8_0 builds on the GPU */
int nhb_repack_q8_0_host(const void* blocks34, int64_t N, int64_t K, int64_t n0, int64_t n1, int8_t* q_plane, uint16_t* d_plane);
int nhb_unpack_q8_0_host(const int8_t* q_plane, const uint16_t* d_plane, int64_t rows, int64_t K, void* blocks34);
/* GEMV (1), or GEMM (3) for this M?  The runtime form of the reference's compile-time eval/prompt split. */
int nhb_choose_kernel(int64_t N, int64_t K, int64_t M, int act_mode);
/* the tile shape the tensor-core GEMM takes for `rows` weight rows and M tokens on a GPU with `sms` SMs: 128 rows of one
 * side on the TMEM lanes (tokens when *swapped, else weight rows), *tile_cols (16..256) rows of the other side on the
 * columns, *lane_tiles x *col_tiles CTAs.  Host-only; for tests and for reading performance numbers. */
int nhb_gemm_tile_plan(int64_t rows, int64_t M, int sms, int* swapped, int* tile_cols, int* lane_tiles, int* col_tiles);
/* algorithmic bytes / flops of one mul_mat: N*(K/32)*34 + 4*M*K + 4*M*N and 2*M*N*K */
int64_t nhb_mul_mat_bytes(int64_t N, int64_t K, int64_t M);
int64_t nhb_mul_mat_flops(int64_t N, int64_t K, int64_t M);

/* ---- context: replaces thread_pool<gpu> + memory_buffer<gpu> for this path (cuda/thread_pool.hpp:46-67,
 *      cuda/memory_buffer.hpp:78-152) ---- */
int nhb_ctx_create(nhb_ctx** out, int device, int rank, int world);
int nhb_ctx_destroy(nhb_ctx* ctx);
/* run everything on the caller's cudaStream_t.  NULL selects the context's own non-blocking stream; to name the
 * legacy default stream pass cudaStreamLegacy, not 0. */
int nhb_ctx_set_stream(nhb_ctx* ctx, void* cuda_stream);
/* explicit synchronisation + device status check; the reference syncs after every launch (cuda/cuda_12.hpp:679) */
int nhb_sync(nhb_ctx* ctx);
/* largest M served by the GEMV family under NHB_KERNEL_AUTO (default 8) */
int nhb_ctx_set_gemv_max_m(nhb_ctx* ctx, int max_m);
/* tuning knobs: "pdl" (programmatic dependent launch, default 1), "gemv_kernel" (1, 2 or 4: what AUTO uses for
 * small M), "rows_ctas_per_sm", "prequantize", "ctas_per_sm" (streaming GEMV, 1 or 2), "gemv_max_m", "rows_fat_ctas",
 * "rows_split_long", "rows_double_buffer" (-1 chooses per launch), "fused_gather", "peer_window" and "peer_wait_us" (see
 * nhb_symm_alloc), "gemm_keep_planes" (default 1: the tensor-core GEMM keeps an fp16 copy of a weight's quants and its
 * scales in block-major order with the weight, 2.125 bytes per weight, made at the weight's first GEMM; 0: they are rebuilt
 * into one buffer of the context in front of every GEMM -- the memory of the largest weight instead of the whole model's,
 * for about 45 us more per GEMM of a 14336 x 4096 weight: +30 % at 512 tokens, +8 % at 2048; same results), and the placement policy "replicate_below_mb": with world > 1, a weight smaller
 * than that many MiB is kept whole on every rank (n0 = 0, n1 = N; every rank computes every row, no exchange) instead of
 * row-sharded -- set it before uploading; 0 (default) shards everything */
int nhb_ctx_set_option(nhb_ctx* ctx, const char* name, int value);
/* kernels this context has launched so far (upload, mul_mat, gather ...) */
long long nhb_ctx_launch_count(const nhb_ctx* ctx);
/* asynchronous copies on the context stream: memory_transfer<gpu>::host_to_device / device_to_host
 * (cuda/memory_buffer.hpp:33-74) without the blocking */
int nhb_memcpy_h2d(nhb_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int nhb_memcpy_d2h(nhb_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
/* plain device memory on the context's GPU for activations and outputs: what memory_buffer<gpu>::init does for the
 * reference's arena (cuda/memory_buffer.hpp:78-152).  256-byte aligned; not for use during graph capture. */
int nhb_device_alloc(nhb_ctx* ctx, size_t bytes, void** out_dev);
int nhb_device_free(nhb_ctx* ctx, void* dev);

/* ---- weights: replaces the verbatim 34-byte upload of infra/model_parser.hpp:151-154, :933-937 ---- */
/* host_blocks34 = the tensor's bytes as they sit in the GGUF file (N*(K/32)*34 bytes, whole tensor);
 * only this context's row shard is copied to the GPU and repacked there into the two planes. */
int nhb_weight_upload_q8_0(nhb_ctx* ctx, const void* host_blocks34, int64_t N, int64_t K, nhb_weight** out);
int nhb_weight_free(nhb_ctx* ctx, nhb_weight* w);
int nhb_weight_info_get(const nhb_weight* w, nhb_weight_info* info);
/* planes back to 34-byte blocks on the host (rows n0..n1 only) -- for round-trip checks */
int nhb_weight_download_q8_0(nhb_ctx* ctx, const nhb_weight* w, void* host_blocks34_shard);

/* ---- the operator: fills the empty GPU cores of cuda/cuda_12.hpp:803-952; arithmetic of cpu/avx_2.hpp:4749-5004 ----
 * X and Y must not overlap (NHB_ERR_ARG). */
int nhb_mul_mat(nhb_ctx* ctx, const nhb_weight* w, const float* x_dev, int64_t ldx, float* y_dev, int64_t ldy, int64_t M, int act_mode,
	int kernel);
/* several independent mul_mats (q/k/v of one layer, gate/up of one layer ...) in one persistent launch */
int nhb_mul_mat_batch(nhb_ctx* ctx, const nhb_mul_mat_op* ops, int n_ops, int act_mode, int kernel);
/* same operator with HOST activations and outputs: copies X up, runs, copies this shard's Y columns back
 * (asynchronous on the context stream; the buffers must stay valid until nhb_sync) */
int nhb_mul_mat_host(nhb_ctx* ctx, const nhb_weight* w, const float* x_host, int64_t ldx, float* y_host, int64_t ldy, int64_t M,
	int act_mode, int kernel);
/* exact per-block int32 dots of the Q8 arithmetic: dots[((m*rows)+r)*(K/32)+b] for this shard's rows */
int nhb_mul_mat_block_dots(nhb_ctx* ctx, const nhb_weight* w, const float* x_dev, int64_t ldx, int64_t M, int32_t* dots_dev);
/* the activation quantiser alone (quantize_row_q8_0, cpu/avx_2.hpp:4439-4489): int8 [M][K] and f32 scales
 * (the fp16-rounded d, widened) [M][K/32] */
int nhb_quantize_q8_0(nhb_ctx* ctx, const float* x_dev, int64_t ldx, int64_t M, int64_t K, int8_t* q_dev, float* d_dev);

/* ---- the element-wise neighbours of the mul_mats in the reference's FFN and attention cores, fused ----
 * The reference's chains are ffn_gate_mul_mat -> silu -> mul(ffn_up_mul_mat) -> ffn_down_mul_mat -> add(ffn_inp)
 * (infra/core_traits.hpp:976-992) and attn_out_mul_mat -> add(inp_embd) (:768-772).  Its kernels for silu, mul and add are
 * empty (cpu/avx_2.hpp:1946-2075, 5325-5330), the traits name the arithmetic: f32, silu(g) = g / (1 + exp(-g)).
 *   nhb_mul_mat_swiglu_add   y = W . quantise(silu(gate) * up) [+ residual]      W = ffn_down; gate, up [M][ld] with K = W's K
 *   nhb_mul_mat_add          y = W . quantise(x) + residual                      W = attn_output
 * For decode (M <= gemv_max_m) SwiGLU runs inside the GEMV's activation prologue and the residual is added as the row is
 * stored: no intermediate row, no extra launch.  For more tokens the element-wise kernels run around the tensor-core
 * GEMM.  Q8 arithmetic; the values are those of the separate steps (nhb_swiglu, nhb_mul_mat, a float add), bit for bit.
 * residual may be NULL in the first; residual[m * ld_residual + n] belongs to output column n (full width N). */
int nhb_mul_mat_swiglu_add(nhb_ctx* ctx, const nhb_weight* w, const float* gate_dev, const float* up_dev, int64_t ld, const float* residual_dev,
	int64_t ld_residual, float* y_dev, int64_t ldy, int64_t M);
int nhb_mul_mat_add(nhb_ctx* ctx, const nhb_weight* w, const float* x_dev, int64_t ldx, const float* residual_dev, int64_t ld_residual, float* y_dev, int64_t ldy,
	int64_t M);
/* h[m][k] = silu(gate[m][k]) * up[m][k] on its own (16-byte aligned rows, K, ld and ldh multiples of 4) */
int nhb_swiglu(nhb_ctx* ctx, const float* gate_dev, const float* up_dev, int64_t ld, float* h_dev, int64_t ldh, int64_t M, int64_t K);

/* ---- rms_norm x norm-weight: the producer of a projection's activations ----
 * Replaces the reference's rms_norm_mul kernel (cpu/avx_2.hpp:3875-3950) and its helpers simd_sum_squares
 * (:758-779), vec_scale_mul_f32 (:3621-3850) and quantize_row_q8_0_avx2 (:671-721), bit for bit:
 *   scale = 1 / sqrtf_fast(sum_squares(x) / K + eps),  y = (x * norm_w) * scale.
 * sqrt_mode picks which of the reference's two sqrtf_fast builds is reproduced: */
#define NHB_SQRT_IEEE 0     /* the IEEE square root (the NEON build, cpu/common.hpp:310-312) */
#define NHB_SQRT_X86_FAST 1 /* the x86 build's integer formula (cpu/common.hpp:448-450); as written it returns about
                               2^64 * sqrt(x), so every output carries a factor of about 2^-64 */
/* x [M][ldx] -> y [M][ldy], f32, device pointers 16-byte aligned, ldx and ldy multiples of 4, K % 32 == 0, K <= 51200 */
int nhb_rms_norm_mul(nhb_ctx* ctx, const float* x_dev, int64_t ldx, const float* norm_w_dev, float eps, int sqrt_mode, float* y_dev,
	int64_t ldy, int64_t M, int64_t K);
/* the same rows quantised with quantize_row_q8_0: 34-byte Q8_0 blocks [M][K/32] in device memory */
int nhb_rms_norm_mul_q8_0(nhb_ctx* ctx, const float* x_dev, int64_t ldx, const float* norm_w_dev, float eps, int sqrt_mode,
	void* blocks_dev, int64_t M, int64_t K);
/* rms_norm x norm-weight feeding a batch of Q8-arithmetic mul_mats (q/k/v, or gate/up): ops[i].x is the row BEFORE the
 * norm and must be the same pointer, ldx and K in every op.  Results are bit-identical to nhb_rms_norm_mul followed by
 * nhb_mul_mat_batch(NHB_ACT_Q8).  For decode (the warp-per-row GEMV) the norm kernel writes the quantised row once
 * and the GEMV stages it as is; for larger M the normalised rows go through a scratch buffer of the context. */
int nhb_rms_norm_mul_mat_batch(nhb_ctx* ctx, const nhb_mul_mat_op* ops, int n_ops, const float* norm_w_dev, float eps, int sqrt_mode,
	int kernel);

/* ---- the Q8_0 consumers around the projections ---- */
/* Token-embedding gather: y[m][k] = f32(d) * float(q) of row token_ids[m] of a Q8_0 table [N = vocabulary][K = embedding
 * length], f32 rows out.  Stands in for the reference's two live GPU kernels (cuda/cuda_12.hpp:560-601 prompt, :691-722
 * eval) with the prompt kernel's arithmetic in both phases: the reference's eval kernel ignores the token id and reads
 * row 0 (:710).  The table must be whole on this rank; an id outside [0, N) leaves its row untouched and makes the next
 * nhb_sync return NHB_ERR_ARG.  token_ids_dev: device int32 [M]; y_dev 16-byte aligned, ldy >= K and a multiple of 4. */
int nhb_get_rows_q8_0(nhb_ctx* ctx, const nhb_weight* table, const int32_t* token_ids_dev, int64_t M, float* y_dev, int64_t ldy);
/* The mul_mat side of final_norm_and_sampling (infra/core_traits.hpp:1184-1193): the last of seq_len hidden rows ->
 * rms_norm x output_norm -> logits = W_output . quantise(row), one launch for decode shapes.  logits_dev: f32 [N]. */
int nhb_last_token_logits(nhb_ctx* ctx, const nhb_weight* w_output, const float* hidden_dev, int64_t ld, int64_t seq_len, const float* norm_w_dev, float eps,
	int sqrt_mode, float* logits_dev);

/* ---- cache of repacked weights ---- */
/* The two planes of this context's shard of a weight as one file (header with shape, rows, rank and world, a checksum, then
 * the planes), and back: a later start reads the planes straight into device memory instead of reading, sharding and
 * repacking the tensor's 34-byte blocks (the reference maps and copies the GGUF tensor at every start,
 * infra/model_parser.hpp:897-940).  nhb_weight_load takes the weight's full shape and refuses a file whose rows are not the
 * ones this context would own for it (another rank, world size or placement policy), a truncated file or a bad checksum. */
int nhb_weight_save(nhb_ctx* ctx, const nhb_weight* w, const char* path);
int nhb_weight_load(nhb_ctx* ctx, const char* path, int64_t N, int64_t K, nhb_weight** out);

/* ---- GGUF reader in front of the upload ----
 * Stands in for the reference's model file parser on this path (infra/model_parser.hpp:635-671 header and metadata,
 * :855-880 tensor table, :890-940 data placement): same magic, limits (100000 tensors, 10000 key/values, 4 dimensions,
 * 2^32 per dimension), data section located from the end of the file, offsets rounded up to general.alignment.  The
 * file is mapped read-only; tensor data is never copied on the host except into the upload's pinned staging. */
typedef struct nhb_gguf nhb_gguf;
typedef struct nhb_gguf_tensor {
	const char* name; /* valid until nhb_gguf_close */
	int n_dims;
	int64_t dims[4]; /* ne0 (contiguous) first; unused dimensions are 1 */
	int type;		 /* ggml type id: 0 f32, 1 f16, 8 q8_0 ... (common/config.hpp:179-201) */
	int64_t bytes;
	int64_t offset;	  /* absolute file offset of the data */
	const void* data; /* the mapped bytes */
} nhb_gguf_tensor;
int nhb_gguf_open(const char* path, nhb_gguf** out);
const char* nhb_gguf_last_error(void); /* why the last nhb_gguf_open on this thread failed */
int nhb_gguf_close(nhb_gguf* g);
int64_t nhb_gguf_tensor_count(const nhb_gguf* g);
int64_t nhb_gguf_find(const nhb_gguf* g, const char* name); /* index or -1 */
int nhb_gguf_tensor_get(const nhb_gguf* g, int64_t index, nhb_gguf_tensor* out);
/* scalar metadata by key (integers, floats and booleans as double; e.g. "llama.attention.layer_norm_rms_epsilon") */
int nhb_gguf_get_number(const nhb_gguf* g, const char* key, double* out);
const char* nhb_gguf_get_string(const nhb_gguf* g, const char* key); /* NULL when absent */
/* a Q8_0 matrix [ne1 = N rows][ne0 = K] by tensor name, e.g. "blk.0.attn_q.weight": sharded, repacked, uploaded */
int nhb_gguf_upload_q8_0(nhb_ctx* ctx, const nhb_gguf* g, const char* name, nhb_weight** out);
/* an f32 tensor (norm weights) copied out of the mapping; count must equal its element count */
int nhb_gguf_read_f32(const nhb_gguf* g, const char* name, float* dst, int64_t count);

/* ---- for callers that cannot allocate ---- */
/* No counterpart in the reference.  The decode GEMV (Q8 arithmetic, M <= 4) without a context, a weight handle or
 * any allocation: the caller passes the two device planes of a weight (as nhb_weight_info_get returns them, or as
 * nhb_repack_q8_0_host lays them out: int8 [rows][K], 32-byte aligned, and fp16 [rows][K/32]), device activations
 * and outputs, and a cudaStream_t.  It is meant for hosts that must not call cudaMalloc where they run the
 * operator: an engine that split one device arena at start-up by a fixed memory plan, or a token loop that cannot
 * afford the device-wide synchronisation an allocation may cause.  The only temporary -- the Q8_0-quantised activations -- lives in a
 * fixed 96 KiB array inside the library image (every GPU that loads the library holds it until the process
 * exits), so a call is rejected with NHB_ERR_UNSUPPORTED unless M <= 4 and M * (K + K/8) <= 98304 bytes.
 * The first call on each device looks up the array's device address; make that first call outside any stream
 * capture.  All calls share the array and it keeps what the last call wrote (each call rewrites every byte it
 * later reads, so nothing needs clearing): calls that overlap on the GPU -- two streams, two host threads -- race
 * on it and must be serialised by the caller.  Never calls cudaMalloc, cudaFree or any allocating routine. */
int nhb_mul_mat_q8_0_noalloc(const void* q_plane, const void* d_plane, int64_t rows, int64_t K, const float* x_dev, int64_t ldx,
	float* y_dev, int64_t ldy, int64_t M, void* cuda_stream);
/* capacity of that array in bytes (98304) and the last error text of this thread for the call above */
int64_t nhb_noalloc_max_bytes(void);
const char* nhb_noalloc_last_error(void);

/* ---- a token's whole sequence of decode stages, recorded once ----
 * Stands in for what thread_pool<gpu>::execute_tasks does per token (cuda/thread_pool.hpp:46-67: the input core, the
 * per-block cores of every layer, the output core, one after the other) on the mul_mat side of those cores.
 * `ops` lists the stages back to back, ops_per_stage[s] (1..8) independent mul_mats each (q/k/v; o; gate/up; down; ...
 * lm_head); ops of one stage that read the same activations quantise them once.  Every op of stage s+1 may read any
 * output of stage s.  nhb_chain_create checks the arguments and builds the launch descriptors once; nhb_chain_launch
 * enqueues one warp-per-row GEMV launch per stage with programmatic dependent launch between them (a stage's weight
 * stream starts while the stage before it drains), without per-call argument checks, and can itself be captured with
 * nhb_graph_begin.  Q8 arithmetic, 1 <= M <= 4 (the same M in every op), K % 32 == 0 and M rows of every distinct input
 * of a stage within 96 KB of shared memory (NHB_ERR_UNSUPPORTED otherwise: run such stages with nhb_mul_mat_batch).
 * Results are bit-identical to nhb_mul_mat_batch stage by stage.  The op list is read at create time; the activations
 * and outputs it names must stay valid for every launch.  With world > 1 the rules of nhb_symm_alloc apply per stage:
 * outputs in symmetric memory are delivered to every rank, a stage that reads them waits for the ranks that deliver
 * them, and the outputs of the LAST stage are whole after nhb_all_gather (or nhb_sync).
 * (A single persistent kernel for the whole sequence, with a device-side barrier between stages, was built and measured
 * slower than these launches -- the barrier and the per-stage prologue cost more than a launch boundary -- and is not
 * part of the library.) */
int nhb_chain_create(nhb_ctx* ctx, const nhb_mul_mat_op* ops, const int* ops_per_stage, int n_stages, nhb_chain** out);
int nhb_chain_launch(nhb_ctx* ctx, nhb_chain* chain);
int nhb_chain_free(nhb_ctx* ctx, nhb_chain* chain);

/* ---- launch-overhead removal: record a sequence of nhb_mul_mat* calls once, replay it per token ---- */
int nhb_graph_begin(nhb_ctx* ctx);
int nhb_graph_end(nhb_ctx* ctx, nhb_graph** out);
int nhb_graph_launch(nhb_ctx* ctx, nhb_graph* g);
int nhb_graph_free(nhb_ctx* ctx, nhb_graph* g);

/* ---- multi-GPU (one context per GPU / per process); no counterpart in the reference ---- */
/* 128-byte NCCL unique id made by rank 0 and handed to every rank by the caller's own transport */
int nhb_comm_unique_id(void* id128);
int nhb_comm_init(nhb_ctx* ctx, const void* id128);
/* Output memory for the fused all-gather of the decode GEMV.  Collective: every rank calls it after nhb_comm_init, with
 * the same size, in the same order; each rank gets its own allocation and a mapping of every other rank's (CUDA IPC, so
 * one process per GPU and peer access between the GPUs are required).  When every output of a GEMV launch (M <= 8) lies
 * in such memory at the same offset on every rank, the kernel stores each value into all ranks' copies (plain stores
 * over NVLink) and counts itself a completed "delivering launch"; nhb_all_gather on such an output enqueues no collective.
 * All ranks must issue the same sequence of delivering launches.
 *
 * When the rows are whole.  Delivery is asynchronous: the NEXT launch of the context (any nhb_mul_mat*, nhb_chain_launch,
 * nhb_all_gather*, nhb_sync) first announces this rank's completed deliveries to every rank, and a launch waits for the
 * other ranks' announcements only as far as it must:
 *   - a GEMV launch that READS delivered rows (activations, SwiGLU operand, residual in symmetric memory) waits in its
 *     prologue, after its weight stream has started, until every rank has announced the launch that delivers them;
 *   - every other entry point that may read them (the GEMM path, rms_norm, nhb_get_rows_q8_0, nhb_memcpy_d2h,
 *     nhb_all_gather*, nhb_sync) waits for everything delivered so far;
 *   - kernels of the caller's own on the same stream must be preceded by nhb_all_gather* on the outputs they read.
 * Everything else runs on while the exchange is in flight.
 *
 * When a buffer may be written again.  A delivering launch writes into the peers' copies, so the peers must be done
 * with the previous contents.  What this library's own GEMV launches read and write is tracked: a delivering launch that
 * rewrites rows an earlier launch of this context read (or wrote without delivering them: a weight kept whole on every
 * rank) waits until every rank has announced the first delivering launch enqueued at or after that launch, and any
 * launch that writes rows still being delivered waits for that delivery.  So a reader that delivers rows itself may be
 * followed directly by the launch that rewrites what it read (a stage sequence that ping-pongs between two buffers);
 * after a launch that delivers nothing, at least one other delivering launch must come before its rows are delivered
 * into.  Independently, every second delivering launch checks that the
 * slowest rank is within "peer_window" (option, default 4) delivering launches, so no launch runs more than
 * peer_window + 1 ahead; rows read by kernels this library does not know of may therefore be rewritten once
 * peer_window + 2 further delivering launches have been enqueued after that reader, or once the ranks have met on the
 * host after their nhb_sync.  "peer_window" = 0 makes every launch wait for every earlier delivery (ranks in lock step).
 *
 * Every wait is bounded by option "peer_wait_us" (default 2 000 000): a peer that never shows up ends it, the kernel
 * carries on and finishes, and nhb_sync returns NHB_ERR_TIMEOUT and resets this rank's side of the exchange (every rank
 * must then pass an nhb_sync, and the ranks must meet on the host, before the next delivering launch).  Option
 * "fused_gather" = 0 keeps NCCL. */
int nhb_symm_alloc(nhb_ctx* ctx, size_t bytes, void** out_dev);
int nhb_symm_free(nhb_ctx* ctx, void* dev);
/* The same for ONE process that drives several GPUs from one thread, as the reference's host does (one process, one
 * thread per model: cuda/thread_pool.hpp:46-67): ctxs[i] is rank i of a world of n, all created in this process on
 * distinct devices with peer access.  nhb_symm_alloc_local allocates `bytes` on every context's device and gives every
 * context plain pointers to the others' allocations (no IPC handles, no NCCL); out_dev[i] is rank i's buffer.  The fused
 * all-gather of the decode GEMV then works as described above; enqueue each step's calls for all contexts (rank 0, rank
 * 1, ...) before blocking on any of them, and block with nhb_sync_all, which first enqueues every context's wait for its
 * peers and only then synchronises -- nhb_sync on one context alone would wait for announcements the other contexts have
 * not been asked to make yet.  nhb_all_gather_local completes Y[M][N] on every rank for outputs that were not delivered
 * by a fused launch (the GEMM path): peer copies of every rank's column slice (nhb_shard_rows) ordered by events across
 * the contexts' streams; y_dev[i] is rank i's buffer, all with the same ldy.  Free with nhb_symm_free per context. */
int nhb_symm_alloc_local(nhb_ctx* const* ctxs, int n, size_t bytes, void** out_dev);
int nhb_all_gather_local(nhb_ctx* const* ctxs, int n, float* const* y_dev, int64_t ldy, int64_t M, int64_t N);
int nhb_sync_all(nhb_ctx* const* ctxs, int n);
/* The decisions behind "a launch waits only as far as it must", on their own and without a GPU: feed the planner the
 * symmetric allocations and then, in enqueue order, what every warp-per-row launch reads and (if it delivers) completes
 * on every rank; it answers whether that launch polls the peers' announcements and with which lag (it waits until every
 * peer has announced this rank's completed delivering launches minus lag).  nhb_wait_planner_wait_all stands for nhb_sync /
 * nhb_all_gather* (returns 1 if a wait was needed).  The library runs the same code; tests replay programs against a
 * model of ranks that drift apart (tests/test_wait_planner.py). */
typedef struct nhb_wait_planner nhb_wait_planner;
nhb_wait_planner* nhb_wait_planner_create(int peer_window);
void nhb_wait_planner_destroy(nhb_wait_planner* p);
int nhb_wait_planner_add_region(nhb_wait_planner* p, const void* base, size_t bytes);
int nhb_wait_planner_launch(nhb_wait_planner* p, const void* const* in, const size_t* in_bytes, int n_in, const void* const* out, const size_t* out_bytes,
	int n_out, int delivers, int* waits, int* lag);
int nhb_wait_planner_wait_all(nhb_wait_planner* p);
long long nhb_wait_planner_seq(const nhb_wait_planner* p);
/* what nhb_graph_begin / nhb_graph_end / nhb_graph_launch do to the bookkeeping: the launches planned between begin and end keep
 * their answers for every replay; _capture_end returns the recording's number, _replayed accounts for one replay of it */
void nhb_wait_planner_capture_begin(nhb_wait_planner* p);
int nhb_wait_planner_capture_end(nhb_wait_planner* p);
int nhb_wait_planner_replayed(nhb_wait_planner* p, int recording);
/* complete Y[M][N] (ldy) on every rank from the column slices each rank wrote */
int nhb_all_gather(nhb_ctx* ctx, float* y_dev, int64_t ldy, int64_t M, int64_t N);
/* several outputs in one grouped collective (q/k/v, gate/up) */
int nhb_all_gather_batch(nhb_ctx* ctx, float* const* y_dev, const int64_t* ldy, const int64_t* M, const int64_t* N, int n);

#ifdef __cplusplus
}
#endif
#endif
