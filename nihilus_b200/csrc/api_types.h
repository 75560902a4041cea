// Host-side types and helpers shared by the translation units behind the C ABI (api.cu, extras.cu).  Not part of the ABI.
#pragma once
#include <algorithm>
#include <string>
#include <vector>

#include "deliveries.h"
#include "internal.h"

typedef struct ncclComm* ncclComm_t;

struct nhb_ctx {
	int device		   = 0;
	int rank		   = 0;
	int world		   = 1;
	int sm_count	   = 148;
	cudaStream_t own   = nullptr;
	cudaStream_t stream = nullptr;
	int* dev_status	   = nullptr;
	int* host_status   = nullptr;// pinned
	void* scratch	   = nullptr;
	size_t scratch_cap = 0;
	unsigned* gemm_counters = nullptr;// arrival counters of the GEMM's split tiles
	bool gemm_keep_planes	= true;// false: a weight's fp16 operand planes are rebuilt before every GEMM instead of kept with the weight
	void* plane_buf			= nullptr;
	size_t plane_cap		= 0;
	void* io		   = nullptr;
	size_t io_cap	   = 0;
	ncclComm_t comm	   = nullptr;
	bool pdl		   = true;
	int gemv_max_m	   = 8;
	int ctas_per_sm	   = 1;// streaming GEMV: persistent CTAs per SM
	int rows_cps	   = 3;// warp-per-row GEMV: grid cap in CTAs per SM
	int preq		   = 0;// warp-per-row GEMV: quantise activations in a separate kernel
	// set only while nhb_rms_norm_mul_mat_batch runs: the GEMV's activations come from the norm kernel, already quantised
	const float* norm_w = nullptr;
	float norm_eps		= 0.f;
	int norm_sqrt		= 0;
	void* norm_buf		= nullptr;// normalised f32 rows for the paths that quantise for themselves
	size_t norm_cap		= 0;
	int rows_db		   = -1;// warp-per-row GEMV: two items in flight per warp (1), one (0), or chosen per launch (-1)
	int rows_cluster   = 1;// warp-per-row GEMV: CTAs per cluster sharing the activation quantisation
	int rows_fat	   = 1;// warp-per-row GEMV: one 24-warp CTA per SM for launches with enough rows
	int rows_split	   = 1;// ... and within those, the item-parallel kernel for rows longer than 4096
	int gemv_default   = NHB_KERNEL_GEMV_ROWS;
	bool capturing	   = false;
	long long launches = 0;
	std::string err;
	// fused all-gather (decode GEMV): peer-mapped output regions, the flag array every rank can write, local counters
	struct symm_region {
		char* local	 = nullptr;
		size_t bytes = 0;
		char* peer[NHB_MAX_WORLD] = {};// this rank's own entry is `local`
		bool ipc = true;// the other ranks' entries are CUDA IPC mappings (to be closed); false: plain pointers of this process
	};
	// outputs whose rows are already whole on every rank (delivered by a fused launch, or computed from a replicated
	// weight): nhb_all_gather has nothing to do for them.  Keyed by the output pointer the caller passes.
	std::vector<const void*> complete;
	int64_t replicate_below = 0;// bytes: smaller weights are kept whole on every rank instead of row-sharded
	std::vector<symm_region> regions;
	// upload staging: two pinned host buffers, two device buffers, an event each (kept for the next upload)
	void* up_pinned[2]	   = { nullptr, nullptr };
	void* up_dev[2]		   = { nullptr, nullptr };
	cudaEvent_t up_done[2] = { nullptr, nullptr };
	size_t up_cap		   = 0;
	unsigned* push_local = nullptr;// [0] CTAs done in the running launch, [1] delivering launches completed, [2] the count last announced to the peers
	int fused_gather	 = 1;
	nhb_deliveries dl;
	unsigned long long cap_seq0 = 0;// dl.seq when the open capture began
	int peer_window		 = 4;// a launch never runs further ahead of the slowest rank than this many delivering launches
	long long peer_wait_us = 2000000;// bound of a kernel's wait for the other ranks' announcements
	int symm_loopback	 = 0;// test aid: "peer" mappings alias this rank's own memory, so no announcement ever arrives
	unsigned long long err_seq = 0;
	cudaEvent_t group_ev[2] = { nullptr, nullptr };// cross-stream ordering of nhb_all_gather_local
};

struct nhb_weight {
	int64_t N = 0, K = 0, n0 = 0, n1 = 0;
	int8_t* q	= nullptr;
	__half* d	= nullptr;
	__half* w16 = nullptr;// fp16 copy of the quants for the tensor-core GEMM, made on first use
	float* wdT	= nullptr;// f32 block-major copy of the scales [K/32][gemm_tc_pad(rows)], made with it
	int device	= 0;
};

// A recorded sequence of dependent decode stages (nhb_chain_*): one warp-per-row GEMV launch per stage, each told what the
// next one will read first
struct nhb_chain {
	std::vector<nhb::rows_batch> stages;// launch descriptors, prefetch hints included
	int M = 0;
	std::vector<const void*> delivered;// outputs the launches complete on every rank
	std::vector<const void*> written;// every output pointer they write
	std::vector<char> delivers;// per stage: its rows go to the other ranks
	std::vector<std::vector<nhb_span>> in, out;// per stage: what it reads, what it completes on every rank
	int device = 0;
};

struct nhb_graph {
	cudaGraph_t graph	 = nullptr;
	cudaGraphExec_t exec = nullptr;
	nhb::replay_record replay;// what one replay adds to the context's delivery bookkeeping
};

namespace nhb {

	// records the message for nhb_last_error (this thread, and the context if there is one) and returns `code`
	int fail(nhb_ctx* ctx, int code, const std::string& msg);
	int fail_cuda(nhb_ctx* ctx, cudaError_t e, const char* what);

#define NHB_CUDA(ctx, call) \
	do { \
		cudaError_t e__ = (call); \
		if (e__ != cudaSuccess) \
			return nhb::fail_cuda(ctx, e__, #call); \
	} while (0)

	// makes `dev` the current device for the lifetime of the guard
	struct device_guard {
		int prev = -1;
		bool ok	 = true;
		explicit device_guard(int dev) {
			if (cudaGetDevice(&prev) != cudaSuccess) {
				ok = false;
				return;
			}
			if (prev != dev && cudaSetDevice(dev) != cudaSuccess)
				ok = false;
		}
		~device_guard() {
			if (prev >= 0)
				cudaSetDevice(prev);
		}
	};

	launch_cfg cfg_of(nhb_ctx* ctx);
	// grows *buf to `need` bytes (refused during graph capture)
	int ensure(nhb_ctx* ctx, void** buf, size_t* cap, size_t need, const char* what);
	// in front of work that reads rows another rank may still be delivering: a one-warp kernel that waits for the peers
	int wait_pending(nhb_ctx* ctx);
	// Decides what a warp-per-row launch waits for in its prologue and records what it reads and delivers.
	// in / out: the byte ranges it reads (activations, residual) and writes; `delivers`: the rows in `out` are completed on every rank.
	void plan_peer_wait(nhb_ctx* ctx, nhb::push_ctl& pc, const nhb_span* in, int n_in, const nhb_span* out, int n_out, bool delivers);

}
