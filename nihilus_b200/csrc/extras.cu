// The Q8_0 consumers on either side of the projection mul_mats, and the on-disk cache of repacked weights:
//   nhb_get_rows_q8_0      the token-embedding gather (the reference's only live GPU kernels,
//                          include/nihilus-incl/cuda/cuda_12.hpp:560-601 prompt, :691-722 eval)
//   nhb_last_token_logits  last-token view -> final rms_norm x output_norm -> logits mul_mat
//                          (include/nihilus-incl/infra/core_traits.hpp:1184-1193)
//   nhb_weight_save/load   the two planes of a weight shard as a file, so that a later start skips reading, splitting and
//                          repacking the 34-byte blocks (the reference re-reads the GGUF tensor every start,
//                          include/nihilus-incl/infra/model_parser.hpp:897-940)
#include <cstdio>
#include <cstring>

#include "api_types.h"
#include "ptx.cuh"

using namespace nhb;

namespace {

	// out[m][k] = f32(d[t][k / 32]) * float(q[t][k]) for t = ids[m]: the prompt kernel's arithmetic (cuda_12.hpp:587-598).  The
	// reference's eval-time kernel skips the token id and always reads row 0 (:710); here both phases honour the id.
	// One thread per 16 quants.  An id outside the table is reported through the status word and its row left untouched.
	__global__ void get_rows_q8_0_kernel(const int8_t* __restrict__ q, const __half* __restrict__ d, int rows, int K, const int32_t* __restrict__ ids, int M,
		float* __restrict__ y, long long ldy, int* __restrict__ status) {
		pdl_launch_dependents();
		pdl_wait_prior_grids();
		const int cpr		= K >> 4;// 16-quant chunks per row
		const long long tot = static_cast<long long>(M) * cpr;
		for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < tot; i += static_cast<long long>(gridDim.x) * blockDim.x) {
			const int m = static_cast<int>(i / cpr);
			const int c = static_cast<int>(i - static_cast<long long>(m) * cpr);
			const int t = __ldg(ids + m);
			if (t < 0 || t >= rows) {
				if (c == 0)
					atomicExch(status, DEV_BAD_INDEX);
				continue;
			}
			const uint4 v		= __ldg(reinterpret_cast<const uint4*>(q + static_cast<size_t>(t) * K) + c);
			const float scale	= __half2float(d[static_cast<size_t>(t) * (K >> 5) + (c >> 1)]);
			const uint32_t w[4] = { v.x, v.y, v.z, v.w };
			float4* dst			= reinterpret_cast<float4*>(y + static_cast<size_t>(m) * ldy) + c * 4;
#pragma unroll
			for (int j = 0; j < 4; ++j)
				dst[j] = make_float4(__fmul_rn(scale, static_cast<float>(static_cast<int8_t>(w[j] & 0xff))),
					__fmul_rn(scale, static_cast<float>(static_cast<int8_t>((w[j] >> 8) & 0xff))), __fmul_rn(scale, static_cast<float>(static_cast<int8_t>((w[j] >> 16) & 0xff))),
					__fmul_rn(scale, static_cast<float>(static_cast<int8_t>(w[j] >> 24))));
		}
	}

	// ---- weight cache file: header, int8 plane, fp16 plane ----
	struct cache_header {
		char magic[8];// "NHBQ8W01"
		int64_t N, K, n0, n1;
		int32_t world, rank;
		uint64_t q_bytes, d_bytes;
		uint64_t checksum;// FNV-1a over both planes
	};
	constexpr char CACHE_MAGIC[8] = { 'N', 'H', 'B', 'Q', '8', 'W', '0', '1' };

	uint64_t fnv1a(uint64_t h, const unsigned char* p, size_t n) {
		for (size_t i = 0; i < n; ++i)
			h = (h ^ p[i]) * 1099511628211ull;
		return h;
	}

}

extern "C" {

int nhb_get_rows_q8_0(nhb_ctx* ctx, const nhb_weight* table, const int32_t* token_ids_dev, int64_t M, float* y_dev, int64_t ldy) {
	if (!ctx || !table)
		return fail(ctx, NHB_ERR_ARG, "nhb_get_rows_q8_0: null context or table");
	if (table->device != ctx->device)
		return fail(ctx, NHB_ERR_ARG, "nhb_get_rows_q8_0: the table was uploaded through a context of another device");
	if (M < 0 || M > INT32_MAX || ldy < table->K || (ldy & 3))
		return fail(ctx, NHB_ERR_ARG, "nhb_get_rows_q8_0: bad M or leading dimension (ldy >= K, a multiple of 4)");
	if (table->n0 != 0 || table->n1 != table->N)
		return fail(ctx, NHB_ERR_UNSUPPORTED,
			"nhb_get_rows_q8_0: the table must be whole on this rank (upload it with \"replicate_below_mb\" above its size): any token may be asked for");
	if (M == 0)
		return NHB_OK;
	if (!token_ids_dev || !y_dev || (reinterpret_cast<uintptr_t>(y_dev) & 15) || (reinterpret_cast<uintptr_t>(token_ids_dev) & 3))
		return fail(ctx, NHB_ERR_ARG, "nhb_get_rows_q8_0: null or misaligned pointer (outputs 16-byte aligned)");
	device_guard g(ctx->device);
	if (int rc = wait_pending(ctx); rc != NHB_OK)
		return rc;
	const long long tot = M * (table->K >> 4);
	long long grid		= (tot + 255) / 256;
	grid				= grid > 148 * 8 ? 148 * 8 : grid;
	cudaLaunchConfig_t lc{};
	lc.gridDim	= dim3(static_cast<unsigned>(grid));
	lc.blockDim = dim3(256);
	lc.stream	= ctx->stream;
	cudaLaunchAttribute attr[1];
	attr[0].id										   = cudaLaunchAttributeProgrammaticStreamSerialization;
	attr[0].val.programmaticStreamSerializationAllowed = 1;
	lc.attrs										   = attr;
	lc.numAttrs										   = ctx->pdl ? 1 : 0;
	cudaError_t e = cudaLaunchKernelEx(&lc, get_rows_q8_0_kernel, static_cast<const int8_t*>(table->q), static_cast<const __half*>(table->d), static_cast<int>(table->N),
		static_cast<int>(table->K), token_ids_dev, static_cast<int>(M), y_dev, static_cast<long long>(ldy), ctx->dev_status);
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "get_rows_q8_0 launch");
	ctx->launches += 1;
	return NHB_OK;
}

int nhb_last_token_logits(nhb_ctx* ctx, const nhb_weight* w_output, const float* hidden_dev, int64_t ld, int64_t seq_len, const float* norm_w_dev, float eps,
	int sqrt_mode, float* logits_dev) {
	if (!ctx || !w_output || seq_len < 1 || (seq_len > 0 && !hidden_dev) || ld < w_output->K)
		return fail(ctx, NHB_ERR_ARG, "nhb_last_token_logits: bad arguments (seq_len >= 1, ld >= K)");
	// the view: row seq_len - 1 of the hidden states; then the norm fused in front of the one-token mul_mat
	nhb_mul_mat_op op{ w_output, hidden_dev + (seq_len - 1) * ld, ld, logits_dev, w_output->N, 1 };
	return nhb_rms_norm_mul_mat_batch(ctx, &op, 1, norm_w_dev, eps, sqrt_mode, NHB_KERNEL_AUTO);
}

int nhb_weight_save(nhb_ctx* ctx, const nhb_weight* w, const char* path) {
	if (!ctx || !w || !path)
		return fail(ctx, NHB_ERR_ARG, "nhb_weight_save: null argument");
	if (ctx->capturing)
		return fail(ctx, NHB_ERR_UNSUPPORTED, "nhb_weight_save during graph capture");
	device_guard g(ctx->device);
	cache_header h{};
	std::memcpy(h.magic, CACHE_MAGIC, 8);
	h.N		  = w->N;
	h.K		  = w->K;
	h.n0	  = w->n0;
	h.n1	  = w->n1;
	h.world	  = ctx->world;
	h.rank	  = ctx->rank;
	h.q_bytes = static_cast<uint64_t>(w->n1 - w->n0) * w->K;
	h.d_bytes = static_cast<uint64_t>(w->n1 - w->n0) * (w->K / 32) * 2;
	std::vector<unsigned char> host(h.q_bytes + h.d_bytes);
	if (!host.empty()) {
		NHB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
		NHB_CUDA(ctx, cudaMemcpy(host.data(), w->q, h.q_bytes, cudaMemcpyDeviceToHost));
		NHB_CUDA(ctx, cudaMemcpy(host.data() + h.q_bytes, w->d, h.d_bytes, cudaMemcpyDeviceToHost));
	}
	h.checksum = fnv1a(14695981039346656037ull, host.data(), host.size());
	const std::string tmp = std::string(path) + ".tmp";
	FILE* f				  = std::fopen(tmp.c_str(), "wb");
	if (!f)
		return fail(ctx, NHB_ERR_ARG, std::string("nhb_weight_save: cannot create ") + tmp);
	const bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1 && (host.empty() || std::fwrite(host.data(), host.size(), 1, f) == 1);
	const bool closed = std::fclose(f) == 0;
	if (!ok || !closed || std::rename(tmp.c_str(), path) != 0) {
		std::remove(tmp.c_str());
		return fail(ctx, NHB_ERR_ARG, std::string("nhb_weight_save: writing ") + path + " failed");
	}
	return NHB_OK;
}

int nhb_weight_load(nhb_ctx* ctx, const char* path, int64_t N, int64_t K, nhb_weight** out) {
	if (!ctx || !path || !out)
		return fail(ctx, NHB_ERR_ARG, "nhb_weight_load: null argument");
	*out = nullptr;
	if (ctx->capturing)
		return fail(ctx, NHB_ERR_UNSUPPORTED, "nhb_weight_load during graph capture");
	FILE* f = std::fopen(path, "rb");
	if (!f)
		return fail(ctx, NHB_ERR_ARG, std::string("nhb_weight_load: cannot open ") + path);
	cache_header h{};
	int rc = NHB_OK;
	if (std::fread(&h, sizeof(h), 1, f) != 1 || std::memcmp(h.magic, CACHE_MAGIC, 8) != 0)
		rc = fail(ctx, NHB_ERR_ARG, std::string("nhb_weight_load: ") + path + " is not a weight cache file of this version");
	int64_t n0 = 0, n1 = 0;
	if (rc == NHB_OK) {
		// the file must hold exactly the rows this context would give itself for this weight: same shape, same placement
		nhb_place_rows(N, K, ctx->world, ctx->rank, ctx->replicate_below, &n0, &n1);
		if (h.N != N || h.K != K || K <= 0 || K % 32 != 0 || h.n0 != n0 || h.n1 != n1 || h.q_bytes != static_cast<uint64_t>(n1 - n0) * K ||
			h.d_bytes != static_cast<uint64_t>(n1 - n0) * (K / 32) * 2)
			rc = fail(ctx, NHB_ERR_ARG,
				std::string("nhb_weight_load: ") + path + " holds rows [" + std::to_string(h.n0) + ", " + std::to_string(h.n1) + ") of a " + std::to_string(h.N) + " x " +
					std::to_string(h.K) + " weight; this context needs rows [" + std::to_string(n0) + ", " + std::to_string(n1) + ") of " + std::to_string(N) + " x " +
					std::to_string(K));
	}
	std::vector<unsigned char> host;
	if (rc == NHB_OK) {
		host.resize(h.q_bytes + h.d_bytes);
		if (!host.empty() && std::fread(host.data(), host.size(), 1, f) != 1)
			rc = fail(ctx, NHB_ERR_ARG, std::string("nhb_weight_load: ") + path + " is truncated");
		else if (fnv1a(14695981039346656037ull, host.data(), host.size()) != h.checksum)
			rc = fail(ctx, NHB_ERR_ARG, std::string("nhb_weight_load: ") + path + " fails its checksum");
	}
	std::fclose(f);
	if (rc != NHB_OK)
		return rc;
	device_guard g(ctx->device);
	nhb_weight* w = new nhb_weight();
	w->N		  = N;
	w->K		  = K;
	w->n0		  = n0;
	w->n1		  = n1;
	w->device	  = ctx->device;
	if (!host.empty()) {
		cudaError_t e = cudaMalloc(&w->q, h.q_bytes);
		if (e == cudaSuccess)
			e = cudaMalloc(&w->d, h.d_bytes);
		if (e == cudaSuccess)
			e = cudaMemcpy(w->q, host.data(), h.q_bytes, cudaMemcpyHostToDevice);
		if (e == cudaSuccess)
			e = cudaMemcpy(w->d, host.data() + h.q_bytes, h.d_bytes, cudaMemcpyHostToDevice);
		if (e != cudaSuccess) {
			if (w->q)
				cudaFree(w->q);
			if (w->d)
				cudaFree(w->d);
			delete w;
			return fail_cuda(ctx, e, "nhb_weight_load");
		}
	}
	*out = w;
	return NHB_OK;
}
}

// ---- the wait planner on its own (host only): the decisions of the fused all-gather for a sequence of launches, so that
//      they can be checked on a machine without a GPU ----
struct nhb_wait_planner {
	nhb_deliveries d;
	std::vector<nhb_span> regions;
	int window = 4;
	unsigned long long cap_seq0 = 0;
	std::vector<nhb::replay_record> recordings;
};

extern "C" {

nhb_wait_planner* nhb_wait_planner_create(int peer_window) {
	nhb_wait_planner* p = new nhb_wait_planner();
	p->window			= peer_window < 0 ? 0 : peer_window;
	return p;
}

void nhb_wait_planner_destroy(nhb_wait_planner* p) {
	delete p;
}

int nhb_wait_planner_add_region(nhb_wait_planner* p, const void* base, size_t bytes) {
	if (!p || !base || bytes == 0)
		return NHB_ERR_ARG;
	p->regions.push_back(nhb_span{ static_cast<const char*>(base), static_cast<const char*>(base) + bytes, 0 });
	return NHB_OK;
}

int nhb_wait_planner_launch(nhb_wait_planner* p, const void* const* in, const size_t* in_bytes, int n_in, const void* const* out, const size_t* out_bytes, int n_out,
	int delivers, int* waits, int* lag) {
	if (!p || n_in < 0 || n_out < 0 || (n_in > 0 && (!in || !in_bytes)) || (n_out > 0 && (!out || !out_bytes)) || !waits || !lag)
		return NHB_ERR_ARG;
	std::vector<nhb_span> si, so;
	for (int i = 0; i < n_in; ++i)
		si.push_back(nhb_span{ static_cast<const char*>(in[i]), static_cast<const char*>(in[i]) + in_bytes[i], 0 });
	for (int i = 0; i < n_out; ++i)
		so.push_back(nhb_span{ static_cast<const char*>(out[i]), static_cast<const char*>(out[i]) + out_bytes[i], 0 });
	const nhb::wait_plan plan = nhb::plan_wait(p->d, p->window, p->regions.data(), static_cast<int>(p->regions.size()), si.data(), n_in, so.data(), n_out, delivers != 0);
	*waits = plan.wait ? 1 : 0;
	*lag   = plan.lag;
	return NHB_OK;
}

int nhb_wait_planner_wait_all(nhb_wait_planner* p) {
	return p && nhb::plan_wait_all(p->d) ? 1 : 0;
}

long long nhb_wait_planner_seq(const nhb_wait_planner* p) {
	return p ? static_cast<long long>(p->d.seq) : 0;
}

void nhb_wait_planner_capture_begin(nhb_wait_planner* p) {
	if (p)
		p->cap_seq0 = nhb::capture_begin(p->d);
}

int nhb_wait_planner_capture_end(nhb_wait_planner* p) {
	if (!p)
		return -1;
	p->recordings.push_back(nhb::capture_end(p->d, p->cap_seq0));
	return static_cast<int>(p->recordings.size()) - 1;
}

int nhb_wait_planner_replayed(nhb_wait_planner* p, int recording) {
	if (!p || recording < 0 || recording >= static_cast<int>(p->recordings.size()))
		return NHB_ERR_ARG;
	nhb::replayed(p->d, p->recordings[static_cast<size_t>(recording)]);
	return NHB_OK;
}
}
