// extern "C" layer of libnihilus_b200.so: contexts, weight upload + repack + row sharding, the mul_mat
// dispatch by M, graphs, NCCL all-gather.  Host code only; kernels live in gemv.cu, gemm_tc.cu, repack.cu.
//
// There is deliberately no CPU fallback: when a CUDA call fails the entry point returns NHB_ERR_CUDA.
#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "api_types.h"

using namespace nhb;

// ---------------------------------------------------------------------------------------------------------------
// NCCL is bound at run time (dlopen) so that the library loads on machines without it and shares the copy a host
// process (e.g. PyTorch) has already loaded.
// ---------------------------------------------------------------------------------------------------------------
namespace {

	struct nccl_uid {
		char internal[128];
	};
	enum { nccl_float = 7, nccl_success = 0 };

	struct nccl_api {
		void* handle											  = nullptr;
		int (*GetUniqueId)(nccl_uid*)							  = nullptr;
		int (*CommInitRank)(ncclComm_t*, int, nccl_uid, int)	  = nullptr;
		int (*CommDestroy)(ncclComm_t)							  = nullptr;
		int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t)	   = nullptr;
		int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
		int (*GroupStart)()										  = nullptr;
		int (*GroupEnd)()										  = nullptr;
		const char* (*GetErrorString)(int)						  = nullptr;
		bool ok													  = false;
	};

	nccl_api& nccl() {
		static nccl_api api;
		static std::once_flag once;
		std::call_once(once, [] {
			const char* names[] = { "libnccl.so.2", "libnccl.so" };
			for (const char* n: names) {
				api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
				if (api.handle)
					break;
			}
			if (!api.handle)
				return;
#define NHB_SYM(field, name) api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, name))
			NHB_SYM(GetUniqueId, "ncclGetUniqueId");
			NHB_SYM(CommInitRank, "ncclCommInitRank");
			NHB_SYM(CommDestroy, "ncclCommDestroy");
			NHB_SYM(AllGather, "ncclAllGather");
			NHB_SYM(Broadcast, "ncclBroadcast");
			NHB_SYM(GroupStart, "ncclGroupStart");
			NHB_SYM(GroupEnd, "ncclGroupEnd");
			NHB_SYM(GetErrorString, "ncclGetErrorString");
#undef NHB_SYM
			api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.Broadcast && api.GroupStart && api.GroupEnd;
		});
		return api;
	}

	thread_local std::string g_err;
	thread_local unsigned long long g_err_seq = 0;
	std::atomic<unsigned long long> g_err_counter{ 0 };

}

namespace nhb {

	int fail(nhb_ctx* ctx, int code, const std::string& msg) {
		g_err	  = msg;
		g_err_seq = ++g_err_counter;
		if (ctx) {
			ctx->err	 = msg;
			ctx->err_seq = g_err_seq;
		}
		return code;
	}

	int fail_cuda(nhb_ctx* ctx, cudaError_t e, const char* what) {
		return fail(ctx, NHB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
	}

	launch_cfg cfg_of(nhb_ctx* ctx) {
		launch_cfg c;
		c.stream	 = ctx->stream;
		c.sm_count	 = ctx->sm_count;
		c.pdl		 = ctx->pdl;
		c.dev_status = ctx->dev_status;
		return c;
	}

}

namespace {

	int env_int(const char* name, int dflt) {
		const char* v = std::getenv(name);
		return (v && *v) ? std::atoi(v) : dflt;
	}

}

namespace nhb {
	int ensure(nhb_ctx* ctx, void** buf, size_t* cap, size_t need, const char* what) {
		if (need <= *cap)
			return NHB_OK;
		if (ctx->capturing)
			return fail(ctx, NHB_ERR_UNSUPPORTED, std::string(what) + " must grow during graph capture; run the same calls once before nhb_graph_begin");
		NHB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
		if (*buf)
			NHB_CUDA(ctx, cudaFree(*buf));
		*buf = nullptr;
		*cap = 0;
		need = (need + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
		NHB_CUDA(ctx, cudaMalloc(buf, need));
		*cap = need;
		return NHB_OK;
	}

}

namespace {

	int check_mm_args(nhb_ctx* ctx, const nhb_weight* w, const float* x, int64_t ldx, float* y, int64_t ldy, int64_t M) {
		if (!ctx || !w)
			return fail(ctx, NHB_ERR_ARG, "null context or weight");
		if (w->device != ctx->device)
			return fail(ctx, NHB_ERR_ARG, "weight was uploaded through a context of another device");
		if (M < 0)
			return fail(ctx, NHB_ERR_ARG, "M < 0");
		if (M == 0)
			return NHB_OK;
		if (!x || (!y && w->N > 0))
			return fail(ctx, NHB_ERR_ARG, "null activation or output pointer");
		if (ldx < w->K || ldy < w->N)
			return fail(ctx, NHB_ERR_ARG, "leading dimension smaller than the row length");
		if ((reinterpret_cast<uintptr_t>(x) & 15) || (ldx & 3))
			return fail(ctx, NHB_ERR_ARG, "activations must be 16-byte aligned with ldx a multiple of 4");
		if (M > (int64_t(1) << 20))
			return fail(ctx, NHB_ERR_ARG, "M too large");
		if (y && w->N > 0) {
			// y = W x is never computed in place: rows of y are stored while other rows of x are still being read (and, with
			// several GPUs, delivered into the peers' copies while they still read theirs)
			const char* x0 = reinterpret_cast<const char*>(x);
			const char* x1 = reinterpret_cast<const char*>(x + (M - 1) * ldx + w->K);
			const char* y0 = reinterpret_cast<const char*>(y);
			const char* y1 = reinterpret_cast<const char*>(y + (M - 1) * ldy + w->N);
			if (x0 < y1 && y0 < x1)
				return fail(ctx, NHB_ERR_ARG, "activations and outputs overlap");
		}
		return NHB_OK;
	}

	nhb_ctx::symm_region* find_region(nhb_ctx* ctx, const void* p, size_t bytes) {
		const char* c = static_cast<const char*>(p);
		for (auto& r: ctx->regions)
			if (c >= r.local && c + bytes <= r.local + r.bytes)
				return &r;
		return nullptr;
	}

	// Allocates `bytes` on this rank and maps the matching allocation of every other rank (CUDA IPC; the 64-byte
	// handles travel through an NCCL all-gather).  Collective: every rank calls it with the same size, in the same order.
	int symm_alloc_impl(nhb_ctx* ctx, size_t bytes, nhb_ctx::symm_region* out) {
		if (ctx->world > NHB_MAX_WORLD)
			return fail(ctx, NHB_ERR_UNSUPPORTED, "symmetric memory supports at most 8 ranks");
		nhb_ctx::symm_region reg;
		reg.bytes = bytes;
		void* p	  = nullptr;
		NHB_CUDA(ctx, cudaMalloc(&p, bytes));
		reg.local			= static_cast<char*>(p);
		reg.peer[ctx->rank] = reg.local;
		cudaError_t e		= cudaMemsetAsync(p, 0, bytes, ctx->stream);
		if (e == cudaSuccess && ctx->world > 1 && ctx->symm_loopback) {
			// every "peer" is this rank's own allocation: stores meant for the peers land on the values already there, and
			// no other rank ever announces anything -- the waits of the following launches run into their time limit
			for (int r = 0; r < ctx->world; ++r)
				reg.peer[r] = reg.local;
			e = cudaStreamSynchronize(ctx->stream);
		} else if (e == cudaSuccess && ctx->world > 1) {
			if (!ctx->comm) {
				cudaFree(p);
				return fail(ctx, NHB_ERR_NCCL, "symmetric memory needs nhb_comm_init first (the handles travel over NCCL)");
			}
			cudaIpcMemHandle_t mine;
			e = cudaIpcGetMemHandle(&mine, p);
			unsigned char* stage = nullptr;
			const size_t hb		 = sizeof(cudaIpcMemHandle_t);
			if (e == cudaSuccess)
				e = cudaMalloc(&stage, hb * ctx->world);
			if (e == cudaSuccess)
				e = cudaMemcpyAsync(stage + hb * ctx->rank, &mine, hb, cudaMemcpyHostToDevice, ctx->stream);
			int nrc = nccl_success;
			if (e == cudaSuccess)
				nrc = nccl().AllGather(stage + hb * ctx->rank, stage, hb, /*ncclUint8*/ 1, ctx->comm, ctx->stream);
			std::vector<cudaIpcMemHandle_t> all(ctx->world);
			if (e == cudaSuccess && nrc == nccl_success)
				e = cudaMemcpyAsync(all.data(), stage, hb * ctx->world, cudaMemcpyDeviceToHost, ctx->stream);
			if (e == cudaSuccess)
				e = cudaStreamSynchronize(ctx->stream);
			if (stage)
				cudaFree(stage);
			if (nrc != nccl_success) {
				cudaFree(p);
				return fail(ctx, NHB_ERR_NCCL, "exchange of memory handles failed");
			}
			for (int r = 0; r < ctx->world && e == cudaSuccess; ++r) {
				if (r == ctx->rank)
					continue;
				void* q = nullptr;
				e		= cudaIpcOpenMemHandle(&q, all[r], cudaIpcMemLazyEnablePeerAccess);
				reg.peer[r] = static_cast<char*>(q);
			}
		}
		if (e != cudaSuccess) {
			for (int r = 0; r < ctx->world; ++r)
				if (r != ctx->rank && reg.peer[r])
					cudaIpcCloseMemHandle(reg.peer[r]);
			cudaFree(p);
			return fail_cuda(ctx, e, "symmetric allocation (one process per GPU with peer access is required)");
		}
		*out = reg;
		return NHB_OK;
	}

	void symm_release(nhb_ctx* ctx, nhb_ctx::symm_region& reg) {
		for (int r = 0; r < ctx->world && reg.ipc; ++r)
			if (r != ctx->rank && reg.peer[r] && reg.peer[r] != reg.local)
				cudaIpcCloseMemHandle(reg.peer[r]);
		if (reg.local)
			cudaFree(reg.local);
		reg = nhb_ctx::symm_region();
	}

	// Fills the fused all-gather part of a warp-per-row launch when every output of the batch lies in symmetric memory.
	// regions[0] is the control region holding the flag array.
	// The waiting half: every launch of a context that has symmetric memory first waits for the other ranks' announcements.
	void setup_peer_wait(nhb_ctx* ctx, push_ctl& pc) {
		pc.status = ctx->dev_status;
		if (ctx->world <= 1 || ctx->regions.empty() || !ctx->push_local)
			return;
		pc.wait_world  = ctx->world;
		pc.peers	   = ctx->world;
		pc.rank		   = ctx->rank;
		pc.wait_ns	   = static_cast<unsigned long long>(ctx->peer_wait_us) * 1000ull;
		pc.epoch	   = ctx->push_local + 1;
		pc.announced   = ctx->push_local + 2;
		pc.flags_local = reinterpret_cast<unsigned*>(ctx->regions[0].local);
		for (int r = 0; r < ctx->world; ++r)
			pc.flags_peer[r] = reinterpret_cast<unsigned*>(ctx->regions[0].peer[r]);
	}

	bool setup_push(nhb_ctx* ctx, rows_batch& b, const nhb_mul_mat_op* const* src_ops, int mt, int64_t m0) {
		if (ctx->world <= 1 || !ctx->fused_gather || ctx->regions.empty() || !ctx->push_local || b.n_ops == 0)
			return false;
		nhb_ctx::symm_region* regs[NHB_MAX_BATCH];
		for (int i = 0; i < b.n_ops; ++i) {
			const nhb_mul_mat_op* op = src_ops[i];
			regs[i]					 = nullptr;
			if (op->w->n1 - op->w->n0 == op->w->N)
				continue;// replicated: nothing to deliver, the output may live anywhere
			// the whole row range this launch completes must be inside one region
			float* first = op->y + m0 * op->ldy;
			regs[i]		 = find_region(ctx, first, (static_cast<size_t>(mt - 1) * op->ldy + op->w->N) * sizeof(float));
			if (!regs[i] || regs[i] == &ctx->regions[0])
				return false;
		}
		bool any = false;
		for (int i = 0; i < b.n_ops; ++i) {
			const nhb_weight* w = src_ops[i]->w;
			if (w->n1 - w->n0 == w->N)
				continue;// replicated weight: every rank computes every row, nothing to deliver (y_peer stays null)
			const char* y_local = reinterpret_cast<const char*>(b.op[i].y);
			const size_t off	= static_cast<size_t>(y_local - regs[i]->local);
			for (int r = 0; r < ctx->world; ++r)
				b.y_peer[i][r] = reinterpret_cast<float*>(regs[i]->peer[r] + off);
			any = true;
		}
		if (!any)
			return false;
		b.push.world	   = ctx->world;
		b.push.rank		   = ctx->rank;
		b.push.done_ctas   = ctx->push_local;
		b.push.epoch	   = ctx->push_local + 1;
		b.push.flags_local = reinterpret_cast<unsigned*>(ctx->regions[0].local);
		for (int r = 0; r < ctx->world; ++r)
			b.push.flags_peer[r] = reinterpret_cast<unsigned*>(ctx->regions[0].peer[r]);
		b.push.status = ctx->dev_status;
		return true;
	}

	// One launch's worth of ops as the warp-per-row kernels see them: this rank's row shard of every weight (ops it owns no
	// rows of are left out), token rows [m0, m0 + mt), and one shared-memory slot per distinct activation input.  Returns
	// the shared memory the quantised activations take.
	size_t fill_rows_batch(const nhb_mul_mat_op* ops, int n_ops, int64_t m0, int mt, bool f32act, rows_batch& b, const nhb_mul_mat_op** src_ops) {
		size_t off = 0;
		for (int i = 0; i < n_ops; ++i) {
			const nhb_weight* w = ops[i].w;
			if (w->n1 == w->n0)
				continue;
			src_ops[b.n_ops] = &ops[i];
			rows_op& ro		 = b.op[b.n_ops];
			ro.wq			 = w->q;
			ro.wd			 = w->d;
			ro.x			 = ops[i].x + m0 * ops[i].ldx;
			ro.y			 = ops[i].y + m0 * ops[i].ldy + w->n0;
			ro.ldx			 = ops[i].ldx;
			ro.ldy			 = ops[i].ldy;
			ro.rows			 = static_cast<int>(w->n1 - w->n0);
			ro.K			 = static_cast<int>(w->K);
			int slot		 = -1;
			for (int s = 0; s < b.n_slots; ++s) {
				const rows_op& so = b.op[b.slot_op[s]];
				if (so.x == ro.x && so.ldx == ro.ldx && so.K == ro.K)
					slot = s;
			}
			if (slot < 0) {
				b.slot_op[b.n_slots++] = b.n_ops;
				ro.act_off			   = static_cast<int>(off);
				ro.preq_off			   = static_cast<int>(off);
				off += gemv_rows_act_bytes(ro.K, mt, f32act);
			} else {
				ro.act_off	= b.op[b.slot_op[slot]].act_off;
				ro.preq_off = ro.act_off;
			}
			++b.n_ops;
		}
		b.act_bytes = static_cast<int>(off);
		b.f32act	= f32act ? 1 : 0;
		return off;
	}

	// The byte ranges a warp-per-row launch reads (activations, the second SwiGLU operand, the residual) and the rows it
	// writes (whole rows: in a delivering launch they are completed on every rank).
	struct batch_spans {
		nhb_span in[3 * NHB_MAX_BATCH];
		nhb_span out[NHB_MAX_BATCH];
		int n_in = 0, n_out = 0;
	};
	void spans_of(const rows_batch& b, const nhb_mul_mat_op* const* src_ops, int mt, int64_t m0, batch_spans& sp) {
		sp.n_in = sp.n_out = 0;
		for (int i = 0; i < b.n_ops; ++i) {
			const rows_op& ro = b.op[i];
			const size_t xb	  = (static_cast<size_t>(mt - 1) * ro.ldx + ro.K) * sizeof(float);
			sp.in[sp.n_in++]  = nhb_span{ reinterpret_cast<const char*>(ro.x), reinterpret_cast<const char*>(ro.x) + xb, 0 };
			if (ro.x2)
				sp.in[sp.n_in++] = nhb_span{ reinterpret_cast<const char*>(ro.x2), reinterpret_cast<const char*>(ro.x2) + xb, 0 };
			if (ro.res)
				sp.in[sp.n_in++] = nhb_span{ reinterpret_cast<const char*>(ro.res),
					reinterpret_cast<const char*>(ro.res) + (static_cast<size_t>(mt - 1) * ro.ldr + ro.rows) * sizeof(float), 0 };
			const nhb_mul_mat_op* op = src_ops[i];
			const char* y0			 = reinterpret_cast<const char*>(op->y + m0 * op->ldy);
			sp.out[sp.n_out++]		 = nhb_span{ y0, y0 + (static_cast<size_t>(mt - 1) * op->ldy + op->w->N) * sizeof(float), 0 };
		}
	}

	// Which register-fed kernel a launch takes.  A short launch (a q/k/v or attn_output stage: a few rows of one 4 KB item
	// per warp) is over before a single-buffered warp has hidden one memory latency, so it runs the variant with two
	// items in flight per warp, at two 8-warp CTAs per SM: everything it needs is then requested before it waits for
	// the kernel in front of it (attn_output 6.1 -> 4.5 us, q+k+v 7.0 -> 6.1 us on a B200).  Long launches keep one 24-warp
	// CTA per SM, whose steady state is faster (gate+up 21.6 against 23.0 us).  The choice never shows in the results.
	bool pick_double_buffer(const nhb_ctx* ctx, const rows_batch& b, int mt, bool delivers) {
		if (ctx->rows_db >= 0)
			return ctx->rows_db != 0;
		if (b.f32act || b.norm_w || b.preq || mt > 4 || delivers || ctx->rows_cluster > 1)
			return false;
		int64_t bytes = 0;
		for (int i = 0; i < b.n_ops; ++i) {
			if (b.op[i].K > 4096)
				return false;
			bytes += static_cast<int64_t>(b.op[i].rows) * (b.op[i].K + (b.op[i].K >> 4));
		}
		return bytes >= (int64_t(4) << 20) && bytes <= (int64_t(40) << 20);
	}

}

namespace {


}

namespace nhb {
	// What a warp-per-row launch waits for in its prologue (deliveries.h: plan_wait), and the record of what it reads and delivers
	void plan_peer_wait(nhb_ctx* ctx, push_ctl& pc, const nhb_span* in, int n_in, const nhb_span* out, int n_out, bool delivers) {
		setup_peer_wait(ctx, pc);
		pc.wait_lag = 0;
		if (pc.wait_world <= 1)
			return;
		std::vector<nhb_span> regions;
		for (size_t i = 1; i < ctx->regions.size(); ++i)// regions[0] holds the flags
			regions.push_back(nhb_span{ ctx->regions[i].local, ctx->regions[i].local + ctx->regions[i].bytes, 0 });
		const wait_plan plan = plan_wait(ctx->dl, ctx->peer_window, regions.data(), static_cast<int>(regions.size()), in, n_in, out, n_out, delivers);
		if (plan.wait)
			pc.wait_lag = plan.lag;
		else
			pc.wait_world = 0;// nothing has been delivered that this launch could depend on
	}

	// Rows delivered by a fused launch are whole on this rank only after the other ranks' announcements have arrived.  The
	// decode GEMV kernels wait for what they read in their own prologue; in front of anything else that may read such rows
	// (other kernels, copies to the host, the end of nhb_sync) this enqueues a one-warp kernel that waits for everything.
	int wait_pending(nhb_ctx* ctx) {
		if (ctx->dl.pending.empty())
			return NHB_OK;
		push_ctl pc{};
		setup_peer_wait(ctx, pc);
		pc.wait_lag	  = 0;
		int launches  = 0;
		cudaError_t e = launch_peer_wait(pc, cfg_of(ctx), &launches);
		if (e != cudaSuccess)
			return fail_cuda(ctx, e, "peer-wait launch");
		ctx->launches += launches;
		plan_wait_all(ctx->dl);
		return NHB_OK;
	}
}

namespace {

	// GEMV family over M rows (looping over row groups the kernels support)
	int run_gemv(nhb_ctx* ctx, const nhb_mul_mat_op* ops, int n_ops, int act_mode, int kernel) {
		const int64_t M = ops[0].M;
		launch_cfg cfg	= cfg_of(ctx);
		int launches	= 0;
		if (kernel == NHB_KERNEL_AUTO)
			kernel = ctx->gemv_default;
		// ---- warp-per-row GEMV: the default ----
		const bool f32act = act_mode == NHB_ACT_F32;
		if (!(kernel == NHB_KERNEL_GEMV_ROWS && !ctx->preq && !ctx->norm_w)) {
			int rc = wait_pending(ctx);// kernels without the wait in their own prologue
			if (rc != NHB_OK)
				return rc;
		}
		if (kernel == NHB_KERNEL_GEMV_ROWS) {
			// rows per pass: 4 in general; up to 8 for the plain Q8 kernel on rows of one 4 KB item (K <= 4096), where a
			// pass of 8 costs less than two passes of 4 over the weights
			int mt_max = (f32act || ctx->rows_db > 0 || ctx->rows_cluster > 1 || ctx->norm_w || ctx->preq || M <= 4) ? 4 : 8;
			for (int i = 0; i < n_ops; ++i)
				if (ops[i].w->K > 4096)
					mt_max = std::min(mt_max, 4);
			for (int i = 0; i < n_ops; ++i)
				while (mt_max > 0 && !gemv_rows_supports(ops[i].w->K, mt_max, f32act))
					--mt_max;
			// the shared-memory budget counts every distinct input once
			size_t act_total = 0;
			for (int i = 0; i < n_ops && mt_max > 0; ++i) {
				bool seen = false;
				for (int j = 0; j < i; ++j)
					seen = seen || (ops[j].x == ops[i].x && ops[j].ldx == ops[i].ldx && ops[j].w->K == ops[i].w->K);
				if (!seen)
					act_total += gemv_rows_act_bytes(ops[i].w->K, 1, f32act);
			}
			while (mt_max > 1 && act_total * mt_max > 96 * 1024)
				--mt_max;
			if (mt_max >= 1 && act_total <= 96 * 1024) {
				for (int64_t m0 = 0; m0 < M; m0 += mt_max) {
					const int mt = static_cast<int>(std::min<int64_t>(mt_max, M - m0));
					rows_batch b{};
					const nhb_mul_mat_op* src_ops[NHB_MAX_BATCH];
					const size_t off = fill_rows_batch(ops, n_ops, m0, mt, f32act, b, src_ops);
					if (b.n_ops == 0)
						break;
					// rms_norm in front of the quantiser: inside the GEMV when its rows fit the shared memory, else its own kernel
					int rows_total = 0;
					for (int i = 0; i < b.n_ops; ++i)
						rows_total += b.op[i].rows;
					const bool norm_inside = ctx->norm_w && !f32act && ctx->rows_db <= 0 && b.n_ops > 0 &&
						gemv_rows_norm_inside(rows_total, off, b.op[0].K, mt, cfg.sm_count, ctx->rows_fat != 0);
					if (norm_inside) {
						b.norm_w	= ctx->norm_w;
						b.norm_eps	= ctx->norm_eps;
						b.norm_sqrt = ctx->norm_sqrt;
					}
					if ((ctx->preq || ctx->norm_w) && !f32act && !norm_inside) {
						int rc = ensure(ctx, &ctx->scratch, &ctx->scratch_cap, off, "activation scratch");
						if (rc != NHB_OK)
							return rc;
						b.preq		= 1;
						b.preq_base = static_cast<const unsigned char*>(ctx->scratch);
						for (int s = 0; s < b.n_slots; ++s) {
							const rows_op& so = b.op[b.slot_op[s]];
							int8_t* q		  = static_cast<int8_t*>(ctx->scratch) + so.preq_off;
							float* d		  = reinterpret_cast<float*>(q + static_cast<size_t>(mt) * so.K);
							cudaError_t e;
							if (ctx->norm_w) {
								const norm_out no{ nullptr, 0, q, d, nullptr };
								e = launch_rms_norm(so.x, so.ldx, ctx->norm_w, ctx->norm_eps, ctx->norm_sqrt, mt, so.K, no, ctx->stream, ctx->pdl);
							} else {
								e = launch_quantize(so.x, so.ldx, mt, so.K, q, d, ctx->stream, ctx->pdl);
							}
							if (e != cudaSuccess)
								return fail_cuda(ctx, e, "activation quantise launch");
							++launches;
						}
					}
					// a batch in which some rank owns no rows of some op would leave the ranks with different launch counts
					bool all_ranks_have_rows = true;
					for (int i = 0; i < n_ops; ++i)
						all_ranks_have_rows = all_ranks_have_rows && ops[i].w->N >= ctx->world;
					const bool pushed = ctx->rows_db <= 0 && ctx->rows_cluster <= 1 && all_ranks_have_rows && setup_push(ctx, b, src_ops, mt, m0);
					if (pushed && m0 + mt >= M)
						for (int i = 0; i < b.n_ops; ++i)
							if (b.y_peer[i][0])
								ctx->complete.push_back(src_ops[i]->y);
					batch_spans sp;
					spans_of(b, src_ops, mt, m0, sp);
					plan_peer_wait(ctx, b.push, sp.in, sp.n_in, sp.out, sp.n_out, pushed);
					const bool db = pick_double_buffer(ctx, b, mt, pushed);
					cudaError_t e = launch_gemv_rows(b, mt, cfg, db && ctx->rows_db < 0 ? 2 : ctx->rows_cps, &launches, db, ctx->rows_cluster, ctx->rows_fat != 0, ctx->rows_split != 0);
					if (e != cudaSuccess)
						return fail_cuda(ctx, e, "gemv_q8_rows launch");
				}
				ctx->launches += launches;
				return NHB_OK;
			}
			if (ctx->norm_w)
				return fail(ctx, NHB_ERR_UNSUPPORTED, "fused rms_norm needs the warp-per-row GEMV");
			if (kernel == NHB_KERNEL_GEMV_ROWS && ctx->gemv_default != NHB_KERNEL_GEMV_ROWS)
				return fail(ctx, NHB_ERR_UNSUPPORTED, "K too large for the warp-per-row GEMV's shared memory");
			kernel = NHB_KERNEL_GEMV_LDG;
		}
		bool stream_ok	= act_mode == NHB_ACT_Q8 && kernel == NHB_KERNEL_GEMV_STREAM;
		for (int i = 0; i < n_ops && stream_ok; ++i)
			stream_ok = gemv_stream_supports(ops[i].w->K, 1);
		if (kernel == NHB_KERNEL_GEMV_STREAM && !stream_ok)
			return fail(ctx, NHB_ERR_UNSUPPORTED, "streaming GEMV needs Q8 activations, K % 256 == 0 and 1024 <= K <= 16384");
		if (stream_ok) {
			int64_t kmax = 0;
			for (int i = 0; i < n_ops; ++i)
				kmax = std::max<int64_t>(kmax, ops[i].w->K);
			int mt_max = 1;
			while (mt_max < 8 && gemv_stream_supports(kmax, mt_max + 1))
				++mt_max;
			for (int64_t m0 = 0; m0 < M; m0 += mt_max) {
				const int mt = static_cast<int>(std::min<int64_t>(mt_max, M - m0));
				stream_batch b{};
				b.n_ops = 0;
				for (int i = 0; i < n_ops; ++i) {
					const nhb_weight* w = ops[i].w;
					if (w->n1 == w->n0)
						continue;
					stream_op& so = b.op[b.n_ops++];
					so.wq		  = w->q;
					so.wd		  = w->d;
					so.x		  = ops[i].x + m0 * ops[i].ldx;
					so.y		  = ops[i].y + m0 * ops[i].ldy + w->n0;
					so.ldx		  = ops[i].ldx;
					so.ldy		  = ops[i].ldy;
					so.rows		  = static_cast<int>(w->n1 - w->n0);
					so.K		  = static_cast<int>(w->K);
				}
				if (b.n_ops == 0)
					break;
				cudaError_t e = launch_gemv_stream(b, mt, cfg, ctx->ctas_per_sm, &launches);
				if (e != cudaSuccess)
					return fail_cuda(ctx, e, "gemv_q8_stream launch");
			}
		} else {
			for (int i = 0; i < n_ops; ++i) {
				const nhb_weight* w = ops[i].w;
				const int rows		= static_cast<int>(w->n1 - w->n0);
				if (rows == 0)
					continue;
				const int mt_max = gemv_ldg_max_m(w->K, act_mode);
				if (mt_max < 1)
					return fail(ctx, NHB_ERR_UNSUPPORTED, "K too large for the GEMV fallback's shared memory");
				for (int64_t m0 = 0; m0 < M; m0 += mt_max) {
					const int mt  = static_cast<int>(std::min<int64_t>(mt_max, M - m0));
					cudaError_t e = launch_gemv_ldg(w->q, w->d, ops[i].x + m0 * ops[i].ldx, ops[i].ldx, ops[i].y + m0 * ops[i].ldy + w->n0, ops[i].ldy, rows,
						static_cast<int>(w->K), mt, act_mode, cfg, &launches);
					if (e != cudaSuccess)
						return fail_cuda(ctx, e, "gemv_q8_ldg launch");
				}
			}
		}
		ctx->launches += launches;
		return NHB_OK;
	}

	// `same_input`: the scratch already holds the quantised activations of this very input (left by the previous op of the batch)
	int run_gemm(nhb_ctx* ctx, const nhb_mul_mat_op& op, bool same_input = false) {
		const nhb_weight* w = op.w;
		const int rows		= static_cast<int>(w->n1 - w->n0);
		if (rows == 0)
			return NHB_OK;
		const size_t need = gemm_tc_scratch_bytes(w->K, op.M, rows, ctx->sm_count);
		int rc			  = ensure(ctx, &ctx->scratch, &ctx->scratch_cap, need, "GEMM scratch");
		if (rc == NHB_OK && !ctx->gemm_counters) {
			// the arrival counters of split tiles: zero now, and zero again after every launch that used them
			if (ctx->capturing)
				return fail(ctx, NHB_ERR_UNSUPPORTED, "the GEMM's counters must exist before graph capture; run the GEMM once first");
			NHB_CUDA(ctx, cudaMalloc(&ctx->gemm_counters, gemm_tc_counter_bytes()));
			NHB_CUDA(ctx, cudaMemsetAsync(ctx->gemm_counters, 0, gemm_tc_counter_bytes(), ctx->stream));
		}
		if (rc == NHB_OK)
			rc = wait_pending(ctx);
		if (rc != NHB_OK)
			return rc;
		int launches		= 0;
		const __half* w16	= w->w16;
		const float* wdT	= w->wdT;
		const size_t sb		= static_cast<size_t>(w->K / 32) * gemm_tc_pad(rows) * sizeof(float);
		const size_t w16_b	= (static_cast<size_t>(rows) * w->K * sizeof(__half) + 255) & ~size_t(255);
		if (!w->w16 && !ctx->gemm_keep_planes) {
			// The tensor cores take fp16 operands.  Option "gemm_keep_planes" = 0: the fp16 copy of the quants and the
			// block-major scales are rebuilt into one buffer of the context in front of every GEMM (2 bytes per weight of
			// the largest weight instead of 2 bytes per weight of the whole model; 45 us more per GEMM of a 14336 x 4096 weight).
			// Rows past the shard in the scale plane hold whatever was there: their outputs are never stored.
			rc = ensure(ctx, &ctx->plane_buf, &ctx->plane_cap, w16_b + sb, "GEMM weight planes");
			if (rc != NHB_OK)
				return rc;
			__half* p16 = static_cast<__half*>(ctx->plane_buf);
			float* pdT	= reinterpret_cast<float*>(static_cast<char*>(ctx->plane_buf) + w16_b);
			cudaError_t ew = launch_weight_gemm_planes(w->q, w->d, rows, w->K, p16, pdT, ctx->stream);
			if (ew != cudaSuccess)
				return fail_cuda(ctx, ew, "GEMM weight planes");
			launches += 2;
			w16 = p16;
			wdT = pdT;
		} else if (!w->w16) {
			// keep an exact fp16 copy of the int8 plane (2 bytes per weight) and the scales as f32, block-major, so that a
			// tile's scales of one block are contiguous
			if (ctx->capturing)
				return fail(ctx, NHB_ERR_UNSUPPORTED, "the weight's GEMM planes must exist before graph capture; run the GEMM once first");
			nhb_weight* wm = const_cast<nhb_weight*>(w);
			NHB_CUDA(ctx, cudaMalloc(&wm->w16, static_cast<size_t>(rows) * w->K * sizeof(__half)));
			cudaError_t ew = cudaMalloc(&wm->wdT, sb);
			if (ew == cudaSuccess)
				ew = cudaMemsetAsync(wm->wdT, 0, sb, ctx->stream);
			if (ew == cudaSuccess)
				ew = launch_weight_gemm_planes(w->q, w->d, rows, w->K, wm->w16, wm->wdT, ctx->stream);
			if (ew != cudaSuccess) {
				cudaFree(wm->w16);
				wm->w16 = nullptr;
				if (wm->wdT)
					cudaFree(wm->wdT);
				wm->wdT = nullptr;
				return fail_cuda(ctx, ew, "GEMM weight planes");
			}
			NHB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));// a programmatic-dependent launch after it must not overtake it
			launches += 2;
			w16 = wm->w16;
			wdT = wm->wdT;
		}
		std::string err;
		cudaError_t e = launch_gemm_tc(w16, wdT, op.x, op.ldx, op.y + w->n0, op.ldy, rows, static_cast<int>(w->K), static_cast<int>(op.M), ctx->scratch,
			ctx->gemm_counters, cfg_of(ctx), &launches, &err, same_input);
		ctx->launches += launches;
		if (e != cudaSuccess)
			return fail_cuda(ctx, e, err.empty() ? "gemm_q8_tc launch" : err.c_str());
		return NHB_OK;
	}

}

extern "C" {

int nhb_version(void) {
	return NHB_VERSION;
}

int nhb_arch(void) {
	return 100;
}

const char* nhb_last_error(const nhb_ctx* ctx) {
	// the more recent of this context's last error and this thread's last error
	if (ctx && !ctx->err.empty() && ctx->err_seq >= g_err_seq)
		return ctx->err.c_str();
	return g_err.c_str();
}

int nhb_shard_rows(int64_t N, int world, int rank, int64_t* n0, int64_t* n1) {
	if (N < 0 || world < 1 || rank < 0 || rank >= world || !n0 || !n1)
		return fail(nullptr, NHB_ERR_ARG, "nhb_shard_rows: bad arguments");
	const int64_t base = N / world, rem = N % world;
	*n0 = rank * base + std::min<int64_t>(rank, rem);
	*n1 = *n0 + base + (rank < rem ? 1 : 0);
	return NHB_OK;
}

int nhb_place_rows(int64_t N, int64_t K, int world, int rank, int64_t replicate_below_bytes, int64_t* n0, int64_t* n1) {
	if (K <= 0 || K % 32 != 0)
		return fail(nullptr, NHB_ERR_ARG, "nhb_place_rows: K must be a positive multiple of 32");
	int rc = nhb_shard_rows(N, world, rank, n0, n1);
	if (rc != NHB_OK)
		return rc;
	if (world > 1 && N * (K / 32) * 34 < replicate_below_bytes) {
		*n0 = 0;
		*n1 = N;
	}
	return NHB_OK;
}

int nhb_gemm_tile_plan(int64_t rows, int64_t M, int sms, int* swapped, int* tile_cols, int* lane_tiles, int* col_tiles) {
	if (rows < 1 || M < 1 || sms < 1 || !swapped || !tile_cols || !lane_tiles || !col_tiles)
		return fail(nullptr, NHB_ERR_ARG, "nhb_gemm_tile_plan: bad arguments");
	const gemm_plan p = gemm_tc_plan(rows, M, sms);
	*swapped		  = p.swapped;
	*tile_cols		  = p.n_t;
	*lane_tiles		  = p.lane_tiles;
	*col_tiles		  = p.col_tiles;
	return NHB_OK;
}

int nhb_repack_q8_0_host(const void* blocks34, int64_t N, int64_t K, int64_t n0, int64_t n1, int8_t* q_plane, uint16_t* d_plane) {
	if (!blocks34 || !q_plane || !d_plane || N < 0 || K <= 0 || K % 32 != 0 || n0 < 0 || n1 > N || n0 > n1)
		return fail(nullptr, NHB_ERR_ARG, "nhb_repack_q8_0_host: bad arguments");
	const int64_t nb   = K / 32;
	const uint8_t* src = static_cast<const uint8_t*>(blocks34) + n0 * nb * 34;
	for (int64_t i = 0; i < (n1 - n0) * nb; ++i) {
		std::memcpy(&d_plane[i], src + i * 34, 2);
		std::memcpy(q_plane + i * 32, src + i * 34 + 2, 32);
	}
	return NHB_OK;
}

int nhb_unpack_q8_0_host(const int8_t* q_plane, const uint16_t* d_plane, int64_t rows, int64_t K, void* blocks34) {
	if (!blocks34 || !q_plane || !d_plane || rows < 0 || K <= 0 || K % 32 != 0)
		return fail(nullptr, NHB_ERR_ARG, "nhb_unpack_q8_0_host: bad arguments");
	uint8_t* dst = static_cast<uint8_t*>(blocks34);
	for (int64_t i = 0; i < rows * (K / 32); ++i) {
		std::memcpy(dst + i * 34, &d_plane[i], 2);
		std::memcpy(dst + i * 34 + 2, q_plane + i * 32, 32);
	}
	return NHB_OK;
}

int nhb_choose_kernel(int64_t N, int64_t K, int64_t M, int act_mode) {
	(void)N;
	if (act_mode == NHB_ACT_F32)
		return gemv_rows_supports(K, M > 4 ? 4 : (M < 1 ? 1 : M), true) ? NHB_KERNEL_GEMV_ROWS : NHB_KERNEL_GEMV_LDG;
	if (M <= 8)
		return gemv_rows_supports(K, 1) ? NHB_KERNEL_GEMV_ROWS : NHB_KERNEL_GEMV_LDG;
	return NHB_KERNEL_GEMM_TC;
}

int64_t nhb_mul_mat_bytes(int64_t N, int64_t K, int64_t M) {
	return N * (K / 32) * 34 + 4 * M * K + 4 * M * N;
}

int64_t nhb_mul_mat_flops(int64_t N, int64_t K, int64_t M) {
	return 2 * M * N * K;
}

int nhb_ctx_create(nhb_ctx** out, int device, int rank, int world) {
	if (!out || world < 1 || rank < 0 || rank >= world || device < 0)
		return fail(nullptr, NHB_ERR_ARG, "nhb_ctx_create: bad arguments");
	*out = nullptr;
	int n_dev = 0;
	NHB_CUDA(nullptr, cudaGetDeviceCount(&n_dev));
	if (device >= n_dev)
		return fail(nullptr, NHB_ERR_ARG, "nhb_ctx_create: no such device");
	device_guard g(device);
	if (!g.ok)
		return fail(nullptr, NHB_ERR_CUDA, "cudaSetDevice failed");
	cudaDeviceProp prop{};
	NHB_CUDA(nullptr, cudaGetDeviceProperties(&prop, device));
	if (prop.major != 10)
		return fail(nullptr, NHB_ERR_UNSUPPORTED, "this library holds sm_100a code only; device is compute capability " + std::to_string(prop.major) + "." + std::to_string(prop.minor));
	nhb_ctx* ctx  = new nhb_ctx();
	ctx->device	  = device;
	ctx->rank	  = rank;
	ctx->world	  = world;
	ctx->sm_count = prop.multiProcessorCount;
	cudaError_t e = cudaStreamCreateWithFlags(&ctx->own, cudaStreamNonBlocking);
	if (e == cudaSuccess)
		e = cudaMalloc(&ctx->dev_status, NHB_STATUS_WORDS * sizeof(int));
	if (e == cudaSuccess)
		e = cudaMemset(ctx->dev_status, 0, NHB_STATUS_WORDS * sizeof(int));
	if (e == cudaSuccess)
		e = cudaMallocHost(&ctx->host_status, NHB_STATUS_WORDS * sizeof(int));
	if (e != cudaSuccess) {
		int rc = fail_cuda(nullptr, e, "nhb_ctx_create");
		if (ctx->own)
			cudaStreamDestroy(ctx->own);
		if (ctx->dev_status)
			cudaFree(ctx->dev_status);
		delete ctx;
		return rc;
	}
	ctx->stream		 = ctx->own;
	ctx->pdl		 = env_int("NHB_PDL", 1) != 0;
	ctx->gemv_max_m	 = env_int("NHB_GEMV_MAX_M", 8);
	ctx->ctas_per_sm = env_int("NHB_CTAS_PER_SM", 1);
	ctx->rows_cps	 = env_int("NHB_ROWS_CPS", 3);
	ctx->preq		 = env_int("NHB_PREQ", 0);
	ctx->rows_db	 = env_int("NHB_ROWS_DB", -1);
	ctx->rows_cluster = env_int("NHB_ROWS_CLUSTER", 1);
	ctx->replicate_below = static_cast<int64_t>(std::max(0, env_int("NHB_REPLICATE_MB", 0))) << 20;
	ctx->rows_fat	  = env_int("NHB_ROWS_FAT", 1);
	ctx->rows_split	  = env_int("NHB_ROWS_SPLIT", 1);
	{
		const int k = env_int("NHB_GEMV_KERNEL", NHB_KERNEL_GEMV_ROWS);
		if (k == NHB_KERNEL_GEMV_LDG || k == NHB_KERNEL_GEMV_STREAM || k == NHB_KERNEL_GEMV_ROWS)
			ctx->gemv_default = k;
	}
	*out			 = ctx;
	return NHB_OK;
}

int nhb_ctx_destroy(nhb_ctx* ctx) {
	if (!ctx)
		return NHB_OK;
	device_guard g(ctx->device);
	cudaStreamSynchronize(ctx->stream);
	if (ctx->comm && nccl().ok)
		nccl().CommDestroy(ctx->comm);
	for (auto& r: ctx->regions)
		symm_release(ctx, r);
	for (int i = 0; i < 2; ++i) {
		if (ctx->up_pinned[i])
			cudaFreeHost(ctx->up_pinned[i]);
		if (ctx->up_dev[i])
			cudaFree(ctx->up_dev[i]);
		if (ctx->up_done[i])
			cudaEventDestroy(ctx->up_done[i]);
		if (ctx->group_ev[i])
			cudaEventDestroy(ctx->group_ev[i]);
	}
	if (ctx->push_local)
		cudaFree(ctx->push_local);

	if (ctx->scratch)
		cudaFree(ctx->scratch);
	if (ctx->gemm_counters)
		cudaFree(ctx->gemm_counters);
	if (ctx->plane_buf)
		cudaFree(ctx->plane_buf);
	if (ctx->norm_buf)
		cudaFree(ctx->norm_buf);
	if (ctx->io)
		cudaFree(ctx->io);
	if (ctx->dev_status)
		cudaFree(ctx->dev_status);
	if (ctx->host_status)
		cudaFreeHost(ctx->host_status);
	if (ctx->own)
		cudaStreamDestroy(ctx->own);
	delete ctx;
	return NHB_OK;
}

int nhb_ctx_set_stream(nhb_ctx* ctx, void* cuda_stream) {
	if (!ctx)
		return fail(nullptr, NHB_ERR_ARG, "null context");
	ctx->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->own;
	return NHB_OK;
}

int nhb_ctx_set_gemv_max_m(nhb_ctx* ctx, int max_m) {
	if (!ctx || max_m < 1)
		return fail(ctx, NHB_ERR_ARG, "nhb_ctx_set_gemv_max_m: bad arguments");
	ctx->gemv_max_m = max_m;
	return NHB_OK;
}

int nhb_ctx_set_option(nhb_ctx* ctx, const char* name, int value) {
	if (!ctx || !name)
		return fail(ctx, NHB_ERR_ARG, "nhb_ctx_set_option: bad arguments");
	if (!std::strcmp(name, "pdl"))
		ctx->pdl = value != 0;
	else if (!std::strcmp(name, "ctas_per_sm"))
		ctx->ctas_per_sm = value < 1 ? 1 : (value > 2 ? 2 : value);
	else if (!std::strcmp(name, "gemv_max_m"))
		ctx->gemv_max_m = value < 1 ? 1 : value;
	else if (!std::strcmp(name, "rows_ctas_per_sm"))
		ctx->rows_cps = value < 1 ? 1 : (value > 8 ? 8 : value);
	else if (!std::strcmp(name, "prequantize"))
		ctx->preq = value != 0;
	else if (!std::strcmp(name, "gemm_keep_planes"))
		ctx->gemm_keep_planes = value != 0;
	else if (!std::strcmp(name, "peer_window"))
		ctx->peer_window = value < 0 ? 0 : value;
	else if (!std::strcmp(name, "rows_double_buffer"))
		ctx->rows_db = value < 0 ? -1 : (value != 0);
	else if (!std::strcmp(name, "rows_cluster"))
		ctx->rows_cluster = value < 1 ? 1 : value;
	else if (!std::strcmp(name, "replicate_below_mb"))
		ctx->replicate_below = static_cast<int64_t>(value < 0 ? 0 : value) << 20;
	else if (!std::strcmp(name, "fused_gather"))
		ctx->fused_gather = value != 0;
	else if (!std::strcmp(name, "rows_split_long"))
		ctx->rows_split = value != 0;
	else if (!std::strcmp(name, "rows_fat_ctas"))
		ctx->rows_fat = value != 0;
	else if (!std::strcmp(name, "gemv_kernel")) {
		if (value != NHB_KERNEL_GEMV_LDG && value != NHB_KERNEL_GEMV_STREAM && value != NHB_KERNEL_GEMV_ROWS)
			return fail(ctx, NHB_ERR_ARG, "gemv_kernel must be 1, 2 or 4");
		ctx->gemv_default = value;
	} else if (!std::strcmp(name, "peer_wait_us"))
		ctx->peer_wait_us = value < 1 ? 1 : value;
	else if (!std::strcmp(name, "symm_loopback"))
		ctx->symm_loopback = value != 0;
	else
		return fail(ctx, NHB_ERR_ARG, std::string("unknown option ") + name);
	return NHB_OK;
}

long long nhb_ctx_launch_count(const nhb_ctx* ctx) {
	return ctx ? ctx->launches : 0;
}

// nhb_sync in two halves, so that one host thread driving several contexts can enqueue every context's wait for its
// peers before it blocks on any of them
static int sync_enqueue(nhb_ctx* ctx) {
	if (!ctx->capturing) {
		int rc = wait_pending(ctx);// rows other ranks are still delivering belong to "everything enqueued so far"
		if (rc != NHB_OK)
			return rc;
	}
	NHB_CUDA(ctx, cudaMemcpyAsync(ctx->host_status, ctx->dev_status, NHB_STATUS_WORDS * sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
	return NHB_OK;
}

static int sync_finish(nhb_ctx* ctx) {
	NHB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
	if (ctx->host_status[0] != DEV_OK) {
		const int code = ctx->host_status[0];
		cudaMemsetAsync(ctx->dev_status, 0, NHB_STATUS_WORDS * sizeof(int), ctx->stream);
		if (ctx->push_local) {
			// the exchange starts over: no launch counted, no announcement seen (every rank that saw the timeout does the same)
			cudaMemsetAsync(ctx->push_local, 0, 3 * sizeof(unsigned), ctx->stream);
			cudaMemsetAsync(ctx->regions[0].local, 0, ctx->regions[0].bytes, ctx->stream);
		}
		ctx->dl = nhb_deliveries();
		if (ctx->gemm_counters)
			cudaMemsetAsync(ctx->gemm_counters, 0, gemm_tc_counter_bytes(), ctx->stream);// a GEMM that gave up may have left its tiles' counters half-way
		cudaStreamSynchronize(ctx->stream);
		if (code == DEV_BAD_INDEX)
			return fail(ctx, NHB_ERR_ARG, "a token id outside the embedding table reached nhb_get_rows_q8_0; its output row was left untouched");
		return fail(ctx, NHB_ERR_TIMEOUT, "a device-side wait ran out (code " + std::to_string(code) + "); results of the last launches are invalid");
	}
	return NHB_OK;
}

int nhb_sync(nhb_ctx* ctx) {
	if (!ctx)
		return fail(nullptr, NHB_ERR_ARG, "null context");
	device_guard g(ctx->device);
	int rc = sync_enqueue(ctx);
	return rc != NHB_OK ? rc : sync_finish(ctx);
}

int nhb_sync_all(nhb_ctx* const* ctxs, int n) {
	if (!ctxs || n < 1)
		return fail(nullptr, NHB_ERR_ARG, "nhb_sync_all: bad arguments");
	for (int i = 0; i < n; ++i)
		if (!ctxs[i])
			return fail(nullptr, NHB_ERR_ARG, "nhb_sync_all: null context");
	int first = NHB_OK;
	for (int i = 0; i < n; ++i) {
		device_guard g(ctxs[i]->device);
		const int rc = sync_enqueue(ctxs[i]);
		if (rc != NHB_OK && first == NHB_OK)
			first = rc;
	}
	for (int i = 0; i < n; ++i) {
		device_guard g(ctxs[i]->device);
		const int rc = sync_finish(ctxs[i]);
		if (rc != NHB_OK && first == NHB_OK)
			first = rc;
	}
	return first;
}

int nhb_memcpy_h2d(nhb_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
	if (!ctx || (bytes && (!dst_dev || !src_host)))
		return fail(ctx, NHB_ERR_ARG, "nhb_memcpy_h2d: bad arguments");
	device_guard g(ctx->device);
	NHB_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
	return NHB_OK;
}

int nhb_memcpy_d2h(nhb_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
	if (!ctx || (bytes && (!dst_host || !src_dev)))
		return fail(ctx, NHB_ERR_ARG, "nhb_memcpy_d2h: bad arguments");
	device_guard g(ctx->device);
	NHB_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
	return NHB_OK;
}

int nhb_device_alloc(nhb_ctx* ctx, size_t bytes, void** out_dev) {
	if (!ctx || !out_dev)
		return fail(ctx, NHB_ERR_ARG, "nhb_device_alloc: null argument");
	*out_dev = nullptr;
	if (ctx->capturing)
		return fail(ctx, NHB_ERR_UNSUPPORTED, "allocation during graph capture");
	if (bytes == 0)
		return NHB_OK;
	device_guard g(ctx->device);
	cudaError_t e = cudaMalloc(out_dev, bytes);
	if (e == cudaErrorMemoryAllocation) {
		cudaGetLastError();
		return fail(ctx, NHB_ERR_NOMEM, "nhb_device_alloc: out of device memory");
	}
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "cudaMalloc");
	return NHB_OK;
}

int nhb_device_free(nhb_ctx* ctx, void* dev) {
	if (!ctx)
		return fail(nullptr, NHB_ERR_ARG, "null context");
	if (!dev)
		return NHB_OK;
	device_guard g(ctx->device);
	NHB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
	NHB_CUDA(ctx, cudaFree(dev));
	return NHB_OK;
}

int nhb_weight_upload_q8_0(nhb_ctx* ctx, const void* host_blocks34, int64_t N, int64_t K, nhb_weight** out) {
	if (!ctx || !out)
		return fail(ctx, NHB_ERR_ARG, "nhb_weight_upload_q8_0: null context or output");
	*out = nullptr;
	if (N < 0 || K <= 0 || K % 32 != 0)
		return fail(ctx, NHB_ERR_ARG, "nhb_weight_upload_q8_0: K must be a positive multiple of 32 and N >= 0");
	if (N > 0 && !host_blocks34)
		return fail(ctx, NHB_ERR_ARG, "nhb_weight_upload_q8_0: null tensor data");
	if (K > INT32_MAX || N > (int64_t(1) << 30) * ctx->world)
		return fail(ctx, NHB_ERR_ARG, "nhb_weight_upload_q8_0: K beyond 2^31 - 1 or more than 2^30 rows per rank (the kernels index rows and columns with 32-bit integers)");
	if (ctx->capturing)
		return fail(ctx, NHB_ERR_UNSUPPORTED, "weight upload during graph capture");
	device_guard g(ctx->device);
	nhb_weight* w = new nhb_weight();
	w->N		  = N;
	w->K		  = K;
	w->device	  = ctx->device;
	// placement policy: a weight under the threshold costs less to stream whole on every rank than to shard and exchange
	nhb_place_rows(N, K, ctx->world, ctx->rank, ctx->replicate_below, &w->n0, &w->n1);
	const int64_t rows = w->n1 - w->n0;
	const int64_t nb   = K / 32;
	if (rows > 0) {
		cudaError_t e = cudaMalloc(&w->q, static_cast<size_t>(rows) * K);
		if (e == cudaSuccess)
			e = cudaMalloc(&w->d, static_cast<size_t>(rows) * nb * sizeof(__half));
		if (e != cudaSuccess) {
			if (w->q)
				cudaFree(w->q);
			delete w;
			return fail_cuda(ctx, e, "weight plane allocation");
		}
		// Raw blocks travel in row chunks of <= 32 MiB through two pinned host buffers and two device buffers, and are
		// split on the device.  The caller's memory is usually pageable (a mapped GGUF file): copying it into pinned
		// memory on this thread while the previous chunk is on the bus and in the repack kernel roughly triples the
		// rate of handing pageable memory to cudaMemcpyAsync chunk by chunk.
		const int64_t row_bytes	 = nb * 34;
		const int64_t chunk_rows = std::max<int64_t>(1, (int64_t(32) << 20) / row_bytes);
		const size_t stage_bytes = static_cast<size_t>(std::min(chunk_rows, rows) * row_bytes);
		const uint8_t* src		 = static_cast<const uint8_t*>(host_blocks34) + w->n0 * row_bytes;
		e						 = cudaSuccess;
		for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
			if (ctx->up_cap < stage_bytes || !ctx->up_pinned[i]) {
				if (ctx->up_pinned[i])
					cudaFreeHost(ctx->up_pinned[i]);
				if (ctx->up_dev[i])
					cudaFree(ctx->up_dev[i]);
				ctx->up_pinned[i] = nullptr;
				ctx->up_dev[i]	  = nullptr;
				e				  = cudaMallocHost(&ctx->up_pinned[i], stage_bytes);
				if (e == cudaSuccess)
					e = cudaMalloc(&ctx->up_dev[i], stage_bytes);
			}
			if (e == cudaSuccess && !ctx->up_done[i])
				e = cudaEventCreateWithFlags(&ctx->up_done[i], cudaEventDisableTiming);
		}
		if (e == cudaSuccess && ctx->up_cap < stage_bytes)
			ctx->up_cap = stage_bytes;
		int slot = 0;
		bool used[2] = { false, false };
		for (int64_t r0 = 0; r0 < rows && e == cudaSuccess; r0 += chunk_rows, slot ^= 1) {
			const int64_t rr   = std::min(chunk_rows, rows - r0);
			const size_t bytes = static_cast<size_t>(rr * row_bytes);
			if (used[slot])
				e = cudaEventSynchronize(ctx->up_done[slot]);// the chunk that used this pair two steps ago has left it
			if (e != cudaSuccess)
				break;
			std::memcpy(ctx->up_pinned[slot], src + r0 * row_bytes, bytes);
			e = cudaMemcpyAsync(ctx->up_dev[slot], ctx->up_pinned[slot], bytes, cudaMemcpyHostToDevice, ctx->stream);
			if (e == cudaSuccess)
				e = launch_repack(static_cast<const uint8_t*>(ctx->up_dev[slot]), rr, K, w->q + r0 * K, w->d + r0 * nb, ctx->stream);
			if (e == cudaSuccess)
				e = cudaEventRecord(ctx->up_done[slot], ctx->stream);
			used[slot] = true;
		}
		if (e == cudaSuccess)
			e = cudaStreamSynchronize(ctx->stream);// the weight is usable, and the caller's buffer released, on return
		if (e != cudaSuccess) {
			cudaFree(w->q);
			cudaFree(w->d);
			delete w;
			return fail_cuda(ctx, e, "weight upload");
		}
		ctx->launches += (rows + chunk_rows - 1) / chunk_rows;
	}
	*out = w;
	return NHB_OK;
}

int nhb_weight_free(nhb_ctx* ctx, nhb_weight* w) {
	if (!w)
		return NHB_OK;
	device_guard g(w->device);
	if (ctx)
		cudaStreamSynchronize(ctx->stream);
	if (w->q)
		cudaFree(w->q);
	if (w->d)
		cudaFree(w->d);
	if (w->w16)
		cudaFree(w->w16);
	if (w->wdT)
		cudaFree(w->wdT);
	delete w;
	return NHB_OK;
}

int nhb_weight_info_get(const nhb_weight* w, nhb_weight_info* info) {
	if (!w || !info)
		return fail(nullptr, NHB_ERR_ARG, "nhb_weight_info_get: null argument");
	info->N		   = w->N;
	info->K		   = w->K;
	info->n0	   = w->n0;
	info->n1	   = w->n1;
	info->q		   = w->q;
	info->d		   = w->d;
	info->bytes_q8 = (w->n1 - w->n0) * (w->K / 32) * 34;
	return NHB_OK;
}

int nhb_weight_download_q8_0(nhb_ctx* ctx, const nhb_weight* w, void* host_blocks34_shard) {
	if (!ctx || !w || !host_blocks34_shard)
		return fail(ctx, NHB_ERR_ARG, "nhb_weight_download_q8_0: null argument");
	device_guard g(ctx->device);
	const int64_t rows = w->n1 - w->n0;
	if (rows == 0)
		return NHB_OK;
	const size_t bytes = static_cast<size_t>(rows) * (w->K / 32) * 34;
	void* stage		   = nullptr;
	NHB_CUDA(ctx, cudaMalloc(&stage, bytes));
	cudaError_t e = launch_unpack(w->q, w->d, rows, w->K, static_cast<uint8_t*>(stage), ctx->stream);
	if (e == cudaSuccess)
		e = cudaMemcpyAsync(host_blocks34_shard, stage, bytes, cudaMemcpyDeviceToHost, ctx->stream);
	if (e == cudaSuccess)
		e = cudaStreamSynchronize(ctx->stream);
	cudaFree(stage);
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "weight download");
	ctx->launches += 1;
	return NHB_OK;
}

int nhb_mul_mat_batch(nhb_ctx* ctx, const nhb_mul_mat_op* ops, int n_ops, int act_mode, int kernel) {
	if (!ctx || (n_ops > 0 && !ops) || n_ops < 0 || n_ops > NHB_MAX_BATCH)
		return fail(ctx, NHB_ERR_ARG, "nhb_mul_mat_batch: bad batch (at most 8 ops)");
	if (act_mode != NHB_ACT_Q8 && act_mode != NHB_ACT_F32)
		return fail(ctx, NHB_ERR_ARG, "unknown activation mode");
	if (kernel < NHB_KERNEL_AUTO || kernel > NHB_KERNEL_GEMV_ROWS)
		return fail(ctx, NHB_ERR_ARG, "unknown kernel id");
	if (n_ops == 0)
		return NHB_OK;
	for (int i = 0; i < n_ops; ++i) {
		int rc = check_mm_args(ctx, ops[i].w, ops[i].x, ops[i].ldx, ops[i].y, ops[i].ldy, ops[i].M);
		if (rc != NHB_OK)
			return rc;
		if (ops[i].M != ops[0].M)
			return fail(ctx, NHB_ERR_ARG, "all ops of a batch must share M");
	}
	const int64_t M = ops[0].M;
	if (M == 0)
		return NHB_OK;
	device_guard g(ctx->device);
	// whatever this call writes is this rank's slice only, until a fused launch below says otherwise
	for (int i = 0; i < n_ops && ctx->world > 1; ++i) {
		auto& c = ctx->complete;
		c.erase(std::remove(c.begin(), c.end(), static_cast<const void*>(ops[i].y)), c.end());
		if (ops[i].w->n1 - ops[i].w->n0 == ops[i].w->N)
			c.push_back(ops[i].y);// replicated weight: this rank writes the whole row itself
	}
	const int forced = env_int("NHB_FORCE_KERNEL", 0);
	if (kernel == NHB_KERNEL_AUTO && forced >= 1 && forced <= 4)
		kernel = forced;
	bool use_gemm = false;
	if (kernel == NHB_KERNEL_GEMM_TC) {
		use_gemm = true;
	} else if (kernel == NHB_KERNEL_AUTO) {
		use_gemm = act_mode == NHB_ACT_Q8 && M > ctx->gemv_max_m;
		for (int i = 0; i < n_ops && use_gemm; ++i)
			use_gemm = gemm_tc_supports(ops[i].w->n1 - ops[i].w->n0, ops[i].w->K, M) || ops[i].w->n1 == ops[i].w->n0;
	}
	if (use_gemm) {
		if (act_mode != NHB_ACT_Q8)
			return fail(ctx, NHB_ERR_UNSUPPORTED, "the tensor-core GEMM implements the Q8-activation arithmetic only");
		int last = -1;// the last op that actually ran (a rank may own no rows of an op)
		for (int i = 0; i < n_ops; ++i) {
			if (ops[i].w->n1 > ops[i].w->n0 && !gemm_tc_supports(ops[i].w->n1 - ops[i].w->n0, ops[i].w->K, M))
				return fail(ctx, NHB_ERR_UNSUPPORTED, "shape not supported by the tensor-core GEMM (needs K % 64 == 0)");
			// ops that share their input (q/k/v, gate/up) quantise it once: the scratch is only rewritten by another input
			const bool same = last >= 0 && ops[last].x == ops[i].x && ops[last].ldx == ops[i].ldx && ops[last].w->K == ops[i].w->K;
			int rc			= run_gemm(ctx, ops[i], same);
			if (rc != NHB_OK)
				return rc;
			if (ops[i].w->n1 > ops[i].w->n0)
				last = i;
		}
		return NHB_OK;
	}
	return run_gemv(ctx, ops, n_ops, act_mode, kernel);
}

int nhb_mul_mat(nhb_ctx* ctx, const nhb_weight* w, const float* x_dev, int64_t ldx, float* y_dev, int64_t ldy, int64_t M, int act_mode, int kernel) {
	nhb_mul_mat_op op{ w, x_dev, ldx, y_dev, ldy, M };
	return nhb_mul_mat_batch(ctx, &op, 1, act_mode, kernel);
}

int nhb_mul_mat_host(nhb_ctx* ctx, const nhb_weight* w, const float* x_host, int64_t ldx, float* y_host, int64_t ldy, int64_t M, int act_mode,
	int kernel) {
	if (!ctx || !w)
		return fail(ctx, NHB_ERR_ARG, "null context or weight");
	if (M < 0 || (M > 0 && (!x_host || !y_host)) || ldx < w->K || ldy < w->N)
		return fail(ctx, NHB_ERR_ARG, "nhb_mul_mat_host: bad arguments");
	if (M == 0)
		return NHB_OK;
	device_guard g(ctx->device);
	const int64_t rows = w->n1 - w->n0;
	const size_t xb	   = static_cast<size_t>(M) * w->K * 4;
	const size_t xpad  = (xb + 255) & ~size_t(255);
	const size_t yb	   = static_cast<size_t>(M) * w->N * 4;
	int rc			   = ensure(ctx, &ctx->io, &ctx->io_cap, xpad + yb, "host-I/O staging");
	if (rc != NHB_OK)
		return rc;
	float* xd = static_cast<float*>(ctx->io);
	float* yd = reinterpret_cast<float*>(static_cast<char*>(ctx->io) + xpad);
	NHB_CUDA(ctx, cudaMemcpy2DAsync(xd, w->K * 4, x_host, ldx * 4, w->K * 4, M, cudaMemcpyHostToDevice, ctx->stream));
	rc = nhb_mul_mat(ctx, w, xd, w->K, yd, w->N, M, act_mode, kernel);
	if (rc != NHB_OK)
		return rc;
	if (rows > 0)
		NHB_CUDA(ctx, cudaMemcpy2DAsync(y_host + w->n0, ldy * 4, yd + w->n0, w->N * 4, rows * 4, M, cudaMemcpyDeviceToHost, ctx->stream));
	return NHB_OK;
}

namespace {
	// y = W . act(x [, x2]) [+ res]: the GEMV family with the element-wise neighbours fused into its prologue and epilogue, or
	// -- for more tokens than it takes -- the two element-wise kernels around the tensor-core GEMM.  Same values either way.
	int run_fused(nhb_ctx* ctx, const nhb_weight* w, const float* x, const float* x2, int64_t ldx, const float* res, int64_t ldr, float* y, int64_t ldy, int64_t M,
		const char* who) {
		int rc = check_mm_args(ctx, w, x, ldx, y, ldy, M);
		if (rc != NHB_OK)
			return rc;
		if (M == 0)
			return NHB_OK;
		if (x2 && (reinterpret_cast<uintptr_t>(x2) & 15))
			return fail(ctx, NHB_ERR_ARG, std::string(who) + ": the up projection's rows must be 16-byte aligned");
		if (res && ldr < w->N)
			return fail(ctx, NHB_ERR_ARG, std::string(who) + ": residual leading dimension smaller than the row length");
		device_guard g(ctx->device);
		const int64_t rows = w->n1 - w->n0;
		auto& c			   = ctx->complete;
		if (ctx->world > 1) {
			c.erase(std::remove(c.begin(), c.end(), static_cast<const void*>(y)), c.end());
			if (rows == w->N)
				c.push_back(y);
		}
		if (rows == 0)
			return NHB_OK;
		const bool gemv = M <= ctx->gemv_max_m && gemv_rows_supports(w->K, std::min<int64_t>(M, 4)) && gemv_rows_act_bytes(w->K, 1) <= 96 * 1024;
		if (gemv) {
			const launch_cfg cfg = cfg_of(ctx);
			int launches		 = 0;
			int mt_max			 = 4;
			while (mt_max > 1 && gemv_rows_act_bytes(w->K, mt_max) > 96 * 1024)
				--mt_max;
			for (int64_t m0 = 0; m0 < M; m0 += mt_max) {
				const int mt = static_cast<int>(std::min<int64_t>(mt_max, M - m0));
				nhb_mul_mat_op op{ w, x, ldx, y, ldy, M };
				rows_batch b{};
				const nhb_mul_mat_op* src_ops[NHB_MAX_BATCH];
				fill_rows_batch(&op, 1, m0, mt, false, b, src_ops);
				b.op[0].x2	= x2 ? x2 + m0 * ldx : nullptr;
				b.op[0].res = res ? res + m0 * ldr + w->n0 : nullptr;
				b.op[0].ldr = ldr;
				const bool pushed = ctx->rows_cluster <= 1 && w->N >= ctx->world && setup_push(ctx, b, src_ops, mt, m0);
				if (pushed && m0 + mt >= M)
					c.push_back(y);
				batch_spans sp;
				spans_of(b, src_ops, mt, m0, sp);
				plan_peer_wait(ctx, b.push, sp.in, sp.n_in, sp.out, sp.n_out, pushed);
				cudaError_t e = launch_gemv_rows(b, mt, cfg, ctx->rows_cps, &launches, false, 1, ctx->rows_fat != 0, ctx->rows_split != 0);
				if (e != cudaSuccess)
					return fail_cuda(ctx, e, "gemv_q8_rows launch (fused element-wise)");
			}
			ctx->launches += launches;
			return NHB_OK;
		}
		// the GEMM path: SwiGLU into a scratch row block, the contraction, then the residual on this rank's columns
		if (!gemm_tc_supports(rows, w->K, M))
			return fail(ctx, NHB_ERR_UNSUPPORTED, std::string(who) + ": shape not supported by the tensor-core GEMM (needs K % 64 == 0)");
		const float* act = x;
		int64_t ld_act	 = ldx;
		if (x2) {
			rc = ensure(ctx, &ctx->norm_buf, &ctx->norm_cap, static_cast<size_t>(M) * w->K * 4, "SwiGLU scratch");
			if (rc == NHB_OK)
				rc = wait_pending(ctx);
			if (rc != NHB_OK)
				return rc;
			cudaError_t e = launch_swiglu(x, x2, ldx, static_cast<float*>(ctx->norm_buf), w->K, static_cast<int>(M), static_cast<int>(w->K), ctx->stream, ctx->pdl);
			if (e != cudaSuccess)
				return fail_cuda(ctx, e, "swiglu launch");
			ctx->launches += 1;
			act	   = static_cast<const float*>(ctx->norm_buf);
			ld_act = w->K;
		}
		nhb_mul_mat_op op{ w, act, ld_act, y, ldy, M };
		rc = run_gemm(ctx, op);
		if (rc != NHB_OK)
			return rc;
		if (res) {
			cudaError_t e = launch_add_rows(y + w->n0, ldy, res + w->n0, ldr, static_cast<int>(M), static_cast<int>(rows), ctx->stream, ctx->pdl);
			if (e != cudaSuccess)
				return fail_cuda(ctx, e, "residual add launch");
			ctx->launches += 1;
		}
		return NHB_OK;
	}
}

int nhb_mul_mat_swiglu_add(nhb_ctx* ctx, const nhb_weight* w, const float* gate_dev, const float* up_dev, int64_t ld, const float* residual_dev, int64_t ld_residual,
	float* y_dev, int64_t ldy, int64_t M) {
	if (M > 0 && !up_dev)
		return fail(ctx, NHB_ERR_ARG, "nhb_mul_mat_swiglu_add: null up-projection pointer");
	return run_fused(ctx, w, gate_dev, up_dev, ld, residual_dev, ld_residual, y_dev, ldy, M, "nhb_mul_mat_swiglu_add");
}

int nhb_mul_mat_add(nhb_ctx* ctx, const nhb_weight* w, const float* x_dev, int64_t ldx, const float* residual_dev, int64_t ld_residual, float* y_dev, int64_t ldy,
	int64_t M) {
	if (M > 0 && !residual_dev)
		return fail(ctx, NHB_ERR_ARG, "nhb_mul_mat_add: null residual pointer");
	return run_fused(ctx, w, x_dev, nullptr, ldx, residual_dev, ld_residual, y_dev, ldy, M, "nhb_mul_mat_add");
}

int nhb_swiglu(nhb_ctx* ctx, const float* gate_dev, const float* up_dev, int64_t ld, float* h_dev, int64_t ldh, int64_t M, int64_t K) {
	if (!ctx || M < 0 || K < 0 || K % 4 != 0 || ld < K || ldh < K || (ld & 3) || (ldh & 3) || M > INT32_MAX || K > INT32_MAX)
		return fail(ctx, NHB_ERR_ARG, "nhb_swiglu: bad arguments (K, ld and ldh are multiples of 4)");
	if (M == 0 || K == 0)
		return NHB_OK;
	if (!gate_dev || !up_dev || !h_dev || ((reinterpret_cast<uintptr_t>(gate_dev) | reinterpret_cast<uintptr_t>(up_dev) | reinterpret_cast<uintptr_t>(h_dev)) & 15))
		return fail(ctx, NHB_ERR_ARG, "nhb_swiglu: null or misaligned pointer");
	device_guard g(ctx->device);
	if (int rc = wait_pending(ctx); rc != NHB_OK)
		return rc;
	cudaError_t e = launch_swiglu(gate_dev, up_dev, ld, h_dev, ldh, static_cast<int>(M), static_cast<int>(K), ctx->stream, ctx->pdl);
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "swiglu launch");
	ctx->launches += 1;
	return NHB_OK;
}

int nhb_quantize_q8_0(nhb_ctx* ctx, const float* x_dev, int64_t ldx, int64_t M, int64_t K, int8_t* q_dev, float* d_dev) {
	if (!ctx || M < 0 || K <= 0 || K % 32 != 0 || ldx < K)
		return fail(ctx, NHB_ERR_ARG, "nhb_quantize_q8_0: bad arguments");
	if (M == 0)
		return NHB_OK;
	if (!x_dev || !q_dev || !d_dev || (reinterpret_cast<uintptr_t>(x_dev) & 15) || (ldx & 3) || (reinterpret_cast<uintptr_t>(q_dev) & 15))
		return fail(ctx, NHB_ERR_ARG, "nhb_quantize_q8_0: null or misaligned pointer");
	device_guard g(ctx->device);
	if (int rc = wait_pending(ctx); rc != NHB_OK)
		return rc;
	cudaError_t e = launch_quantize(x_dev, ldx, static_cast<int>(M), static_cast<int>(K), q_dev, d_dev, ctx->stream);
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "quantize_q8 launch");
	ctx->launches += 1;
	return NHB_OK;
}

namespace {
	int check_norm_args(nhb_ctx* ctx, const float* x, int64_t ldx, const float* w, int sqrt_mode, int64_t M, int64_t K, const char* who) {
		if (!ctx || M < 0 || K <= 0 || K % 32 != 0 || ldx < K || (sqrt_mode != NHB_SQRT_IEEE && sqrt_mode != NHB_SQRT_X86_FAST))
			return fail(ctx, NHB_ERR_ARG, std::string(who) + ": bad arguments");
		if (!rms_norm_supports(K))
			return fail(ctx, NHB_ERR_UNSUPPORTED, std::string(who) + ": K too large for one CTA's shared memory (K <= 51200)");
		if (M > 0 && (!x || !w || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (ldx & 3)))
			return fail(ctx, NHB_ERR_ARG, std::string(who) + ": null or misaligned pointer");
		if (M > INT32_MAX)
			return fail(ctx, NHB_ERR_ARG, std::string(who) + ": M too large");
		return NHB_OK;
	}
}

int nhb_rms_norm_mul(nhb_ctx* ctx, const float* x_dev, int64_t ldx, const float* norm_w_dev, float eps, int sqrt_mode, float* y_dev, int64_t ldy,
	int64_t M, int64_t K) {
	int rc = check_norm_args(ctx, x_dev, ldx, norm_w_dev, sqrt_mode, M, K, "nhb_rms_norm_mul");
	if (rc != NHB_OK)
		return rc;
	if (M == 0)
		return NHB_OK;
	if (!y_dev || (reinterpret_cast<uintptr_t>(y_dev) & 15) || (ldy & 3) || ldy < K)
		return fail(ctx, NHB_ERR_ARG, "nhb_rms_norm_mul: null or misaligned output");
	device_guard g(ctx->device);
	if (int rcw = wait_pending(ctx); rcw != NHB_OK)
		return rcw;
	const norm_out no{ y_dev, ldy, nullptr, nullptr, nullptr };
	cudaError_t e = launch_rms_norm(x_dev, ldx, norm_w_dev, eps, sqrt_mode, static_cast<int>(M), static_cast<int>(K), no, ctx->stream, ctx->pdl);
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "rms_norm_mul launch");
	ctx->launches += 1;
	return NHB_OK;
}

int nhb_rms_norm_mul_q8_0(nhb_ctx* ctx, const float* x_dev, int64_t ldx, const float* norm_w_dev, float eps, int sqrt_mode, void* blocks_dev, int64_t M,
	int64_t K) {
	int rc = check_norm_args(ctx, x_dev, ldx, norm_w_dev, sqrt_mode, M, K, "nhb_rms_norm_mul_q8_0");
	if (rc != NHB_OK)
		return rc;
	if (M == 0)
		return NHB_OK;
	if (!blocks_dev || (reinterpret_cast<uintptr_t>(blocks_dev) & 1))
		return fail(ctx, NHB_ERR_ARG, "nhb_rms_norm_mul_q8_0: null or odd output address");
	device_guard g(ctx->device);
	if (int rcw = wait_pending(ctx); rcw != NHB_OK)
		return rcw;
	const norm_out no{ nullptr, 0, nullptr, nullptr, static_cast<unsigned char*>(blocks_dev) };
	cudaError_t e = launch_rms_norm(x_dev, ldx, norm_w_dev, eps, sqrt_mode, static_cast<int>(M), static_cast<int>(K), no, ctx->stream, ctx->pdl);
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "rms_norm_mul_q8_0 launch");
	ctx->launches += 1;
	return NHB_OK;
}

int nhb_rms_norm_mul_mat_batch(nhb_ctx* ctx, const nhb_mul_mat_op* ops, int n_ops, const float* norm_w_dev, float eps, int sqrt_mode, int kernel) {
	if (!ctx || (n_ops > 0 && !ops) || n_ops < 0 || n_ops > NHB_MAX_BATCH)
		return fail(ctx, NHB_ERR_ARG, "nhb_rms_norm_mul_mat_batch: bad batch (at most 8 ops)");
	if (kernel < NHB_KERNEL_AUTO || kernel > NHB_KERNEL_GEMV_ROWS)
		return fail(ctx, NHB_ERR_ARG, "unknown kernel id");
	if (n_ops == 0)
		return NHB_OK;
	for (int i = 0; i < n_ops; ++i) {
		int rc = check_mm_args(ctx, ops[i].w, ops[i].x, ops[i].ldx, ops[i].y, ops[i].ldy, ops[i].M);
		if (rc != NHB_OK)
			return rc;
		if (ops[i].x != ops[0].x || ops[i].ldx != ops[0].ldx || ops[i].M != ops[0].M || ops[i].w->K != ops[0].w->K)
			return fail(ctx, NHB_ERR_ARG, "nhb_rms_norm_mul_mat_batch: every op must read the same rows (x, ldx, M, K)");
	}
	const int64_t M = ops[0].M, K = ops[0].w->K;
	int rc = check_norm_args(ctx, ops[0].x, ops[0].ldx, norm_w_dev, sqrt_mode, M, K, "nhb_rms_norm_mul_mat_batch");
	if (rc != NHB_OK)
		return rc;
	if (M == 0)
		return NHB_OK;
	device_guard g(ctx->device);
	// decode: the norm kernel hands the GEMV its quantised rows directly
	int resolved = kernel;
	if (resolved == NHB_KERNEL_AUTO) {
		const int forced = env_int("NHB_FORCE_KERNEL", 0);
		resolved		 = forced >= 1 && forced <= 4 ? forced : (M > ctx->gemv_max_m ? NHB_KERNEL_GEMM_TC : ctx->gemv_default);
	}
	if (resolved == NHB_KERNEL_GEMV_ROWS && gemv_rows_supports(K, 1) && gemv_rows_act_bytes(K, 1) <= 96 * 1024) {
		ctx->norm_w	   = norm_w_dev;
		ctx->norm_eps  = eps;
		ctx->norm_sqrt = sqrt_mode;
		rc			   = nhb_mul_mat_batch(ctx, ops, n_ops, NHB_ACT_Q8, NHB_KERNEL_GEMV_ROWS);
		ctx->norm_w	   = nullptr;
		return rc;
	}
	// everything else: normalised f32 rows through a scratch buffer, then the ordinary operator
	rc = ensure(ctx, &ctx->norm_buf, &ctx->norm_cap, static_cast<size_t>(M) * K * 4, "rms_norm scratch");
	if (rc == NHB_OK)
		rc = wait_pending(ctx);
	if (rc != NHB_OK)
		return rc;
	const norm_out no{ static_cast<float*>(ctx->norm_buf), K, nullptr, nullptr, nullptr };
	cudaError_t e = launch_rms_norm(ops[0].x, ops[0].ldx, norm_w_dev, eps, sqrt_mode, static_cast<int>(M), static_cast<int>(K), no, ctx->stream, ctx->pdl);
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "rms_norm_mul launch");
	ctx->launches += 1;
	nhb_mul_mat_op normed[NHB_MAX_BATCH];
	for (int i = 0; i < n_ops; ++i) {
		normed[i]	  = ops[i];
		normed[i].x	  = static_cast<const float*>(ctx->norm_buf);
		normed[i].ldx = K;
	}
	return nhb_mul_mat_batch(ctx, normed, n_ops, NHB_ACT_Q8, kernel);
}

int nhb_mul_mat_block_dots(nhb_ctx* ctx, const nhb_weight* w, const float* x_dev, int64_t ldx, int64_t M, int32_t* dots_dev) {
	if (!ctx || !w || M < 0 || (M > 0 && (!x_dev || !dots_dev)) || ldx < w->K)
		return fail(ctx, NHB_ERR_ARG, "nhb_mul_mat_block_dots: bad arguments");
	if ((reinterpret_cast<uintptr_t>(x_dev) & 15) || (ldx & 3))
		return fail(ctx, NHB_ERR_ARG, "activations must be 16-byte aligned with ldx a multiple of 4");
	const int64_t rows = w->n1 - w->n0;
	if (M == 0 || rows == 0)
		return NHB_OK;
	device_guard g(ctx->device);
	const size_t qb = (static_cast<size_t>(M) * w->K + 255) & ~size_t(255);
	int rc			= ensure(ctx, &ctx->scratch, &ctx->scratch_cap, qb + static_cast<size_t>(M) * (w->K / 32) * 4, "block-dot scratch");
	if (rc != NHB_OK)
		return rc;
	int8_t* qa	  = static_cast<int8_t*>(ctx->scratch);
	float* da	  = reinterpret_cast<float*>(static_cast<char*>(ctx->scratch) + qb);
	rc			  = wait_pending(ctx);
	if (rc != NHB_OK)
		return rc;
	cudaError_t e = launch_quantize(x_dev, ldx, static_cast<int>(M), static_cast<int>(w->K), qa, da, ctx->stream);
	if (e == cudaSuccess)
		e = launch_block_dots(w->q, qa, static_cast<int>(rows), static_cast<int>(w->K), static_cast<int>(M), dots_dev, ctx->stream);
	if (e != cudaSuccess)
		return fail_cuda(ctx, e, "block-dot launch");
	ctx->launches += 2;
	return NHB_OK;
}

int nhb_chain_create(nhb_ctx* ctx, const nhb_mul_mat_op* ops, const int* ops_per_stage, int n_stages, nhb_chain** out) {
	if (!ctx || !out || n_stages < 0 || (n_stages > 0 && (!ops || !ops_per_stage)))
		return fail(ctx, NHB_ERR_ARG, "nhb_chain_create: bad arguments");
	*out = nullptr;
	nhb_chain* ch = new nhb_chain();
	ch->device	  = ctx->device;
	ch->stages.resize(static_cast<size_t>(n_stages));
	ch->delivers.assign(static_cast<size_t>(n_stages), 0);
	int64_t M				 = -1;
	const nhb_mul_mat_op* op = ops;
	for (int s = 0; s < n_stages; ++s) {
		const int n = ops_per_stage[s];
		if (n < 1 || n > NHB_MAX_BATCH) {
			delete ch;
			return fail(ctx, NHB_ERR_ARG, "nhb_chain_create: a stage holds 1 to 8 ops");
		}
		size_t act_total = 0;
		for (int i = 0; i < n; ++i) {
			int rc = check_mm_args(ctx, op[i].w, op[i].x, op[i].ldx, op[i].y, op[i].ldy, op[i].M);
			if (rc == NHB_OK && M >= 0 && op[i].M != M)
				rc = fail(ctx, NHB_ERR_ARG, "nhb_chain_create: all ops of a chain must share M");
			if (rc == NHB_OK && (op[i].M < 1 || op[i].M > 4 || !gemv_rows_supports(op[i].w->K, op[i].M)))
				rc = fail(ctx, NHB_ERR_UNSUPPORTED, "nhb_chain_create: needs 1 <= M <= 4 and rows the warp-per-row GEMV takes; run other stages with nhb_mul_mat_batch");
			if (rc != NHB_OK) {
				delete ch;
				return rc;
			}
			M = op[i].M;
		}
		rows_batch& b = ch->stages[static_cast<size_t>(s)];
		b			  = rows_batch{};
		const nhb_mul_mat_op* src_ops[NHB_MAX_BATCH];
		act_total = fill_rows_batch(op, n, 0, static_cast<int>(M), false, b, src_ops);
		if (act_total > 96 * 1024) {
			delete ch;
			return fail(ctx, NHB_ERR_UNSUPPORTED, "nhb_chain_create: a stage's distinct activation inputs exceed the GEMV's shared memory");
		}
		bool all_ranks_have_rows = true;
		for (int i = 0; i < n; ++i)
			all_ranks_have_rows = all_ranks_have_rows && op[i].w->N >= ctx->world;
		const bool pushed = b.n_ops > 0 && all_ranks_have_rows && setup_push(ctx, b, src_ops, static_cast<int>(M), 0);
		setup_peer_wait(ctx, b.push);
		batch_spans sp;
		spans_of(b, src_ops, static_cast<int>(M), 0, sp);
		ch->in.emplace_back(sp.in, sp.in + sp.n_in);
		ch->out.emplace_back(sp.out, sp.out + sp.n_out);
		for (int i = 0; i < n; ++i) {
			ch->written.push_back(op[i].y);
			if (op[i].w->n1 - op[i].w->n0 == op[i].w->N && ctx->world > 1)
				ch->delivered.push_back(op[i].y);// replicated weight: this rank writes the whole row itself
		}
		for (int i = 0; i < b.n_ops && pushed; ++i)
			if (b.y_peer[i][0])
				ch->delivered.push_back(src_ops[i]->y);
		ch->delivers[static_cast<size_t>(s)] = pushed ? 1 : 0;
		op += n;
	}
	ch->M = static_cast<int>(M < 0 ? 0 : M);
	*out = ch;
	return NHB_OK;
}

int nhb_chain_launch(nhb_ctx* ctx, nhb_chain* ch) {
	if (!ctx || !ch)
		return fail(ctx, NHB_ERR_ARG, "nhb_chain_launch: null argument");
	if (ch->device != ctx->device)
		return fail(ctx, NHB_ERR_ARG, "nhb_chain_launch: the chain belongs to a context of another device");
	if (ch->stages.empty() || ch->M == 0)
		return NHB_OK;
	device_guard g(ctx->device);
	// what these launches write is this rank's slice only, except where they deliver the rows themselves
	if (ctx->world > 1) {
		auto& c = ctx->complete;
		for (const void* y: ch->written)
			c.erase(std::remove(c.begin(), c.end(), y), c.end());
		for (const void* y: ch->delivered)
			c.push_back(y);
	}
	const launch_cfg cfg = cfg_of(ctx);
	int launches		 = 0;
	for (size_t s = 0; s < ch->stages.size(); ++s) {
		const bool db = pick_double_buffer(ctx, ch->stages[s], ch->M, ch->delivers[s] != 0);
		plan_peer_wait(ctx, ch->stages[s].push, ch->in[s].data(), static_cast<int>(ch->in[s].size()), ch->out[s].data(), static_cast<int>(ch->out[s].size()),
			ch->delivers[s] != 0);
		cudaError_t e = launch_gemv_rows(ch->stages[s], ch->M, cfg, db && ctx->rows_db < 0 ? 2 : ctx->rows_cps, &launches, db, 1, ctx->rows_fat != 0, ctx->rows_split != 0);
		if (e != cudaSuccess)
			return fail_cuda(ctx, e, "gemv_q8_rows launch (chain)");
	}
	ctx->launches += launches;
	return NHB_OK;
}

int nhb_chain_free(nhb_ctx* ctx, nhb_chain* ch) {
	(void)ctx;
	delete ch;
	return NHB_OK;
}

int nhb_graph_begin(nhb_ctx* ctx) {
	if (!ctx)
		return fail(nullptr, NHB_ERR_ARG, "null context");
	if (ctx->capturing)
		return fail(ctx, NHB_ERR_ARG, "a capture is already open");
	device_guard g(ctx->device);
	NHB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
	ctx->capturing = true;
	// a replay may follow anything (deliveries.h: capture_begin)
	ctx->cap_seq0 = ctx->world > 1 ? capture_begin(ctx->dl) : ctx->dl.seq;
	return NHB_OK;
}

int nhb_graph_end(nhb_ctx* ctx, nhb_graph** out) {
	if (!ctx || !out)
		return fail(ctx, NHB_ERR_ARG, "nhb_graph_end: null argument");
	if (!ctx->capturing)
		return fail(ctx, NHB_ERR_ARG, "no capture is open");
	device_guard g(ctx->device);
	ctx->capturing = false;
	nhb_graph* gr  = new nhb_graph();
	cudaError_t e  = cudaStreamEndCapture(ctx->stream, &gr->graph);
	if (e == cudaSuccess)
		e = cudaGraphInstantiate(&gr->exec, gr->graph, 0);
	if (e != cudaSuccess) {
		if (gr->graph)
			cudaGraphDestroy(gr->graph);
		delete gr;
		return fail_cuda(ctx, e, "graph capture");
	}
	gr->replay = capture_end(ctx->dl, ctx->cap_seq0);// what a replay leaves behind, relative to where it starts
	*out = gr;
	return NHB_OK;
}

int nhb_graph_launch(nhb_ctx* ctx, nhb_graph* gr) {
	if (!ctx || !gr || !gr->exec)
		return fail(ctx, NHB_ERR_ARG, "nhb_graph_launch: null argument");
	device_guard g(ctx->device);
	NHB_CUDA(ctx, cudaGraphLaunch(gr->exec, ctx->stream));
	replayed(ctx->dl, gr->replay);
	return NHB_OK;
}

int nhb_graph_free(nhb_ctx* ctx, nhb_graph* gr) {
	if (!gr)
		return NHB_OK;
	if (ctx) {
		device_guard g(ctx->device);
		cudaStreamSynchronize(ctx->stream);
		if (gr->exec)
			cudaGraphExecDestroy(gr->exec);
		if (gr->graph)
			cudaGraphDestroy(gr->graph);
	}
	delete gr;
	return NHB_OK;
}

int nhb_comm_unique_id(void* id128) {
	if (!id128)
		return fail(nullptr, NHB_ERR_ARG, "null id buffer");
	if (!nccl().ok)
		return fail(nullptr, NHB_ERR_NCCL, "libnccl.so.2 could not be loaded");
	nccl_uid id;
	int rc = nccl().GetUniqueId(&id);
	if (rc != nccl_success)
		return fail(nullptr, NHB_ERR_NCCL, std::string("ncclGetUniqueId: ") + (nccl().GetErrorString ? nccl().GetErrorString(rc) : "error"));
	std::memcpy(id128, &id, sizeof(id));
	return NHB_OK;
}

int nhb_comm_init(nhb_ctx* ctx, const void* id128) {
	if (!ctx || !id128)
		return fail(ctx, NHB_ERR_ARG, "nhb_comm_init: null argument");
	if (ctx->world == 1)
		return NHB_OK;
	if (!nccl().ok)
		return fail(ctx, NHB_ERR_NCCL, "libnccl.so.2 could not be loaded");
	if (ctx->comm)
		return fail(ctx, NHB_ERR_ARG, "communicator already initialised");
	device_guard g(ctx->device);
	nccl_uid id;
	std::memcpy(&id, id128, sizeof(id));
	int rc = nccl().CommInitRank(&ctx->comm, ctx->world, id, ctx->rank);
	if (rc != nccl_success) {
		ctx->comm = nullptr;
		return fail(ctx, NHB_ERR_NCCL, std::string("ncclCommInitRank: ") + (nccl().GetErrorString ? nccl().GetErrorString(rc) : "error"));
	}
	return NHB_OK;
}

int nhb_symm_alloc(nhb_ctx* ctx, size_t bytes, void** out_dev) {
	if (!ctx || !out_dev || bytes == 0)
		return fail(ctx, NHB_ERR_ARG, "nhb_symm_alloc: bad arguments");
	*out_dev = nullptr;
	if (ctx->capturing)
		return fail(ctx, NHB_ERR_UNSUPPORTED, "allocation during graph capture");
	device_guard g(ctx->device);
	if (ctx->regions.empty()) {
		// first use: the flag array every rank writes into (region 0) and this rank's two counters
		nhb_ctx::symm_region ctl;
		int rc = symm_alloc_impl(ctx, 256, &ctl);
		if (rc != NHB_OK)
			return rc;
		cudaError_t e = cudaMalloc(&ctx->push_local, 256);
		if (e == cudaSuccess)
			e = cudaMemset(ctx->push_local, 0, 256);
		if (e != cudaSuccess) {
			symm_release(ctx, ctl);
			return fail_cuda(ctx, e, "nhb_symm_alloc: control block");
		}
		ctx->regions.reserve(64);
		ctx->regions.push_back(ctl);
	}
	nhb_ctx::symm_region reg;
	int rc = symm_alloc_impl(ctx, (bytes + 255) & ~size_t(255), &reg);
	if (rc != NHB_OK)
		return rc;
	ctx->regions.push_back(reg);
	*out_dev = reg.local;
	return NHB_OK;
}

// ---- one process driving several GPUs ----
static int check_group(nhb_ctx* const* ctxs, int n, const char* who) {
	if (!ctxs || n < 1 || n > NHB_MAX_WORLD)
		return fail(nullptr, NHB_ERR_ARG, std::string(who) + ": 1 to 8 contexts");
	for (int i = 0; i < n; ++i) {
		if (!ctxs[i])
			return fail(nullptr, NHB_ERR_ARG, std::string(who) + ": null context");
		if (ctxs[i]->world != n || ctxs[i]->rank != i)
			return fail(ctxs[i], NHB_ERR_ARG, std::string(who) + ": ctxs[i] must be rank i of a world of n");
		for (int j = 0; j < i; ++j)
			if (ctxs[j]->device == ctxs[i]->device)
				return fail(ctxs[i], NHB_ERR_ARG, std::string(who) + ": two contexts share a device");
	}
	return NHB_OK;
}

// the same allocation on every context's device, each context holding plain pointers to the others' (peer access)
static int symm_alloc_group(nhb_ctx* const* ctxs, int n, size_t bytes, nhb_ctx::symm_region* regs) {
	for (int i = 0; i < n; ++i)
		regs[i] = nhb_ctx::symm_region();
	cudaError_t e = cudaSuccess;
	for (int i = 0; i < n && e == cudaSuccess; ++i) {
		device_guard g(ctxs[i]->device);
		void* p = nullptr;
		e		= cudaMalloc(&p, bytes);
		if (e == cudaSuccess) {
			regs[i].local = static_cast<char*>(p);
			regs[i].bytes = bytes;
			regs[i].ipc	  = false;
			e			  = cudaMemsetAsync(p, 0, bytes, ctxs[i]->stream);
		}
		if (e == cudaSuccess)
			e = cudaStreamSynchronize(ctxs[i]->stream);
	}
	if (e != cudaSuccess) {
		for (int i = 0; i < n; ++i)
			if (regs[i].local) {
				device_guard g(ctxs[i]->device);
				cudaFree(regs[i].local);
			}
		return fail_cuda(ctxs[0], e, "nhb_symm_alloc_local");
	}
	for (int i = 0; i < n; ++i)
		for (int r = 0; r < n; ++r)
			regs[i].peer[r] = regs[r].local;
	return NHB_OK;
}

int nhb_symm_alloc_local(nhb_ctx* const* ctxs, int n, size_t bytes, void** out_dev) {
	int rc = check_group(ctxs, n, "nhb_symm_alloc_local");
	if (rc != NHB_OK)
		return rc;
	if (!out_dev || bytes == 0)
		return fail(ctxs[0], NHB_ERR_ARG, "nhb_symm_alloc_local: bad arguments");
	for (int i = 0; i < n; ++i) {
		out_dev[i] = nullptr;
		if (ctxs[i]->capturing)
			return fail(ctxs[i], NHB_ERR_UNSUPPORTED, "allocation during graph capture");
		if (ctxs[i]->regions.empty() != ctxs[0]->regions.empty())
			return fail(ctxs[i], NHB_ERR_ARG, "nhb_symm_alloc_local: the contexts must have made the same symmetric allocations so far");
	}
	// every device must be able to store into every other
	for (int i = 0; i < n; ++i) {
		device_guard g(ctxs[i]->device);
		for (int j = 0; j < n; ++j) {
			if (j == i)
				continue;
			int can = 0;
			cudaError_t e = cudaDeviceCanAccessPeer(&can, ctxs[i]->device, ctxs[j]->device);
			if (e != cudaSuccess || !can)
				return fail(ctxs[i], NHB_ERR_UNSUPPORTED, "nhb_symm_alloc_local: no peer access between the contexts' devices");
			e = cudaDeviceEnablePeerAccess(ctxs[j]->device, 0);
			if (e == cudaErrorPeerAccessAlreadyEnabled)
				cudaGetLastError();
			else if (e != cudaSuccess)
				return fail_cuda(ctxs[i], e, "cudaDeviceEnablePeerAccess");
		}
	}
	nhb_ctx::symm_region regs[NHB_MAX_WORLD];
	if (ctxs[0]->regions.empty()) {
		// first use: the flag array every rank writes into (region 0) and each rank's counters
		rc = symm_alloc_group(ctxs, n, 256, regs);
		if (rc != NHB_OK)
			return rc;
		for (int i = 0; i < n; ++i) {
			device_guard g(ctxs[i]->device);
			cudaError_t e = cudaMalloc(&ctxs[i]->push_local, 256);
			if (e == cudaSuccess)
				e = cudaMemset(ctxs[i]->push_local, 0, 256);
			if (e != cudaSuccess)
				return fail_cuda(ctxs[i], e, "nhb_symm_alloc_local: control block");
			ctxs[i]->regions.reserve(64);
			ctxs[i]->regions.push_back(regs[i]);
		}
	}
	rc = symm_alloc_group(ctxs, n, (bytes + 255) & ~size_t(255), regs);
	if (rc != NHB_OK)
		return rc;
	for (int i = 0; i < n; ++i) {
		ctxs[i]->regions.push_back(regs[i]);
		out_dev[i] = regs[i].local;
	}
	return NHB_OK;
}

int nhb_all_gather_local(nhb_ctx* const* ctxs, int n, float* const* y_dev, int64_t ldy, int64_t M, int64_t N) {
	int rc = check_group(ctxs, n, "nhb_all_gather_local");
	if (rc != NHB_OK)
		return rc;
	if (!y_dev || M < 0 || N < 0 || ldy < N)
		return fail(ctxs[0], NHB_ERR_ARG, "nhb_all_gather_local: bad arguments");
	if (n == 1 || M == 0 || N == 0)
		return NHB_OK;
	bool all_complete = true;
	for (int i = 0; i < n; ++i) {
		if (!y_dev[i])
			return fail(ctxs[i], NHB_ERR_ARG, "nhb_all_gather_local: null output");
		const auto& c = ctxs[i]->complete;
		all_complete  = all_complete && std::find(c.begin(), c.end(), static_cast<const void*>(y_dev[i])) != c.end();
	}
	if (all_complete) {
		// delivered by fused launches: whole once every rank's announcements are in
		for (int i = 0; i < n; ++i) {
			device_guard g(ctxs[i]->device);
			rc = wait_pending(ctxs[i]);
			if (rc != NHB_OK)
				return rc;
		}
		return NHB_OK;
	}
	// Peer copies of every rank's column slice into every other rank's buffer, on the owning rank's stream.  Two rounds of
	// events order them: no copy starts before every rank has finished what it had enqueued (its buffer may still be read),
	// and no rank goes on before every copy into its buffer has landed.
	for (int i = 0; i < n; ++i) {
		device_guard g(ctxs[i]->device);
		for (int k = 0; k < 2; ++k)
			if (!ctxs[i]->group_ev[k])
				NHB_CUDA(ctxs[i], cudaEventCreateWithFlags(&ctxs[i]->group_ev[k], cudaEventDisableTiming));
		NHB_CUDA(ctxs[i], cudaEventRecord(ctxs[i]->group_ev[0], ctxs[i]->stream));
	}
	for (int i = 0; i < n; ++i) {
		device_guard g(ctxs[i]->device);
		for (int j = 0; j < n; ++j)
			if (j != i)
				NHB_CUDA(ctxs[i], cudaStreamWaitEvent(ctxs[i]->stream, ctxs[j]->group_ev[0], 0));
		int64_t a, b;
		nhb_shard_rows(N, n, i, &a, &b);
		for (int j = 0; j < n && b > a; ++j)
			if (j != i)
				NHB_CUDA(ctxs[i], cudaMemcpy2DAsync(y_dev[j] + a, static_cast<size_t>(ldy) * sizeof(float), y_dev[i] + a, static_cast<size_t>(ldy) * sizeof(float),
										static_cast<size_t>(b - a) * sizeof(float), static_cast<size_t>(M), cudaMemcpyDeviceToDevice, ctxs[i]->stream));
		NHB_CUDA(ctxs[i], cudaEventRecord(ctxs[i]->group_ev[1], ctxs[i]->stream));
	}
	for (int i = 0; i < n; ++i) {
		device_guard g(ctxs[i]->device);
		for (int j = 0; j < n; ++j)
			if (j != i)
				NHB_CUDA(ctxs[i], cudaStreamWaitEvent(ctxs[i]->stream, ctxs[j]->group_ev[1], 0));
	}
	return NHB_OK;
}

int nhb_symm_free(nhb_ctx* ctx, void* dev) {
	if (!ctx)
		return fail(nullptr, NHB_ERR_ARG, "null context");
	if (!dev)
		return NHB_OK;
	device_guard g(ctx->device);
	for (size_t i = 1; i < ctx->regions.size(); ++i) {
		if (ctx->regions[i].local == dev) {
			NHB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
			symm_release(ctx, ctx->regions[i]);
			ctx->regions.erase(ctx->regions.begin() + static_cast<long>(i));
			return NHB_OK;
		}
	}
	return fail(ctx, NHB_ERR_ARG, "nhb_symm_free: not a pointer nhb_symm_alloc returned");
}

int nhb_all_gather_batch(nhb_ctx* ctx, float* const* y_dev, const int64_t* ldy, const int64_t* M, const int64_t* N, int n) {
	if (!ctx || n < 0 || (n > 0 && (!y_dev || !ldy || !M || !N)))
		return fail(ctx, NHB_ERR_ARG, "nhb_all_gather_batch: bad arguments");
	if (ctx->world == 1 || n == 0)
		return NHB_OK;
	device_guard g(ctx->device);
	// outputs a fused GEMV launch has already completed on every rank need no collective
	auto is_complete = [&](const void* y) { return std::find(ctx->complete.begin(), ctx->complete.end(), y) != ctx->complete.end(); };
	bool any_left = false, any_done = false;
	for (int i = 0; i < n; ++i) {
		any_left = any_left || !is_complete(y_dev[i]);
		any_done = any_done || is_complete(y_dev[i]);
	}
	if (any_done) {
		// delivered by a fused launch: whole once the other ranks' announcements are in (nothing to do for rows this rank
		// computed itself from a replicated weight, or when a later launch has already waited)
		int rc = wait_pending(ctx);
		if (rc != NHB_OK)
			return rc;
	}
	if (!any_left)
		return NHB_OK;
	if (!ctx->comm)
		return fail(ctx, NHB_ERR_NCCL, "nhb_comm_init has not been called (contexts of one process complete their rows with nhb_all_gather_local)");
	nccl_api& nc = nccl();
	int rc		 = nc.GroupStart();
	for (int i = 0; i < n && rc == nccl_success; ++i) {
		if (M[i] < 0 || N[i] < 0 || ldy[i] < N[i] || (M[i] > 0 && !y_dev[i])) {
			nc.GroupEnd();
			return fail(ctx, NHB_ERR_ARG, "nhb_all_gather_batch: bad entry");
		}
		if (is_complete(y_dev[i]))
			continue;
		const bool even = N[i] % ctx->world == 0;
		for (int64_t m = 0; m < M[i] && rc == nccl_success; ++m) {
			float* row = y_dev[i] + m * ldy[i];
			if (even) {
				const int64_t cnt = N[i] / ctx->world;
				rc				  = nc.AllGather(row + ctx->rank * cnt, row, static_cast<size_t>(cnt), nccl_float, ctx->comm, ctx->stream);
			} else {
				for (int r = 0; r < ctx->world && rc == nccl_success; ++r) {
					int64_t a, b;
					nhb_shard_rows(N[i], ctx->world, r, &a, &b);
					if (b > a)
						rc = nc.Broadcast(row + a, row + a, static_cast<size_t>(b - a), nccl_float, r, ctx->comm, ctx->stream);
				}
			}
		}
	}
	int rc2 = nc.GroupEnd();
	if (rc == nccl_success)
		rc = rc2;
	if (rc != nccl_success)
		return fail(ctx, NHB_ERR_NCCL, std::string("all-gather: ") + (nc.GetErrorString ? nc.GetErrorString(rc) : "error"));
	ctx->launches += 1;
	return NHB_OK;
}

int nhb_all_gather(nhb_ctx* ctx, float* y_dev, int64_t ldy, int64_t M, int64_t N) {
	return nhb_all_gather_batch(ctx, &y_dev, &ldy, &M, &N, 1);
}
}
