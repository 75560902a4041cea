// Device code shared by the decode GEMV kernels (gemv_rows.cu): the activation prologue that every CTA
// runs (quantize_row_q8_0 of the reference, include/nihilus-incl/cpu/avx_2.hpp:4439-4489, optionally behind the
// rms_norm x norm-weight producer) and the two halves of the fused all-gather: announcing a finished launch to
// the other ranks, and waiting for theirs before activations are read.
#pragma once
#include "internal.h"
#include "ptx.cuh"
#include "q8_device.cuh"

namespace nhb {

	__device__ __forceinline__ int rows_find_op(const rows_batch& b, int row, int cur) {
		while (cur + 1 < b.n_ops && row >= b.op[cur + 1].row_begin)
			++cur;
		return cur;
	}

	// barrier over the first `nthreads` threads of the CTA (a multiple of 32); id 0 is the CTA-wide barrier
	__device__ __forceinline__ void group_sync(int bar_id, int nthreads) {
		if (bar_id == 0)
			__syncthreads();
		else
			asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
	}

	// activations another SM may have written earlier in this same kernel must not come from this SM's L1
	template<bool COHERENT> __device__ __forceinline__ float4 ld_act4(const float4* p) {
		if constexpr (COHERENT)
			return __ldcg(p);
		else
			return __ldg(p);
	}

	// Prologue of the GEMV kernels: quantise every distinct input of the batch into shared memory.  Run by `nthreads` threads
	// (tid 0 .. nthreads-1) that meet at named barrier `bar_id` (0: the whole CTA).  COHERENT: read the activations past L1.
	// SWIGLU: honour rows_op::x2 (the activation is silu(x) * x2).
	// Layout of one input, per row m: the first 16 bytes of every block (uint4 [nb]), then the second 16 bytes
	// (uint4 [nb]) -- two planes, so that a warp reading one block per lane touches consecutive 16-byte words (no bank
	// conflicts) -- and after all MT rows the f32 scales [MT][nb].
	template<int MT, bool NORM = false, bool COHERENT = false, bool SWIGLU = false> __device__ __forceinline__ void quantize_inputs(const rows_batch& b, unsigned char* act_smem, int tid, int nthreads, int bar_id = 0) {
		const uint32_t cn = cluster_size();
		const uint32_t cr = cluster_rank();
		for (int s = 0; s < b.n_slots; ++s) {
			const rows_op* op  = &b.op[b.slot_op[s]];
			unsigned char* act = act_smem + op->act_off;
			const int K		   = op->K;
			const int nb	   = K >> 5;
			float* sda		   = reinterpret_cast<float*>(act + static_cast<size_t>(MT) * K);
			if constexpr (NORM) {
				// rms_norm x norm-weight in front of the quantiser (rms_norm.cu has the arithmetic and its source):
				// the rows are staged as f32, eight lanes per row run the sum-of-squares chains -- K / 8 dependent fma
				// steps, which overlap the weight loads this CTA issued before it waited for the previous kernel -- and
				// the quantiser below then reads (x * w) * scale instead of x.  Every CTA does this for itself: the
				// rows are a few KB out of L2 and a separate kernel would put its launch on the critical path.
				const int KS   = K + 8;// row stride: the MT chains of a step hit different banks
				float* rows	   = reinterpret_cast<float*>(act_smem + b.norm_off);
				float* prod	   = rows + MT * KS;// x * w, formed while the row is staged, so nothing is fetched after the chains
				float* s_scale = prod + MT * KS;
				const int k4   = K >> 2;
				for (int i = tid; i < MT * k4; i += nthreads) {
					const int m		= i / k4;
					const int j		= i - m * k4;
					const float4 xv = ld_act4<COHERENT>(reinterpret_cast<const float4*>(op->x + static_cast<size_t>(m) * op->ldx) + j);
					const float4 wv = __ldg(reinterpret_cast<const float4*>(b.norm_w) + j);
					reinterpret_cast<float4*>(rows + m * KS)[j] = xv;
					reinterpret_cast<float4*>(prod + m * KS)[j] =
						make_float4(__fmul_rn(xv.x, wv.x), __fmul_rn(xv.y, wv.y), __fmul_rn(xv.z, wv.z), __fmul_rn(xv.w, wv.w));
				}
				group_sync(bar_id, nthreads);
				if (tid < 8 * MT) {
					constexpr unsigned mask = MT >= 4 ? 0xffffffffu : ((1u << (8 * MT)) - 1u);
					const float acc			= sum_squares_lane(rows + (tid >> 3) * KS + (tid & 7), K >> 3);
					const float quad = __fadd_rn(acc, __shfl_down_sync(mask, acc, 4, 8));
					const float dual = __fadd_rn(quad, __shfl_down_sync(mask, quad, 2, 8));
					const float sum	 = __fadd_rn(dual, __shfl_down_sync(mask, dual, 1, 8));
					if ((tid & 7) == 0) {
						const float v = __fadd_rn(__fdiv_rn(sum, static_cast<float>(K)), b.norm_eps);
						const float root =
							b.norm_sqrt == NHB_SQRT_X86_FAST ? __uint_as_float(((__float_as_uint(v) + 0x3f800000u) >> 1) + 0x20000000u) : __fsqrt_rn(v);
						s_scale[tid >> 3] = __fdiv_rn(1.0f, root);
					}
				}
				group_sync(bar_id, nthreads);
				const int n = MT * nb * 2;// quantiser work items: half a block (16 values) each
				for (int i = tid; i < n; i += nthreads) {
					const int hb	 = i >> 1;
					const int m		 = hb / nb;
					const int blk	 = hb - m * nb;
					const float sc_n = s_scale[m];
					const float4* p	 = reinterpret_cast<const float4*>(prod + m * KS + blk * QK) + (i & 1) * 4;
					float4 v[4];
#pragma unroll
					for (int j = 0; j < 4; ++j) {
						const float4 t = p[j];
						v[j]		   = make_float4(__fmul_rn(t.x, sc_n), __fmul_rn(t.y, sc_n), __fmul_rn(t.z, sc_n), __fmul_rn(t.w, sc_n));
					}
					float amax		   = absmax4(v[0], absmax4(v[1], absmax4(v[2], absmax4(v[3], 0.f))));
					amax			   = fmaxf(amax, __shfl_xor_sync(__activemask(), amax, 1));
					const act_scale sc = q8_scales(amax);
					reinterpret_cast<uint4*>(act + static_cast<size_t>(m) * K)[(i & 1) * nb + blk] =
						make_uint4(q8_pack4(v[0].x, v[0].y, v[0].z, v[0].w, sc.id), q8_pack4(v[1].x, v[1].y, v[1].z, v[1].w, sc.id),
							q8_pack4(v[2].x, v[2].y, v[2].z, v[2].w, sc.id), q8_pack4(v[3].x, v[3].y, v[3].z, v[3].w, sc.id));
					if ((i & 1) == 0)
						sda[hb] = sc.d;
				}
				group_sync(bar_id, nthreads);// the staged rows are reused by the next slot
			} else
			if (b.preq) {
				// quantised by quantize_q8_kernel into global scratch: int8 [MT][K] then f32 [MT][nb]
				const unsigned char* src = b.preq_base + op->preq_off;
				for (int i = tid; i < MT * nb * 2; i += nthreads) {
					const int hb  = i >> 1;
					const int m	  = hb / nb;
					const int blk = hb - m * nb;
					reinterpret_cast<uint4*>(act + static_cast<size_t>(m) * K)[(i & 1) * nb + blk] = __ldg(reinterpret_cast<const uint4*>(src) + i);
				}
				const float* sd = reinterpret_cast<const float*>(src + static_cast<size_t>(MT) * K);
				for (int i = tid; i < MT * nb; i += nthreads)
					sda[i] = __ldg(sd + i);
			} else {
				// two threads per 32-wide block (16 floats each); the pair shares its absmax by shuffle.  In a cluster
				// launch every CTA quantises 1/cn of the input and writes it into the shared memory of all cn CTAs.
				const float* x		= op->x;
				const long long ldx = op->ldx;
				const int n			= MT * nb * 2;
				const int per		= ((n / 2 + static_cast<int>(cn) - 1) / static_cast<int>(cn)) * 2;
				const int i_begin	= static_cast<int>(cr) * per;
				const int i_end		= min(n, i_begin + per);
				for (int i = i_begin + tid; i < i_end; i += nthreads) {
					const int hb	= i >> 1;
					const int m		= hb / nb;
					const int blk	= hb - m * nb;
					const size_t at = static_cast<size_t>(m) * ldx + static_cast<size_t>(blk) * QK + (i & 1) * 16;
					const float4* p = reinterpret_cast<const float4*>(x + at);
					float4 v0 = ld_act4<COHERENT>(p), v1 = ld_act4<COHERENT>(p + 1), v2 = ld_act4<COHERENT>(p + 2), v3 = ld_act4<COHERENT>(p + 3);
					if constexpr (SWIGLU) {
						if (op->x2) {// SwiGLU in front of the quantiser: x holds the gate projection's rows, x2 the up projection's
							const float4* u = reinterpret_cast<const float4*>(op->x2 + at);
							v0				= swiglu4(v0, ld_act4<COHERENT>(u));
							v1				= swiglu4(v1, ld_act4<COHERENT>(u + 1));
							v2				= swiglu4(v2, ld_act4<COHERENT>(u + 2));
							v3				= swiglu4(v3, ld_act4<COHERENT>(u + 3));
						}
					}
					float amax		= absmax4(v0, absmax4(v1, absmax4(v2, absmax4(v3, 0.f))));
					amax			= fmaxf(amax, __shfl_xor_sync(__activemask(), amax, 1));
					const act_scale sc = q8_scales(amax);
					const uint4 qv	   = make_uint4(q8_pack4(v0.x, v0.y, v0.z, v0.w, sc.id), q8_pack4(v1.x, v1.y, v1.z, v1.w, sc.id),
						   q8_pack4(v2.x, v2.y, v2.z, v2.w, sc.id), q8_pack4(v3.x, v3.y, v3.z, v3.w, sc.id));
					uint4* dst		   = reinterpret_cast<uint4*>(act + static_cast<size_t>(m) * K) + ((i & 1) * nb + blk);
					if (cn == 1) {
						*dst = qv;
						if ((i & 1) == 0)
							sda[hb] = sc.d;
					} else {
						const uint32_t a_q = smem_u32(dst);
						const uint32_t a_d = smem_u32(sda + hb);
						for (uint32_t r = 0; r < cn; ++r) {
							cluster_st_v4(cluster_map(a_q, r), qv);
							if ((i & 1) == 0)
								cluster_st_f32(cluster_map(a_d, r), sc.d);
						}
					}
				}
			}
		}
		// everyone's activations are complete (own writes and, in a cluster, the peers' remote stores)
		if (cn == 1)
			group_sync(bar_id, nthreads);
		else
			cluster_barrier();
	}

	__device__ __forceinline__ void st_relaxed_sys(unsigned* p, unsigned v) {
		asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
	}
	__device__ __forceinline__ unsigned ld_relaxed_sys(const unsigned* p) {
		unsigned v;
		asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
		return v;
	}
	__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
		unsigned v;
		asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
		return v;
	}
	__device__ __forceinline__ unsigned long long global_timer_ns() {
		unsigned long long t;
		asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
		return t;
	}

	// End of a launch that delivered its rows to the other ranks: the CTAs count themselves done and the last one bumps
	// this rank's count of completed delivering launches.  No fence and no announcement here -- a fence at this point
	// would have every CTA wait for its NVLink stores to be acknowledged before the kernel may end.  The kernel boundary
	// orders the stores; the next launch of the context announces them (push_publish).
	__device__ __forceinline__ void push_done(const push_ctl& pc, int tid) {
		__syncthreads();
		if (tid != 0)
			return;
		const unsigned prev = atomicAdd(pc.done_ctas, 1u);
		if (prev != gridDim.x * gridDim.y * gridDim.z - 1)
			return;
		*reinterpret_cast<volatile unsigned*>(pc.done_ctas) = 0u;
		*reinterpret_cast<volatile unsigned*>(pc.epoch)	   = *reinterpret_cast<volatile unsigned*>(pc.epoch) + 1u;
	}

	// Start of every launch of a context that shares outputs with other ranks, after the wait for the previous kernels of
	// this stream (whose stores, the ones that crossed NVLink included, are then complete): one thread tells every rank
	// "this rank has finished delivering launch number e" if that is news.  The system-scope fence orders those kernels'
	// stores before the flag stores for every observer.
	__device__ __forceinline__ void push_publish(const push_ctl& pc, int tid) {
		if (pc.peers > 1 && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
			const unsigned e = *reinterpret_cast<volatile unsigned*>(pc.epoch);
			if (*reinterpret_cast<volatile unsigned*>(pc.announced) != e) {
				asm volatile("fence.acq_rel.sys;" ::: "memory");
				for (int r = 0; r < pc.peers; ++r)
					st_relaxed_sys(pc.flags_peer[r] + pc.rank, e);
				*reinterpret_cast<volatile unsigned*>(pc.announced) = e;
			}
		}
	}

	// Then the launch waits for the peers as far as the host found it must (plan_peer_wait): until every rank has announced
	// delivering launch number (this rank's completed count - wait_lag).  One thread per CTA polls this rank's own flag
	// array (local memory, written by the peers) for at most wait_ns nanoseconds, then records DEV_TIMEOUT_PEER and carries
	// on, so that the kernel always ends and the host learns of it from nhb_sync.  A rank announces before it waits, and an
	// announcement only depends on that rank's own earlier kernels, so ranks cannot wait on each other in a cycle.  Called
	// by the `nthreads` threads that go on to read the activations; ends with their barrier (group_sync).
	__device__ __forceinline__ void push_wait_peers(const push_ctl& pc, int tid, int nthreads = 0, int bar_id = 0) {
		push_publish(pc, tid);
		if (pc.wait_world > 1) {
			if (tid < 32) {
				// lane r watches rank r's flag: one round trip to L2 for all peers together when the flags are already there
				const unsigned e = *reinterpret_cast<volatile unsigned*>(pc.epoch) - static_cast<unsigned>(pc.wait_lag);
				bool ok			 = true;
				if (tid < pc.wait_world && tid != pc.rank) {
					const unsigned* flag = pc.flags_local + tid;
					if (static_cast<int>(ld_acquire_sys(flag) - e) < 0) {
						const unsigned long long t0 = global_timer_ns();
						for (;;) {
							if (static_cast<int>(ld_relaxed_sys(flag) - e) >= 0) {
								ok = static_cast<int>(ld_acquire_sys(flag) - e) >= 0;
								break;
							}
							__nanosleep(20);
							if (global_timer_ns() - t0 > pc.wait_ns) {
								ok = false;
								break;
							}
						}
					}
				}
				if (!__all_sync(0xffffffffu, ok) && tid == 0)
					atomicExch(pc.status, DEV_TIMEOUT_PEER);
			}
			group_sync(bar_id, nthreads);
		}
	}

}
