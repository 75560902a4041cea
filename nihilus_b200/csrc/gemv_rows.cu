// gemv_q8_rows: the decode GEMV (sm_100a).  One warp per weight row, 256-bit coalesced loads of the int8
// plane, packed int8 dot products (dp4a) against Q8_0-quantised activations staged in shared memory,
// warp-shuffle reduction.  Several independent mul_mats (q/k/v, gate/up) run in one launch.
//
// Built for back-to-back launches: every warp issues the loads of its first weight rows BEFORE it waits for
// the previous kernel (programmatic dependent launch) -- weights never depend on an earlier kernel, the
// activations do -- so the weight stream of launch i+1 overlaps the tail of launch i.
//
// Arithmetic: quantize_row_q8_0 + vec_dot_q8_0_q8_0 of the reference (include/nihilus-incl/cpu/avx_2.hpp
// :4439-4489, :4749-4780); per 32-wide block  acc = fma(float(exact int32 block dot), d_w * d_a, acc).  The
// summation order depends on K only, so any row sharding gives bit-identical outputs.
#include <algorithm>

#include "internal.h"
#include "ptx.cuh"
#include "q8_device.cuh"

namespace nhb {

	namespace {

		// Two CTA shapes.  Wide launches use one CTA of 24 warps per SM: the activations are quantised once per SM
		// instead of three times.  Launches with too few rows for that keep 8-warp CTAs, several per SM.
		constexpr int ROWS_WARPS	 = 8;
		constexpr int ROWS_TPB		 = ROWS_WARPS * 32;
		constexpr int ROWS_WARPS_FAT = 24;
		constexpr int ROWS_TPB_FAT	 = ROWS_WARPS_FAT * 32;
		constexpr int ITEM		 = 4;// 32-byte Q8 blocks per lane per step: 4 KB of a row per warp

		__device__ __forceinline__ int rows_find_op(const rows_batch& b, int row, int cur) {
			while (cur + 1 < b.n_ops && row >= b.op[cur + 1].row_begin)
				++cur;
			return cur;
		}

		struct blk32 {
			uint4 lo, hi;
		};

		// one whole 32-byte block per lane: 256-bit load, streamed past L1, first to leave L2
		__device__ __forceinline__ blk32 ldg_block(const void* p) {
			blk32 v;
			asm("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
						 : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x), "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
						 : "l"(p));
			return v;
		}

		struct item_regs {
			blk32 w[ITEM];
			uint16_t d[ITEM];
		};

		// everything a warp needs to stream one weight row, held in registers
		struct row_desc {
			const int8_t* wrow;
			const uint16_t* drow;
			int nb;
		};

		__device__ __forceinline__ row_desc make_row(const rows_op* op, int lrow) {
			row_desc r;
			const int K = op->K;
			r.nb		= K >> 5;
			r.wrow		= op->wq + static_cast<size_t>(lrow) * K;
			r.drow		= reinterpret_cast<const uint16_t*>(op->wd) + static_cast<size_t>(lrow) * r.nb;
			return r;
		}

		// blocks b0 + lane + 32*i of the row
		__device__ __forceinline__ void load_item(item_regs& r, const row_desc rd, int b0, int lane) {
#pragma unroll
			for (int i = 0; i < ITEM; ++i) {
				const int blk = b0 + lane + 32 * i;
				if (blk < rd.nb) {
					r.w[i] = ldg_block(rd.wrow + static_cast<size_t>(blk) * QK);
					r.d[i] = __ldg(rd.drow + blk);
				}
			}
		}

		// Activations of one input in shared memory, per row m: the first 16 bytes of every block (uint4 [nb]), then the
		// second 16 bytes (uint4 [nb]) -- two planes, so that a warp reading one block per lane touches consecutive
		// 16-byte words (no bank conflicts) -- and after all MT rows the f32 scales [MT][nb].
#ifdef NHB_ROWS_PROF
		__device__ unsigned long long rows_prof[8];
		__device__ __forceinline__ unsigned long long gtimer() {
			unsigned long long t;
			asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
			return t;
		}
#define ROWS_STAMP(i) \
	if (blockIdx.x == 0 && threadIdx.x == 0) \
	rows_prof[i] = gtimer()
#else
#define ROWS_STAMP(i)
#endif
		template<int MT> __device__ __forceinline__ void compute_item(const item_regs& r, float (&acc)[MT], const unsigned char* act, int nb, int b0, int lane) {
			const float* da = reinterpret_cast<const float*>(act + static_cast<size_t>(MT) * nb * QK);
#pragma unroll
			for (int i = 0; i < ITEM; ++i) {
				const int blk = b0 + lane + 32 * i;
				if (blk < nb) {
					const float dw = __half2float(__ushort_as_half(r.d[i]));
#pragma unroll
					for (int m = 0; m < MT; ++m) {
						const uint4* lo = reinterpret_cast<const uint4*>(act + static_cast<size_t>(m) * nb * QK);
						// copy to registers first: a reference into shared memory would be read word by word
						const uint4 a0 = lo[blk];
						const uint4 a1 = lo[nb + blk];
						const int sumi = dot16(r.w[i].lo, a0) + dot16(r.w[i].hi, a1);// the exact block dot
						acc[m]		   = fmaf(static_cast<float>(sumi), dw * da[m * nb + blk], acc[m]);
					}
				}
			}
		}

		// f32-activation arithmetic (vec_dot_q8_f32, include/nihilus-incl/cpu/avx_2.hpp:4782-4852): per block
		// s = sum_j x_j * float(q_j), acc += s * d_w.  Activations sit in shared memory as float4 [MT][8][nb]: chunk c of
		// block blk at (c * nb + blk), so a warp reading one block per lane touches consecutive 16-byte words.
		template<int MT> __device__ __forceinline__ void compute_item_f32(const item_regs& r, float (&acc)[MT], const unsigned char* act, int nb, int b0, int lane) {
#pragma unroll
			for (int i = 0; i < ITEM; ++i) {
				const int blk = b0 + lane + 32 * i;
				if (blk < nb) {
					const float dw		= __half2float(__ushort_as_half(r.d[i]));
					const uint32_t w[8] = { r.w[i].lo.x, r.w[i].lo.y, r.w[i].lo.z, r.w[i].lo.w, r.w[i].hi.x, r.w[i].hi.y, r.w[i].hi.z, r.w[i].hi.w };
#pragma unroll
					for (int m = 0; m < MT; ++m) {
						const float4* xs = reinterpret_cast<const float4*>(act) + static_cast<size_t>(m) * 8 * nb;
						float s0 = 0.f, s1 = 0.f;// two chains: the 32 fmas of a block would otherwise be one dependent run
#pragma unroll
						for (int c = 0; c < 8; ++c) {
							const float4 xv = xs[c * nb + blk];
							const int q0 = static_cast<int8_t>(w[c] & 0xff), q1 = static_cast<int8_t>((w[c] >> 8) & 0xff);
							const int q2 = static_cast<int8_t>((w[c] >> 16) & 0xff), q3 = static_cast<int8_t>(w[c] >> 24);
							s0 = fmaf(xv.x, static_cast<float>(q0), s0);
							s1 = fmaf(xv.y, static_cast<float>(q1), s1);
							s0 = fmaf(xv.z, static_cast<float>(q2), s0);
							s1 = fmaf(xv.w, static_cast<float>(q3), s1);
						}
						acc[m] = fmaf(s0 + s1, dw, acc[m]);
					}
				}
			}
		}

		// Prologue of the f32-activation mode: copy every distinct input into shared memory in the chunk-major layout above.
		template<int MT> __device__ __forceinline__ void stage_inputs_f32(const rows_batch& b, unsigned char* act_smem, int tid) {
			for (int s = 0; s < b.n_slots; ++s) {
				const rows_op* op = &b.op[b.slot_op[s]];
				float4* dst		  = reinterpret_cast<float4*>(act_smem + op->act_off);
				const int nb	  = op->K >> 5;
				for (int i = tid; i < MT * nb * 8; i += static_cast<int>(blockDim.x)) {
					const int m	  = i / (nb * 8);
					const int j	  = i - m * nb * 8;// float4 index inside the row: block j / 8, chunk j % 8
					const float4 v = __ldg(reinterpret_cast<const float4*>(op->x + static_cast<size_t>(m) * op->ldx) + j);
					dst[static_cast<size_t>(m) * 8 * nb + (j & 7) * nb + (j >> 3)] = v;
				}
			}
			__syncthreads();
		}

		// Prologue of both GEMV variants: quantise every distinct input of the batch into shared memory.
		template<int MT, bool NORM = false> __device__ __forceinline__ void quantize_inputs(const rows_batch& b, unsigned char* act_smem, int tid) {
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
				for (int i = tid; i < MT * k4; i += static_cast<int>(blockDim.x)) {
					const int m		= i / k4;
					const int j		= i - m * k4;
					const float4 xv = __ldg(reinterpret_cast<const float4*>(op->x + static_cast<size_t>(m) * op->ldx) + j);
					const float4 wv = __ldg(reinterpret_cast<const float4*>(b.norm_w) + j);
					reinterpret_cast<float4*>(rows + m * KS)[j] = xv;
					reinterpret_cast<float4*>(prod + m * KS)[j] =
						make_float4(__fmul_rn(xv.x, wv.x), __fmul_rn(xv.y, wv.y), __fmul_rn(xv.z, wv.z), __fmul_rn(xv.w, wv.w));
				}
				__syncthreads();
				ROWS_STAMP(2);
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
				ROWS_STAMP(3);
				__syncthreads();
				const int n = MT * nb * 2;// quantiser work items: half a block (16 values) each
				for (int i = tid; i < n; i += static_cast<int>(blockDim.x)) {
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
				__syncthreads();// the staged rows are reused by the next slot
			} else
			if (b.preq) {
				// quantised by quantize_q8_kernel into global scratch: int8 [MT][K] then f32 [MT][nb]
				const unsigned char* src = b.preq_base + op->preq_off;
				for (int i = tid; i < MT * nb * 2; i += static_cast<int>(blockDim.x)) {
					const int hb  = i >> 1;
					const int m	  = hb / nb;
					const int blk = hb - m * nb;
					reinterpret_cast<uint4*>(act + static_cast<size_t>(m) * K)[(i & 1) * nb + blk] = __ldg(reinterpret_cast<const uint4*>(src) + i);
				}
				const float* sd = reinterpret_cast<const float*>(src + static_cast<size_t>(MT) * K);
				for (int i = tid; i < MT * nb; i += static_cast<int>(blockDim.x))
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
				for (int i = i_begin + tid; i < i_end; i += static_cast<int>(blockDim.x)) {
					const int hb	= i >> 1;
					const int m		= hb / nb;
					const int blk	= hb - m * nb;
					const float4* p = reinterpret_cast<const float4*>(x + static_cast<size_t>(m) * ldx + static_cast<size_t>(blk) * QK) + (i & 1) * 4;
					const float4 v0 = __ldg(p), v1 = __ldg(p + 1), v2 = __ldg(p + 2), v3 = __ldg(p + 3);
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
			__syncthreads();
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

		// End of a fused launch.  Every CTA orders its stores (CTA barrier, then a device-scope fence by thread 0) and
		// counts itself done; the last one issues the launch's single system-scope fence, tells every rank "this rank
		// has finished launch number e" and then waits, for a bounded time, until all ranks have said the same.
		// System-scope fences wait for the stores that crossed NVLink to be acknowledged, so there is exactly one on the
		// critical path; the polls are relaxed loads and one acquire load closes the wait.  Nothing here waits on a CTA
		// of this grid that has not run yet, and a peer's flag only depends on that peer's own kernel, so ranks cannot
		// wait on each other in a cycle.
		__device__ __forceinline__ void push_finish(const push_ctl& pc, int tid) {
			__syncthreads();
			if (tid != 0)
				return;
			asm volatile("fence.acq_rel.gpu;" ::: "memory");
			const unsigned prev = atomicAdd(pc.done_ctas, 1u);
			if (prev != gridDim.x - 1)
				return;
			asm volatile("fence.acq_rel.sys;" ::: "memory");
			const unsigned e = *reinterpret_cast<volatile unsigned*>(pc.epoch) + 1u;
			for (int r = 0; r < pc.world; ++r)
				st_relaxed_sys(pc.flags_peer[r] + pc.rank, e);
			bool ok = true;
			for (int r = 0; r < pc.world && ok; ++r) {
				ok = false;
				for (uint32_t i = 0; i < NHB_SPIN_LIMIT; ++i) {
					if (static_cast<int>(ld_relaxed_sys(pc.flags_local + r) - e) >= 0) {
						ok = static_cast<int>(ld_acquire_sys(pc.flags_local + r) - e) >= 0;
						break;
					}
					if (i > 4096)
						__nanosleep(20);
				}
			}
			*reinterpret_cast<volatile unsigned*>(pc.done_ctas) = 0u;
			*reinterpret_cast<volatile unsigned*>(pc.epoch)	   = e;
			if (!ok)
				atomicExch(pc.status, DEV_TIMEOUT_PEER);
		}

		// NORM: the rms_norm x norm-weight producer runs inside the prologue (its own instantiation, so that the plain
		// kernels keep their register allocation)
		template<int MT, int OCC, int TPB = ROWS_TPB, bool F32 = false, bool NORM = false> __global__ void __launch_bounds__(TPB, OCC)
			gemv_q8_rows(const __grid_constant__ rows_batch b) {
			constexpr int WARPS = TPB / 32;
			extern __shared__ __align__(128) unsigned char act_smem[];
			const int tid		 = threadIdx.x;
			const int lane		 = tid & 31;
			const int warp		 = tid >> 5;
			const int W			 = gridDim.x * WARPS;
			const int row0		 = blockIdx.x * WARPS + warp;
			const int total_rows = b.total_rows;
			const int n_ops		 = b.n_ops;
			int cur				 = 0;
			bool pre			 = false;
			item_regs regs;
			// ---- weights first: they never depend on the previous kernel ----
			if (row0 < total_rows) {
				cur = rows_find_op(b, row0, 0);
				load_item(regs, make_row(&b.op[cur], row0 - b.op[cur].row_begin), 0, lane);
				pre = true;
			}
			ROWS_STAMP(0);
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			ROWS_STAMP(1);
			if constexpr (F32)
				stage_inputs_f32<MT>(b, act_smem, tid);
			else
				quantize_inputs<MT, NORM>(b, act_smem, tid);
			ROWS_STAMP(4);
			// ---- rows ----
			for (int row = row0; row < total_rows; row += W) {
				while (cur + 1 < n_ops && row >= b.op[cur + 1].row_begin)
					++cur;
				const rows_op* op		 = &b.op[cur];
				const int lrow			 = row - op->row_begin;
				const row_desc rd		 = make_row(op, lrow);
				const unsigned char* act = act_smem + op->act_off;
				float* const yrow		 = op->y + lrow;
				const long long ldy		 = op->ldy;
				// A row's value is the sum, in ascending order, of its 4 KB items' totals; an item's total is the warp
				// reduction of the lanes' partial sums.  (One item per row for K = 4096.)  Every kernel of this file sums
				// in this order, so which warp computes which item never shows in the result.
				float rowacc[MT];
#pragma unroll
				for (int m = 0; m < MT; ++m)
					rowacc[m] = 0.f;
				for (int b0 = 0; b0 < rd.nb; b0 += 32 * ITEM) {
					if (!pre)
						load_item(regs, rd, b0, lane);
					pre = false;
					float acc[MT];
#pragma unroll
					for (int m = 0; m < MT; ++m)
						acc[m] = 0.f;
					if constexpr (F32)
						compute_item_f32<MT>(regs, acc, act, rd.nb, b0, lane);
					else
						compute_item<MT>(regs, acc, act, rd.nb, b0, lane);
#pragma unroll
					for (int m = 0; m < MT; ++m)
						rowacc[m] += warp_sum(acc[m]);
				}
				if (lane == 0) {
#pragma unroll
					for (int m = 0; m < MT; ++m)
						yrow[static_cast<size_t>(m) * ldy] = rowacc[m];
				}
			}
			ROWS_STAMP(5);
			if (b.push.world > 1) {
				// Fused all-gather.  In pass i the warps of this CTA finished WARPS consecutive rows; once they are all
				// written (CTA barrier) one warp per pass copies that run to every other rank in one coalesced store per
				// rank and token, instead of one 4-byte store across NVLink per row.
				__syncthreads();
				int pcur = 0;
				for (int base = blockIdx.x * WARPS + warp * W; base < total_rows; base += WARPS * W) {
					const int row = base + lane;
					if (lane < WARPS && row < total_rows) {
						pcur			   = rows_find_op(b, row, pcur);
						const rows_op* op  = &b.op[pcur];
						const int lrow	   = row - op->row_begin;
						const long long ld = op->ldy;
#pragma unroll
						for (int m = 0; m < MT; ++m) {
							const float v = __ldcg(op->y + static_cast<size_t>(m) * ld + lrow);
							for (int r = 0; r < b.push.world; ++r)
								if (r != b.push.rank && b.y_peer[pcur][r])
									b.y_peer[pcur][r][static_cast<size_t>(m) * ld + lrow] = v;
						}
					}
				}
				push_finish(b.push, tid);
			}
		}


		// ---- item-parallel variant for long rows (K > 4096) ----
		// With one warp per row a 14336-wide row is four 4 KB items fetched one after the other, and 4096 such rows leave
		// most warps with one or two of these chains: the kernel is bound by that chain, not by bandwidth.  Here a CTA
		// owns a contiguous run of rows (every SM gets the same share) and deals their items to its 24 warps, so the
		// items of one row are in flight in different warps at the same time; item totals meet in shared memory and are
		// added per row in ascending order -- the same order, hence the same bits, as the one-warp-per-row kernels.
		// All ops of the launch must share K.
		constexpr int SPLIT_MAX_ROWS = 64;// rows per CTA the partial-sum array is sized for
		template<int MT, bool F32 = false> __global__ void __launch_bounds__(ROWS_TPB_FAT, 1) gemv_q8_rows_split(const __grid_constant__ rows_batch b) {
			constexpr int WARPS = ROWS_WARPS_FAT;
			extern __shared__ __align__(128) unsigned char act_smem[];
			__shared__ float part[SPLIT_MAX_ROWS * 8 * MT];// [row][item][m]
			const int tid		 = threadIdx.x;
			const int lane		 = tid & 31;
			const int warp		 = tid >> 5;
			const int total_rows = b.total_rows;
			const int nb		 = b.op[0].K >> 5;
			const int ipr		 = (nb + 32 * ITEM - 1) / (32 * ITEM);// items per row
			// this CTA's rows: an even contiguous split of the batch-wide row list
			const int r_lo	  = static_cast<int>(static_cast<long long>(total_rows) * blockIdx.x / gridDim.x);
			const int r_hi	  = static_cast<int>(static_cast<long long>(total_rows) * (blockIdx.x + 1) / gridDim.x);
			const int n_items = (r_hi - r_lo) * ipr;
			item_regs regs;
			bool pre = false;
			int cur	 = 0;
			// ---- weights first: they never depend on the previous kernel ----
			if (warp < n_items) {
				const int row = r_lo + warp / ipr;
				cur			  = rows_find_op(b, row, 0);
				load_item(regs, make_row(&b.op[cur], row - b.op[cur].row_begin), (warp % ipr) * 32 * ITEM, lane);
				pre = true;
			}
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			if constexpr (F32)
				stage_inputs_f32<MT>(b, act_smem, tid);
			else
				quantize_inputs<MT>(b, act_smem, tid);
			for (int it = warp; it < n_items; it += WARPS) {
				const int rl  = it / ipr;
				const int b0  = (it - rl * ipr) * 32 * ITEM;
				const int row = r_lo + rl;
				cur			  = rows_find_op(b, row, cur);
				const rows_op* op = &b.op[cur];
				const row_desc rd = make_row(op, row - op->row_begin);
				if (!pre)
					load_item(regs, rd, b0, lane);
				pre = false;
				float acc[MT];
#pragma unroll
				for (int m = 0; m < MT; ++m)
					acc[m] = 0.f;
				if constexpr (F32)
					compute_item_f32<MT>(regs, acc, act_smem + op->act_off, rd.nb, b0, lane);
				else
					compute_item<MT>(regs, acc, act_smem + op->act_off, rd.nb, b0, lane);
#pragma unroll
				for (int m = 0; m < MT; ++m) {
					const float v = warp_sum(acc[m]);
					if (lane == 0)
						part[(rl * 8 + (it - rl * ipr)) * MT + m] = v;
				}
			}
			__syncthreads();
			// one thread per (row, token): item totals in ascending order, store, and in a fused launch the peers' copies
			int ocur = 0;
			for (int i = tid; i < (r_hi - r_lo) * MT; i += ROWS_TPB_FAT) {
				const int m	 = i / (r_hi - r_lo);
				const int rl = i - m * (r_hi - r_lo);// consecutive threads -> consecutive rows: coalesced stores
				float v		 = 0.f;
				for (int k = 0; k < ipr; ++k)
					v += part[(rl * 8 + k) * MT + m];
				const int row	  = r_lo + rl;
				ocur			  = rows_find_op(b, row, 0);
				const rows_op* op = &b.op[ocur];
				const size_t off  = static_cast<size_t>(m) * op->ldy + (row - op->row_begin);
				op->y[off]		  = v;
				if (b.push.world > 1)
					for (int r = 0; r < b.push.world; ++r)
						if (r != b.push.rank && b.y_peer[ocur][r])
							b.y_peer[ocur][r][off] = v;
			}
			if (b.push.world > 1)
				push_finish(b.push, tid);
		}

		// ---- double-buffered variant: two 4 KB items in flight per warp ----
		// A position in a warp's work list: one item (32*ITEM blocks) of one row, with everything needed to stream it.
		struct item_pos {
			row_desc rd;
			const unsigned char* act;
			float* yrow;
			long long ldy;
			int row;// batch-wide row index; >= total_rows means "past the end"
			int b0;
			int cur;// op index
		};

		__device__ __forceinline__ void pos_set_row(item_pos& p, const rows_batch& b, const unsigned char* act_smem, int row, int total_rows, int n_ops) {
			p.row = row;
			p.b0  = 0;
			if (row < total_rows) {
				while (p.cur + 1 < n_ops && row >= b.op[p.cur + 1].row_begin)
					++p.cur;
				const rows_op* op = &b.op[p.cur];
				const int lrow	  = row - op->row_begin;
				p.rd			  = make_row(op, lrow);
				p.act			  = act_smem + op->act_off;
				p.yrow			  = op->y + lrow;
				p.ldy			  = op->ldy;
			}
		}

		// the item after `p` in this warp's list
		__device__ __forceinline__ item_pos pos_next(const item_pos& p, const rows_batch& b, const unsigned char* act_smem, int W, int total_rows, int n_ops) {
			item_pos n = p;
			n.b0	   = p.b0 + 32 * ITEM;
			if (n.b0 >= p.rd.nb)
				pos_set_row(n, b, act_smem, p.row + W, total_rows, n_ops);
			return n;
		}

		template<int MT> __global__ void __launch_bounds__(ROWS_TPB, 2) gemv_q8_rows_db(const __grid_constant__ rows_batch b) {
			extern __shared__ __align__(128) unsigned char act_smem[];
			const int tid		 = threadIdx.x;
			const int lane		 = tid & 31;
			const int warp		 = tid >> 5;
			const int W			 = gridDim.x * ROWS_WARPS;
			const int total_rows = b.total_rows;
			const int n_ops		 = b.n_ops;
			item_regs ra, rb;
			item_pos pa, pb;
			pa.cur = 0;
			pos_set_row(pa, b, act_smem, blockIdx.x * ROWS_WARPS + warp, total_rows, n_ops);
			// ---- weights first: both buffers are filled before waiting for the previous kernel ----
			if (pa.row < total_rows)
				load_item(ra, pa.rd, pa.b0, lane);
			pb = pa;
			if (pa.row < total_rows) {
				pb = pos_next(pa, b, act_smem, W, total_rows, n_ops);
				if (pb.row < total_rows)
					load_item(rb, pb.rd, pb.b0, lane);
			}
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			quantize_inputs<MT>(b, act_smem, tid);
			float acc[MT], rowacc[MT];
#pragma unroll
			for (int m = 0; m < MT; ++m)
				acc[m] = rowacc[m] = 0.f;
			// same summation order as gemv_q8_rows: item totals added in ascending order
			auto finish_item = [&]() {
#pragma unroll
				for (int m = 0; m < MT; ++m) {
					rowacc[m] += warp_sum(acc[m]);
					acc[m] = 0.f;
				}
			};
			auto finish_row = [&](const item_pos& p) {
#pragma unroll
				for (int m = 0; m < MT; ++m) {
					if (lane == 0)
						p.yrow[static_cast<size_t>(m) * p.ldy] = rowacc[m];
					rowacc[m] = 0.f;
				}
			};
			while (true) {
				if (pa.row >= total_rows)
					break;
				compute_item<MT>(ra, acc, pa.act, pa.rd.nb, pa.b0, lane);
				finish_item();
				{
					const bool row_end = pa.b0 + 32 * ITEM >= pa.rd.nb;
					const item_pos done = pa;
					pa = pos_next(pb, b, act_smem, W, total_rows, n_ops);
					if (pb.row < total_rows && pa.row < total_rows)
						load_item(ra, pa.rd, pa.b0, lane);
					if (row_end)
						finish_row(done);
				}
				if (pb.row >= total_rows)
					break;
				compute_item<MT>(rb, acc, pb.act, pb.rd.nb, pb.b0, lane);
				finish_item();
				{
					const bool row_end = pb.b0 + 32 * ITEM >= pb.rd.nb;
					const item_pos done = pb;
					pb = pos_next(pa, b, act_smem, W, total_rows, n_ops);
					if (pa.row < total_rows && pb.row < total_rows)
						load_item(rb, pb.rd, pb.b0, lane);
					if (row_end)
						finish_row(done);
				}
			}
		}
	}

	size_t gemv_rows_act_bytes(int64_t K, int M, bool f32act) {
		const int64_t per_row = f32act ? K * 4 : K + (K / 32) * 4;
		return static_cast<size_t>((M * per_row + 127) & ~int64_t(127));
	}

	// dynamic shared memory a launch with the in-kernel rms_norm may ask for: one CTA per SM, or two
	size_t gemv_rows_norm_smem_cap(bool fat) {
		return fat ? 200 * 1024 : 100 * 1024;
	}

	// whether a launch of `total_rows` rows can run the rms_norm in its prologue (else the caller uses rms_norm.cu's kernel)
	bool gemv_rows_norm_inside(int total_rows, size_t act_bytes, int64_t K, int M, int sm_count, bool fat_ctas) {
		const bool fat = fat_ctas && total_rows >= sm_count * ROWS_WARPS_FAT;
		return ((act_bytes + 127) & ~size_t(127)) + gemv_rows_norm_bytes(K, M) <= gemv_rows_norm_smem_cap(fat);
	}

	size_t gemv_rows_norm_bytes(int64_t K, int M) {
		return 2 * static_cast<size_t>(M) * static_cast<size_t>(K + 8) * 4 + 128;// the staged rows and their products with the norm weight
	}

	bool gemv_rows_supports(int64_t K, int64_t M, bool f32act) {
		// up to 4 rows per pass in every shape of the kernel; 5 to 8 in the plain Q8 shape (8-warp CTAs, two per SM) only
		return K % 32 == 0 && M >= 1 && M <= (f32act ? 4 : 8) && gemv_rows_act_bytes(K, static_cast<int>(M), f32act) <= 96 * 1024;
	}

	// `b` arrives with op pointers/shapes, act_off/slot tables and preq fields filled by the caller.
	cudaError_t launch_gemv_rows(const rows_batch& b_in, int M, const launch_cfg& cfg, int ctas_per_sm, int* launches, bool double_buffer, int cluster, bool fat_ctas,
		bool split_long_rows) {
		rows_batch b = b_in;
		int rows	 = 0;
		for (int i = 0; i < b.n_ops; ++i) {
			b.op[i].row_begin = rows;
			rows += b.op[i].rows;
		}
		b.total_rows = rows;
		if (rows == 0)
			return cudaSuccess;
		if (ctas_per_sm < 1)
			ctas_per_sm = 1;
		// one 24-warp CTA per SM when every one of those warps gets a row, else 8-warp CTAs
		if (b.f32act) {// one shape family for the f32 mode: no double buffering, no clusters, 2 CTAs per SM when not fat
			double_buffer = false;
			cluster		  = 1;
			ctas_per_sm	  = 2;
		}
		if (b.norm_w) {// the in-kernel rms_norm: two shapes only (24-warp CTAs, or 8-warp CTAs at two per SM), this CTA's shared memory only
			if (b.f32act)
				return cudaErrorInvalidValue;
			double_buffer	= false;
			cluster			= 1;
			split_long_rows = false;
			ctas_per_sm		= 2;
		}
		if (M > 4) {// 5 to 8 rows per pass: one kernel shape (more rows per pass means more shared-memory traffic per weight byte, not more HBM)
			if (b.f32act || b.norm_w)
				return cudaErrorInvalidValue;
			double_buffer	= false;
			cluster			= 1;
			split_long_rows = false;
			fat_ctas		= false;
			ctas_per_sm		= 2;
		}
		const bool fat	= fat_ctas && !double_buffer && cluster <= 1 && rows >= cfg.sm_count * ROWS_WARPS_FAT;
		const int warps = fat ? ROWS_WARPS_FAT : ROWS_WARPS;
		if (fat)
			ctas_per_sm = 1;
		int grid	  = (rows + warps - 1) / warps;
		const int cap = cfg.sm_count * ctas_per_sm;
		if (grid > cap) {
			// even split: every warp gets ceil(rows / W) or one fewer rows, with as few short warps as possible
			const int per_warp = (rows + cap * warps - 1) / (cap * warps);
			grid			   = (rows + per_warp * warps - 1) / (per_warp * warps);
		}
		// long rows: the item-parallel kernel, one CTA per SM, when all ops share K and a CTA's rows fit its partial-sum array
		// (for rows of a single item the same distribution loses: decode set 4702 against 4884 GB/s)
		bool split = fat && split_long_rows && (b.op[0].K >> 5) > 32 * ITEM && (b.op[0].K >> 5) <= 8 * 32 * ITEM &&
			(rows + cfg.sm_count - 1) / cfg.sm_count <= SPLIT_MAX_ROWS;
		for (int i = 1; i < b.n_ops && split; ++i)
			split = b.op[i].K == b.op[0].K;
		if (split)
			grid = cfg.sm_count;
		if (b.norm_w)
			b.norm_off = (b.act_bytes + 127) & ~127;
		const size_t smem = b.norm_w ? static_cast<size_t>(b.norm_off) + gemv_rows_norm_bytes(b.op[0].K, M) : static_cast<size_t>(b.act_bytes);
		if (smem > (b.norm_w ? gemv_rows_norm_smem_cap(fat) : 100 * 1024))
			return cudaErrorInvalidValue;
		cudaError_t e = cudaErrorInvalidValue;
		cudaLaunchConfig_t lc{};
		lc.gridDim			= dim3(grid);
		lc.blockDim			= dim3(warps * 32);
		lc.dynamicSmemBytes = smem;
		lc.stream			= cfg.stream;
		cudaLaunchAttribute attr[2];
		int n_attr = 0;
		if (cfg.pdl) {
			attr[n_attr].id											= cudaLaunchAttributeProgrammaticStreamSerialization;
			attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
			++n_attr;
		}
		if (cluster > 1 && !b.preq) {
			cluster = cluster >= 8 ? 8 : (cluster >= 4 ? 4 : 2);
			grid	= ((grid + cluster - 1) / cluster) * cluster;
			attr[n_attr].id				  = cudaLaunchAttributeClusterDimension;
			attr[n_attr].val.clusterDim.x = static_cast<unsigned>(cluster);
			attr[n_attr].val.clusterDim.y = 1;
			attr[n_attr].val.clusterDim.z = 1;
			++n_attr;
			lc.gridDim = dim3(grid);
		}
		lc.attrs	= attr;
		lc.numAttrs = n_attr;
		// registers per thread are capped by the occupancy the grid was sized for (2, 3 or 4 CTAs per SM)
		const int occ = double_buffer ? 0 : (ctas_per_sm >= 4 ? 4 : (ctas_per_sm == 3 ? 3 : 2));
#define NHB_ROWS_NORM_CASE(MT) \
	if (b.norm_w && M == MT) { \
		e = cudaSuccess; \
		if (fat) { \
			auto kern = gemv_q8_rows<MT, 1, ROWS_TPB_FAT, false, true>; \
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} else { \
			auto kern = gemv_q8_rows<MT, 2, ROWS_TPB, false, true>; \
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} \
	}
		NHB_ROWS_NORM_CASE(1)
		NHB_ROWS_NORM_CASE(2)
		NHB_ROWS_NORM_CASE(3)
		NHB_ROWS_NORM_CASE(4)
#undef NHB_ROWS_NORM_CASE
#define NHB_ROWS_F32_CASE(MT) \
	if (b.f32act && M == MT) { \
		e = cudaSuccess; \
		if (split) { \
			auto kern = gemv_q8_rows_split<MT, true>; \
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} else if (fat) { \
			auto kern = gemv_q8_rows<MT, 1, ROWS_TPB_FAT, true>; \
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} else { \
			auto kern = gemv_q8_rows<MT, 2, ROWS_TPB, true>; \
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} \
	}
		NHB_ROWS_F32_CASE(1)
		NHB_ROWS_F32_CASE(2)
		NHB_ROWS_F32_CASE(3)
		NHB_ROWS_F32_CASE(4)
#undef NHB_ROWS_F32_CASE
#define NHB_ROWS_SPLIT_CASE(MT) \
	if (!b.f32act && !b.norm_w && split && M == MT) { \
		auto kern = gemv_q8_rows_split<MT>; \
		e		  = cudaSuccess; \
		if (smem > 40 * 1024) \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
		if (e == cudaSuccess) \
			e = cudaLaunchKernelEx(&lc, kern, b); \
	}
		NHB_ROWS_SPLIT_CASE(1)
		NHB_ROWS_SPLIT_CASE(2)
		NHB_ROWS_SPLIT_CASE(3)
		NHB_ROWS_SPLIT_CASE(4)
#undef NHB_ROWS_SPLIT_CASE
#define NHB_ROWS_FAT_CASE(MT) \
	if (!b.f32act && !b.norm_w && fat && !split && M == MT) { \
		auto kern = gemv_q8_rows<MT, 1, ROWS_TPB_FAT>; \
		e		  = cudaSuccess; \
		if (smem > 48 * 1024) \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
		if (e == cudaSuccess) \
			e = cudaLaunchKernelEx(&lc, kern, b); \
	}
		NHB_ROWS_FAT_CASE(1)
		NHB_ROWS_FAT_CASE(2)
		NHB_ROWS_FAT_CASE(3)
		NHB_ROWS_FAT_CASE(4)
#undef NHB_ROWS_FAT_CASE
#define NHB_ROWS_CASE(MT, OCC) \
	if (!b.f32act && !b.norm_w && !fat && M == MT && occ == OCC) { \
		auto kern = gemv_q8_rows<MT, OCC>; \
		e		  = cudaSuccess; \
		if (smem > 48 * 1024) \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
		if (e == cudaSuccess) \
			e = cudaLaunchKernelEx(&lc, kern, b); \
	}
		NHB_ROWS_CASE(1, 2)
		NHB_ROWS_CASE(1, 3)
		NHB_ROWS_CASE(1, 4)
		NHB_ROWS_CASE(2, 2)
		NHB_ROWS_CASE(2, 3)
		NHB_ROWS_CASE(2, 4)
		NHB_ROWS_CASE(3, 2)
		NHB_ROWS_CASE(3, 3)
		NHB_ROWS_CASE(3, 4)
		NHB_ROWS_CASE(4, 2)
		NHB_ROWS_CASE(4, 3)
		NHB_ROWS_CASE(4, 4)
#undef NHB_ROWS_CASE
#define NHB_ROWS_WIDE_CASE(MT) \
	if (M == MT) { \
		auto kern = gemv_q8_rows<MT, 2>; \
		e		  = cudaSuccess; \
		if (smem > 48 * 1024) \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
		if (e == cudaSuccess) \
			e = cudaLaunchKernelEx(&lc, kern, b); \
	}
		NHB_ROWS_WIDE_CASE(5)
		NHB_ROWS_WIDE_CASE(6)
		NHB_ROWS_WIDE_CASE(7)
		NHB_ROWS_WIDE_CASE(8)
#undef NHB_ROWS_WIDE_CASE
#define NHB_ROWS_DB_CASE(MT) \
	if (!b.f32act && !b.norm_w && double_buffer && M == MT) { \
		auto kern = gemv_q8_rows_db<MT>; \
		e		  = cudaSuccess; \
		if (smem > 48 * 1024) \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
		if (e == cudaSuccess) \
			e = cudaLaunchKernelEx(&lc, kern, b); \
	}
		NHB_ROWS_DB_CASE(1)
		NHB_ROWS_DB_CASE(2)
		NHB_ROWS_DB_CASE(3)
		NHB_ROWS_DB_CASE(4)
#undef NHB_ROWS_DB_CASE
		if (e == cudaSuccess && launches)
			*launches += 1;
		return e;
	}

}

#ifdef NHB_ROWS_PROF
extern "C" int nhb_debug_rows_prof(unsigned long long* out8) {
	return static_cast<int>(cudaMemcpyFromSymbol(out8, nhb::rows_prof, 64));
}
#endif
