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

#include "gemv_common.cuh"

namespace nhb {

	namespace {

		// Two CTA shapes.  Wide launches use one CTA of 24 warps per SM: the activations are quantised once per SM
		// instead of three times.  Launches with too few rows for that keep 8-warp CTAs, several per SM.
		constexpr int ROWS_WARPS	 = 8;
		constexpr int ROWS_TPB		 = ROWS_WARPS * 32;
		constexpr int ROWS_WARPS_FAT = 24;
		constexpr int ROWS_TPB_FAT	 = ROWS_WARPS_FAT * 32;
		constexpr int ITEM		 = 4;// 32-byte Q8 blocks per lane per step: 4 KB of a row per warp

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


		// NORM: the rms_norm x norm-weight producer runs inside the prologue (its own instantiation, so that the plain
		// kernels keep their register allocation)
		// EPI: the element-wise neighbours fused in -- SwiGLU in front of the quantiser (rows_op::x2) and the residual added to the
		// output (rows_op::res); its own instantiations, so that the plain kernels keep their register allocation
		template<int MT, int OCC, int TPB = ROWS_TPB, bool F32 = false, bool NORM = false, bool EPI = false> __global__ void __launch_bounds__(TPB, OCC)
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
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			push_wait_peers(b.push, tid);
			if constexpr (F32)
				stage_inputs_f32<MT>(b, act_smem, tid);
			else
				quantize_inputs<MT, NORM, false, EPI>(b, act_smem, tid, TPB);
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
						yrow[static_cast<size_t>(m) * ldy] = (EPI && op->res) ? rowacc[m] + op->res[static_cast<size_t>(m) * op->ldr + lrow] : rowacc[m];
				}
			}
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
				push_done(b.push, tid);
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
		template<int MT, bool F32 = false, bool EPI = false> __global__ void __launch_bounds__(ROWS_TPB_FAT, 1) gemv_q8_rows_split(const __grid_constant__ rows_batch b) {
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
			push_wait_peers(b.push, tid);
			if constexpr (F32)
				stage_inputs_f32<MT>(b, act_smem, tid);
			else
				quantize_inputs<MT, false, false, EPI>(b, act_smem, tid, ROWS_TPB_FAT);
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
				if constexpr (EPI) {
					if (op->res)
						v += op->res[static_cast<size_t>(m) * op->ldr + (row - op->row_begin)];
				}
				op->y[off] = v;
				if (b.push.world > 1)
					for (int r = 0; r < b.push.world; ++r)
						if (r != b.push.rank && b.y_peer[ocur][r])
							b.y_peer[ocur][r][off] = v;
			}
			if (b.push.world > 1)
				push_done(b.push, tid);
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
			push_wait_peers(b.push, tid);
			quantize_inputs<MT>(b, act_smem, tid, ROWS_TPB);
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

	namespace {
		__global__ void __launch_bounds__(32) peer_wait_kernel(const push_ctl pc) {
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			push_wait_peers(pc, threadIdx.x);
		}
	}

	cudaError_t launch_peer_wait(const push_ctl& pc, const launch_cfg& cfg, int* launches) {
		cudaLaunchConfig_t lc{};
		lc.gridDim	= dim3(1);
		lc.blockDim = dim3(32);
		lc.stream	= cfg.stream;
		cudaLaunchAttribute attr[1];
		attr[0].id										   = cudaLaunchAttributeProgrammaticStreamSerialization;
		attr[0].val.programmaticStreamSerializationAllowed = 1;
		lc.attrs										   = attr;
		lc.numAttrs										   = cfg.pdl ? 1 : 0;
		cudaError_t e									   = cudaLaunchKernelEx(&lc, peer_wait_kernel, pc);
		if (e == cudaSuccess && launches)
			*launches += 1;
		return e;
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

	namespace {
		struct rows_flags {
			int ctas_per_sm;
			bool double_buffer;
			int cluster;
			bool fat_ctas, split_long_rows;
		};

		// which of the options a batch of this kind can take; false = a combination no kernel shape serves
		bool settle_flags(const rows_batch& b, int M, rows_flags& f) {
			if (f.ctas_per_sm < 1)
				f.ctas_per_sm = 1;
			if (b.f32act) {// one shape family for the f32 mode: no double buffering, no clusters, 2 CTAs per SM when not fat
				f.double_buffer = false;
				f.cluster		= 1;
				f.ctas_per_sm	= 2;
			}
			if (b.norm_w) {// the in-kernel rms_norm: two shapes only (24-warp CTAs, or 8-warp CTAs at two per SM), this CTA's shared memory only
				if (b.f32act)
					return false;
				f.double_buffer	  = false;
				f.cluster		  = 1;
				f.split_long_rows = false;
				f.ctas_per_sm	  = 2;
			}
			bool epi = false;
			for (int i = 0; i < b.n_ops; ++i)
				epi = epi || b.op[i].x2 || b.op[i].res;
			if (epi) {// fused SwiGLU / residual: the plain Q8 shapes at one 24-warp CTA or two 8-warp CTAs per SM
				if (b.f32act || b.norm_w || b.preq || M > 4)
					return false;
				f.double_buffer = false;
				f.cluster		= 1;
				f.ctas_per_sm	= 2;
			}
			if (M > 4) {// 5 to 8 rows per pass: one kernel shape (more rows per pass means more shared-memory traffic per weight byte, not more HBM)
				if (b.f32act || b.norm_w)
					return false;
				f.double_buffer	  = false;
				f.cluster		  = 1;
				f.split_long_rows = false;
				f.fat_ctas		  = false;
				f.ctas_per_sm	  = 2;
			}
			return true;
		}

		// one 24-warp CTA per SM when every one of those warps gets a row, else 8-warp CTAs
		rows_shape shape_of(const rows_batch& b, int rows, int sm_count, rows_flags& f) {
			rows_shape sh{};
			sh.fat	 = f.fat_ctas && !f.double_buffer && f.cluster <= 1 && rows >= sm_count * ROWS_WARPS_FAT;
			sh.warps = sh.fat ? ROWS_WARPS_FAT : ROWS_WARPS;
			if (sh.fat)
				f.ctas_per_sm = 1;
			sh.grid		  = (rows + sh.warps - 1) / sh.warps;
			const int cap = sm_count * f.ctas_per_sm;
			if (sh.grid > cap) {
				// even split: every warp gets ceil(rows / W) or one fewer rows, with as few short warps as possible
				const int per_warp = (rows + cap * sh.warps - 1) / (cap * sh.warps);
				sh.grid			   = (rows + per_warp * sh.warps - 1) / (per_warp * sh.warps);
			}
			// long rows: the item-parallel kernel, one CTA per SM, when all ops share K and a CTA's rows fit its partial-sum array
			// (for rows of a single item the same distribution loses: decode set 4702 against 4884 GB/s)
			sh.split = sh.fat && f.split_long_rows && (b.op[0].K >> 5) > 32 * ITEM && (b.op[0].K >> 5) <= 8 * 32 * ITEM &&
				(rows + sm_count - 1) / sm_count <= SPLIT_MAX_ROWS;
			for (int i = 1; i < b.n_ops && sh.split; ++i)
				sh.split = b.op[i].K == b.op[0].K;
			if (sh.split)
				sh.grid = sm_count;
			return sh;
		}
	}

	rows_shape gemv_rows_shape(const rows_batch& b, int M, int sm_count, int ctas_per_sm, bool double_buffer, int cluster, bool fat_ctas, bool split_long_rows) {
		rows_flags f{ ctas_per_sm, double_buffer, cluster, fat_ctas, split_long_rows };
		int rows = 0;
		for (int i = 0; i < b.n_ops; ++i)
			rows += b.op[i].rows;
		if (rows == 0 || !settle_flags(b, M, f))
			return rows_shape{};
		return shape_of(b, rows, sm_count, f);
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
		rows_flags f{ ctas_per_sm, double_buffer, cluster, fat_ctas, split_long_rows };
		if (!settle_flags(b, M, f))
			return cudaErrorInvalidValue;
		const rows_shape sh = shape_of(b, rows, cfg.sm_count, f);
		ctas_per_sm			= f.ctas_per_sm;
		double_buffer		= f.double_buffer;
		cluster				= f.cluster;
		const bool fat = sh.fat, split = sh.split;
		const int warps = sh.warps;
		int grid		= sh.grid;
		if (b.norm_w)
			b.norm_off = (b.act_bytes + 127) & ~127;
		const size_t smem = b.norm_w ? static_cast<size_t>(b.norm_off) + gemv_rows_norm_bytes(b.op[0].K, M) : static_cast<size_t>(b.act_bytes);
		if (smem > (b.norm_w ? gemv_rows_norm_smem_cap(fat) : 100 * 1024))
			return cudaErrorInvalidValue;
		bool epi = false;// a fused element-wise neighbour somewhere in the batch: the EPI instantiations (plain Q8 shapes only)
		for (int i = 0; i < b.n_ops; ++i)
			epi = epi || b.op[i].x2 || b.op[i].res;
		if (epi && (b.f32act || b.norm_w || b.preq || double_buffer || cluster > 1 || M > 4))
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
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
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
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} else if (fat) { \
			auto kern = gemv_q8_rows<MT, 1, ROWS_TPB_FAT, true>; \
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} else { \
			auto kern = gemv_q8_rows<MT, 2, ROWS_TPB, true>; \
			e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} \
	}
		NHB_ROWS_F32_CASE(1)
		NHB_ROWS_F32_CASE(2)
		NHB_ROWS_F32_CASE(3)
		NHB_ROWS_F32_CASE(4)
#undef NHB_ROWS_F32_CASE
#define NHB_ROWS_EPI_CASE(MT) \
	if (epi && M == MT) { \
		e = cudaSuccess; \
		if (split) { \
			auto kern = gemv_q8_rows_split<MT, false, true>; \
			if (smem > 32 * 1024) \
				e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} else if (fat) { \
			auto kern = gemv_q8_rows<MT, 1, ROWS_TPB_FAT, false, false, true>; \
			if (smem > 48 * 1024) \
				e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} else { \
			auto kern = gemv_q8_rows<MT, 2, ROWS_TPB, false, false, true>; \
			if (smem > 48 * 1024) \
				e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
			if (e == cudaSuccess) \
				e = cudaLaunchKernelEx(&lc, kern, b); \
		} \
	}
		NHB_ROWS_EPI_CASE(1)
		NHB_ROWS_EPI_CASE(2)
		NHB_ROWS_EPI_CASE(3)
		NHB_ROWS_EPI_CASE(4)
#undef NHB_ROWS_EPI_CASE
#define NHB_ROWS_SPLIT_CASE(MT) \
	if (!epi && !b.f32act && !b.norm_w && split && M == MT) { \
		auto kern = gemv_q8_rows_split<MT>; \
		e		  = cudaSuccess; \
		if (smem > 32 * 1024) /* the kernel also has static shared memory */ \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
		if (e == cudaSuccess) \
			e = cudaLaunchKernelEx(&lc, kern, b); \
	}
		NHB_ROWS_SPLIT_CASE(1)
		NHB_ROWS_SPLIT_CASE(2)
		NHB_ROWS_SPLIT_CASE(3)
		NHB_ROWS_SPLIT_CASE(4)
#undef NHB_ROWS_SPLIT_CASE
#define NHB_ROWS_FAT_CASE(MT) \
	if (!epi && !b.f32act && !b.norm_w && fat && !split && M == MT) { \
		auto kern = gemv_q8_rows<MT, 1, ROWS_TPB_FAT>; \
		e		  = cudaSuccess; \
		if (smem > 48 * 1024) \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
		if (e == cudaSuccess) \
			e = cudaLaunchKernelEx(&lc, kern, b); \
	}
		NHB_ROWS_FAT_CASE(1)
		NHB_ROWS_FAT_CASE(2)
		NHB_ROWS_FAT_CASE(3)
		NHB_ROWS_FAT_CASE(4)
#undef NHB_ROWS_FAT_CASE
#define NHB_ROWS_CASE(MT, OCC) \
	if (!epi && !b.f32act && !b.norm_w && !fat && M == MT && occ == OCC) { \
		auto kern = gemv_q8_rows<MT, OCC>; \
		e		  = cudaSuccess; \
		if (smem > 48 * 1024) \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
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
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
		if (e == cudaSuccess) \
			e = cudaLaunchKernelEx(&lc, kern, b); \
	}
		NHB_ROWS_WIDE_CASE(5)
		NHB_ROWS_WIDE_CASE(6)
		NHB_ROWS_WIDE_CASE(7)
		NHB_ROWS_WIDE_CASE(8)
#undef NHB_ROWS_WIDE_CASE
#define NHB_ROWS_DB_CASE(MT) \
	if (!epi && !b.f32act && !b.norm_w && double_buffer && M == MT) { \
		auto kern = gemv_q8_rows_db<MT>; \
		e		  = cudaSuccess; \
		if (smem > 48 * 1024) \
			e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
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

