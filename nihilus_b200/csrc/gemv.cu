// Q8_0 GEMV kernels for decode-sized M (sm_100a).
//
// Arithmetic (NHB_ACT_Q8): the reference's quantize_row_q8_0 + vec_dot_q8_0_q8_0
// (include/nihilus-incl/cpu/avx_2.hpp:4439-4489, :4749-4780): activations are quantised per 32-wide
// block, every block contributes float(exact int dot) * (d_weight * d_activation) by fused multiply-add.
// Only the order in which block terms are added differs from the CPU code.  The order here depends on
// K alone -- not on the grid, the row shard or the GPU count -- so results are bit-identical across
// shardings.
//
// HBM-bound: each launch reads N*(K/32)*34 bytes of weights exactly once; x and y are noise.
//
//  gemv_q8_stream  persistent CTAs; one producer thread streams row tiles of both weight planes into a
//                  shared-memory ring with bulk (TMA) copies, 8 consumer warps dot them against
//                  activations that live in registers.  Several independent mul_mats run in one launch.
//  gemv_q8_ldg     fallback for any K % 32 == 0 and for f32 activations: coalesced 128-bit loads.
#include "internal.h"
#include "ptx.cuh"
#include "q8_device.cuh"

namespace nhb {

	namespace {

		constexpr int NCW		  = 8;// consumer warps
		constexpr int NCT		  = NCW * 32;// consumer threads
		constexpr int STREAM_TPB  = NCT + 32;// + one producer warp
		constexpr int MAX_ROWS	  = 32;// rows per ring slot, upper bound
		constexpr int STAGE_TARGET = 17408;// 4 rows of K = 4096: 16384 quant bytes + 1024 scale bytes
		constexpr int RING_ALIGN  = 128;

		struct stream_smem_hdr {
			uint64_t full[16];
			uint64_t empty[16];
			int abort_flag;
			int consumed;
			int pad[2];
		};

		__device__ __forceinline__ int find_op(const stream_batch& b, int tile, int cur) {
			while (cur + 1 < b.n_ops && tile >= b.op[cur + 1].tile_begin)
				++cur;
			return cur;
		}

		// CH: 16-byte chunks of a row owned by one consumer thread (K <= CH * 4096); MT: activation rows
		template<int CH, int MT> __global__ void __launch_bounds__(STREAM_TPB, 1)
			gemv_q8_stream(const __grid_constant__ stream_batch b, int* __restrict__ dev_status) {
			extern __shared__ __align__(128) unsigned char smem_raw[];
			stream_smem_hdr* hdr = reinterpret_cast<stream_smem_hdr*>(smem_raw);
			float* partial		 = reinterpret_cast<float*>(smem_raw + sizeof(stream_smem_hdr));// [2][MAX_ROWS][NCW][MT]
			constexpr int partial_bytes = 2 * MAX_ROWS * NCW * MT * 4;
			unsigned char* ring = smem_raw + ((sizeof(stream_smem_hdr) + partial_bytes + RING_ALIGN - 1) / RING_ALIGN) * RING_ALIGN;

			const int tid	  = threadIdx.x;
			const int S		  = b.n_stages;
			const int n_tiles = b.total_tiles;

			if (tid == 0) {
				for (int s = 0; s < S; ++s) {
					mbar_init(&hdr->full[s], 1);
					mbar_init(&hdr->empty[s], 1);
				}
				hdr->abort_flag = 0;
				hdr->consumed	= 0;
				fence_mbar_init();
			}
			__syncthreads();
			pdl_launch_dependents();

			int issued = 0;
			if (tid >= NCT) {
				// ---- producer: weights never depend on an earlier kernel, so it does not wait for prior grids ----
				if (tid == NCT) {
					const uint64_t pol = l2_policy_evict_first();
					int cur			   = 0;
					int it			   = 0;
					for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
						const int s = it % S;
						if (it >= S) {
							if (!mbar_wait(&hdr->empty[s], ((it / S) - 1) & 1)) {
								atomicExch(dev_status, DEV_TIMEOUT_EMPTY);
								break;
							}
						}
						if (*reinterpret_cast<volatile int*>(&hdr->abort_flag))
							break;
						cur					= find_op(b, tile, cur);
						const stream_op& op = b.op[cur];
						const int row0		= (tile - op.tile_begin) * op.rows_per_tile;
						const int rows		= min(op.rows_per_tile, op.rows - row0);
						const uint32_t bq	= static_cast<uint32_t>(rows) * static_cast<uint32_t>(op.K);
						const uint32_t bd	= bq >> 4;
						unsigned char* slot = ring + static_cast<size_t>(s) * b.stage_bytes;
						mbar_expect_tx(&hdr->full[s], bq + bd);
						bulk_g2s(slot, op.wq + static_cast<size_t>(row0) * op.K, bq, &hdr->full[s], pol);
						bulk_g2s(slot + static_cast<size_t>(op.rows_per_tile) * op.K, op.wd + static_cast<size_t>(row0) * (op.K >> 5), bd, &hdr->full[s], pol);
						issued = it + 1;
					}
				}
			} else {
				// ---- consumers ----
				const int lane = tid & 31;
				const int warp = tid >> 5;
				uint4 qa[MT][CH];
				float da[MT][CH];
				int cur	   = -1;
				int buf	   = 0;
				int it	   = 0;
				bool alive = true;
				pdl_wait_prior_grids();// x may be the previous kernel's output; y may still be read by it
				for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++it) {
					const int ncur = find_op(b, tile, cur < 0 ? 0 : cur);
					if (ncur != cur) {
						cur					= ncur;
						const stream_op& op = b.op[cur];
						const int cpr		= op.K >> 4;
#pragma unroll
						for (int m = 0; m < MT; ++m) {
#pragma unroll
							for (int j = 0; j < CH; ++j) {
								const int c		 = tid + j * NCT;
								const bool valid = c < cpr;
								float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0, v2 = v0, v3 = v0;
								if (valid) {
									const float4* p = reinterpret_cast<const float4*>(op.x + static_cast<size_t>(m) * op.ldx + static_cast<size_t>(c) * 16);
									v0				= __ldg(p);
									v1				= __ldg(p + 1);
									v2				= __ldg(p + 2);
									v3				= __ldg(p + 3);
								}
								float amax = absmax4(v0, absmax4(v1, absmax4(v2, absmax4(v3, 0.f))));
								amax	   = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));// the other half of the 32-wide block
								const act_scale sc = q8_scales(amax);
								qa[m][j].x		   = q8_pack4(v0.x, v0.y, v0.z, v0.w, sc.id);
								qa[m][j].y		   = q8_pack4(v1.x, v1.y, v1.z, v1.w, sc.id);
								qa[m][j].z		   = q8_pack4(v2.x, v2.y, v2.z, v2.w, sc.id);
								qa[m][j].w		   = q8_pack4(v3.x, v3.y, v3.z, v3.w, sc.id);
								da[m][j]		   = sc.d;
							}
						}
					}
					const stream_op& op = b.op[cur];
					const int K			= op.K;
					const int cpr		= K >> 4;
					const int row0		= (tile - op.tile_begin) * op.rows_per_tile;
					const int rows		= min(op.rows_per_tile, op.rows - row0);
					const int s			= it % S;
					bool ok				= mbar_wait(&hdr->full[s], (it / S) & 1);
					float* part			= partial + buf * (MAX_ROWS * NCW * MT);
					if (ok) {
						const unsigned char* sq = ring + static_cast<size_t>(s) * b.stage_bytes;
						const __half* sd		= reinterpret_cast<const __half*>(sq + static_cast<size_t>(op.rows_per_tile) * K);
#pragma unroll 4
						for (int r = 0; r < rows; ++r) {
							float acc[MT];
#pragma unroll
							for (int m = 0; m < MT; ++m)
								acc[m] = 0.f;
#pragma unroll
							for (int j = 0; j < CH; ++j) {
								const int c = tid + j * NCT;
								if (c < cpr) {
									const uint4 w  = *reinterpret_cast<const uint4*>(sq + static_cast<size_t>(r) * K + static_cast<size_t>(c) * 16);
									const float dw = __half2float(sd[r * (K >> 5) + (c >> 1)]);
#pragma unroll
									for (int m = 0; m < MT; ++m)
										acc[m] = fmaf(static_cast<float>(dot16(w, qa[m][j])), dw * da[m][j], acc[m]);
								}
							}
#pragma unroll
							for (int m = 0; m < MT; ++m) {
								const float v = warp_sum(acc[m]);
								if (lane == 0)
									part[(r * NCW + warp) * MT + m] = v;
							}
						}
					}
					// all consumers meet here; a failed wait anywhere makes every consumer leave together
					ok = named_bar_and(1, NCT, ok);
					if (!ok) {
						if (tid == 0) {
							atomicExch(dev_status, DEV_TIMEOUT_FULL);
							*reinterpret_cast<volatile int*>(&hdr->abort_flag) = 1;
						}
						alive = false;
						break;
					}
					if (tid < rows * MT) {
						const int r = tid / MT;
						const int m = tid - r * MT;
						float v		= 0.f;
#pragma unroll
						for (int w = 0; w < NCW; ++w)
							v += part[(r * NCW + w) * MT + m];
						op.y[static_cast<size_t>(m) * op.ldy + row0 + r] = v;
					}
					if (tid == 0) {
						mbar_arrive(&hdr->empty[s]);
						hdr->consumed = it + 1;
					}
					buf ^= 1;
				}
			}
			__syncthreads();
			// abnormal exit only: do not leave while bulk copies may still land in this CTA's shared memory
			if (tid == NCT && issued > hdr->consumed) {
				for (int it = hdr->consumed; it < issued; ++it) {
					if (!mbar_wait(&hdr->full[it % S], (it / S) & 1)) {
						atomicExch(dev_status, DEV_TIMEOUT_DRAIN);
						break;
					}
				}
			}
		}

		// ---- fallback: one warp per row, 128-bit coalesced loads of the quant plane ----
		template<int MT, bool F32ACT> __global__ void __launch_bounds__(256)
			gemv_q8_ldg(const int8_t* __restrict__ wq, const __half* __restrict__ wd, const float* __restrict__ x, long long ldx, float* __restrict__ y,
				long long ldy, int rows, int K) {
			extern __shared__ __align__(128) unsigned char smem_raw[];
			const int tid  = threadIdx.x;
			const int lane = tid & 31;
			const int warp = tid >> 5;
			const int nb   = K >> 5;
			const int cpr  = K >> 4;
			// Q8: int8 [MT][K] then f32 scales [MT][nb];  F32: f32 [MT][K]
			int8_t* sqa = reinterpret_cast<int8_t*>(smem_raw);
			float* sda	= reinterpret_cast<float*>(smem_raw + static_cast<size_t>(MT) * K);
			float* sx	= reinterpret_cast<float*>(smem_raw);
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			if constexpr (F32ACT) {
				for (int m = 0; m < MT; ++m)
					for (int k = tid; k < K; k += blockDim.x)
						sx[m * K + k] = x[static_cast<size_t>(m) * ldx + k];
			} else {
				for (int m = 0; m < MT; ++m) {
					for (int blk = tid; blk < nb; blk += blockDim.x) {
						const float4* p = reinterpret_cast<const float4*>(x + static_cast<size_t>(m) * ldx + static_cast<size_t>(blk) * QK);
						float4 v[8];
						float amax = 0.f;
#pragma unroll
						for (int i = 0; i < 8; ++i) {
							v[i] = __ldg(p + i);
							amax = absmax4(v[i], amax);
						}
						const act_scale sc = q8_scales(amax);
						uint32_t* dst	   = reinterpret_cast<uint32_t*>(sqa + static_cast<size_t>(m) * K + static_cast<size_t>(blk) * QK);
#pragma unroll
						for (int i = 0; i < 8; ++i)
							dst[i] = q8_pack4(v[i].x, v[i].y, v[i].z, v[i].w, sc.id);
						sda[m * nb + blk] = sc.d;
					}
				}
			}
			__syncthreads();
			const int wpb = blockDim.x >> 5;
			for (int row = blockIdx.x * wpb + warp; row < rows; row += gridDim.x * wpb) {
				const uint4* wrow  = reinterpret_cast<const uint4*>(wq + static_cast<size_t>(row) * K);
				const __half* drow = wd + static_cast<size_t>(row) * nb;
				float acc[MT];
#pragma unroll
				for (int m = 0; m < MT; ++m)
					acc[m] = 0.f;
#pragma unroll 4
				for (int c = lane; c < cpr; c += 32) {
					const uint4 w  = __ldg(wrow + c);
					const float dw = __half2float(drow[c >> 1]);
					if constexpr (F32ACT) {
						// vec_dot_q8_f32 (cpu/avx_2.hpp:4800-4815): (sum_j x_j * float(q_j)) * d, here over a half block
						const uint32_t ww[4] = { w.x, w.y, w.z, w.w };
#pragma unroll
						for (int m = 0; m < MT; ++m) {
							const float4* xp = reinterpret_cast<const float4*>(sx + static_cast<size_t>(m) * K + static_cast<size_t>(c) * 16);
							float s			 = 0.f;
#pragma unroll
							for (int i = 0; i < 4; ++i) {
								const float4 xv = xp[i];
								const int q0 = static_cast<int8_t>(ww[i] & 0xff), q1 = static_cast<int8_t>((ww[i] >> 8) & 0xff);
								const int q2 = static_cast<int8_t>((ww[i] >> 16) & 0xff), q3 = static_cast<int8_t>(ww[i] >> 24);
								s = fmaf(xv.x, static_cast<float>(q0), s);
								s = fmaf(xv.y, static_cast<float>(q1), s);
								s = fmaf(xv.z, static_cast<float>(q2), s);
								s = fmaf(xv.w, static_cast<float>(q3), s);
							}
							acc[m] = fmaf(s, dw, acc[m]);
						}
					} else {
#pragma unroll
						for (int m = 0; m < MT; ++m) {
							const uint4 a = *reinterpret_cast<const uint4*>(sqa + static_cast<size_t>(m) * K + static_cast<size_t>(c) * 16);
							acc[m]		  = fmaf(static_cast<float>(dot16(w, a)), dw * sda[m * nb + (c >> 1)], acc[m]);
						}
					}
				}
#pragma unroll
				for (int m = 0; m < MT; ++m) {
					const float v = warp_sum(acc[m]);
					if (lane == 0)
						y[static_cast<size_t>(m) * ldy + row] = v;
				}
			}
		}

		// quantize_row_q8_0 on its own: one thread per 32-wide block
		__global__ void quantize_q8_kernel(const float* __restrict__ x, long long ldx, int M, int K, int8_t* __restrict__ q, float* __restrict__ d) {
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			const int nb		= K >> 5;
			const long long tot = static_cast<long long>(M) * nb;
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < tot; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				const int m		= static_cast<int>(i / nb);
				const int blk	= static_cast<int>(i - static_cast<long long>(m) * nb);
				const float4* p = reinterpret_cast<const float4*>(x + static_cast<size_t>(m) * ldx + static_cast<size_t>(blk) * QK);
				float4 v[8];
				float amax = 0.f;
#pragma unroll
				for (int j = 0; j < 8; ++j) {
					v[j] = __ldg(p + j);
					amax = absmax4(v[j], amax);
				}
				const act_scale sc = q8_scales(amax);
				uint32_t* dst	   = reinterpret_cast<uint32_t*>(q + static_cast<size_t>(m) * K + static_cast<size_t>(blk) * QK);
#pragma unroll
				for (int j = 0; j < 8; ++j)
					dst[j] = q8_pack4(v[j].x, v[j].y, v[j].z, v[j].w, sc.id);
				d[i] = sc.d;
			}
		}

		// exact int32 dot of every (activation row, weight row, block)
		__global__ void block_dots_kernel(const int8_t* __restrict__ wq, const int8_t* __restrict__ qa, int rows, int K, int M, int32_t* __restrict__ dots) {
			const int nb		= K >> 5;
			const long long tot = static_cast<long long>(M) * rows * nb;
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < tot; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				const int blk	   = static_cast<int>(i % nb);
				const long long mr = i / nb;
				const int r		   = static_cast<int>(mr % rows);
				const int m		   = static_cast<int>(mr / rows);
				const uint4* w	   = reinterpret_cast<const uint4*>(wq + static_cast<size_t>(r) * K + static_cast<size_t>(blk) * QK);
				const uint4* a	   = reinterpret_cast<const uint4*>(qa + static_cast<size_t>(m) * K + static_cast<size_t>(blk) * QK);
				dots[i]			   = dot16(w[0], a[0]) + dot16(w[1], a[1]);
			}
		}

		template<typename kern_t, typename... args_t>
		cudaError_t launch_pdl(kern_t kern, dim3 grid, dim3 block, size_t smem, const launch_cfg& cfg, args_t... args) {
			cudaLaunchConfig_t lc{};
			lc.gridDim			= grid;
			lc.blockDim			= block;
			lc.dynamicSmemBytes = smem;
			lc.stream			= cfg.stream;
			cudaLaunchAttribute attr[1];
			attr[0].id										   = cudaLaunchAttributeProgrammaticStreamSerialization;
			attr[0].val.programmaticStreamSerializationAllowed = 1;
			lc.attrs										   = attr;
			lc.numAttrs										   = cfg.pdl ? 1 : 0;
			return cudaLaunchKernelEx(&lc, kern, args...);
		}

		size_t stream_smem_bytes(int MT, int stage_bytes, int n_stages) {
			const size_t head = ((sizeof(stream_smem_hdr) + 2 * MAX_ROWS * NCW * MT * 4 + RING_ALIGN - 1) / RING_ALIGN) * RING_ALIGN;
			return head + static_cast<size_t>(stage_bytes) * n_stages;
		}

		template<int CH, int MT> cudaError_t launch_stream_t(const stream_batch& b, const launch_cfg& cfg, int grid, size_t smem) {
			auto kern = gemv_q8_stream<CH, MT>;
			static size_t set_max[64] = {};// per device: the attribute belongs to the device's copy of the kernel
			int dev					  = 0;
			cudaGetDevice(&dev);
			dev &= 63;
			if (smem > set_max[dev]) {
				cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
				if (e != cudaSuccess)
					return e;
				set_max[dev] = smem;
			}
			return launch_pdl(kern, dim3(grid), dim3(STREAM_TPB), smem, cfg, b, cfg.dev_status);
		}

	}

	bool gemv_stream_supports(int64_t K, int64_t M) {
		if (K % 256 != 0 || K < 1024 || K > 16384)
			return false;
		const int ch = static_cast<int>((K / 16 + NCT - 1) / NCT);
		return M >= 1 && M * ch <= 8 && M <= 8;
	}

	// Fills rows_per_tile / tile_begin / stage geometry of `b` (ops' pointers and shapes already set) and launches.
	cudaError_t launch_gemv_stream(const stream_batch& b_in, int M, const launch_cfg& cfg, int ctas_per_sm, int* launches) {
		stream_batch b = b_in;
		int ch_max	   = 1;
		int stage	   = 0;
		int tiles	   = 0;
		for (int i = 0; i < b.n_ops; ++i) {
			stream_op& op	  = b.op[i];
			const int per_row = op.K + (op.K >> 4);
			int rpt			  = STAGE_TARGET / per_row;
			rpt				  = rpt < 1 ? 1 : (rpt > MAX_ROWS ? MAX_ROWS : rpt);
			op.rows_per_tile  = rpt;
			op.tile_begin	  = tiles;
			tiles += (op.rows + rpt - 1) / rpt;
			const int need = ((rpt * per_row + RING_ALIGN - 1) / RING_ALIGN) * RING_ALIGN;
			stage		   = need > stage ? need : stage;
			const int ch   = (op.K / 16 + NCT - 1) / NCT;
			ch_max		   = ch > ch_max ? ch : ch_max;
		}
		if (tiles == 0)
			return cudaSuccess;
		b.total_tiles = tiles;
		b.stage_bytes = stage;
		if (ctas_per_sm < 1)
			ctas_per_sm = 1;
		const size_t budget = (ctas_per_sm == 1 ? 200 * 1024 : 110 * 1024);
		int n_stages		= static_cast<int>((budget - stream_smem_bytes(M, 0, 0)) / stage);
		n_stages			= n_stages > 16 ? 16 : n_stages;
		if (n_stages < 2)
			return cudaErrorInvalidConfiguration;
		b.n_stages		  = n_stages;
		const size_t smem = stream_smem_bytes(M, stage, n_stages);
		int grid		  = cfg.sm_count * ctas_per_sm;
		grid			  = grid > tiles ? tiles : grid;
		cudaError_t e	  = cudaErrorInvalidValue;
#define NHB_STREAM_CASE(CH, MT) \
	if (ch_max == CH && M == MT) \
		e = launch_stream_t<CH, MT>(b, cfg, grid, smem);
		NHB_STREAM_CASE(1, 1)
		NHB_STREAM_CASE(2, 1)
		NHB_STREAM_CASE(3, 1)
		NHB_STREAM_CASE(4, 1)
		NHB_STREAM_CASE(1, 2)
		NHB_STREAM_CASE(2, 2)
		NHB_STREAM_CASE(3, 2)
		NHB_STREAM_CASE(4, 2)
		NHB_STREAM_CASE(1, 3)
		NHB_STREAM_CASE(2, 3)
		NHB_STREAM_CASE(1, 4)
		NHB_STREAM_CASE(2, 4)
		NHB_STREAM_CASE(1, 5)
		NHB_STREAM_CASE(1, 6)
		NHB_STREAM_CASE(1, 7)
		NHB_STREAM_CASE(1, 8)
#undef NHB_STREAM_CASE
		if (e == cudaSuccess && launches)
			*launches += 1;
		return e;
	}

	int gemv_ldg_max_m(int64_t K, int act_mode) {
		const int64_t per_m = act_mode == NHB_ACT_F32 ? K * 4 : K + (K / 32) * 4;
		int64_t m			= (160 * 1024) / per_m;
		if (m > 4)
			m = 4;
		return static_cast<int>(m);
	}

	cudaError_t launch_gemv_ldg(const int8_t* wq, const __half* wd, const float* x, long long ldx, float* y, long long ldy, int rows, int K, int M,
		int act_mode, const launch_cfg& cfg, int* launches) {
		const bool f32	  = act_mode == NHB_ACT_F32;
		const size_t smem = f32 ? static_cast<size_t>(M) * K * 4 : static_cast<size_t>(M) * (K + (K / 32) * 4);
		int grid		  = (rows + 7) / 8;
		const int cap	  = cfg.sm_count * 4;
		grid			  = grid > cap ? cap : grid;
		if (grid < 1)
			return cudaSuccess;
		cudaError_t e = cudaErrorInvalidValue;
#define NHB_LDG_CASE(MT, F) \
	if (M == MT && f32 == F) { \
		auto kern = gemv_q8_ldg<MT, F>; \
		e		  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem > 48 * 1024 ? smem : 48 * 1024)); \
		if (e == cudaSuccess) \
			e = launch_pdl(kern, dim3(grid), dim3(256), smem, cfg, wq, wd, x, ldx, y, ldy, rows, K); \
	}
		NHB_LDG_CASE(1, false)
		NHB_LDG_CASE(2, false)
		NHB_LDG_CASE(3, false)
		NHB_LDG_CASE(4, false)
		NHB_LDG_CASE(1, true)
		NHB_LDG_CASE(2, true)
		NHB_LDG_CASE(3, true)
		NHB_LDG_CASE(4, true)
#undef NHB_LDG_CASE
		if (e == cudaSuccess && launches)
			*launches += 1;
		return e;
	}

	cudaError_t launch_quantize(const float* x, long long ldx, int M, int K, int8_t* q, float* d, cudaStream_t s, bool pdl) {
		const long long tot = static_cast<long long>(M) * (K / 32);
		if (tot == 0)
			return cudaSuccess;
		long long grid = (tot + 127) / 128;
		grid		   = grid > 148 * 16 ? 148 * 16 : grid;
		launch_cfg cfg{};
		cfg.stream = s;
		cfg.pdl	   = pdl;
		return launch_pdl(quantize_q8_kernel, dim3(static_cast<int>(grid)), dim3(128), 0, cfg, x, ldx, M, K, q, d);
	}

	cudaError_t launch_block_dots(const int8_t* wq, const int8_t* qa, int rows, int K, int M, int32_t* dots, cudaStream_t s) {
		const long long tot = static_cast<long long>(M) * rows * (K / 32);
		if (tot == 0)
			return cudaSuccess;
		long long grid = (tot + 255) / 256;
		grid		   = grid > 148 * 16 ? 148 * 16 : grid;
		block_dots_kernel<<<static_cast<int>(grid), 256, 0, s>>>(wq, qa, rows, K, M, dots);
		return cudaGetLastError();
	}

}
