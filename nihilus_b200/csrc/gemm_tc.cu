// gemm_q8_tc: the prefill GEMM (sm_100a) -- TMA-fed tcgen05.mma with accumulators in tensor memory.
//
// Arithmetic is the reference's quantize_row_q8_0 + vec_dot_q8_0_q8_0 (include/nihilus-incl/cpu/avx_2.hpp
// :4439-4489, :4749-4780), unchanged: activations are quantised to Q8_0, every 32-wide block contributes
// float(exact int dot) * (d_w * d_a).  The tensor cores compute the exact int dot: both operands are the int8
// quants widened to fp16 (|q| <= 127 is exact in fp16, products and their 32-term sums are exact in the fp32
// accumulator), one accumulator stage per Q8 block, never accumulated across blocks.  The per-block scales
// are applied by the epilogue warps while the next block's MMA runs on the other accumulator stage.
//
// Layout per CTA: D[128 weight rows][N_T tokens] in TMEM (row = lane, token = column), two stages.
//   warp 0      TMA producer: A tile [128][64] fp16 of the weight's fp16 plane, B tile [N_T][64] fp16 of the
//               quantised activations (both K-major, 128-byte swizzle), and the activation scales of the two
//               Q8 blocks of the K slice (plain bulk copies).  No multicast.
//   warp 1      allocates TMEM, issues tcgen05.mma.kind::f16 (2 x K=16 per Q8 block) and the commits.
//   warps 4-19  epilogue (4 token-column groups x 4 TMEM lane quarters): tcgen05.ld the block's int dots,
//               acc = fma(P * d_w, d_a, acc) in registers, store Y.
// Every mbarrier wait is bounded; when one runs out the CTA records a code for the host, stops, frees its
// tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "internal.h"
#include "ptx.cuh"
#include "q8_device.cuh"

namespace nhb {

	namespace {

		constexpr int GM_ROWS	 = 128;// weight rows per CTA = MMA M
		constexpr int GM_KSLICE	 = 64;// fp16 elements per smem stage row = 128 bytes = two Q8 blocks
		constexpr int GM_EPI_WARPS = 16;// four per scheduler: their TMEM loads and FMAs overlap without manual pipelining
		constexpr int GM_THREADS   = (4 + GM_EPI_WARPS) * 32;// warpgroup 0: producer warp, MMA warp, two idle warps; then the epilogue warpgroups

		// ---- PTX: TMA, tcgen05 ----
		__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
			asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
							 smem_u32(dst_smem)),
				"l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
				: "memory");
		}
		__device__ __forceinline__ void bulk_g2s_plain(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
			asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)), "l"(src),
				"r"(bytes), "r"(smem_u32(bar))
				: "memory");
		}
		__device__ __forceinline__ void tmem_alloc(uint32_t* slot_smem, uint32_t ncols) {
			asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "r"(ncols) : "memory");
			asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
		}
		__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
			asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
		}
		__device__ __forceinline__ void tc_fence_before() {
			asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
		}
		__device__ __forceinline__ void tc_fence_after() {
			asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
		}
		// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate = 0 overwrites D
		__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
			asm volatile(
				"{\n"
				".reg .pred p;\n"
				"setp.ne.b32 p, %4, 0;\n"
				"tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
				"}\n" ::"r"(d_tmem),
				"l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
				: "memory");
		}
		// arrive on `bar` once every tcgen05 operation this thread issued so far has completed
		__device__ __forceinline__ void umma_commit(uint64_t* bar) {
			asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
		}
		[[maybe_unused]] __device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
			asm volatile(
				"tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
				: "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
				"=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
				"=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
				"=r"(v[31])
				: "r"(taddr)
				: "memory");
		}
		__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[32]) {
			asm volatile(
				"tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
				: "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
				"=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
				: "r"(taddr)
				: "memory");
		}
		__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[32]) {
			asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
						 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
						 : "r"(taddr)
						 : "memory");
		}
		__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&v)[32]) {
			asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr) : "memory");
		}
		__device__ __forceinline__ void tmem_ld_wait() {
			asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
		}

		// shared-memory matrix descriptor: K-major, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024 bytes apart
		__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
			uint64_t d = 0;
			d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);// start address
			d |= static_cast<uint64_t>(1) << 16;// leading byte offset (unused for swizzled K-major; canonical value 1)
			d |= static_cast<uint64_t>(1024 >> 4) << 32;// stride byte offset
			d |= static_cast<uint64_t>(1) << 46;// descriptor version (Blackwell)
			d |= static_cast<uint64_t>(2) << 61;// SWIZZLE_128B
			return d;
		}

		// instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n
		__host__ __device__ constexpr uint32_t idesc_f16(int n) {
			return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(GM_ROWS >> 4) << 24);
		}

		struct gemm_params {
			const __half* wd;// [rows][K/32] weight scales
			const float* daT;// [K/32][m_pad] activation scales, block-major
			float* y;// output, already offset to this shard's first column
			long long ldy;
			int rows;
			int K;
			int M;
			int m_pad;
		};

		template<int N_T> struct gemm_smem {
			static constexpr int a_bytes	 = GM_ROWS * GM_KSLICE * 2;// 16 KiB
			static constexpr int b_bytes	 = N_T * GM_KSLICE * 2;
			static constexpr int da_bytes	 = 2 * N_T * 4;// two Q8 blocks
			static constexpr int stage_bytes = a_bytes + b_bytes + ((da_bytes + 1023) / 1024) * 1024;
			static constexpr int stages		 = (200 * 1024) / stage_bytes > 6 ? 6 : (200 * 1024) / stage_bytes;
			static constexpr int head_bytes	 = 1024;// barriers + tmem slot
			static constexpr int total		 = head_bytes + stages * stage_bytes + 1024;// + alignment slack
		};

		struct gemm_head {
			uint64_t full[8];
			uint64_t empty[8];
			uint64_t tmem_full[2];
			uint64_t tmem_empty[2];
			uint32_t tmem_base;
			int abort_flag;
		};

		template<int N_T> __global__ void __launch_bounds__(GM_THREADS, 1)
			gemm_q8_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const gemm_params p, int* __restrict__ dev_status) {
			using L = gemm_smem<N_T>;
			constexpr int S			= L::stages;
			constexpr int CW		= N_T / 4;// token columns per epilogue warp
			constexpr uint32_t TCOLS = (2 * N_T) < 32 ? 32 : (2 * N_T);
			extern __shared__ unsigned char smem_raw[];
			// 1024-byte alignment for the 128-byte swizzle atoms
			unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
			gemm_head* hd		= reinterpret_cast<gemm_head*>(base);
			unsigned char* ring = base + L::head_bytes;

			const int tid	= threadIdx.x;
			const int warp	= tid >> 5;
			const int lane	= tid & 31;
			const int n0	= blockIdx.x * GM_ROWS;
			const int m0	= blockIdx.y * N_T;
			const int n_kb	= p.K / GM_KSLICE;
			const int n_blk = n_kb * 2;

			if (tid == 0) {
				for (int s = 0; s < S; ++s) {
					mbar_init(&hd->full[s], 1);
					mbar_init(&hd->empty[s], 1 + GM_EPI_WARPS);
				}
				for (int a = 0; a < 2; ++a) {
					mbar_init(&hd->tmem_full[a], 1);
					mbar_init(&hd->tmem_empty[a], GM_EPI_WARPS);
				}
				hd->abort_flag = 0;
				fence_mbar_init();
			}
			if (warp == 1)
				tmem_alloc(&hd->tmem_base, TCOLS);
			tc_fence_before();
			__syncthreads();
			tc_fence_after();
			const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&hd->tmem_base);
			pdl_launch_dependents();
			pdl_wait_prior_grids();// the quantised activations come from the kernel before this one

			// Registers follow the work: 20 warps put five on every scheduler, which caps a uniform allocation at 96 per
			// thread; warpgroup 0 (copy and MMA issue, a handful of registers) hands most of its share to the epilogue.
			if (warp < 4) {
				asm volatile("setmaxnreg.dec.sync.aligned.u32 32;" ::: "memory");
			if (warp == 0) {
				// ---------------- TMA producer ----------------
				if (lane == 0) {
					for (int kb = 0; kb < n_kb; ++kb) {
						const int s = kb % S;
						if (kb >= S && !mbar_wait(&hd->empty[s], ((kb / S) - 1) & 1)) {
							atomicExch(dev_status, DEV_TIMEOUT_EMPTY);
							break;
						}
						unsigned char* st = ring + static_cast<size_t>(s) * L::stage_bytes;
						mbar_expect_tx(&hd->full[s], L::a_bytes + L::b_bytes + L::da_bytes);
						tma_load_2d(st, &map_a, kb * GM_KSLICE, n0, &hd->full[s]);
						tma_load_2d(st + L::a_bytes, &map_b, kb * GM_KSLICE, m0, &hd->full[s]);
						float* da_s = reinterpret_cast<float*>(st + L::a_bytes + L::b_bytes);
						bulk_g2s_plain(da_s, p.daT + static_cast<size_t>(2 * kb) * p.m_pad + m0, N_T * 4, &hd->full[s]);
						bulk_g2s_plain(da_s + N_T, p.daT + static_cast<size_t>(2 * kb + 1) * p.m_pad + m0, N_T * 4, &hd->full[s]);
					}
				}
			} else if (warp == 1) {
				// ---------------- MMA issuer ----------------
				if (lane == 0) {
					constexpr uint32_t idesc = idesc_f16(N_T);
					for (int kb = 0; kb < n_kb; ++kb) {
						const int s = kb % S;
						if (!mbar_wait(&hd->full[s], (kb / S) & 1)) {
							atomicExch(dev_status, DEV_TIMEOUT_FULL);
							break;
						}
						tc_fence_after();
						const uint32_t a_addr = smem_u32(ring + static_cast<size_t>(s) * L::stage_bytes);
						const uint32_t b_addr = a_addr + L::a_bytes;
						bool ok				  = true;
#pragma unroll
						for (int j = 0; j < 2; ++j) {
							const int t = 2 * kb + j;// Q8 block index
							const int a = t & 1;// accumulator stage
							const int u = t >> 1;
							if (u >= 1 && !mbar_wait(&hd->tmem_empty[a], (u - 1) & 1)) {
								atomicExch(dev_status, DEV_TIMEOUT_MMA);
								ok = false;
								break;
							}
							tc_fence_after();
							const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(a * N_T);
#pragma unroll
							for (int k2 = 0; k2 < 2; ++k2) {
								const uint32_t off = static_cast<uint32_t>(j * 64 + k2 * 32);// bytes inside the 128-byte row
								umma_f16(d_tmem, smem_desc_sw128(a_addr + off), smem_desc_sw128(b_addr + off), idesc, k2);
							}
							umma_commit(&hd->tmem_full[a]);
						}
						if (!ok)
							break;
						umma_commit(&hd->empty[s]);// the slot's operands are free once these MMAs have run
					}
				}
			}
			} else {
				// ---------------- epilogue ----------------
				asm volatile("setmaxnreg.inc.sync.aligned.u32 112;" ::: "memory");
				const int e		   = warp - 4;// 0..15
				const int q		   = warp & 3;// TMEM lane quarter this warp may touch
				const int g		   = e >> 2;// which quarter of the token columns
				const int n_local  = q * 32 + lane;
				const int n		   = n0 + n_local;
				const bool n_valid = n < p.rows;
				const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
				const uint4* dw_row		 = reinterpret_cast<const uint4*>(p.wd + static_cast<size_t>(n_valid ? n : 0) * (p.K >> 5));
				float acc[CW];
#pragma unroll
				for (int i = 0; i < CW; ++i)
					acc[i] = 0.f;
				uint4 dw8 = make_uint4(0, 0, 0, 0);
				bool ok	  = true;
				for (int t = 0; t < n_blk && ok; ++t) {
					const int a	 = t & 1;
					const int u	 = t >> 1;
					const int kb = t >> 1;
					const int s	 = kb % S;
					if ((t & 7) == 0 && n_valid)
						dw8 = __ldg(dw_row + (t >> 3));// this row's next eight block scales
					if ((t & 1) == 0) {
						// the activation scales of this K slice were written by the async proxy: acquire them
						if (!mbar_wait(&hd->full[s], (kb / S) & 1)) {
							ok = false;
							break;
						}
					}
					if (!mbar_wait(&hd->tmem_full[a], u & 1)) {
						ok = false;
						break;
					}
					tc_fence_after();
					const uint32_t w32 = (t & 7) < 2 ? dw8.x : ((t & 7) < 4 ? dw8.y : ((t & 7) < 6 ? dw8.z : dw8.w));
					const float dw	   = __half2float(__ushort_as_half(static_cast<unsigned short>((t & 1) ? (w32 >> 16) : (w32 & 0xffffu))));
					const float* da_s  = reinterpret_cast<const float*>(ring + static_cast<size_t>(s) * L::stage_bytes + L::a_bytes + L::b_bytes) + (t & 1) * N_T + g * CW;
					const uint32_t col = static_cast<uint32_t>(a * N_T + g * CW);
					constexpr int CH   = CW >= 16 ? 16 : CW;// columns per tcgen05.ld
#pragma unroll
					for (int c0 = 0; c0 < CW; c0 += CH) {
						uint32_t v[32];
						if constexpr (CH == 16)
							tmem_ld16(lane_base + col + c0, v);
						else if constexpr (CH == 8)
							tmem_ld8(lane_base + col + c0, v);
						else
							tmem_ld4(lane_base + col + c0, v);
						tmem_ld_wait();
						if (c0 + CH >= CW) {
							// all of this block's dots are in registers: hand the accumulator stage back to the MMA warp
							tc_fence_before();
							__syncwarp();
							if (lane == 0)
								mbar_arrive(&hd->tmem_empty[a]);
						}
#pragma unroll
						for (int i = 0; i < CH; i += 4) {
							const float4 d4 = *reinterpret_cast<const float4*>(da_s + c0 + i);
							acc[c0 + i + 0] = fmaf(__uint_as_float(v[i + 0]) * dw, d4.x, acc[c0 + i + 0]);
							acc[c0 + i + 1] = fmaf(__uint_as_float(v[i + 1]) * dw, d4.y, acc[c0 + i + 1]);
							acc[c0 + i + 2] = fmaf(__uint_as_float(v[i + 2]) * dw, d4.z, acc[c0 + i + 2]);
							acc[c0 + i + 3] = fmaf(__uint_as_float(v[i + 3]) * dw, d4.w, acc[c0 + i + 3]);
						}
					}
					if (t & 1) {
						// done with the activation scales of this smem slot
						__syncwarp();
						if (lane == 0)
							mbar_arrive(&hd->empty[s]);
					}
				}
				if (!ok) {
					if (lane == 0)
						atomicExch(dev_status, DEV_TIMEOUT_MMA);
				} else if (n_valid) {
#pragma unroll
					for (int i = 0; i < CW; ++i) {
						const int m = m0 + g * CW + i;
						if (m < p.M)
							p.y[static_cast<size_t>(m) * p.ldy + n] = acc[i];
					}
				}
			}
			tc_fence_before();
			__syncthreads();
			if (warp == 1) {
				tc_fence_after();
				tmem_dealloc(tmem_base, TCOLS);
			}
		}

		// ---- helper kernels ----
		// int8 plane -> fp16 plane (exact), 16 values per thread
		__global__ void widen_i8_f16_kernel(const int8_t* __restrict__ q, __half* __restrict__ out, long long n16) {
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n16; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				const uint4 v		= __ldg(reinterpret_cast<const uint4*>(q) + i);
				const uint32_t w[4] = { v.x, v.y, v.z, v.w };
				__half2 o[8];
#pragma unroll
				for (int j = 0; j < 4; ++j) {
					o[2 * j]	 = __floats2half2_rn(static_cast<float>(static_cast<int8_t>(w[j] & 0xff)), static_cast<float>(static_cast<int8_t>((w[j] >> 8) & 0xff)));
					o[2 * j + 1] = __floats2half2_rn(static_cast<float>(static_cast<int8_t>((w[j] >> 16) & 0xff)), static_cast<float>(static_cast<int8_t>(w[j] >> 24)));
				}
				uint4* dst = reinterpret_cast<uint4*>(out) + 2 * i;
				dst[0]	   = *reinterpret_cast<uint4*>(&o[0]);
				dst[1]	   = *reinterpret_cast<uint4*>(&o[4]);
			}
		}

		// quantize_row_q8_0 for the GEMM: quants as fp16 [m_pad][K] (rows >= M zero), scales block-major [K/32][m_pad]
		__global__ void quantize_for_gemm_kernel(const float* __restrict__ x, long long ldx, int M, int m_pad, int K, __half* __restrict__ qa16,
			float* __restrict__ daT) {
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			const int nb		= K >> 5;
			const long long tot = static_cast<long long>(m_pad) * nb;
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < tot; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				const int m	  = static_cast<int>(i / nb);
				const int blk = static_cast<int>(i - static_cast<long long>(m) * nb);
				uint4* dst	  = reinterpret_cast<uint4*>(qa16 + static_cast<size_t>(m) * K + static_cast<size_t>(blk) * QK);
				if (m >= M) {
					const uint4 z = make_uint4(0, 0, 0, 0);
					dst[0] = z, dst[1] = z, dst[2] = z, dst[3] = z;
					daT[static_cast<size_t>(blk) * m_pad + m] = 0.f;
					continue;
				}
				const float4* p = reinterpret_cast<const float4*>(x + static_cast<size_t>(m) * ldx + static_cast<size_t>(blk) * QK);
				float4 v[8];
				float amax = 0.f;
#pragma unroll
				for (int j = 0; j < 8; ++j) {
					v[j] = __ldg(p + j);
					amax = fmaxf(fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))), amax);
				}
				const act_scale sc = q8_scales(amax);
				const float d	   = sc.d;
				__half2 o[16];
#pragma unroll
				for (int j = 0; j < 8; ++j) {
					const int q0 = q8_quant(v[j].x, sc.id);
					const int q1 = q8_quant(v[j].y, sc.id);
					const int q2 = q8_quant(v[j].z, sc.id);
					const int q3 = q8_quant(v[j].w, sc.id);
					o[2 * j]	 = __floats2half2_rn(static_cast<float>(q0), static_cast<float>(q1));
					o[2 * j + 1] = __floats2half2_rn(static_cast<float>(q2), static_cast<float>(q3));
				}
#pragma unroll
				for (int j = 0; j < 4; ++j)
					dst[j] = *reinterpret_cast<uint4*>(&o[4 * j]);
				daT[static_cast<size_t>(blk) * m_pad + m] = d;
			}
		}

		// ---- tensor maps ----
		typedef CUresult (*encode_fn_t)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
			const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

		encode_fn_t encode_fn() {
			static encode_fn_t fn = nullptr;
			static std::once_flag once;
			std::call_once(once, [] {
				void* p = nullptr;
				cudaDriverEntryPointQueryResult qres;
				if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
					fn = reinterpret_cast<encode_fn_t>(p);
			});
			return fn;
		}

		// fp16 [rows][K] row-major, box [box_rows][64], 128-byte swizzle, out-of-range rows read as zero
		bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
			encode_fn_t fn = encode_fn();
			if (!fn)
				return false;
			const cuuint64_t dims[2]	= { K, rows };
			const cuuint64_t strides[1] = { K * 2 };
			const cuuint32_t box[2]		= { GM_KSLICE, box_rows };
			const cuuint32_t estr[2]	= { 1, 1 };
			return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
					   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
		}

		int pick_nt(int M) {
			return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
		}

		template<int N_T> cudaError_t launch_t(const CUtensorMap& ma, const CUtensorMap& mb, const gemm_params& p, const launch_cfg& cfg) {
			auto kern		  = gemm_q8_tc<N_T>;
			const size_t smem = gemm_smem<N_T>::total;
			cudaError_t e	  = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
			if (e != cudaSuccess)
				return e;
			cudaLaunchConfig_t lc{};
			lc.gridDim			= dim3((p.rows + GM_ROWS - 1) / GM_ROWS, p.m_pad / N_T);
			lc.blockDim			= dim3(GM_THREADS);
			lc.dynamicSmemBytes = smem;
			lc.stream			= cfg.stream;
			cudaLaunchAttribute attr[1];
			attr[0].id										   = cudaLaunchAttributeProgrammaticStreamSerialization;
			attr[0].val.programmaticStreamSerializationAllowed = 1;
			lc.attrs										   = attr;
			lc.numAttrs										   = cfg.pdl ? 1 : 0;
			return cudaLaunchKernelEx(&lc, kern, ma, mb, p, cfg.dev_status);
		}

	}

	bool gemm_tc_supports(int64_t rows, int64_t K, int64_t M) {
		return rows >= 1 && K % 256 == 0 && K >= 256 && M >= 1 && M <= (1 << 16);
	}

	int gemm_tc_m_pad(int64_t M) {
		const int nt = pick_nt(static_cast<int>(M > 256 ? 256 : M));
		return static_cast<int>(((M + nt - 1) / nt) * nt);
	}

	// quantised activations: fp16 quants [m_pad][K], then block-major scales [K/32][m_pad]
	size_t gemm_tc_scratch_bytes(int64_t K, int64_t M) {
		const int64_t m_pad = gemm_tc_m_pad(M);
		return static_cast<size_t>(((m_pad * K * 2 + 255) & ~int64_t(255)) + (K / 32) * m_pad * 4);
	}

	cudaError_t launch_widen_i8_f16(const int8_t* q, __half* out, int64_t rows, int64_t K, cudaStream_t s) {
		const long long n16 = rows * K / 16;
		if (n16 == 0)
			return cudaSuccess;
		long long grid = (n16 + 255) / 256;
		grid		   = grid > 148 * 16 ? 148 * 16 : grid;
		widen_i8_f16_kernel<<<static_cast<int>(grid), 256, 0, s>>>(q, out, n16);
		return cudaGetLastError();
	}

	cudaError_t launch_gemm_tc(const __half* w16, const __half* wd, const float* x, long long ldx, float* y, long long ldy, int rows, int K, int M,
		void* scratch, const launch_cfg& cfg, int* launches, std::string* err) {
		const int nt	= pick_nt(M);
		const int m_pad = gemm_tc_m_pad(M);
		__half* qa16	= static_cast<__half*>(scratch);
		float* daT		= reinterpret_cast<float*>(static_cast<char*>(scratch) + ((static_cast<size_t>(m_pad) * K * 2 + 255) & ~size_t(255)));
		// 1. quantise the activations (fp16-widened quants + block-major scales)
		{
			const long long tot = static_cast<long long>(m_pad) * (K / 32);
			long long grid		= (tot + 127) / 128;
			grid				= grid > 148 * 16 ? 148 * 16 : grid;
			cudaLaunchConfig_t lc{};
			lc.gridDim	= dim3(static_cast<unsigned>(grid));
			lc.blockDim = dim3(128);
			lc.stream	= cfg.stream;
			cudaLaunchAttribute attr[1];
			attr[0].id										   = cudaLaunchAttributeProgrammaticStreamSerialization;
			attr[0].val.programmaticStreamSerializationAllowed = 1;
			lc.attrs										   = attr;
			lc.numAttrs										   = cfg.pdl ? 1 : 0;
			cudaError_t e = cudaLaunchKernelEx(&lc, quantize_for_gemm_kernel, x, ldx, M, m_pad, K, qa16, daT);
			if (e != cudaSuccess) {
				if (err)
					*err = "quantize_for_gemm launch";
				return e;
			}
			if (launches)
				*launches += 1;
		}
		// 2. tensor maps + the GEMM
		CUtensorMap ma, mb;
		if (!make_map(&ma, w16, static_cast<uint64_t>(rows), static_cast<uint64_t>(K), GM_ROWS) ||
			!make_map(&mb, qa16, static_cast<uint64_t>(m_pad), static_cast<uint64_t>(K), static_cast<uint32_t>(nt))) {
			if (err)
				*err = "cuTensorMapEncodeTiled failed";
			return cudaErrorInvalidValue;
		}
		gemm_params p{};
		p.wd	= wd;
		p.daT	= daT;
		p.y		= y;
		p.ldy	= ldy;
		p.rows	= rows;
		p.K		= K;
		p.M		= M;
		p.m_pad = m_pad;
		cudaError_t e;
		switch (nt) {
			case 16:
				e = launch_t<16>(ma, mb, p, cfg);
				break;
			case 32:
				e = launch_t<32>(ma, mb, p, cfg);
				break;
			case 64:
				e = launch_t<64>(ma, mb, p, cfg);
				break;
			case 128:
				e = launch_t<128>(ma, mb, p, cfg);
				break;
			default:
				e = launch_t<256>(ma, mb, p, cfg);
				break;
		}
		if (e != cudaSuccess) {
			if (err)
				*err = "gemm_q8_tc launch";
			return e;
		}
		if (launches)
			*launches += 1;
		return cudaSuccess;
	}

}
