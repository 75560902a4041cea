// gemm_q8_tc: the prefill GEMM (sm_100a) -- TMA-fed tcgen05.mma with accumulators in tensor memory.
//
// Arithmetic is the reference's quantize_row_q8_0 + vec_dot_q8_0_q8_0 (include/nihilus-incl/cpu/avx_2.hpp
// :4439-4489, :4749-4780), unchanged: activations are quantised to Q8_0, every 32-wide block contributes
// fma(float(exact int dot), d_w * d_a, acc).  The tensor cores compute the exact int dot: both operands are the
// int8 quants widened to fp16 (|q| <= 127 is exact in fp16, products and their 32-term sums are exact in the fp32
// accumulator), one accumulator stage per Q8 block, never accumulated across blocks.  The per-block scales are
// applied by the epilogue warps while the next block's MMA runs on the other accumulator stage.
//
// One CTA owns a tile of 128 "lane" rows x N_T "column" rows of the output, where either side may be the weight:
//   tokens < 128:  lanes = weight rows, columns = tokens (N_T = tokens rounded up to 16)
//   otherwise:     lanes = tokens,      columns = weight rows (N_T picked so the tile count fills whole waves)
// D[128][N_T] sits in TMEM (lane = TMEM lane, column = TMEM column), two stages of 256 columns.
//   warp 0      TMA producer: A tile [128][64] fp16, B tile [N_T][64] fp16 (both K-major, 128-byte swizzle) and the
//               f32 scales of the two Q8 blocks of the K slice for both sides (plain bulk copies).  No multicast.
//   warp 1      allocates TMEM, issues tcgen05.mma.kind::f16 (2 x K=16 per Q8 block) and the commits.
//   warps 4-19  epilogue (4 TMEM lane quarters x 4 column groups).  They read the accumulator with the 16x256b
//               shape, which gives every thread 4 lanes x 2 adjacent columns per 8 columns: a column scale fetched
//               from shared memory serves 4 rows (a lane-per-thread shape needs one shared-memory broadcast per
//               element and saturates the load/store unit), the 4 row scales live in registers.
// Every mbarrier wait is bounded; when one runs out the CTA records a code for the host, stops, frees its
// tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "internal.h"
#include "ptx.cuh"
#include "q8_device.cuh"

namespace nhb {

	namespace {

		constexpr int GM_ROWS	 = 128;// weight rows per CTA = MMA M
		constexpr int GM_KSLICE	 = 64;// fp16 elements per smem stage row = 128 bytes = two Q8 blocks
		// Epilogue warps: 4 TMEM lane quarters x 2, 3 or 4 column groups.  A warp pays a fixed cost per Q8 block (waits,
		// fences, scale fetches), so wide tiles do better with fewer, fatter warps -- as long as enough warps remain to
		// cover each other's TMEM round trips.  Measured (us, 12 against 16 warps): 512 tokens x 14336 rows 159 / 179,
		// 2048 x 14336 551 / 646, but 112-column tiles 165 / 151.  Eight warps with 232 registers: 208-column tiles
		// 143 against 159 with twelve (512 x 128256: 1203 / 1349), 224-column tiles 559 / 552.  32-column TMEM loads were
		// slower than 16-column ones in every shape.
		__host__ __device__ constexpr int gemm_epi_warps(int n_t) {
			return n_t >= 224 ? 12 : (n_t >= 208 ? 8 : (n_t >= 144 ? 12 : 16));
		}
		constexpr int GM_LDU = 2;// 8-column units fetched per TMEM load
		// Up to 32 tokens (tiles of 16 or 32 columns) sum K in chunks of 16 slices = 1024 values: a chunk is accumulated from
		// zero and the chunk totals are added in ascending order.  That order does not depend on how many CTAs share a tile, so
		// a tile's chunks can be dealt to several CTAs (K = 4096 walked by one CTA is 128 Q8 blocks in series, about 30 us
		// whatever the tile holds) and the result stays the same bits for every split, shard and GPU count.
		constexpr int GM_CHUNK_SLICES	  = 16;
		constexpr int GM_CHUNK_MAX_TOKENS = 32;
		constexpr size_t GM_COUNTER_BYTES = 16 * 1024;// one counter per tile of a split launch (fewer tiles than SMs)

		// ---- PTX: TMA, tcgen05 ----
		__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
			asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
							 dst_smem),
				"l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
				: "memory");
		}
		__device__ __forceinline__ void bulk_g2s_plain(uint32_t dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
			asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem), "l"(src),
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
		// mbarrier operations on a 32-bit shared address (the hot loops keep barrier addresses in registers)
		__device__ __forceinline__ bool mbar_try_a(uint32_t bar, uint32_t parity) {
			uint32_t ok;
			asm volatile(
				"{\n"
				".reg .pred p;\n"
				"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
				"selp.u32 %0, 1, 0, p;\n"
				"}\n"
				: "=r"(ok)
				: "r"(bar), "r"(parity)
				: "memory");
			return ok != 0;
		}
		// bounded wait; false = gave up.  The first poll usually succeeds, the loop is kept out of line of sight.
		__device__ __forceinline__ bool mbar_wait_a(uint32_t bar, uint32_t parity) {
			if (mbar_try_a(bar, parity))
				return true;
			for (uint32_t i = 0; i < NHB_SPIN_LIMIT; ++i) {
				if (mbar_try_a(bar, parity))
					return true;
				if (i > 32)
					__nanosleep(40);
			}
			return false;
		}
		__device__ __forceinline__ void mbar_arrive_a(uint32_t bar) {
			asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
		}
		__device__ __forceinline__ void umma_commit_a(uint32_t bar) {
			asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
		}
		// D[tmem] = A * B (overwrite) and D[tmem] += A * B, descriptors given as (low word, constant high word)
		__device__ __forceinline__ void umma_f16_set(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
			asm volatile(
				"{\n"
				".reg .pred p;\n"
				".reg .b64 da, db;\n"
				"setp.ne.b32 p, 0, 0;\n"
				"mov.b64 da, {%1, %3};\n"
				"mov.b64 db, {%2, %3};\n"
				"tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n"
				"}\n" ::"r"(d_tmem),
				"r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc)
				: "memory");
		}
		__device__ __forceinline__ void umma_f16_acc(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc) {
			asm volatile(
				"{\n"
				".reg .pred p;\n"
				".reg .b64 da, db;\n"
				"setp.eq.b32 p, 0, 0;\n"
				"mov.b64 da, {%1, %3};\n"
				"mov.b64 db, {%2, %3};\n"
				"tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n"
				"}\n" ::"r"(d_tmem),
				"r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc)
				: "memory");
		}
		// the two words of the shared-memory matrix descriptor below: only the 14-bit address field in the low word
		// changes from tile to tile (shared addresses stay below 256 KiB, so adding (bytes >> 4) never carries out of it)
		constexpr uint32_t GM_DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);// stride 1024 B, version 1, 128-byte swizzle
		__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) {
			return ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
		}


		// instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n
		__host__ __device__ constexpr uint32_t idesc_f16(int n) {
			return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(GM_ROWS >> 4) << 24);
		}

		constexpr int GM_TMEM_COLS = 512;// the whole tensor memory of the SM: one CTA per SM
		// accumulator stages: as many as fit, so the MMA warp can run several Q8 blocks ahead of the epilogue (narrow
		// tiles are bound by the latency of the MMA -> epilogue -> MMA hand-over, which more stages overlap)
		__host__ __device__ constexpr int gemm_stage_cols(int n_t) {
			return n_t <= 64 ? 64 : (n_t <= 128 ? 128 : 256);
		}

		struct gemm_params {
			const float* row_scale;// [K/32][lanes_pad]  scales of the lane side, block-major
			const float* col_scale;// [K/32][cols_pad]   scales of the column side, block-major
			float* y;// output, already offset to this shard's first column
			long long ldy;
			int lanes_pad, cols_pad;
			int lane_rows;// valid rows on the lane side (weight rows, or tokens when swapped)
			int col_rows;// valid rows on the column side
			int K;
			int swapped;// 0: lanes = weight rows, columns = tokens; 1: lanes = tokens, columns = weight rows
			int stages;
			// up to 32 tokens only (see GM_CHUNK_SLICES): K slices per CTA (a whole number of chunks), the scratch for
			// the chunk totals [chunk][tile][128][N_T] and one arrival counter per tile
			int chunked;// 1: at most 32 tokens
			int kb_per_cta;
			float* partial;
			unsigned* counters;
		};

		struct gemm_head {
			uint64_t full[8];
			uint64_t empty[8];
			uint64_t tmem_full[8];
			uint64_t tmem_empty[8];
			uint32_t tmem_base;
			int abort_flag;
			int last_cta;// split tiles: this CTA was the last of its tile to deliver its chunk totals
		};

		constexpr int GM_HEAD_BYTES = 1024;
		constexpr int GM_A_BYTES	= GM_ROWS * GM_KSLICE * 2;// 16 KiB

		// bytes of one pipeline stage: A tile, B tile, then [2 blocks][128 row scales + n_t column scales] floats
		__host__ __device__ constexpr int gemm_stage_bytes(int n_t) {
			return GM_A_BYTES + n_t * GM_KSLICE * 2 + ((2 * (GM_ROWS + n_t) * 4 + 1023) / 1024) * 1024;
		}

		// packed fp32 pairs: one issue slot, two IEEE fp32 results
		__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
			uint64_t r;
			asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
			return r;
		}
		__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
			asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
		}
		__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
			uint64_t r;
			asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
			return r;
		}
		__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
			uint64_t r;
			asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
			return r;
		}
		__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
			uint64_t r;
			asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
			return r;
		}
		__device__ __forceinline__ float lds_f32(uint32_t addr) {
			float v;
			asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
			return v;
		}
		__device__ __forceinline__ uint64_t lds_b64(uint32_t addr) {
			uint64_t v;
			asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(addr));
			return v;
		}
		// 16 lanes x 16 columns: thread t receives, for k = 0, 1: r[4k], r[4k+1] = lane t/4, columns
		// 8k + 2(t%4), +1 and r[4k+2], r[4k+3] = lane t/4 + 8, same columns (lanes relative to the lane in taddr)
		__device__ __forceinline__ void tmem_ld_16x256b(uint32_t taddr, uint32_t (&r)[8]) {
			asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
						 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
						 : "r"(taddr)
						 : "memory");
		}
		// Waits for the loads in flight.  The registers pass through the statement so that no use of them can be
		// scheduled ahead of the wait.
		__device__ __forceinline__ void tmem_ld_wait_regs(uint32_t (&a)[8], uint32_t (&b)[8]) {
			asm volatile("tcgen05.wait::ld.sync.aligned;"
						 : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]),
						 "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7])
						 :
						 : "memory");
		}
		__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) {
			uint64_t r;
			asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
			return r;
		}

		template<int N_T> __global__ void __launch_bounds__((4 + gemm_epi_warps(N_T)) * 32, 1)
			gemm_q8_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const gemm_params p, int* __restrict__ dev_status) {
			constexpr int STAGE_BYTES = gemm_stage_bytes(N_T);
			constexpr int B_BYTES	  = N_T * GM_KSLICE * 2;
			constexpr int SC_FLOATS	  = GM_ROWS + N_T;// scales of one Q8 block: lane side, then column side
			constexpr int UNITS		  = N_T / 8;// 8-column units in the tile, dealt to the four column groups
			constexpr int GM_EPI_WARPS = gemm_epi_warps(N_T);
			constexpr int GM_NG		   = GM_EPI_WARPS / 4;// column groups
			constexpr int BASE		  = UNITS / GM_NG;
			constexpr int REM		  = UNITS % GM_NG;
			constexpr int MAXU		  = BASE + (REM ? 1 : 0);
			constexpr int STAGE_COLS  = gemm_stage_cols(N_T);
			constexpr int NS		  = GM_TMEM_COLS / STAGE_COLS;// 2, 4 or 8 accumulator stages
			constexpr int PAIRS		  = (MAXU + GM_LDU - 1) / GM_LDU;// load groups of GM_LDU units
			extern __shared__ unsigned char smem_raw[];
			// 1024-byte alignment for the 128-byte swizzle atoms
			unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
			gemm_head* hd		= reinterpret_cast<gemm_head*>(base);
			const uint32_t ring = smem_u32(base + GM_HEAD_BYTES);

			const int tid	= threadIdx.x;
			const int warp	= tid >> 5;
			const int lane	= tid & 31;
			const int S		= p.stages;
			const int lane0 = blockIdx.x * GM_ROWS;// first lane-side row of this tile
			const int col0	= blockIdx.y * N_T;// first column-side row of this tile
			constexpr bool CAN_CHUNK = N_T <= GM_CHUNK_MAX_TOKENS;
			// chunked summation is a property of the token count alone (at most 32 tokens, which always sit on the columns), never
			// of the tile a shard happens to get: p.chunked is the host's (M <= 32)
			const bool chunked	 = CAN_CHUNK && p.chunked != 0;
			const int n_kb_all	 = p.K / GM_KSLICE;
			const int kb0		 = chunked ? static_cast<int>(blockIdx.z) * p.kb_per_cta : 0;// this CTA's first K slice
			const int n_kb		 = chunked ? min(p.kb_per_cta, n_kb_all - kb0) : n_kb_all;

			if (tid == 0) {
				for (int s = 0; s < S; ++s) {
					mbar_init(&hd->full[s], 1);
					mbar_init(&hd->empty[s], 1 + GM_EPI_WARPS);
				}
				for (int a = 0; a < NS; ++a) {
					mbar_init(&hd->tmem_full[a], 1);
					mbar_init(&hd->tmem_empty[a], GM_EPI_WARPS);
				}
				hd->abort_flag = 0;
				fence_mbar_init();
			}
			if (warp == 1)
				tmem_alloc(&hd->tmem_base, GM_TMEM_COLS);
			tc_fence_before();
			__syncthreads();
			tc_fence_after();
			const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&hd->tmem_base);
			pdl_launch_dependents();
			pdl_wait_prior_grids();// the quantised activations come from the kernel before this one

			// Registers follow the work: warpgroup 0 (copy and MMA issue, a handful of registers) hands most of its share
			// to the epilogue warps.
			if (warp < 4) {
				asm volatile("setmaxnreg.dec.sync.aligned.u32 32;" ::: "memory");
				if (warp == 0) {
					// ---------------- TMA producer ----------------
					if (lane == 0) {
						constexpr uint32_t tx = static_cast<uint32_t>(GM_A_BYTES + B_BYTES + 2 * SC_FLOATS * 4);
						const float* rsrc	  = p.row_scale + lane0 + static_cast<size_t>(2 * kb0) * p.lanes_pad;
						const float* csrc	  = p.col_scale + col0 + static_cast<size_t>(2 * kb0) * p.cols_pad;
						const uint32_t full0  = smem_u32(&hd->full[0]);
						const uint32_t empty0 = smem_u32(&hd->empty[0]);
						int s				  = 0;
						uint32_t ph			  = 1;// a fresh barrier reads as "phase 1 complete": the first S waits pass at once
						for (int kb = 0; kb < n_kb; ++kb) {
							if (!mbar_wait_a(empty0 + 8 * s, ph)) {
								atomicExch(dev_status, DEV_TIMEOUT_EMPTY);
								break;
							}
							const uint32_t st = ring + static_cast<uint32_t>(s) * STAGE_BYTES;
							mbar_expect_tx(&hd->full[s], tx);
							tma_load_2d(st, &map_a, (kb0 + kb) * GM_KSLICE, lane0, &hd->full[s]);
							tma_load_2d(st + GM_A_BYTES, &map_b, (kb0 + kb) * GM_KSLICE, col0, &hd->full[s]);
							const uint32_t sc = st + GM_A_BYTES + B_BYTES;
#pragma unroll
							for (int j = 0; j < 2; ++j) {
								bulk_g2s_plain(sc + j * SC_FLOATS * 4, rsrc, GM_ROWS * 4, &hd->full[s]);
								bulk_g2s_plain(sc + (j * SC_FLOATS + GM_ROWS) * 4, csrc, N_T * 4, &hd->full[s]);
								rsrc += p.lanes_pad;
								csrc += p.cols_pad;
							}
							if (++s == S) {
								s = 0;
								ph ^= 1;
							}
						}
					}
				} else if (warp == 1 || (NS >= 8 && warp == 2)) {
					// ---------------- MMA issuers ----------------
					// A thread that issues every MMA and commit of a K slice is the critical path of narrow tiles (about 370
					// cycles per Q8 block, all of it issue latency).  For tiles of up to 64 columns (eight accumulator stages) two
					// warps take alternate K slices: they then own disjoint accumulator stages and (the ring depth is even)
					// disjoint ring slots, so each barrier still has a single waiter that is never more than one phase ahead of
					// it.  Wider tiles are bound by the epilogue, where a second polling warp only costs issue slots (measured:
					// 2048 tokens x 4096 rows 163 -> 181 us), and with two stages both issuers would share them and a parity wait
					// could pass a phase early; there one warp issues everything.
					// Barrier addresses and descriptor words live in registers and only get incremented.
					constexpr uint32_t ISSUERS = NS >= 8 ? 2 : 1;
					if (lane == 0 && static_cast<uint32_t>(warp - 1) < ISSUERS) {
						const uint32_t first = static_cast<uint32_t>(warp - 1);// 0 or 1
						constexpr uint32_t idesc   = idesc_f16(N_T);
						const uint32_t full0	   = smem_u32(&hd->full[0]);
						const uint32_t empty0	   = smem_u32(&hd->empty[0]);
						const uint32_t tmem_full0  = smem_u32(&hd->tmem_full[0]);
						const uint32_t tmem_empty0 = smem_u32(&hd->tmem_empty[0]);
						uint32_t s = first, ph = 0;
						if (s >= static_cast<uint32_t>(S)) {// a one-slot ring: slice 1 is the second use of slot 0
							s -= S;
							ph ^= 1;
						}
						bool ok = true;
						for (int kb = static_cast<int>(first); kb < n_kb && ok; kb += ISSUERS) {
							const uint32_t a_lo = smem_desc_lo(ring + s * STAGE_BYTES);// descriptor low word of this slot's A tile
							if (!mbar_wait_a(full0 + 8 * s, ph)) {
								atomicExch(dev_status, DEV_TIMEOUT_FULL);
								break;
							}
							tc_fence_after();
							const uint32_t b_lo = a_lo + (GM_A_BYTES >> 4);
							// Q8 block t = 2 kb + j goes to accumulator stage t % NS, in its (t / NS)-th use
							const uint32_t a0	  = static_cast<uint32_t>(2 * kb) & (NS - 1);
							const uint32_t use_ph = (static_cast<uint32_t>(2 * kb) / NS) & 1u;
#pragma unroll
							for (uint32_t j = 0; j < 2; ++j) {
								const uint32_t a = a0 + j;
								if (!mbar_wait_a(tmem_empty0 + 8 * a, use_ph ^ 1u)) {
									atomicExch(dev_status, DEV_TIMEOUT_MMA);
									ok = false;
									break;
								}
								tc_fence_after();
								const uint32_t d_tmem = tmem_base + a * STAGE_COLS;
								// the block's two K = 16 steps sit 32 bytes apart inside the 128-byte rows: (j * 64 + k2 * 32) >> 4
								umma_f16_set(d_tmem, a_lo + 4 * j, b_lo + 4 * j, GM_DESC_HI, idesc);
								umma_f16_acc(d_tmem, a_lo + 4 * j + 2, b_lo + 4 * j + 2, GM_DESC_HI, idesc);
								umma_commit_a(tmem_full0 + 8 * a);
							}
							if (ok)
								umma_commit_a(empty0 + 8 * s);// the slot's operands are free once these MMAs have run
							s += ISSUERS;
							while (s >= static_cast<uint32_t>(S)) {
								s -= S;
								ph ^= 1;
							}
						}
					}
				}
			} else {
				// ---------------- epilogue ----------------
				// The CTA can only redistribute what it was launched with: 20 warps launch with 96 registers per thread, 128
				// threads release 64 each and 512 take 16 (-> 112); 16 warps launch with 128, 128 threads release 96 each and
				// 384 take 32 (-> 160).  Asking for more would wait forever for registers that never come.
				if constexpr (GM_EPI_WARPS == 16)
					asm volatile("setmaxnreg.inc.sync.aligned.u32 112;" ::: "memory");
				else if constexpr (GM_EPI_WARPS == 12)
					asm volatile("setmaxnreg.inc.sync.aligned.u32 160;" ::: "memory");
				else
					asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");// 12 warps launch with 168: 128 x 136 released >= 256 x 64 taken
				const int q		   = warp & 3;// TMEM lane quarter this warp may touch
				const int g		   = (warp - 4) >> 2;// column group
				const int t4	   = lane & 3;
				const int my_units = BASE + (g < REM ? 1 : 0);
				const int my_pairs = (my_units + GM_LDU - 1) / GM_LDU;
				const int col_off  = (BASE * g + (g < REM ? g : REM)) * 8;// first column of this warp inside the tile
				const int r0	   = q * 32 + (lane >> 2);// this thread's rows inside the tile: r0 + 8j, j = 0..3
				const uint32_t tl0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(col_off);
				const uint32_t tl1 = tl0 + (16u << 16);
				const uint32_t rs_off = static_cast<uint32_t>(GM_A_BYTES + B_BYTES + r0 * 4);
				const uint32_t cs_off = static_cast<uint32_t>(GM_A_BYTES + B_BYTES + (GM_ROWS + col_off + 2 * t4) * 4);
				uint64_t acc[4][MAXU > 0 ? MAXU : 1];
				uint64_t tot[4][(CAN_CHUNK && MAXU > 0) ? MAXU : 1];// chunk totals added up (narrow tiles walked by one CTA)
#pragma unroll
				for (int j = 0; j < 4; ++j)
#pragma unroll
					for (int i = 0; i < MAXU; ++i) {
						acc[j][i] = 0ull;
						if constexpr (CAN_CHUNK)
							tot[j][i] = 0ull;
					}
				// split tiles: where this thread's values sit inside a [128][N_T] tile of the scratch, and the tile's number
				const size_t n_tiles  = static_cast<size_t>(gridDim.x) * gridDim.y;
				const size_t tile_id  = static_cast<size_t>(blockIdx.x) * gridDim.y + blockIdx.y;
				const bool split_tile = chunked && gridDim.z > 1;
				const uint32_t full0	   = smem_u32(&hd->full[0]);
				const uint32_t empty0	   = smem_u32(&hd->empty[0]);
				const uint32_t tmem_full0  = smem_u32(&hd->tmem_full[0]);
				const uint32_t tmem_empty0 = smem_u32(&hd->tmem_empty[0]);
				bool ok		= true;
				int s		= 0;
				uint32_t ph = 0;
				// (two loops: the chunk boundary sits outside the loop over K slices, so that it is a branch taken once per chunk
				// and not a set of predicated moves in every slice)
				for (int kb = 0; kb < n_kb && ok;) {
				const int k_end = chunked ? min(n_kb, kb + GM_CHUNK_SLICES) : n_kb;
				for (; kb < k_end && ok; ++kb) {
					// the scales of this K slice were written by the async proxy: acquire them
					if (!mbar_wait_a(full0 + 8 * s, ph)) {
						ok = false;
						break;
					}
					const uint32_t st	  = ring + static_cast<uint32_t>(s) * STAGE_BYTES;
					const int a0		  = (2 * kb) & (NS - 1);
					const uint32_t use_ph = static_cast<uint32_t>((2 * kb) / NS) & 1u;
#pragma unroll
					for (int j = 0; j < 2; ++j) {
						const int a = a0 + j;
						uint64_t rs2[4];
#pragma unroll
						for (int i = 0; i < 4; ++i) {
							const float r = lds_f32(st + rs_off + (j * SC_FLOATS + 8 * i) * 4);
							rs2[i]		  = pack2(r, r);
						}
						if (!mbar_wait_a(tmem_full0 + 8 * a, use_ph)) {
							ok = false;
							break;
						}
						tc_fence_after();
						if (MAXU == 0 || my_units == 0) {
							// a narrow tile leaves this column group empty; the stage still counts this warp's release
							__syncwarp();
							if (lane == 0)
								mbar_arrive_a(tmem_empty0 + 8 * a);
						}
#pragma unroll
						for (int pr = 0; pr < PAIRS; ++pr) {
							if (pr < my_pairs) {
								uint32_t ra[4 * GM_LDU], rb[4 * GM_LDU];
								uint64_t va[2 * GM_LDU], vb[2 * GM_LDU], cs2[GM_LDU];
#pragma unroll
								for (int h = 0; h < GM_LDU; ++h)
									cs2[h] = lds_b64(st + cs_off + (j * SC_FLOATS + 8 * (GM_LDU * pr + h)) * 4);
								tmem_ld_16x256b(tl0 + a * STAGE_COLS + 8 * GM_LDU * pr, ra);
								tmem_ld_16x256b(tl1 + a * STAGE_COLS + 8 * GM_LDU * pr, rb);
								tmem_ld_wait_regs(ra, rb);
#pragma unroll
								for (int i = 0; i < 2 * GM_LDU; ++i) {
									va[i] = pack2u(ra[2 * i], ra[2 * i + 1]);
									vb[i] = pack2u(rb[2 * i], rb[2 * i + 1]);
								}
								if (pr == my_pairs - 1) {
									// all of this block's dots are in registers: hand the accumulator stage back to the MMA warp
									tc_fence_before();
									__syncwarp();
									if (lane == 0)
										mbar_arrive_a(tmem_empty0 + 8 * a);
								}
#pragma unroll
								for (int h = 0; h < GM_LDU; ++h) {
									const int un = GM_LDU * pr + h;
									const int ui = un < MAXU ? un : 0;// keeps the index in range where the unrolled body is dead
									if (un < MAXU && un < my_units) {
										acc[0][ui] = fma2(va[2 * h], mul2(rs2[0], cs2[h]), acc[0][ui]);
										acc[1][ui] = fma2(va[2 * h + 1], mul2(rs2[1], cs2[h]), acc[1][ui]);
										acc[2][ui] = fma2(vb[2 * h], mul2(rs2[2], cs2[h]), acc[2][ui]);
										acc[3][ui] = fma2(vb[2 * h + 1], mul2(rs2[3], cs2[h]), acc[3][ui]);
									}
								}
							}
						}
					}
					// done with the scales of this smem slot
					__syncwarp();
					if (ok && lane == 0)
						mbar_arrive_a(empty0 + 8 * s);
					if (++s == S) {
						s = 0;
						ph ^= 1;
					}
				}
					if constexpr (CAN_CHUNK) {
						if (chunked && ok) {
							// a chunk is complete: its total joins the running sum, or goes to the scratch for the CTA that sums the tile
							const size_t at = (static_cast<size_t>((kb0 + kb - 1) / GM_CHUNK_SLICES) * n_tiles + tile_id) * (GM_ROWS * N_T);
#pragma unroll
							for (int j = 0; j < 4; ++j)
#pragma unroll
								for (int un = 0; un < MAXU; ++un) {
									if (un < my_units) {
										if (split_tile)
											*reinterpret_cast<uint64_t*>(p.partial + at + (r0 + 8 * j) * N_T + col_off + 8 * un + 2 * t4) = acc[j][un];
										else
											tot[j][un] = add2(tot[j][un], acc[j][un]);
									}
									acc[j][un] = 0ull;
								}
						}
					}
				}
				const bool failed = !ok;
				bool writer		  = true;// this CTA stores the tile
				if constexpr (CAN_CHUNK) {
					if (split_tile) {
						// Every CTA of the tile has stored its chunk totals; the last one to arrive adds all chunks of the tile in
						// ascending order.  All epilogue warps pass both barriers whatever happened before (no early exit).
						__threadfence();
						asm volatile("bar.sync 1, %0;" ::"n"(GM_EPI_WARPS * 32) : "memory");
						if (tid == 128) {
							const unsigned prev = atomicAdd(p.counters + tile_id, 1u);
							const int last		= prev == gridDim.z - 1 ? 1 : 0;
							if (last)
								p.counters[tile_id] = 0u;// ready for the next launch
							hd->last_cta = last;
						}
						asm volatile("bar.sync 1, %0;" ::"n"(GM_EPI_WARPS * 32) : "memory");
						writer = *reinterpret_cast<volatile int*>(&hd->last_cta) != 0;
						if (writer) {
							__threadfence();
							const int n_chunks = (n_kb_all + GM_CHUNK_SLICES - 1) / GM_CHUNK_SLICES;
							constexpr int RB   = MAXU <= 1 ? 4 : 2;// chunks fetched together: the loads of a batch are all in flight before the first add
							for (int c0 = 0; c0 < n_chunks; c0 += RB) {
								float2 v[RB][4][MAXU > 0 ? MAXU : 1];
#pragma unroll
								for (int cc = 0; cc < RB; ++cc) {
									const float* src = p.partial + (static_cast<size_t>(min(c0 + cc, n_chunks - 1)) * n_tiles + tile_id) * (GM_ROWS * N_T);
#pragma unroll
									for (int j = 0; j < 4; ++j)
#pragma unroll
										for (int un = 0; un < MAXU; ++un)
											if (un < my_units)
												v[cc][j][un] = __ldcg(reinterpret_cast<const float2*>(src + (r0 + 8 * j) * N_T + col_off + 8 * un + 2 * t4));
								}
#pragma unroll
								for (int cc = 0; cc < RB; ++cc)
									if (c0 + cc < n_chunks) {
#pragma unroll
										for (int j = 0; j < 4; ++j)
#pragma unroll
											for (int un = 0; un < MAXU; ++un)
												if (un < my_units)
													tot[j][un] = add2(tot[j][un], pack2(v[cc][j][un].x, v[cc][j][un].y));
									}
							}
						}
					}
					if (chunked) {
#pragma unroll
						for (int j = 0; j < 4; ++j)
#pragma unroll
							for (int un = 0; un < MAXU; ++un)
								acc[j][un] = tot[j][un];
					}
				}
				if (failed) {
					if (lane == 0)
						atomicExch(dev_status, DEV_TIMEOUT_MMA);
				} else if (writer) {
#pragma unroll
					for (int j = 0; j < 4; ++j) {
						const int lr = lane0 + r0 + 8 * j;// lane-side row
						if (lr < p.lane_rows) {
#pragma unroll
							for (int un = 0; un < MAXU; ++un) {
								if (un < my_units) {
									float v[2];
									unpack2(acc[j][un], v[0], v[1]);
#pragma unroll
									for (int c = 0; c < 2; ++c) {
										const int cr = col0 + col_off + 8 * un + 2 * t4 + c;// column-side row
										if (cr < p.col_rows) {
											// swapped: lane = token, column = weight row; otherwise the other way round
											const size_t idx = p.swapped ? static_cast<size_t>(lr) * p.ldy + cr : static_cast<size_t>(cr) * p.ldy + lr;
											p.y[idx]		 = v[c];
										}
									}
								}
							}
						}
					}
				}
			}
			tc_fence_before();
			__syncthreads();
			if (warp == 1) {
				tc_fence_after();
				tmem_dealloc(tmem_base, GM_TMEM_COLS);
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

		// weight scales fp16 [rows][nb] -> f32 block-major [nb][rows_pad] through a 32 x 32 shared-memory tile
		__global__ void scales_block_major_kernel(const __half* __restrict__ wd, int rows, int nb, int rows_pad, float* __restrict__ out) {
			__shared__ float tile[32][33];
			const int r_base = blockIdx.x * 32, b_base = blockIdx.y * 32;
			for (int i = threadIdx.y; i < 32; i += blockDim.y) {
				const int r = r_base + i, b = b_base + threadIdx.x;
				tile[i][threadIdx.x] = (r < rows && b < nb) ? __half2float(wd[static_cast<size_t>(r) * nb + b]) : 0.f;
			}
			__syncthreads();
			for (int i = threadIdx.y; i < 32; i += blockDim.y) {
				const int b = b_base + i, r = r_base + threadIdx.x;
				if (b < nb && r < rows_pad)
					out[static_cast<size_t>(b) * rows_pad + r] = tile[threadIdx.x][i];
			}
		}

		// quantize_row_q8_0 for the GEMM: quants as fp16 [M][K], scales block-major [K/32][m_pad]
		__global__ void quantize_for_gemm_kernel(const float* __restrict__ x, long long ldx, int M, int m_pad, int K, __half* __restrict__ qa16,
			float* __restrict__ daT) {
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			const int nb		= K >> 5;
			const long long tot = static_cast<long long>(M) * nb;
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < tot; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				const int m		= static_cast<int>(i / nb);
				const int blk	= static_cast<int>(i - static_cast<long long>(m) * nb);
				uint4* dst		= reinterpret_cast<uint4*>(qa16 + static_cast<size_t>(m) * K + static_cast<size_t>(blk) * QK);
				const float4* p = reinterpret_cast<const float4*>(x + static_cast<size_t>(m) * ldx + static_cast<size_t>(blk) * QK);
				float4 v[8];
				float amax = 0.f;
#pragma unroll
				for (int j = 0; j < 8; ++j) {
					v[j] = __ldg(p + j);
					amax = fmaxf(fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))), amax);
				}
				const act_scale sc = q8_scales(amax);
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
				daT[static_cast<size_t>(blk) * m_pad + m] = sc.d;
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

		int round_up(int v, int m) {
			return ((v + m - 1) / m) * m;
		}

	}

	// Tile shape for `rows` weight rows and M tokens on `sms` SMs.  Both orientations and every column count from 16
	// to 256 are priced as waves x columns per tile; the lane side always holds 128 rows.
	gemm_plan gemm_tc_plan(int64_t rows, int64_t M, int sms) {
		gemm_plan best{};
		double best_cost = 1e300;
		for (int swapped = 0; swapped < (M <= GM_CHUNK_MAX_TOKENS ? 1 : 2); ++swapped) {// up to 32 tokens always sit on the columns
			const int64_t lane_rows = swapped ? M : rows;
			const int64_t col_rows	= swapped ? rows : M;
			const int64_t lane_tiles = (lane_rows + GM_ROWS - 1) / GM_ROWS;
			const int n_t_max		= static_cast<int>(std::min<int64_t>(256, ((col_rows + 15) / 16) * 16));
			for (int n_t = 16; n_t <= n_t_max; n_t += 16) {
				const int64_t col_tiles = (col_rows + n_t - 1) / n_t;
				const int64_t tiles		= lane_tiles * col_tiles;
				const int64_t waves		= (tiles + sms - 1) / sms;
				// measured: a tile's time per Q8 block is close to proportional to its width (0.32 us at 112 columns, 0.62 at
				// 208 and 224) down to a floor of about 64 columns' worth, and 256 columns cost a little more per column
				const double cost = static_cast<double>(waves) * (std::max(n_t, 64) + 8.0) * (n_t > 240 ? 1.08 : 1.0);
				if (cost < best_cost - 1e-9) {
					best_cost	   = cost;
					best.swapped   = swapped;
					best.n_t	   = n_t;
					best.lane_tiles = static_cast<int>(lane_tiles);
					best.col_tiles	= static_cast<int>(col_tiles);
				}
			}
		}
		return best;
	}

	bool gemm_tc_supports(int64_t rows, int64_t K, int64_t M) {
		return rows >= 1 && K % 64 == 0 && K >= 64 && M >= 1 && M <= (1 << 16) && rows <= (int64_t(1) << 30);
	}

	// padded row counts of the block-major scale planes: any tile of up to 256 rows that starts inside stays inside
	int gemm_tc_pad(int64_t n) {
		return round_up(static_cast<int>(n), 256) + 256;
	}

	// How a narrow tile's K chunks are dealt to CTAs: as many CTAs per tile as it takes to put about one CTA on every SM
	// (never more than there are chunks).  Any answer gives the same bits; this one is about speed only.
	static int gemm_tc_ctas_per_tile(const gemm_plan& plan, int K, int64_t M, int sms, int* kb_per_cta) {
		const int n_kb	   = K / GM_KSLICE;
		const int n_chunks = (n_kb + GM_CHUNK_SLICES - 1) / GM_CHUNK_SLICES;
		const int tiles	   = plan.lane_tiles * plan.col_tiles;
		const bool chunked = M <= GM_CHUNK_MAX_TOKENS;
		int want		   = 1;
		if (chunked && tiles < sms)
			want = std::min(n_chunks, std::max(1, sms / tiles));
		const int chunks_per_cta = (n_chunks + want - 1) / want;
		*kb_per_cta				 = chunked ? chunks_per_cta * GM_CHUNK_SLICES : n_kb;
		return chunked ? (n_chunks + chunks_per_cta - 1) / chunks_per_cta : 1;
	}

	// Scratch of the GEMM: the quantised activations (fp16 quants [M][K], block-major scales [K/32][pad(M)]) and, for split
	// tiles, the chunk totals [chunk][tile][128][columns].  The arrival counters of split tiles live in a buffer of their own
	// (gemm_tc_counter_bytes, zero between launches).
	size_t gemm_tc_scratch_bytes(int64_t K, int64_t M, int64_t rows, int sms) {
		size_t n = static_cast<size_t>(((M * K * 2 + 255) & ~int64_t(255)) + (K / 32) * gemm_tc_pad(M) * 4);
		n		 = (n + 255) & ~size_t(255);
		const gemm_plan plan = gemm_tc_plan(rows, M, sms);
		int kb_per_cta		 = 0;
		if (gemm_tc_ctas_per_tile(plan, static_cast<int>(K), M, sms, &kb_per_cta) > 1) {
			const size_t n_chunks = static_cast<size_t>((K / GM_KSLICE + GM_CHUNK_SLICES - 1) / GM_CHUNK_SLICES);
			n += n_chunks * plan.lane_tiles * plan.col_tiles * GM_ROWS * plan.n_t * sizeof(float);
		}
		return n;
	}
	size_t gemm_tc_counter_bytes() {
		return GM_COUNTER_BYTES;
	}

	// fp16 copy of the quants and block-major f32 copy of the scales, made once per weight
	cudaError_t launch_weight_gemm_planes(const int8_t* q, const __half* d, int64_t rows, int64_t K, __half* w16, float* wdT, cudaStream_t s) {
		const long long n16 = rows * K / 16;
		if (n16 == 0)
			return cudaSuccess;
		long long grid = (n16 + 255) / 256;
		grid		   = grid > 148 * 16 ? 148 * 16 : grid;
		widen_i8_f16_kernel<<<static_cast<int>(grid), 256, 0, s>>>(q, w16, n16);
		const int nb	   = static_cast<int>(K / 32);
		const int rows_pad = gemm_tc_pad(rows);
		dim3 g((rows_pad + 31) / 32, (nb + 31) / 32);
		scales_block_major_kernel<<<g, dim3(32, 8), 0, s>>>(d, static_cast<int>(rows), nb, rows_pad, wdT);
		return cudaGetLastError();
	}

	cudaError_t launch_gemm_tc(const __half* w16, const float* wdT, const float* x, long long ldx, float* y, long long ldy, int rows, int K, int M,
		void* scratch, unsigned* counters, const launch_cfg& cfg, int* launches, std::string* err, bool activations_ready) {
		const int m_pad	   = gemm_tc_pad(M);
		char* const sbase  = static_cast<char*>(scratch);
		__half* qa16	   = reinterpret_cast<__half*>(sbase);
		float* daT		   = reinterpret_cast<float*>(sbase + ((static_cast<size_t>(M) * K * 2 + 255) & ~size_t(255)));
		float* partial	   = reinterpret_cast<float*>(
			sbase + ((((static_cast<size_t>(M) * K * 2 + 255) & ~size_t(255)) + static_cast<size_t>(K / 32) * m_pad * 4 + 255) & ~size_t(255)));
		cudaLaunchAttribute attr[1];
		attr[0].id										   = cudaLaunchAttributeProgrammaticStreamSerialization;
		attr[0].val.programmaticStreamSerializationAllowed = 1;
		// 1. quantise the activations (fp16-widened quants + block-major scales), unless the previous mul_mat of the same
		//    batch left exactly these in the scratch (q, k, v and gate, up share their input)
		if (!activations_ready) {
			const long long tot = static_cast<long long>(M) * (K / 32);
			long long grid		= (tot + 127) / 128;
			grid				= grid > 148 * 16 ? 148 * 16 : grid;
			cudaLaunchConfig_t lc{};
			lc.gridDim	= dim3(static_cast<unsigned>(grid));
			lc.blockDim = dim3(128);
			lc.stream	= cfg.stream;
			lc.attrs	= attr;
			lc.numAttrs = cfg.pdl ? 1 : 0;
			cudaError_t e = cudaLaunchKernelEx(&lc, quantize_for_gemm_kernel, x, ldx, M, m_pad, K, qa16, daT);
			if (e != cudaSuccess) {
				if (err)
					*err = "quantize_for_gemm launch";
				return e;
			}
			if (launches)
				*launches += 1;
		}
		// 2. tile shape, tensor maps, the GEMM
		const gemm_plan plan = gemm_tc_plan(rows, M, cfg.sm_count);
		CUtensorMap ma, mb;
		const void* a_base	  = plan.swapped ? static_cast<const void*>(qa16) : static_cast<const void*>(w16);
		const void* b_base	  = plan.swapped ? static_cast<const void*>(w16) : static_cast<const void*>(qa16);
		const uint64_t a_rows = plan.swapped ? M : rows;
		const uint64_t b_rows = plan.swapped ? rows : M;
		if (!make_map(&ma, a_base, a_rows, static_cast<uint64_t>(K), GM_ROWS) || !make_map(&mb, b_base, b_rows, static_cast<uint64_t>(K), static_cast<uint32_t>(plan.n_t))) {
			if (err)
				*err = "cuTensorMapEncodeTiled failed";
			return cudaErrorInvalidValue;
		}
		gemm_params p{};
		p.row_scale	  = plan.swapped ? daT : wdT;
		p.col_scale	  = plan.swapped ? wdT : daT;
		p.lanes_pad	  = plan.swapped ? m_pad : gemm_tc_pad(rows);
		p.cols_pad	  = plan.swapped ? gemm_tc_pad(rows) : m_pad;
		p.y			  = y;
		p.ldy		  = ldy;
		p.lane_rows	  = static_cast<int>(a_rows);
		p.col_rows	  = static_cast<int>(b_rows);
		p.K			  = K;
		p.swapped		  = plan.swapped;
		p.partial		  = partial;
		p.counters		  = counters;
		p.chunked				= M <= GM_CHUNK_MAX_TOKENS ? 1 : 0;
		const int ctas_per_tile = gemm_tc_ctas_per_tile(plan, K, M, cfg.sm_count, &p.kb_per_cta);
		const int stage_b = gemm_stage_bytes(plan.n_t);
		p.stages		  = std::min(8, (200 * 1024) / stage_b);
		if (gemm_stage_cols(plan.n_t) <= 64 && p.stages >= 2)
			p.stages &= ~1;// two issuer warps alternate over the ring: an even depth gives each its own slots
		const size_t smem = static_cast<size_t>(GM_HEAD_BYTES) + static_cast<size_t>(p.stages) * stage_b + 1024;
		void (*kern)(const CUtensorMap, const CUtensorMap, const gemm_params, int*) = nullptr;
		switch (plan.n_t) {
#define NHB_GEMM_CASE(n) \
	case n: \
		kern = gemm_q8_tc<n>; \
		break;
			NHB_GEMM_CASE(16)
			NHB_GEMM_CASE(32)
			NHB_GEMM_CASE(48)
			NHB_GEMM_CASE(64)
			NHB_GEMM_CASE(80)
			NHB_GEMM_CASE(96)
			NHB_GEMM_CASE(112)
			NHB_GEMM_CASE(128)
			NHB_GEMM_CASE(144)
			NHB_GEMM_CASE(160)
			NHB_GEMM_CASE(176)
			NHB_GEMM_CASE(192)
			NHB_GEMM_CASE(208)
			NHB_GEMM_CASE(224)
			NHB_GEMM_CASE(240)
			NHB_GEMM_CASE(256)
#undef NHB_GEMM_CASE
			default:
				if (err)
					*err = "no GEMM kernel for this tile width";
				return cudaErrorInvalidValue;
		}
		const cudaError_t attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
		if (attr_err != cudaSuccess) {
			if (err)
				*err = "cudaFuncSetAttribute(gemm_q8_tc)";
			return attr_err;
		}
		cudaLaunchConfig_t lc{};
		lc.gridDim			= dim3(plan.lane_tiles, plan.col_tiles, ctas_per_tile);
		lc.blockDim			= dim3((4 + gemm_epi_warps(plan.n_t)) * 32);
		lc.dynamicSmemBytes = smem;
		lc.stream			= cfg.stream;
		lc.attrs			= attr;
		lc.numAttrs			= cfg.pdl ? 1 : 0;
		cudaError_t e		= cudaLaunchKernelEx(&lc, kern, ma, mb, p, cfg.dev_status);
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

