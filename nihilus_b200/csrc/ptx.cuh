// Thin inline-PTX wrappers for sm_100a: mbarrier, bulk (TMA) copies, programmatic dependent launch,
// named barriers.  Every wait is bounded: it returns false after NHB_SPIN_LIMIT polls instead of
// spinning forever, and the caller turns that into a status word the host reads.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef NHB_SPIN_LIMIT
#define NHB_SPIN_LIMIT (1u << 21)
#endif

namespace nhb {

	__device__ __forceinline__ uint32_t smem_u32(const void* p) {
		return static_cast<uint32_t>(__cvta_generic_to_shared(p));
	}

	__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
		asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
	}

	__device__ __forceinline__ void fence_mbar_init() {
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}

	__device__ __forceinline__ void fence_proxy_async() {
		asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
	}

	__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
		asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
	}

	__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
		asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
	}

	__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
		uint32_t ok;
		asm volatile(
			"{\n"
			".reg .pred p;\n"
			"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
			"selp.u32 %0, 1, 0, p;\n"
			"}\n"
			: "=r"(ok)
			: "r"(smem_u32(bar)), "r"(parity)
			: "memory");
		return ok != 0;
	}

	// bounded wait; false = gave up
	__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
		for (uint32_t i = 0; i < NHB_SPIN_LIMIT; ++i) {
			if (mbar_try_wait(bar, parity))
				return true;
			if (i > 32)
				__nanosleep(40);
		}
		return false;
	}

	__device__ __forceinline__ uint64_t l2_policy_evict_first() {
		uint64_t pol;
		asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
		return pol;
	}

	// global -> shared bulk copy (TMA engine, no tensor map), completion counted in bytes on `bar`.
	// dst, src and bytes must be multiples of 16.
	__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar, uint64_t policy) {
		asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
						 smem_u32(dst_smem)),
			"l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
			: "memory");
	}

	// programmatic dependent launch: no-ops unless the launch carries the programmatic-serialization attribute
	__device__ __forceinline__ void pdl_launch_dependents() {
		asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
	}
	__device__ __forceinline__ void pdl_wait_prior_grids() {
		asm volatile("griddepcontrol.wait;" ::: "memory");
	}

	// named barrier over `nthreads` threads that also ANDs a predicate across them
	__device__ __forceinline__ bool named_bar_and(uint32_t id, uint32_t nthreads, bool pred) {
		uint32_t out;
		asm volatile(
			"{\n"
			".reg .pred p, q;\n"
			"setp.ne.u32 p, %3, 0;\n"
			"bar.red.and.pred q, %1, %2, p;\n"
			"selp.u32 %0, 1, 0, q;\n"
			"}\n"
			: "=r"(out)
			: "r"(id), "r"(nthreads), "r"(static_cast<uint32_t>(pred))
			: "memory");
		return out != 0;
	}

	// ---- thread-block clusters: distributed shared memory (plain remote stores, no multicast copies) ----
	__device__ __forceinline__ uint32_t cluster_size() {
		uint32_t n;
		asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
		return n;
	}
	__device__ __forceinline__ uint32_t cluster_rank() {
		uint32_t r;
		asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
		return r;
	}
	// address of the same shared-memory location in CTA `rank` of this cluster
	__device__ __forceinline__ uint32_t cluster_map(uint32_t local_smem_addr, uint32_t rank) {
		uint32_t a;
		asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_smem_addr), "r"(rank));
		return a;
	}
	__device__ __forceinline__ void cluster_st_v4(uint32_t addr, const uint4& v) {
		asm volatile("st.shared::cluster.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
	}
	__device__ __forceinline__ void cluster_st_f32(uint32_t addr, float v) {
		asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
	}
	// all threads of all CTAs of the cluster; remote stores issued before it are visible after it
	__device__ __forceinline__ void cluster_barrier() {
		asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
		asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
	}

	__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
		for (int o = 16; o > 0; o >>= 1)
			v += __shfl_xor_sync(0xffffffffu, v, o);
		return v;
	}

}
