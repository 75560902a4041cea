// The element-wise neighbours of the reference's mul_mats in its FFN and attention cores, as kernels of their own for the
// paths where they are not fused into the GEMV (the tensor-core GEMM, and callers that want the intermediate):
//   ffn_silu -> ffn_gate_par   h = silu(gate) * up        (include/nihilus-incl/infra/core_traits.hpp:982-986)
//   residual_add               y = y + residual           (:771-772, :991-992)
// The reference's kernels for them are empty (cpu/avx_2.hpp:1946-2075, 5325-5330); the traits name the arithmetic: f32
// throughout, silu(g) = g / (1 + exp(-g)).
#include "internal.h"
#include "ptx.cuh"
#include "q8_device.cuh"

namespace nhb {

	namespace {

		__global__ void swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up, long long ld, float* __restrict__ h, long long ldh, int M, int K) {
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			const long long k4	= K >> 2;
			const long long tot = static_cast<long long>(M) * k4;
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < tot; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				const long long m = i / k4, j = i - m * k4;
				const float4 g = __ldg(reinterpret_cast<const float4*>(gate + m * ld) + j);
				const float4 u = __ldg(reinterpret_cast<const float4*>(up + m * ld) + j);
				reinterpret_cast<float4*>(h + m * ldh)[j] = swiglu4(g, u);
			}
		}

		// y[m][n] += res[m][n] for n in [0, cols)
		__global__ void add_rows_kernel(float* __restrict__ y, long long ldy, const float* __restrict__ res, long long ldr, int M, int cols) {
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			const long long tot = static_cast<long long>(M) * cols;
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < tot; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				const long long m = i / cols, n = i - m * cols;
				y[m * ldy + n]	  = __fadd_rn(y[m * ldy + n], __ldg(res + m * ldr + n));
			}
		}

		template<typename kern_t, typename... args_t> cudaError_t launch_ew(kern_t kern, long long work, cudaStream_t s, bool pdl, args_t... args) {
			long long grid = (work + 255) / 256;
			grid		   = grid > 148 * 8 ? 148 * 8 : (grid < 1 ? 1 : grid);
			cudaLaunchConfig_t lc{};
			lc.gridDim	= dim3(static_cast<unsigned>(grid));
			lc.blockDim = dim3(256);
			lc.stream	= s;
			cudaLaunchAttribute attr[1];
			attr[0].id										   = cudaLaunchAttributeProgrammaticStreamSerialization;
			attr[0].val.programmaticStreamSerializationAllowed = 1;
			lc.attrs										   = attr;
			lc.numAttrs										   = pdl ? 1 : 0;
			return cudaLaunchKernelEx(&lc, kern, args...);
		}

	}

	// gate, up, h: 16-byte aligned rows (ld, ldh multiples of 4), K % 4 == 0
	cudaError_t launch_swiglu(const float* gate, const float* up, long long ld, float* h, long long ldh, int M, int K, cudaStream_t s, bool pdl) {
		if (M == 0 || K == 0)
			return cudaSuccess;
		return launch_ew(swiglu_kernel, static_cast<long long>(M) * (K >> 2), s, pdl, gate, up, ld, h, ldh, M, K);
	}

	cudaError_t launch_add_rows(float* y, long long ldy, const float* res, long long ldr, int M, int cols, cudaStream_t s, bool pdl) {
		if (M == 0 || cols == 0)
			return cudaSuccess;
		return launch_ew(add_rows_kernel, static_cast<long long>(M) * cols, s, pdl, y, ldy, res, ldr, M, cols);
	}

}
