// rms_norm x norm-weight, the producer of a projection's activations: f32 rows, the int8 + f32-scale planes the
// decode GEMV reads, or 34-byte Q8_0 blocks.
//
// Arithmetic of the reference's rms_norm_mul kernel (include/nihilus-incl/cpu/avx_2.hpp:3907-3915), bit for bit:
//   sum   = simd_sum_squares (:758-779): eight accumulators, lane l takes x[8i + l] through one fma each in ascending i,
//           then (l, l + 4), (l, l + 2), (0, 1) pairwise adds;
//   scale = 1 / sqrtf_fast(sum / K + eps), sqrtf_fast either the IEEE root (cpu/common.hpp:310-312) or the integer
//           formula of the x86 build (cpu/common.hpp:448-450, about 2^64 too large as written);
//   y     = (x * w) * scale, two separate roundings (vec_scale_mul_f32, :3621-3850);
//   Q8_0  = quantize_row_q8_0 of that row (:671-721).
// The eight fma chains are sequential by definition (K / 8 dependent steps: about 1 us for K = 4096); everything
// around them is parallel: one CTA per row stages the row in shared memory with 16-byte loads, eight lanes run the
// chains from there, then every warp scales, quantises and stores 128 elements per pass.
#include "internal.h"
#include "ptx.cuh"
#include "q8_device.cuh"

namespace nhb {

	namespace {

		constexpr int NORM_TPB = 256;

		__global__ void __launch_bounds__(NORM_TPB)
			rms_norm_mul_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w, float eps, int sqrt_mode, int K, norm_out o) {
			extern __shared__ float4 row4[];
			__shared__ float s_scale;
			const float* row = reinterpret_cast<const float*>(row4);
			const int tid	 = threadIdx.x;
			const int m		 = blockIdx.x;
			const int k4	 = K >> 2;
			pdl_launch_dependents();
			pdl_wait_prior_grids();
			const float4* xg = reinterpret_cast<const float4*>(x + static_cast<size_t>(m) * ldx);
			for (int i = tid; i < k4; i += NORM_TPB)
				row4[i] = __ldg(xg + i);
			__syncthreads();
			if (tid < 8) {
				const float acc	 = sum_squares_lane(row + tid, K >> 3);
				const float quad = __fadd_rn(acc, __shfl_down_sync(0xffu, acc, 4));
				const float dual = __fadd_rn(quad, __shfl_down_sync(0xffu, quad, 2));
				const float sum	 = __fadd_rn(dual, __shfl_down_sync(0xffu, dual, 1));
				if (tid == 0) {
					const float v = __fadd_rn(__fdiv_rn(sum, static_cast<float>(K)), eps);
					float root;
					if (sqrt_mode == NHB_SQRT_X86_FAST)
						root = __uint_as_float(((__float_as_uint(v) + 0x3f800000u) >> 1) + 0x20000000u);
					else
						root = __fsqrt_rn(v);
					s_scale = __fdiv_rn(1.0f, root);
				}
			}
			__syncthreads();
			const float scale = s_scale;
			const int lane	  = tid & 31;
			const float4* wg  = reinterpret_cast<const float4*>(w);
			// a warp takes 32 float4 = four Q8 blocks per pass; eight lanes share a block
			for (int base = (tid >> 5) * 32; base < k4; base += NORM_TPB) {
				const int i		  = base + lane;
				const bool active = i < k4;
				float4 v		  = make_float4(0.f, 0.f, 0.f, 0.f);
				if (active) {
					const float4 xv = row4[i];
					const float4 wv = __ldg(wg + i);
					v.x				= __fmul_rn(__fmul_rn(xv.x, wv.x), scale);
					v.y				= __fmul_rn(__fmul_rn(xv.y, wv.y), scale);
					v.z				= __fmul_rn(__fmul_rn(xv.z, wv.z), scale);
					v.w				= __fmul_rn(__fmul_rn(xv.w, wv.w), scale);
					if (o.y)
						reinterpret_cast<float4*>(o.y + static_cast<size_t>(m) * o.ldy)[i] = v;
				}
				if (!o.q && !o.blocks)
					continue;
				float amax = absmax4(v, 0.f);
				amax	   = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
				amax	   = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
				amax	   = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
				if (!active)
					continue;
				const act_scale sc	= q8_scales(amax);
				const uint32_t pack = q8_pack4(v.x, v.y, v.z, v.w, sc.id);
				const int blk		= i >> 3;
				if (o.q) {
					reinterpret_cast<uint32_t*>(o.q + static_cast<size_t>(m) * K)[i] = pack;
					if ((lane & 7) == 0)
						o.d[static_cast<size_t>(m) * (K >> 5) + blk] = sc.d;
				}
				if (o.blocks) {
					// a 34-byte block is only 2-byte aligned: two 16-bit stores per lane
					unsigned char* b = o.blocks + (static_cast<size_t>(m) * (K >> 5) + blk) * 34;
					uint16_t* qs	 = reinterpret_cast<uint16_t*>(b + 2) + (lane & 7) * 2;
					qs[0]			 = static_cast<uint16_t>(pack & 0xffffu);
					qs[1]			 = static_cast<uint16_t>(pack >> 16);
					if ((lane & 7) == 0)
						*reinterpret_cast<uint16_t*>(b) = __half_as_ushort(__float2half_rn(sc.d));
				}
			}
		}

	}

	bool rms_norm_supports(long long K) {
		return K > 0 && K % 32 == 0 && K * 4 <= 200 * 1024;
	}

	cudaError_t launch_rms_norm(const float* x, long long ldx, const float* w, float eps, int sqrt_mode, int M, int K, const norm_out& o, cudaStream_t s,
		bool pdl) {
		if (M == 0)
			return cudaSuccess;
		const size_t smem = static_cast<size_t>(K) * 4;
		static bool raised[64] = {};
		int dev				   = 0;
		cudaGetDevice(&dev);
		if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !raised[dev]) {
			cudaError_t e = cudaFuncSetAttribute(rms_norm_mul_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
			if (e != cudaSuccess)
				return e;
			raised[dev] = true;
		}
		cudaLaunchConfig_t lc{};
		lc.gridDim			= dim3(M);
		lc.blockDim			= dim3(NORM_TPB);
		lc.dynamicSmemBytes = smem;
		lc.stream			= s;
		cudaLaunchAttribute attr[1];
		attr[0].id										   = cudaLaunchAttributeProgrammaticStreamSerialization;
		attr[0].val.programmaticStreamSerializationAllowed = 1;
		lc.attrs										   = attr;
		lc.numAttrs										   = pdl ? 1 : 0;
		return cudaLaunchKernelEx(&lc, rms_norm_mul_kernel, x, ldx, w, eps, sqrt_mode, K, o);
	}

}
