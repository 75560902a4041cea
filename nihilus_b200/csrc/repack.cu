// Upload-time repack of GGUF Q8_0 tensors (sm_100a).
//
// The reference copies each tensor's 34-byte blocks {fp16 d; int8 qs[32]} to the GPU verbatim
// (include/nihilus-incl/infra/model_parser.hpp:151-154).  34-byte strides defeat every aligned vector load,
// so the raw bytes are staged on the device and split once into an int8 plane [rows][K] and an fp16 plane
// [rows][K/32]; both planes start 256-byte aligned and every row of the int8 plane is 32-byte aligned.
#include "internal.h"

namespace nhb {

	namespace {

		// one thread per block; the staging buffer is 2-byte aligned at every block (34 is even)
		__global__ void repack_kernel(const uint16_t* __restrict__ src, long long n_blocks, int8_t* __restrict__ q, __half* __restrict__ d) {
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_blocks; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				const uint16_t* b = src + i * 17;
				uint32_t w[8];
#pragma unroll
				for (int j = 0; j < 8; ++j)
					w[j] = static_cast<uint32_t>(b[1 + 2 * j]) | (static_cast<uint32_t>(b[2 + 2 * j]) << 16);
				reinterpret_cast<__half_raw*>(d)[i].x = b[0];
				uint4* dst							  = reinterpret_cast<uint4*>(q + i * 32);
				dst[0]								  = make_uint4(w[0], w[1], w[2], w[3]);
				dst[1]								  = make_uint4(w[4], w[5], w[6], w[7]);
			}
		}

		__global__ void unpack_kernel(const int8_t* __restrict__ q, const __half* __restrict__ d, long long n_blocks, uint16_t* __restrict__ dst) {
			for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_blocks; i += static_cast<long long>(gridDim.x) * blockDim.x) {
				uint16_t* b		   = dst + i * 17;
				b[0]			   = reinterpret_cast<const __half_raw*>(d)[i].x;
				const uint16_t* qs = reinterpret_cast<const uint16_t*>(q + i * 32);
#pragma unroll
				for (int j = 0; j < 16; ++j)
					b[1 + j] = qs[j];
			}
		}

		int grid_for(long long n) {
			long long g = (n + 255) / 256;
			return static_cast<int>(g > 148 * 32 ? 148 * 32 : (g < 1 ? 1 : g));
		}
	}

	// rows*K/32 consecutive blocks -> planes (the planes are plain row-major, so blocks map 1:1)
	cudaError_t launch_repack(const uint8_t* blocks34, int64_t rows, int64_t K, int8_t* q, __half* d, cudaStream_t s) {
		const long long n = rows * (K / 32);
		if (n == 0)
			return cudaSuccess;
		repack_kernel<<<grid_for(n), 256, 0, s>>>(reinterpret_cast<const uint16_t*>(blocks34), n, q, d);
		return cudaGetLastError();
	}

	cudaError_t launch_unpack(const int8_t* q, const __half* d, int64_t rows, int64_t K, uint8_t* blocks34, cudaStream_t s) {
		const long long n = rows * (K / 32);
		if (n == 0)
			return cudaSuccess;
		unpack_kernel<<<grid_for(n), 256, 0, s>>>(q, d, n, reinterpret_cast<uint16_t*>(blocks34));
		return cudaGetLastError();
	}

}
