// nhb_mul_mat_q8_0_noalloc: the decode GEMV for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a mul_mat: an engine that
// reserved its whole device arena up front and hands out offsets from a fixed memory plan (the reference's
// memory_buffer works this way), or a latency-critical token loop where an allocation would mean an implicit
// device-wide synchronisation.  The regular entry points keep their
// temporary buffers in a context that grows them with cudaMalloc on demand; this one needs no context and no
// weight handle.  Its only temporary -- the activations after Q8_0 quantisation, which the quantiser kernel
// writes and the GEMV kernel reads -- lives in a fixed array that is part of the library image.
#include <mutex>
#include <string>

#include "internal.h"

#define NHB_NOALLOC_SCRATCH_BYTES (96 * 1024)

// Every GPU that loads the library carries these 96 KiB until the process exits.
static __device__ __align__(256) unsigned char nhb_noalloc_scratch[NHB_NOALLOC_SCRATCH_BYTES];

namespace {

	constexpr int MAX_DEVICES = 64;
	std::mutex g_mu;
	unsigned char* g_scratch_dev[MAX_DEVICES] = {};// device address of the array, per device ordinal
	thread_local std::string g_noalloc_err;

	int fail(int code, const std::string& msg) {
		g_noalloc_err = msg;
		return code;
	}

	// In host code `nhb_noalloc_scratch` names a host-side shadow of the symbol, not memory a kernel may touch;
	// the device address has to be asked for, once per device, with that device current.
	int scratch_for_current_device(unsigned char** out, int* device) {
		int dev		  = -1;
		cudaError_t e = cudaGetDevice(&dev);
		if (e != cudaSuccess)
			return fail(NHB_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
		if (dev < 0 || dev >= MAX_DEVICES)
			return fail(NHB_ERR_UNSUPPORTED, "device ordinal beyond 63");
		std::lock_guard<std::mutex> lock(g_mu);
		if (!g_scratch_dev[dev]) {
			void* p = nullptr;
			e		= cudaGetSymbolAddress(&p, nhb_noalloc_scratch);
			if (e != cudaSuccess || !p)
				return fail(NHB_ERR_CUDA, std::string("cudaGetSymbolAddress(nhb_noalloc_scratch): ") + cudaGetErrorString(e));
			g_scratch_dev[dev] = static_cast<unsigned char*>(p);
		}
		*out	= g_scratch_dev[dev];
		*device = dev;
		return NHB_OK;
	}

}

extern "C" {

const char* nhb_noalloc_last_error(void) {
	return g_noalloc_err.c_str();
}

int64_t nhb_noalloc_max_bytes(void) {
	return NHB_NOALLOC_SCRATCH_BYTES;
}

int nhb_mul_mat_q8_0_noalloc(const void* q_plane, const void* d_plane, int64_t rows, int64_t K, const float* x_dev, int64_t ldx, float* y_dev,
	int64_t ldy, int64_t M, void* cuda_stream) {
	using namespace nhb;
	if (rows < 0 || M < 0 || K <= 0 || K % 32 != 0)
		return fail(NHB_ERR_ARG, "rows and M must be >= 0 and K a positive multiple of 32");
	if (rows == 0 || M == 0)
		return NHB_OK;
	if (!q_plane || !d_plane || !x_dev || !y_dev)
		return fail(NHB_ERR_ARG, "null pointer");
	if (ldx < K || ldy < rows)
		return fail(NHB_ERR_ARG, "leading dimension smaller than the row length");
	if ((reinterpret_cast<uintptr_t>(q_plane) & 31) || (reinterpret_cast<uintptr_t>(d_plane) & 1) || (reinterpret_cast<uintptr_t>(x_dev) & 15) || (ldx & 3) ||
		(reinterpret_cast<uintptr_t>(y_dev) & 3))
		return fail(NHB_ERR_ARG, "the int8 plane must be 32-byte aligned, activations 16-byte aligned with ldx a multiple of 4, outputs 4-byte aligned");
	if (rows > (int64_t(1) << 30))
		return fail(NHB_ERR_ARG, "too many rows");
	const size_t need = gemv_rows_act_bytes(K, static_cast<int>(M > 4 ? 4 : M));
	if (M > 4 || need > NHB_NOALLOC_SCRATCH_BYTES || !gemv_rows_supports(K, M))
		return fail(NHB_ERR_UNSUPPORTED,
			"nhb_mul_mat_q8_0_noalloc: M = " + std::to_string(M) + ", K = " + std::to_string(K) + " needs " + std::to_string(M * (K + K / 8)) +
				" bytes of quantised activations; the fixed scratch holds at most M = 4 rows and 98304 bytes (M * (K + K/8) <= 98304)");
	unsigned char* scratch = nullptr;
	int dev				   = 0;
	int rc				   = scratch_for_current_device(&scratch, &dev);
	if (rc != NHB_OK)
		return rc;
	cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
	const int m			= static_cast<int>(M);
	const int k			= static_cast<int>(K);
	// 1. quantise the activations into the fixed array: int8 [M][K] then f32 scales [M][K/32] (every byte the GEMV
	//    reads is rewritten by this launch, so nothing of an earlier call survives where it matters)
	int8_t* qa	  = reinterpret_cast<int8_t*>(scratch);
	float* da	  = reinterpret_cast<float*>(scratch + static_cast<size_t>(m) * k);
	cudaError_t e = launch_quantize(x_dev, ldx, m, k, qa, da, stream, false);
	if (e != cudaSuccess)
		return fail(NHB_ERR_CUDA, std::string("quantize_q8 launch: ") + cudaGetErrorString(e));
	// 2. the warp-per-row GEMV, reading its activations from there
	rows_batch b{};
	b.n_ops		  = 1;
	b.n_slots	  = 1;
	b.slot_op[0]  = 0;
	b.preq		  = 1;
	b.preq_base	  = scratch;
	b.act_bytes	  = static_cast<int>(need);
	rows_op& op	  = b.op[0];
	op.wq		  = static_cast<const int8_t*>(q_plane);
	op.wd		  = static_cast<const __half*>(d_plane);
	op.x		  = x_dev;
	op.y		  = y_dev;
	op.ldx		  = ldx;
	op.ldy		  = ldy;
	op.rows		  = static_cast<int>(rows);
	op.K		  = k;
	op.act_off	  = 0;
	op.preq_off	  = 0;
	int sm_count  = 0;
	e			  = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
	if (e != cudaSuccess)
		return fail(NHB_ERR_CUDA, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
	launch_cfg cfg{};
	cfg.stream	 = stream;
	cfg.sm_count = sm_count;
	cfg.pdl		 = false;
	int launches = 0;
	e			 = launch_gemv_rows(b, m, cfg, 3, &launches);
	if (e != cudaSuccess)
		return fail(NHB_ERR_CUDA, std::string("gemv_q8_rows launch: ") + cudaGetErrorString(e));
	return NHB_OK;
}
}
