// Tensor-core (tcgen05 / TMEM) Q8_0 GEMM for prefill-sized M -- placeholder until the kernel lands.
#include "internal.h"

namespace nhb {

	bool gemm_tc_supports(int64_t, int64_t, int64_t) {
		return false;
	}

	size_t gemm_tc_scratch_bytes(int64_t, int64_t) {
		return 0;
	}

	cudaError_t launch_gemm_tc(const int8_t*, const __half*, const float*, long long, float*, long long, int, int, int, void*, const launch_cfg&, int*,
		std::string* err) {
		if (err)
			*err = "tensor-core GEMM not built";
		return cudaErrorNotSupported;
	}

}
