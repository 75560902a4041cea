// Prelude for compiling the reference's own Q8_0 row-dot and quantiser helpers in place
// -- TEST INFRASTRUCTURE ONLY.
//
// build_ref.sh streams this file, then line ranges of the reference's
// include/nihilus-incl/cpu/common.hpp and cpu/avx_2.hpp (read where they lie, never copied into
// this repository), then ref_postlude.cpp, into one g++ invocation.  The code between prelude and
// postlude is the reference's, unmodified.  This prelude only supplies the few names that code
// expects from headers which cannot be included standalone, and two workarounds:
//
//  * the extracted helpers use aligned 256-bit loads/stores on block_q8_0::qs, which sits at
//    offset 2 of a 34-byte block and is therefore never 32-byte aligned; they are mapped to the
//    unaligned forms (same arithmetic);
//  * _mm_prefetch is called with a static_cast between unrelated pointer types, which is
//    ill-formed; prefetching has no arithmetic effect, so the macro swallows its arguments.
#include <immintrin.h>

#include <bit>
#include <cmath>
#include <cstdint>
#include <cstring>

#define NIHILUS_HOST inline

#undef _mm_prefetch
#define _mm_prefetch(...) (( void )0)
#define _mm256_load_si256 _mm256_loadu_si256
#define _mm256_store_si256 _mm256_storeu_si256
#define _mm256_load_ps _mm256_loadu_ps

namespace nihilus {

	inline constexpr uint64_t Q_SIZE{ 32 };// common/data_types.hpp:28
	using half = int16_t;// common/data_types.hpp:30

	template<typename half_type> struct block_q8_0 {// common/data_types.hpp:37-44
		half_type d;
		int8_t qs[Q_SIZE];
	};
	static_assert(sizeof(block_q8_0<half>) == 34);

	enum class device_types { cpu };

	namespace detail {
		template<typename a_t, typename b_t> constexpr a_t min(a_t a, b_t b) noexcept {// common/utility.hpp:117-120
			return a < static_cast<a_t>(b) ? a : static_cast<a_t>(b);
		}
	}

	constexpr float fp32_from_bits(uint32_t w) noexcept {// cpu/common.hpp:447-449
		return std::bit_cast<float>(w);
	}
	constexpr uint32_t fp32_to_bits(float f) noexcept {// cpu/common.hpp:451-453
		return std::bit_cast<uint32_t>(f);
	}
