#!/usr/bin/env bash
# Builds oracle/_ref/libnihilus_ref.so from the reference's own sources, read where they lie.
# TEST INFRASTRUCTURE ONLY.  Nothing from the reference is written into this repository: the
# extracted line ranges are piped straight into the compiler and only the shared object lands in
# oracle/_ref/ (git-ignored).
#
#   usage: oracle/build_ref.sh <reference-root>     (or set NIHILUS_REFERENCE)
#
# Extracted ranges (all inside the reference's block comment, i.e. dead code there):
#   cpu/common.hpp 215-221   fp32_to_fp16 / fp16_to_fp32 (F16C)
#   cpu/common.hpp 448-450   sqrtf_fast (the x86 build's integer approximation)
#   cpu/avx_2.hpp 671-721    quantize_row_q8_0_avx2
#   cpu/avx_2.hpp 758-779    simd_sum_squares
#   cpu/avx_2.hpp 3621-3850  vec_scale_mul_f32<n>
#   cpu/avx_2.hpp 4418-4677  fp32_to_fp16_f16c, quantize_row_q8_0, int8 pair helpers, vec_dot_q8_0_q8_0<n<=16>
#   cpu/avx_2.hpp 4749-4852  vec_dot_q8_0_q8_0_impl, vec_dot_q8_f32<K>
#   cpu/avx_2.hpp 4881-4907  scalar_dot_product_q8_f32
# Skipped: 4679-4747 (names vec_dot_q8_0_q8_0<device_types::cpu, 1>, which is ill-formed).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ref="${1:-${NIHILUS_REFERENCE:-}}"
if [[ -z "$ref" ]]; then
	echo "build_ref: no reference root given (argument or NIHILUS_REFERENCE)" >&2
	exit 3
fi
common="$ref/include/nihilus-incl/cpu/common.hpp"
avx2="$ref/include/nihilus-incl/cpu/avx_2.hpp"
if [[ ! -f "$common" || ! -f "$avx2" ]]; then
	echo "build_ref: reference sources not found under $ref (keeping any prebuilt oracle/_ref)" >&2
	exit 3
fi
# the line numbers are only trusted while these anchors sit where expected
check() { # file line pattern
	sed -n "${2}p" "$1" | grep -q "$3" || { echo "build_ref: anchor '$3' not at $1:$2" >&2; exit 4; }
}
check "$common" 215 'fp32_to_fp16(float f)'
check "$common" 219 'fp16_to_fp32(half h)'
check "$common" 448 'sqrtf_fast(float x)'
check "$common" 450 '}'
check "$avx2" 671 'quantize_row_q8_0_avx2('
check "$avx2" 721 '}'
check "$avx2" 758 'simd_sum_squares('
check "$avx2" 779 '}'
check "$avx2" 3621 'struct vec_scale_mul_f32 {};'
check "$avx2" 3850 '};'
check "$avx2" 4418 'fp32_to_fp16_f16c(float f)'
check "$avx2" 4439 'quantize_row_q8_0('
check "$avx2" 4677 '};'
check "$avx2" 4749 'vec_dot_q8_0_q8_0_impl('
check "$avx2" 4852 '};'
check "$avx2" 4881 'scalar_dot_product_q8_f32('
check "$avx2" 4907 '}'
mkdir -p "$here/_ref"
{
	cat "$here/ref_prelude.hpp"
	sed -n '215,221p;448,450p' "$common"
	sed -n '671,721p;758,779p;3621,3850p;4418,4677p;4749,4852p;4881,4907p' "$avx2"
	cat "$here/ref_postlude.cpp"
} | g++ -x c++ -std=gnu++20 -O3 -mavx2 -mfma -mf16c -fPIC -shared -pthread -o "$here/_ref/libnihilus_ref.so" -
echo "build_ref: wrote $here/_ref/libnihilus_ref.so"
