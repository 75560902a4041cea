// Compiled (syntax only) by tests/test_cpp_operator.py when the reference's source tree is present: the dispatcher
// specialisations of include/nihilus_b200/mega_dispatch.inc, included unchanged inside namespace nihilus behind the
// reference's OWN forward declaration of kernel_dispatcher_impl (common/kernel_traits.hpp:382-383) and its own
// core_types / device_types / processing_phases, must be specialisations of that template -- and dispatching through
// it must reach them.
#include <nihilus-incl/common/kernel_traits.hpp>

#define NHB_DISPATCH_HOST_TYPES
#include <nihilus_b200/mul_mat_op.hpp>

namespace nihilus {
#include <nihilus_b200/mega_dispatch.inc>
}

namespace {
	using namespace nihilus_b200;
	using cfg	  = gpu_config<true>;
	using qkv	  = llama3_8b::qkv_core;
	using ffn	  = llama3_8b::down_core;
	using attn	  = llama3_8b::attn_out_core;
	using logits  = llama3_8b::logits_core;
	// the reference's primary template, its enumerators, arch index 2: complete types only because the block above
	// specialised them
	using d_qkv = nihilus::kernel_dispatcher_impl<cfg, qkv, nihilus::device_types::gpu, 2, nihilus::core_types::mega_qkv_prep_and_cache_publish,
		nihilus::processing_phases::eval_time>;
	using d_attn = nihilus::kernel_dispatcher_impl<cfg, attn, nihilus::device_types::gpu, 2, nihilus::core_types::mega_attention_apply,
		nihilus::processing_phases::prompt_eval_time>;
	using d_ffn = nihilus::kernel_dispatcher_impl<cfg, ffn, nihilus::device_types::gpu, 2, nihilus::core_types::mega_ffn, nihilus::processing_phases::eval_time>;
	using d_out = nihilus::kernel_dispatcher_impl<cfg, logits, nihilus::device_types::gpu, 2, nihilus::core_types::final_norm_and_sampling,
		nihilus::processing_phases::eval_time>;
	static_assert(sizeof(d_qkv) > 0 && sizeof(d_attn) > 0 && sizeof(d_ffn) > 0 && sizeof(d_out) > 0);
	static_assert(qkv::core_type == nihilus::core_types::mega_qkv_prep_and_cache_publish && logits::core_type == nihilus::core_types::final_norm_and_sampling);
}

void instantiate(qkv& a, attn& b, ffn& c, logits& d) {
	d_qkv::impl(a, 3);
	d_attn::impl(b, 3);
	d_ffn::impl(c, 3);
	d_out::impl(d);
}
