// Host-only C++23 mirror of the reference's operator interface for ONE op: the Q8_0 mul_mat.
//
// The reference describes every op of its graph with compile-time traits and runs it through
//   kernel_dispatcher_impl<config, core_traits, device, arch_index, core_type, phase>::impl(params[, block])
// (include/nihilus-incl/common/kernel_traits.hpp:121-213 dims, :393-417 mul_mat checks, :382-383 dispatcher
// forward declaration; include/nihilus-incl/infra/monolithic_dispatcher.hpp:41-62 call site).  Its GPU
// specialisations exist for arch index 4 only and are empty (include/nihilus-incl/cuda/cuda_12.hpp:803-952).
// This header offers the same shapes in namespace nihilus_b200 with arch index 2 (compute capability 10) and
// forwards each mul_mat to the C ABI of libnihilus_b200.so.  It is never seen by nvcc.  The dispatcher
// specialisations themselves live in mega_dispatch.inc, written against the reference's six template parameters
// and enumerator names, so that the same text can be included inside `namespace nihilus` behind the reference's
// own headers (define NHB_DISPATCH_HOST_TYPES there: this header then leaves the enums and the primary template
// to the host's declarations).
//
// What is mirrored, with the reference's meaning:
//   core_trait_dims<d0,d1,d2,d3[,runtime]>   four extents, ne0 contiguous; `runtime` names the extent that is
//                                             patched per step (the sequence length), 5 = none
//   kernel_traits<kernel_types::mul_mat,...>  in0 = weights [K,N], in1 = activations [K,M], out = [N,M]; the
//                                             same static checks as the reference
//   processing_phases                         eval_time (M = 1) / prompt_eval_time (M = sequence length); here
//                                             the split is taken at run time from M by the library
//   kernel_dispatcher_impl<config, core_traits, device_types::gpu, 2, core_types::mega_*, phase>
//                                             impl(params, current_block) for the per-block cores, impl(params) for
//                                             final_norm_and_sampling
// Errors follow include/nihilus-incl/common/exception.hpp:65-108: a failing call throws (config::exceptions) or
// logs and exits with -1.
#pragma once

#include <array>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <source_location>
#include <stdexcept>
#include <string>
#include <tuple>
#include <type_traits>
#include <utility>

#include "../nihilus_b200.h"

namespace nihilus_b200 {

#ifdef NHB_DISPATCH_HOST_TYPES
	// behind the reference's own headers: its enums are the ones the dispatcher is keyed on
	using ::nihilus::core_types;
	using ::nihilus::device_types;
	using ::nihilus::processing_phases;
	enum class kernel_types : uint8_t { weights, rms_norm, mul, mul_mat };
#else
	enum class device_types : uint8_t { cpu, gpu };
	enum class processing_phases { prompt_eval_time, eval_time };
	enum class kernel_types : uint8_t { weights, rms_norm, mul, mul_mat };
	// the cores of the reference's graph (include/nihilus-incl/common/config.hpp:214-223), same names, same order
	enum class core_types : uint8_t {
		weights,
		global_inputs,
		token_embeddings,
		mega_qkv_prep_and_cache_publish,
		mega_attention_apply,
		mega_ffn,
		final_norm_and_sampling,
		count,
	};
#endif
	enum class data_types : uint64_t { f32 = 0, f16 = 1, q8_0 = 8 };

	// compute-capability major -> the reference's build-time arch index (cmake/detection/main.cpp:33-44): 10 -> 2
	inline constexpr uint64_t gpu_arch_index_sm100 = 2;

	// the 34-byte block of the reference (include/nihilus-incl/common/data_types.hpp:28-44), for sizes only
	struct block_q8_0 {
		uint16_t d;
		int8_t qs[32];
	};
	static_assert(sizeof(block_q8_0) == 34);

	inline constexpr uint64_t no_runtime_dim = 5;

	template<uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t runtime = no_runtime_dim> struct core_trait_dims {
		static_assert(runtime < 4 || runtime == no_runtime_dim, "runtime dimension index must be 0..3 or 5 (none)");
		static constexpr uint64_t runtime_dim = runtime;
		mutable std::array<uint64_t, 4> rt{ d0, d1, d2, d3 };

		static constexpr std::array<uint64_t, 4> get_array() {
			return { d0, d1, d2, d3 };
		}
		std::array<uint64_t, 4> get_array_rt() const {
			return rt;
		}
		// the extent the engine patches before every launch (dim_updater, infra/behavioral_axes.hpp:184-220)
		uint64_t& get_seq_length_dim() const
			requires(runtime < 4)
		{
			return rt[runtime];
		}
	};

	// an operand: extents + element type + where its data lives.  For Q8_0 weights `data` is the nhb_weight handle
	// that nhb_weight_upload_q8_0 returned (per-block weights keep one handle per transformer block).
	template<typename dims_type_new, typename element_type_new, uint64_t block_count = 1> struct operand : public dims_type_new {
		using dims_type	   = dims_type_new;
		using element_type = element_type_new;
		static constexpr uint64_t blocks = block_count;
		std::array<void*, block_count> data{};
		void* get_data(uint64_t block = 0) const {
			return data[block_count == 1 ? 0 : block];
		}
	};

	template<kernel_types, typename...> struct kernel_traits;

	// mul_mat: out[N,M,b2,b3] = in0[K,N,..]^T . in1[K,M,..]; the checks of common/kernel_traits.hpp:403-416
	template<typename output_type_new, typename input_01_type_new, typename input_02_type_new>
	struct kernel_traits<kernel_types::mul_mat, output_type_new, input_01_type_new, input_02_type_new> {
		using output_type	= output_type_new;
		using input_01_type = input_01_type_new;
		using input_02_type = input_02_type_new;
		static constexpr auto input_01_dims = input_01_type::get_array();
		static constexpr auto input_02_dims = input_02_type::get_array();
		static constexpr auto output_dims	= output_type::get_array();
		static_assert(input_01_dims[0] == input_02_dims[0], "mul_mat: inner dimensions must match");
		static_assert(output_dims[0] == input_01_dims[1], "mul_mat: output rows must equal the first input's columns");
		static_assert(output_dims[1] == input_02_dims[1], "mul_mat: output columns must equal the second input's columns");
		static_assert(output_dims[2] == input_01_dims[2] || output_dims[2] == input_02_dims[2], "mul_mat: batch dimension 2 must match an input");
		static_assert(output_dims[3] == input_01_dims[3] || output_dims[3] == input_02_dims[3], "mul_mat: batch dimension 3 must match an input");
		static_assert(std::is_same_v<typename input_01_type::element_type, block_q8_0>, "this library implements Q8_0 weights only");
		static_assert(std::is_same_v<typename input_02_type::element_type, float> && std::is_same_v<typename output_type::element_type, float>,
			"activations and outputs are f32 (kernel_type_profile_traits<q8_gqa>)");
		static_assert(input_01_dims[0] % 32 == 0, "K must be a multiple of the Q8_0 block size");
		static constexpr int64_t K = static_cast<int64_t>(input_01_dims[0]);
		static constexpr int64_t N = static_cast<int64_t>(input_01_dims[1]);
		// output extents as the reference derives them (get_new_dims_new_2, common/kernel_traits.hpp:1115-1150)
		static constexpr std::array<uint64_t, 4> derived_output_dims() {
			return { input_01_dims[1], input_02_dims[1], input_02_dims[2], input_01_dims[3] };
		}
	};

	// rms_norm: one input, output of the same extents (common/kernel_traits.hpp:904-922)
	template<typename output_type_new, typename input_01_type_new> struct kernel_traits<kernel_types::rms_norm, output_type_new, input_01_type_new> {
		using output_type	= output_type_new;
		using input_01_type = input_01_type_new;
		static constexpr auto input_01_dims = input_01_type::get_array();
		static constexpr auto output_dims	= output_type::get_array();
		static_assert(input_01_dims[0] == output_dims[0], "rms_norm: input dimension 0 must match output");
		static_assert(input_01_dims[1] == output_dims[1], "rms_norm: input dimension 1 must match output");
		static_assert(input_01_dims[2] == output_dims[2], "rms_norm: input dimension 2 must match output");
		static_assert(input_01_dims[3] == output_dims[3], "rms_norm: input dimension 3 must match output");
		static_assert(std::is_same_v<typename input_01_type::element_type, float> && std::is_same_v<typename output_type::element_type, float>, "rms_norm works on f32");
		static_assert(input_01_dims[0] % 32 == 0, "the row length must be a multiple of the Q8_0 block size");
		static constexpr int64_t K = static_cast<int64_t>(input_01_dims[0]);
	};

	// mul: element-wise, the second input broadcast over dimensions 1-3 (common/kernel_traits.hpp:446-471)
	template<typename output_type_new, typename input_01_type_new, typename input_02_type_new>
	struct kernel_traits<kernel_types::mul, output_type_new, input_01_type_new, input_02_type_new> {
		using output_type	= output_type_new;
		using input_01_type = input_01_type_new;
		using input_02_type = input_02_type_new;
		static constexpr auto input_01_dims = input_01_type::get_array();
		static constexpr auto input_02_dims = input_02_type::get_array();
		static constexpr auto output_dims	= output_type::get_array();
		static_assert(input_01_dims[0] == input_02_dims[0], "mul: element-wise dimension 0 must match");
		static_assert(input_01_dims[1] == input_02_dims[1] || input_02_dims[1] == 1, "mul: dimension 1 must match or be broadcast");
		static_assert(input_01_dims[2] == input_02_dims[2] || input_02_dims[2] == 1, "mul: dimension 2 must match or be broadcast");
		static_assert(input_01_dims[3] == input_02_dims[3] || input_02_dims[3] == 1, "mul: dimension 3 must match or be broadcast");
		static_assert(output_dims[0] == input_01_dims[0] && output_dims[1] == input_01_dims[1] && output_dims[2] == input_01_dims[2] &&
				output_dims[3] == input_01_dims[3],
			"mul: output dimensions must match the first input");
		static_assert(input_02_dims[1] == 1 && input_02_dims[2] == 1 && input_02_dims[3] == 1, "this library multiplies by a norm weight: one row, broadcast");
	};

	struct mul_mat_error : std::runtime_error {
		int status;
		mul_mat_error(int s, const std::string& m) : std::runtime_error(m), status(s) {
		}
	};

	// the reference's convention: throw when the configuration enables exceptions, otherwise log and exit(-1)
	template<bool exceptions> inline void raise(int status, const char* what, const nhb_ctx* ctx, std::source_location loc = std::source_location::current()) {
		std::string msg = std::string(what) + ": " + nhb_last_error(ctx) + " (" + loc.file_name() + ":" + std::to_string(loc.line()) + ")";
		if constexpr (exceptions) {
			throw mul_mat_error(status, msg);
		} else {
			std::fprintf(stderr, "%s\n", msg.c_str());
			std::exit(-1);
		}
	}

	// One mul_mat of a core: which weight meets which activation.  `activation` and `output` hold device pointers,
	// `weight` holds nhb_weight handles.
	template<typename traits_type_new> struct mul_mat_node {
		using traits_type = traits_type_new;
		typename traits_type::input_01_type weight;
		typename traits_type::input_02_type activation;
		typename traits_type::output_type output;

		// tokens in this step: the activation's runtime extent when it has one, else its static ne1
		int64_t token_count() const {
			using act = typename traits_type::input_02_type;
			if constexpr (act::runtime_dim < 4)
				return static_cast<int64_t>(activation.get_array_rt()[1]);
			else
				return static_cast<int64_t>(traits_type::input_02_dims[1]);
		}
		nhb_mul_mat_op describe(uint64_t block) const {
			nhb_mul_mat_op op{};
			op.w   = static_cast<const nhb_weight*>(weight.get_data(block));
			op.x   = static_cast<const float*>(activation.get_data());
			op.ldx = traits_type::K;
			op.y   = static_cast<float*>(output.get_data());
			op.ldy = traits_type::N;
			op.M   = token_count();
			return op;
		}
	};

	// What a configuration must say for this path (a subset of the reference's model_config).
	template<bool exceptions_new = true, int act_mode_new = NHB_ACT_Q8> struct gpu_config {
		static constexpr device_types device_type = device_types::gpu;
		static constexpr bool exceptions		  = exceptions_new;
		static constexpr int act_mode			  = act_mode_new;
	};

	// A core as the dispatcher sees it: the library context plus the independent mul_mats of one stage
	// (q/k/v share one launch, gate/up share one launch).
	template<core_types core_type_new, typename... node_types> struct mul_mat_core {
		static constexpr core_types core_type = core_type_new;// which of the reference's cores this stage belongs to
		nhb_ctx* ctx						  = nullptr;
		std::tuple<node_types...> nodes;
		static constexpr size_t node_count = sizeof...(node_types);
	};

	// The rms_norm -> mul pair in front of a stage (infra/core_traits.hpp:570-573 and 971-974: attn_norm before q/k/v,
	// ffn_norm before gate/up).  `input` is the hidden state before the norm, `norm_weight` the f32 norm weight row.
	template<typename rms_norm_traits_new, typename mul_traits_new> struct norm_mul_node {
		using rms_norm_traits = rms_norm_traits_new;
		using mul_traits	  = mul_traits_new;
		static_assert(std::is_same_v<typename mul_traits::input_01_type, typename rms_norm_traits::output_type>, "mul takes the rms_norm's output");
		typename rms_norm_traits::input_01_type input;
		typename mul_traits::input_02_type norm_weight;
		float eps	  = 1e-5f;// model_traits: layer_norm_rms_epsilon
		int sqrt_mode = NHB_SQRT_IEEE;
		// first row of `input` the stage reads: 0, or sequence length - 1 for the last-token view in front of the final norm
		// (infra/core_traits.hpp:1184)
		int64_t first_row = 0;
	};

	// A stage whose mul_mats all read the normalised row: the norm is fused in front of them.  The mul_mat nodes'
	// `activation` pointers are not read; their extents still carry the token count.
	template<core_types core_type_new, typename norm_node_type, typename... node_types> struct norm_mul_mat_core {
		static constexpr core_types core_type = core_type_new;
		nhb_ctx* ctx						  = nullptr;
		norm_node_type norm;
		std::tuple<node_types...> nodes;
		static constexpr size_t node_count = sizeof...(node_types);
		static_assert(((node_types::traits_type::K == norm_node_type::rms_norm_traits::K) && ...), "every mul_mat of the stage must read the normalised row");
	};

	// ffn_silu -> ffn_gate_par -> ffn_down_mul_mat -> ffn_residual_add as ONE stage (infra/core_traits.hpp:982-992): the down
	// projection reads silu(gate) * up and adds the residual stream as it stores.  `down.activation` is not read (its extents
	// carry the token count); `residual.data[0] == nullptr` leaves the add out.
	template<typename down_node_type> struct ffn_tail_core {
		static constexpr core_types core_type = core_types::mega_ffn;
		static constexpr size_t node_count	  = 1;
		nhb_ctx* ctx						  = nullptr;
		down_node_type down;
		typename down_node_type::traits_type::input_02_type gate, up;// f32 [FF, tokens], the gate and up projections' outputs
		typename down_node_type::traits_type::output_type residual;// ffn_inp, f32 [E, tokens]
		int run_fused(int64_t block) const {
			using t					= typename down_node_type::traits_type;
			const nhb_mul_mat_op op = down.describe(static_cast<uint64_t>(block));
			return nhb_mul_mat_swiglu_add(ctx, op.w, static_cast<const float*>(gate.get_data()), static_cast<const float*>(up.get_data()), t::K,
				static_cast<const float*>(residual.get_data()), t::N, op.y, op.ldy, op.M);
		}
	};

	// attn_out_mul_mat -> residual_add as one stage (infra/core_traits.hpp:768-772)
	template<typename node_type> struct mul_mat_add_core {
		static constexpr core_types core_type = core_types::mega_attention_apply;
		static constexpr size_t node_count	  = 1;
		nhb_ctx* ctx						  = nullptr;
		node_type node;
		typename node_type::traits_type::output_type residual;// inp_embd, f32 [E, tokens]
		int run_fused(int64_t block) const {
			const nhb_mul_mat_op op = node.describe(static_cast<uint64_t>(block));
			return nhb_mul_mat_add(ctx, op.w, op.x, op.ldx, static_cast<const float*>(residual.get_data()), node_type::traits_type::N, op.y, op.ldy, op.M);
		}
	};

	template<typename config_type, bool eval, typename core_traits_type> inline void dispatch_plain_stage(core_traits_type& params, int64_t current_block);

	// What every specialisation in mega_dispatch.inc does: the independent mul_mats of the stage `params` describes, in one
	// call of the C ABI.  `eval` = the reference's processing_phases::eval_time (one token).
	template<typename config_type, bool eval, typename core_traits_type> inline void dispatch_stage(core_traits_type& params, int64_t current_block) {
		if constexpr (requires { params.run_fused(current_block); }) {
			static_assert(config_type::act_mode == NHB_ACT_Q8, "the fused element-wise stages use the Q8 arithmetic");
			const int rc = params.run_fused(current_block);
			if (rc != NHB_OK)
				raise<config_type::exceptions>(rc, "fused mul_mat stage", params.ctx);
			return;
		} else {
			dispatch_plain_stage<config_type, eval>(params, current_block);
		}
	}

	template<typename config_type, bool eval, typename core_traits_type> inline void dispatch_plain_stage(core_traits_type& params, int64_t current_block) {
		std::array<nhb_mul_mat_op, core_traits_type::node_count> ops{};
		[&]<size_t... i>(std::index_sequence<i...>) {
			((ops[i] = std::get<i>(params.nodes).describe(static_cast<uint64_t>(current_block))), ...);
		}(std::make_index_sequence<core_traits_type::node_count>{});
		if constexpr (eval) {
			for (const auto& op: ops)
				if (op.M != 1)
					raise<config_type::exceptions>(NHB_ERR_ARG, "eval_time dispatch with more than one token", params.ctx);
		}
		if constexpr (requires { params.norm; }) {
			static_assert(config_type::act_mode == NHB_ACT_Q8, "the fused norm produces Q8_0 activations");
			for (auto& op: ops)
				op.x = static_cast<const float*>(params.norm.input.get_data()) + params.norm.first_row * op.ldx;
			const int rc = nhb_rms_norm_mul_mat_batch(params.ctx, ops.data(), static_cast<int>(ops.size()), static_cast<const float*>(params.norm.norm_weight.get_data()),
				params.norm.eps, params.norm.sqrt_mode, NHB_KERNEL_AUTO);
			if (rc != NHB_OK)
				raise<config_type::exceptions>(rc, "nhb_rms_norm_mul_mat_batch", params.ctx);
		} else {
			const int rc = nhb_mul_mat_batch(params.ctx, ops.data(), static_cast<int>(ops.size()), config_type::act_mode, NHB_KERNEL_AUTO);
			if (rc != NHB_OK)
				raise<config_type::exceptions>(rc, "nhb_mul_mat_batch", params.ctx);
		}
	}

#ifndef NHB_DISPATCH_HOST_TYPES
	// the reference's forward declaration, parameter for parameter (include/nihilus-incl/common/kernel_traits.hpp:382-383)
	template<typename config_type, typename core_traits_type, device_types devive_type, uint64_t, core_types core_type, processing_phases processing_phase>
	struct kernel_dispatcher_impl;

#include "mega_dispatch.inc"

	// the reference's entry (infra/monolithic_dispatcher.hpp:53-62) for a GPU configuration: the core names its own core_type
	template<typename config_type, processing_phases processing_phase, typename core_type> struct kernel_dispatcher {
		static void impl(core_type& params, int64_t current_block) {
			kernel_dispatcher_impl<config_type, core_type, config_type::device_type, gpu_arch_index_sm100, core_type::core_type, processing_phase>::impl(params, current_block);
		}
		static void impl(core_type& params) {
			kernel_dispatcher_impl<config_type, core_type, config_type::device_type, gpu_arch_index_sm100, core_type::core_type, processing_phase>::impl(params);
		}
	};
#endif

	// ---- LLaMA-3-8B projection descriptors (infra/model_traits.hpp:49-65, infra/core_traits.hpp:145-209) ----
	namespace llama3_8b {
		inline constexpr uint64_t E = 4096, FF = 14336, KV = 1024, V = 128256, L = 32;
		template<uint64_t K, uint64_t N, uint64_t blocks> using weight_t = operand<core_trait_dims<K, N, 1, 1>, block_q8_0, blocks>;
		template<uint64_t K> using act_t									 = operand<core_trait_dims<K, 1, 1, 1, 1>, float>;// ne1 = tokens, patched per step
		template<uint64_t N> using out_t									 = operand<core_trait_dims<N, 1, 1, 1, 1>, float>;
		template<uint64_t K, uint64_t N, uint64_t blocks = L> using projection =
			mul_mat_node<kernel_traits<kernel_types::mul_mat, out_t<N>, weight_t<K, N, blocks>, act_t<K>>>;
		using attn_q	  = projection<E, E>;
		using attn_k	  = projection<E, KV>;
		using attn_v	  = projection<E, KV>;
		using attn_output = projection<E, E>;
		using ffn_gate	  = projection<E, FF>;
		using ffn_up	  = projection<E, FF>;
		using ffn_down	  = projection<FF, E>;
		using output	  = projection<E, V, 1>;
		// attn_norm / ffn_norm in front of their stage
		using norm_w_t = operand<core_trait_dims<E, 1, 1, 1>, float>;
		using norm_node = norm_mul_node<kernel_traits<kernel_types::rms_norm, act_t<E>, act_t<E>>, kernel_traits<kernel_types::mul, act_t<E>, act_t<E>, norm_w_t>>;
		// the stages of the reference's cores (infra/core_traits.hpp:575-594 q/k/v, :768-769 attn_out, :976-989 gate/up and down,
		// :1192-1193 logits)
		using norm_qkv_core		= norm_mul_mat_core<core_types::mega_qkv_prep_and_cache_publish, norm_node, attn_q, attn_k, attn_v>;
		using norm_gate_up_core = norm_mul_mat_core<core_types::mega_ffn, norm_node, ffn_gate, ffn_up>;
		using qkv_core			= mul_mat_core<core_types::mega_qkv_prep_and_cache_publish, attn_q, attn_k, attn_v>;
		using attn_out_core		= mul_mat_core<core_types::mega_attention_apply, attn_output>;
		using gate_up_core		= mul_mat_core<core_types::mega_ffn, ffn_gate, ffn_up>;
		using down_core			= mul_mat_core<core_types::mega_ffn, ffn_down>;
		using logits_core		= mul_mat_core<core_types::final_norm_and_sampling, output>;
		// last-token view -> final norm -> logits (infra/core_traits.hpp:1184-1193): set norm.first_row = sequence length - 1
		using logits_act_t	   = operand<core_trait_dims<E, 1, 1, 1>, float>;// one token, whatever the sequence length
		using last_token_output = mul_mat_node<kernel_traits<kernel_types::mul_mat, operand<core_trait_dims<V, 1, 1, 1>, float>, weight_t<E, V, 1>, logits_act_t>>;
		using norm_logits_core = norm_mul_mat_core<core_types::final_norm_and_sampling, norm_node, last_token_output>;
		// the fused tails of the FFN and attention cores
		using ffn_tail	   = ffn_tail_core<ffn_down>;
		using attn_out_add = mul_mat_add_core<attn_output>;
	}

}
