// Drives the Q8_0 mul_mat through the C++23 operator interface (include/nihilus_b200/mul_mat_op.hpp) the way the
// reference engine would: upload two per-block weights, patch the runtime sequence length, dispatch one core.
//
//   mul_mat_op_demo check                                  compile-time and host-only checks, no GPU
//   mul_mat_op_demo run <wk.bin> <wv.bin> <x.bin> M <yk.bin> <yv.bin>
//        wk/wv: raw Q8_0 blocks of two 1024 x 4096 weights, x: f32 [M][4096]; writes f32 [M][1024] each
//   mul_mat_op_demo run_norm <wk.bin> <wv.bin> <x.bin> M <yk.bin> <yv.bin> <norm_w.bin>
//        the same with the rms_norm -> mul pair in front (x is the row before the norm, norm_w: f32 [4096], eps 1e-5)
#include <nihilus_b200/mul_mat_op.hpp>

#include <cstring>
#include <fstream>
#include <iostream>
#include <vector>

using namespace nihilus_b200;

// the static contract (same rules as the reference's kernel_traits)
using k_traits = llama3_8b::attn_k::traits_type;
static_assert(k_traits::K == 4096 && k_traits::N == 1024);
static_assert(k_traits::derived_output_dims()[0] == 1024);
static_assert(llama3_8b::ffn_down::traits_type::K == 14336 && llama3_8b::ffn_down::traits_type::N == 4096);
static_assert(llama3_8b::output::traits_type::N == 128256);
static_assert(llama3_8b::qkv_core::node_count == 3 && llama3_8b::gate_up_core::node_count == 2);
static_assert(llama3_8b::act_t<4096>::runtime_dim == 1);
static_assert(llama3_8b::norm_qkv_core::node_count == 3 && llama3_8b::norm_node::rms_norm_traits::K == 4096);

static std::vector<char> slurp(const char* path) {
	std::ifstream f(path, std::ios::binary);
	if (!f)
		throw std::runtime_error(std::string("cannot open ") + path);
	return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

static int check() {
	// a dispatch without a context must surface as the library's error, through the exception convention
	using core_t = mul_mat_core<core_types::mega_qkv_prep_and_cache_publish, llama3_8b::attn_k>;
	core_t core{};
	std::get<0>(core.nodes).activation.get_seq_length_dim() = 1;
	bool threw = false;
	try {
		kernel_dispatcher<gpu_config<true>, processing_phases::eval_time, core_t>::impl(core, 0);
	} catch (const mul_mat_error& e) {
		threw = e.status == NHB_ERR_ARG;
	}
	if (!threw) {
		std::cerr << "expected NHB_ERR_ARG for a null context\n";
		return 1;
	}
	// eval_time is the one-token phase
	std::get<0>(core.nodes).activation.get_seq_length_dim() = 4;
	threw = false;
	try {
		kernel_dispatcher<gpu_config<true>, processing_phases::eval_time, core_t>::impl(core, 0);
	} catch (const mul_mat_error&) {
		threw = true;
	}
	if (!threw) {
		std::cerr << "expected an error for eval_time with 4 tokens\n";
		return 1;
	}
	std::cout << "check ok\n";
	return 0;
}

static int run(char** a, bool with_norm) {
	const auto wk = slurp(a[0]), wv = slurp(a[1]), x = slurp(a[2]);
	const int64_t M = std::atoll(a[3]);
	constexpr int64_t K = 4096, N = 1024;
	if (wk.size() != size_t(N) * (K / 32) * 34 || wv.size() != wk.size() || x.size() != size_t(M) * K * 4)
		throw std::runtime_error("input sizes do not match attn_k / attn_v and M");
	using cfg	 = gpu_config<true>;
	using core_t = mul_mat_core<core_types::mega_qkv_prep_and_cache_publish, llama3_8b::attn_k, llama3_8b::attn_v>;
	nhb_ctx* ctx = nullptr;
	if (nhb_ctx_create(&ctx, 0, 0, 1) != NHB_OK)
		raise<true>(NHB_ERR_CUDA, "nhb_ctx_create", nullptr);
	nhb_weight *hk = nullptr, *hv = nullptr;
	if (nhb_weight_upload_q8_0(ctx, wk.data(), N, K, &hk) != NHB_OK || nhb_weight_upload_q8_0(ctx, wv.data(), N, K, &hv) != NHB_OK)
		raise<true>(NHB_ERR_CUDA, "nhb_weight_upload_q8_0", ctx);
	void *xd = nullptr, *yk = nullptr, *yv = nullptr;
	if (nhb_device_alloc(ctx, x.size(), &xd) != NHB_OK || nhb_device_alloc(ctx, size_t(M) * N * 4, &yk) != NHB_OK ||
		nhb_device_alloc(ctx, size_t(M) * N * 4, &yv) != NHB_OK)
		raise<true>(NHB_ERR_NOMEM, "nhb_device_alloc", ctx);
	nhb_memcpy_h2d(ctx, xd, x.data(), x.size());

	core_t core{};
	core.ctx				= ctx;
	constexpr int64_t block = 3;// any transformer block: each holds its own weight handle
	auto& nk				= std::get<0>(core.nodes);
	auto& nv				= std::get<1>(core.nodes);
	nk.weight.data[block]	= hk;
	nv.weight.data[block]	= hv;
	nk.activation.data[0] = nv.activation.data[0] = xd;
	nk.output.data[0]							  = yk;
	nv.output.data[0]							  = yv;
	nk.activation.get_seq_length_dim() = nv.activation.get_seq_length_dim() = static_cast<uint64_t>(M);
	void* nwd = nullptr;
	if (with_norm) {
		// the same two projections behind attn_norm: the dispatcher takes the hidden state and the norm weight
		const auto nw = slurp(a[6]);
		if (nw.size() != size_t(K) * 4)
			throw std::runtime_error("norm weight must be f32 [4096]");
		if (nhb_device_alloc(ctx, nw.size(), &nwd) != NHB_OK)
			raise<true>(NHB_ERR_NOMEM, "nhb_device_alloc", ctx);
		nhb_memcpy_h2d(ctx, nwd, nw.data(), nw.size());
		using ncore_t = norm_mul_mat_core<core_types::mega_qkv_prep_and_cache_publish, llama3_8b::norm_node, llama3_8b::attn_k, llama3_8b::attn_v>;
		ncore_t ncore{};
		ncore.ctx					   = ctx;
		ncore.norm.input.data[0]	   = xd;
		ncore.norm.norm_weight.data[0] = nwd;
		ncore.norm.eps				   = 1e-5f;
		std::get<0>(ncore.nodes)	   = nk;
		std::get<1>(ncore.nodes)	   = nv;
		if (M == 1)
			kernel_dispatcher<cfg, processing_phases::eval_time, ncore_t>::impl(ncore, block);
		else
			kernel_dispatcher<cfg, processing_phases::prompt_eval_time, ncore_t>::impl(ncore, block);
	} else if (M == 1)
		kernel_dispatcher<cfg, processing_phases::eval_time, core_t>::impl(core, block);
	else
		kernel_dispatcher<cfg, processing_phases::prompt_eval_time, core_t>::impl(core, block);

	std::vector<float> ok(size_t(M) * N), ov(size_t(M) * N);
	nhb_memcpy_d2h(ctx, ok.data(), yk, ok.size() * 4);
	nhb_memcpy_d2h(ctx, ov.data(), yv, ov.size() * 4);
	if (nhb_sync(ctx) != NHB_OK)
		raise<true>(NHB_ERR_CUDA, "nhb_sync", ctx);
	std::ofstream(a[4], std::ios::binary).write(reinterpret_cast<const char*>(ok.data()), ok.size() * 4);
	std::ofstream(a[5], std::ios::binary).write(reinterpret_cast<const char*>(ov.data()), ov.size() * 4);
	nhb_weight_free(ctx, hk);
	nhb_weight_free(ctx, hv);
	nhb_device_free(ctx, xd);
	nhb_device_free(ctx, yk);
	nhb_device_free(ctx, yv);
	if (nwd)
		nhb_device_free(ctx, nwd);
	nhb_ctx_destroy(ctx);
	std::cout << "run ok\n";
	return 0;
}

// ffn tail through the dispatcher: gate.bin up.bin res.bin wdown.bin M y.bin, with a small ffn_down stand-in of 256 rows
static int run_tail(char** a) {
	constexpr uint64_t FF = 14336, E = 256;
	using w_t	 = operand<core_trait_dims<FF, E, 1, 1>, block_q8_0, 2>;
	using act_t	 = operand<core_trait_dims<FF, 1, 1, 1, 1>, float>;
	using out_t	 = operand<core_trait_dims<E, 1, 1, 1, 1>, float>;
	using node_t = mul_mat_node<kernel_traits<kernel_types::mul_mat, out_t, w_t, act_t>>;
	using core_t = ffn_tail_core<node_t>;
	static_assert(core_t::core_type == core_types::mega_ffn);
	const auto gate = slurp(a[0]), up = slurp(a[1]), res = slurp(a[2]), wd = slurp(a[3]);
	const int64_t M = std::atoll(a[4]);
	if (gate.size() != size_t(M) * FF * 4 || up.size() != gate.size() || res.size() != size_t(M) * E * 4 || wd.size() != size_t(E) * (FF / 32) * 34)
		throw std::runtime_error("input sizes do not match the ffn tail stand-in");
	nhb_ctx* ctx = nullptr;
	if (nhb_ctx_create(&ctx, 0, 0, 1) != NHB_OK)
		raise<true>(NHB_ERR_CUDA, "nhb_ctx_create", nullptr);
	nhb_weight* h = nullptr;
	if (nhb_weight_upload_q8_0(ctx, wd.data(), E, FF, &h) != NHB_OK)
		raise<true>(NHB_ERR_CUDA, "nhb_weight_upload_q8_0", ctx);
	void *gd = nullptr, *ud = nullptr, *rd = nullptr, *yd = nullptr;
	if (nhb_device_alloc(ctx, gate.size(), &gd) != NHB_OK || nhb_device_alloc(ctx, up.size(), &ud) != NHB_OK || nhb_device_alloc(ctx, res.size(), &rd) != NHB_OK ||
		nhb_device_alloc(ctx, res.size(), &yd) != NHB_OK)
		raise<true>(NHB_ERR_NOMEM, "nhb_device_alloc", ctx);
	nhb_memcpy_h2d(ctx, gd, gate.data(), gate.size());
	nhb_memcpy_h2d(ctx, ud, up.data(), up.size());
	nhb_memcpy_h2d(ctx, rd, res.data(), res.size());
	core_t core{};
	core.ctx				 = ctx;
	core.down.weight.data[1] = h;
	core.down.output.data[0] = yd;
	core.down.activation.get_seq_length_dim() = static_cast<uint64_t>(M);
	core.gate.data[0]		 = gd;
	core.up.data[0]			 = ud;
	core.residual.data[0]	 = rd;
	if (M == 1)
		kernel_dispatcher<gpu_config<true>, processing_phases::eval_time, core_t>::impl(core, 1);
	else
		kernel_dispatcher<gpu_config<true>, processing_phases::prompt_eval_time, core_t>::impl(core, 1);
	std::vector<float> y(size_t(M) * E);
	nhb_memcpy_d2h(ctx, y.data(), yd, y.size() * 4);
	if (nhb_sync(ctx) != NHB_OK)
		raise<true>(NHB_ERR_CUDA, "nhb_sync", ctx);
	std::ofstream(a[5], std::ios::binary).write(reinterpret_cast<const char*>(y.data()), y.size() * 4);
	nhb_weight_free(ctx, h);
	for (void* p: { gd, ud, rd, yd })
		nhb_device_free(ctx, p);
	nhb_ctx_destroy(ctx);
	std::cout << "run ok\n";
	return 0;
}

int main(int argc, char** argv) {
	try {
		if (argc == 2 && !std::strcmp(argv[1], "check"))
			return check();
		if (argc == 8 && !std::strcmp(argv[1], "run"))
			return run(argv + 2, false);
		if (argc == 9 && !std::strcmp(argv[1], "run_norm"))
			return run(argv + 2, true);
		if (argc == 8 && !std::strcmp(argv[1], "run_tail"))
			return run_tail(argv + 2);
	} catch (const std::exception& e) {
		std::cerr << "error: " << e.what() << "\n";
		return 2;
	}
	std::cerr << "usage: mul_mat_op_demo check | run wk.bin wv.bin x.bin M yk.bin yv.bin | run_norm ... norm_w.bin\n";
	return 64;
}
