"""The C++23 operator interface (include/nihilus_b200/mul_mat_op.hpp) compiled with g++ and driven like the
reference engine drives a core: traits -> kernel_dispatcher -> C ABI.  The host-only part runs without a GPU."""
import os
import shutil
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "mul_mat_op_demo.cpp")


@pytest.fixture(scope="module")
def demo(capi, tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    out = str(tmp_path_factory.mktemp("cpp") / "mul_mat_op_demo")
    lib_dir = os.path.dirname(capi.LIB_PATH)
    cmd = [gxx, "-std=c++23", "-O1", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"), SRC, "-o", out, "-L" + lib_dir,
           "-lnihilus_b200", "-Wl,-rpath," + lib_dir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


def test_traits_compile_and_errors_follow_the_exception_convention(demo):
    r = subprocess.run([demo, "check"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "check ok" in r.stdout


def test_static_checks_reject_a_mismatched_mul_mat(capi, tmp_path):
    """K of the weight and of the activation differ: the trait must refuse to compile, like the reference's."""
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    bad = tmp_path / "bad.cpp"
    bad.write_text(
        "#include <nihilus_b200/mul_mat_op.hpp>\n"
        "using namespace nihilus_b200;\n"
        "using w = operand<core_trait_dims<4096, 1024, 1, 1>, block_q8_0>;\n"
        "using a = operand<core_trait_dims<2048, 1, 1, 1, 1>, float>;\n"
        "using o = operand<core_trait_dims<1024, 1, 1, 1, 1>, float>;\n"
        "using t = kernel_traits<kernel_types::mul_mat, o, w, a>;\n"
        "int main() { return static_cast<int>(t::K); }\n"
    )
    r = subprocess.run([gxx, "-std=c++23", "-fsyntax-only", "-I" + os.path.join(ROOT, "include"), str(bad)], capture_output=True, text=True)
    assert r.returncode != 0
    assert "inner dimensions must match" in r.stderr


# what the reference's cmake would define for an x86-64 Linux CPU build (cmake/flags_and_options.cmake:20-39 and
# cmake/detection/nihilus_detect_cpu_properties.cmake:171-201); only needed to PARSE its headers
REFERENCE_DEFINES = [
    "-DNIHILUS_COMPILER_CUDA=0", "-DNIHILUS_ARCH_X64=1", "-DNIHILUS_ARCH_ARM64=0", "-DNIHILUS_PLATFORM_WINDOWS=0", "-DNIHILUS_PLATFORM_LINUX=1",
    "-DNIHILUS_PLATFORM_MAC=0", "-DNIHILUS_COMPILER_CLANG=0", "-DNIHILUS_COMPILER_MSVC=0", "-DNIHILUS_COMPILER_GNUCXX=1", "-DNIHILUS_DEV=0",
    "-DNIHILUS_CUDA_TENSOR_CORES=0", "-DNIHILUS_CUDA_MAX_REGISTERS=0", "-DNIHILUS_GLOBAL=", "-DNIHILUS_AVX2=1", "-DNIHILUS_AVX512=0", "-DNIHILUS_NEON=0",
    "-DNIHILUS_SVE2=0", "-DNIHILUS_HOST=inline __attribute__((always_inline))", "-DNIHILUS_DEVICE=inline __attribute__((always_inline))",
    "-DNIHILUS_HOST_DEVICE=inline __attribute__((always_inline))", "-mavx2", "-mfma", "-mf16c", "-mbmi", "-mbmi2", "-mlzcnt", "-mpopcnt",
]


def test_specialisations_fit_the_references_own_dispatcher_declaration():
    """With the reference tree present: its kernel_traits.hpp is included in place (nothing copied), our specialisation
    block goes into namespace nihilus unchanged, and dispatching through the reference's primary template reaches it."""
    from oracle import pyoracle

    ref = pyoracle.reference_root()
    if not ref or not os.path.isfile(os.path.join(ref, "include", "nihilus-incl", "common", "kernel_traits.hpp")):
        pytest.skip("reference source tree not present")
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    src = os.path.join(ROOT, "tests", "cpp", "reference_dispatch_check.cpp")
    cmd = [gxx, "-std=c++23", "-fsyntax-only", *REFERENCE_DEFINES, "-I" + os.path.join(ref, "include"), "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(ROOT, "tests", "cpp"), src]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 5, 40])
def test_dispatch_through_the_cpp_interface_matches_the_oracle(demo, oracle, tmp_path, M):
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    N, K = 1024, 4096
    wk, wv = synth.make_weight(N, K, 901), synth.make_weight(N, K, 902)
    x = synth.make_activation(M, K, 903 + M)
    p = {n: str(tmp_path / n) for n in ("wk", "wv", "x", "yk", "yv")}
    wk.tofile(p["wk"])
    wv.tofile(p["wv"])
    x.tofile(p["x"])
    r = subprocess.run([demo, "run", p["wk"], p["wv"], p["x"], str(M), p["yk"], p["yv"]], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    for w, name in ((wk, "yk"), (wv, "yv")):
        y = np.fromfile(p[name], dtype=np.float32).reshape(M, N)
        ref = oracle.mul_mat(po.Q8ACT_LANES, w, x)
        assert float(np.abs(y - ref).max() / np.abs(ref).max()) <= 1e-4


def test_static_checks_reject_a_norm_weight_of_the_wrong_length(capi, tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    bad = tmp_path / "bad_norm.cpp"
    bad.write_text(
        "#include <nihilus_b200/mul_mat_op.hpp>\n"
        "using namespace nihilus_b200;\n"
        "using a = operand<core_trait_dims<4096, 1, 1, 1, 1>, float>;\n"
        "using w = operand<core_trait_dims<2048, 1, 1, 1>, float>;\n"
        "using t = kernel_traits<kernel_types::mul, a, a, w>;\n"
        "int main() { return static_cast<int>(t::output_dims[0]); }\n"
    )
    r = subprocess.run([gxx, "-std=c++23", "-fsyntax-only", "-I" + os.path.join(ROOT, "include"), str(bad)], capture_output=True, text=True)
    assert r.returncode != 0
    assert "element-wise dimension 0 must match" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 3, 40])
def test_norm_stage_through_the_cpp_interface_matches_the_oracle(demo, oracle, tmp_path, M):
    """attn_norm -> (k, v) as one core: the dispatcher hands the hidden state and the norm weight to the library."""
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    N, K = 1024, 4096
    wk, wv = synth.make_weight(N, K, 911), synth.make_weight(N, K, 912)
    x = (synth.make_activation(M, K, 913 + M) * 3.0).astype(np.float32)
    nw = np.random.default_rng(914).uniform(0.5, 1.5, K).astype(np.float32)
    p = {n: str(tmp_path / n) for n in ("wk", "wv", "x", "yk", "yv", "nw")}
    wk.tofile(p["wk"])
    wv.tofile(p["wv"])
    x.tofile(p["x"])
    nw.tofile(p["nw"])
    r = subprocess.run([demo, "run_norm", p["wk"], p["wv"], p["x"], str(M), p["yk"], p["yv"], p["nw"]], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    normed = oracle.rms_norm_mul(x, nw, float(np.float32(1e-5)), 0)
    for w, name in ((wk, "yk"), (wv, "yv")):
        y = np.fromfile(p[name], dtype=np.float32).reshape(M, N)
        ref = oracle.mul_mat(po.Q8ACT_LANES, w, normed)
        assert float(np.abs(y - ref).max() / np.abs(ref).max()) <= 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 20])
def test_ffn_tail_through_the_cpp_interface_matches_the_oracle(demo, oracle, tmp_path, M):
    """silu(gate) * up -> ffn_down -> + residual as one core of type mega_ffn (infra/core_traits.hpp:982-992)."""
    from nihilus_b200 import synth
    from oracle import pyoracle as po

    FF, E = 14336, 256
    w = synth.make_weight(E, FF, 921)
    gate = (synth.make_activation(M, FF, 922 + M) * 2).astype(np.float32)
    up = synth.make_activation(M, FF, 923 + M)
    res = synth.make_activation(M, E, 924 + M)
    p = {n: str(tmp_path / n) for n in ("gate", "up", "res", "w", "y")}
    for name, arr in (("gate", gate), ("up", up), ("res", res), ("w", w)):
        arr.tofile(p[name])
    r = subprocess.run([demo, "run_tail", p["gate"], p["up"], p["res"], p["w"], str(M), p["y"]], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    y = np.fromfile(p["y"], dtype=np.float32).reshape(M, E)
    ref = oracle.add(oracle.mul_mat(po.Q8ACT_LANES, w, oracle.swiglu(gate, up)), res)
    assert float(np.abs(y - ref).max() / np.abs(ref).max()) <= 3e-4  # exp() of the two sides differs in the last bits (see test_gpu_ffn_fusion.py)
