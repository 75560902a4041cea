"""nihilus_b200: B200-native Q8_0 mul_mat (the dominant hot path of the Nihilus LLaMA engine).

The product is the C-ABI shared library built from ``csrc/`` (declared in ``include/nihilus_b200.h``).
This package is the thin Python host side used by tests and benchmarks: it loads that library with
ctypes and uses PyTorch only for device memory, streams and ``torch.distributed`` rendezvous.
There is no CPU or PyTorch fallback: importing :mod:`nihilus_b200.capi` fails loudly if the library is
missing, and every operator call goes through the CUDA kernels.
"""
from .shapes import LLAMA3_8B, decode_set, mul_mat_bytes, mul_mat_flops  # noqa: F401

__all__ = ["LLAMA3_8B", "decode_set", "mul_mat_bytes", "mul_mat_flops"]
