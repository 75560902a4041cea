"""ctypes binding of libnihilus_b200.so (see include/nihilus_b200.h) plus small torch conveniences.

No fallback: if the shared library is absent this module raises at import, and every call below runs
the CUDA kernels through the C ABI.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# NHB_LIB names another build of the same library (experiments with compile-time knobs)
LIB_PATH = os.environ.get("NHB_LIB") or os.path.join(_HERE, "lib", "libnihilus_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m nihilus_b200.build` (nvcc, sm_100a). "
        "nihilus_b200 has no CPU or PyTorch fallback."
    )

lib = C.CDLL(LIB_PATH)

ACT_Q8, ACT_F32 = 0, 1
SQRT_IEEE, SQRT_X86_FAST = 0, 1
KERNEL_AUTO, KERNEL_GEMV_LDG, KERNEL_GEMV_STREAM, KERNEL_GEMM_TC, KERNEL_GEMV_ROWS = 0, 1, 2, 3, 4
OK, ERR_ARG, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_NOMEM = 0, -1, -2, -3, -4, -5, -6

# every symbol include/nihilus_b200.h declares
EXPORTS = (
    "nhb_version", "nhb_arch", "nhb_last_error", "nhb_shard_rows", "nhb_repack_q8_0_host", "nhb_unpack_q8_0_host",
    "nhb_choose_kernel", "nhb_mul_mat_bytes", "nhb_mul_mat_flops", "nhb_ctx_create", "nhb_ctx_destroy", "nhb_ctx_set_stream",
    "nhb_sync", "nhb_ctx_set_gemv_max_m", "nhb_ctx_set_option", "nhb_ctx_launch_count", "nhb_memcpy_h2d", "nhb_memcpy_d2h",
    "nhb_weight_upload_q8_0", "nhb_weight_free", "nhb_weight_info_get", "nhb_weight_download_q8_0", "nhb_mul_mat",
    "nhb_mul_mat_batch", "nhb_mul_mat_host", "nhb_mul_mat_block_dots", "nhb_quantize_q8_0", "nhb_graph_begin", "nhb_graph_end",
    "nhb_graph_launch", "nhb_graph_free", "nhb_comm_unique_id", "nhb_comm_init", "nhb_all_gather", "nhb_all_gather_batch",
    "nhb_mul_mat_q8_0_noalloc", "nhb_noalloc_max_bytes", "nhb_noalloc_last_error", "nhb_device_alloc", "nhb_device_free", "nhb_symm_alloc", "nhb_symm_free", "nhb_symm_alloc_local", "nhb_all_gather_local", "nhb_sync_all", "nhb_wait_planner_create", "nhb_wait_planner_destroy", "nhb_wait_planner_add_region",
    "nhb_wait_planner_launch", "nhb_wait_planner_wait_all", "nhb_wait_planner_seq", "nhb_wait_planner_capture_begin", "nhb_wait_planner_capture_end",
    "nhb_wait_planner_replayed", "nhb_place_rows", "nhb_gemm_tile_plan",
    "nhb_rms_norm_mul", "nhb_rms_norm_mul_q8_0", "nhb_rms_norm_mul_mat_batch",
    "nhb_gguf_open", "nhb_gguf_last_error", "nhb_gguf_close", "nhb_gguf_tensor_count", "nhb_gguf_find", "nhb_gguf_tensor_get",
    "nhb_gguf_get_number", "nhb_gguf_get_string", "nhb_gguf_upload_q8_0", "nhb_gguf_read_f32",
    "nhb_chain_create", "nhb_chain_launch", "nhb_chain_free", "nhb_mul_mat_swiglu_add", "nhb_mul_mat_add", "nhb_swiglu",
    "nhb_get_rows_q8_0", "nhb_last_token_logits", "nhb_weight_save", "nhb_weight_load",
)


class WeightInfo(C.Structure):
    _fields_ = [("N", C.c_int64), ("K", C.c_int64), ("n0", C.c_int64), ("n1", C.c_int64), ("q", C.c_void_p), ("d", C.c_void_p),
                ("bytes_q8", C.c_int64)]


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n_dims", C.c_int), ("dims", C.c_int64 * 4), ("type", C.c_int), ("bytes", C.c_int64),
                ("offset", C.c_int64), ("data", C.c_void_p)]


class MulMatOp(C.Structure):
    _fields_ = [("w", C.c_void_p), ("x", C.c_void_p), ("ldx", C.c_int64), ("y", C.c_void_p), ("ldy", C.c_int64), ("M", C.c_int64)]


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


_vp, _i, _i64 = C.c_void_p, C.c_int, C.c_int64
_sig("nhb_version", _i)
_sig("nhb_gguf_open", _i, C.c_char_p, C.POINTER(_vp))
_sig("nhb_gguf_last_error", C.c_char_p)
_sig("nhb_gguf_close", _i, _vp)
_sig("nhb_gguf_tensor_count", _i64, _vp)
_sig("nhb_gguf_find", _i64, _vp, C.c_char_p)
_sig("nhb_gguf_tensor_get", _i, _vp, _i64, C.POINTER(GgufTensor))
_sig("nhb_gguf_get_number", _i, _vp, C.c_char_p, C.POINTER(C.c_double))
_sig("nhb_gguf_get_string", C.c_char_p, _vp, C.c_char_p)
_sig("nhb_gguf_upload_q8_0", _i, _vp, _vp, C.c_char_p, C.POINTER(_vp))
_sig("nhb_gguf_read_f32", _i, _vp, C.c_char_p, _vp, _i64)
_sig("nhb_rms_norm_mul", _i, _vp, _vp, _i64, _vp, C.c_float, _i, _vp, _i64, _i64, _i64)
_sig("nhb_rms_norm_mul_q8_0", _i, _vp, _vp, _i64, _vp, C.c_float, _i, _vp, _i64, _i64)
_sig("nhb_rms_norm_mul_mat_batch", _i, _vp, C.POINTER(MulMatOp), _i, _vp, C.c_float, _i, _i)
_sig("nhb_arch", _i)
_sig("nhb_last_error", C.c_char_p, _vp)
_sig("nhb_shard_rows", _i, _i64, _i, _i, C.POINTER(_i64), C.POINTER(_i64))
_sig("nhb_place_rows", _i, _i64, _i64, _i, _i, _i64, C.POINTER(_i64), C.POINTER(_i64))
_sig("nhb_gemm_tile_plan", _i, _i64, _i64, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i))
_sig("nhb_repack_q8_0_host", _i, _vp, _i64, _i64, _i64, _i64, _vp, _vp)
_sig("nhb_unpack_q8_0_host", _i, _vp, _vp, _i64, _i64, _vp)
_sig("nhb_choose_kernel", _i, _i64, _i64, _i64, _i)
_sig("nhb_mul_mat_bytes", _i64, _i64, _i64, _i64)
_sig("nhb_mul_mat_flops", _i64, _i64, _i64, _i64)
_sig("nhb_ctx_create", _i, C.POINTER(_vp), _i, _i, _i)
_sig("nhb_ctx_destroy", _i, _vp)
_sig("nhb_ctx_set_stream", _i, _vp, _vp)
_sig("nhb_sync", _i, _vp)
_sig("nhb_ctx_set_gemv_max_m", _i, _vp, _i)
_sig("nhb_ctx_set_option", _i, _vp, C.c_char_p, _i)
_sig("nhb_ctx_launch_count", C.c_longlong, _vp)
_sig("nhb_memcpy_h2d", _i, _vp, _vp, _vp, C.c_size_t)
_sig("nhb_memcpy_d2h", _i, _vp, _vp, _vp, C.c_size_t)
_sig("nhb_device_alloc", _i, _vp, C.c_size_t, C.POINTER(_vp))
_sig("nhb_device_free", _i, _vp, _vp)
_sig("nhb_symm_alloc", _i, _vp, C.c_size_t, C.POINTER(_vp))
_sig("nhb_symm_alloc_local", _i, C.POINTER(_vp), _i, C.c_size_t, C.POINTER(_vp))
_sig("nhb_all_gather_local", _i, C.POINTER(_vp), _i, C.POINTER(_vp), _i64, _i64, _i64)
_sig("nhb_sync_all", _i, C.POINTER(_vp), _i)
_sig("nhb_wait_planner_create", _vp, _i)
_sig("nhb_wait_planner_destroy", None, _vp)
_sig("nhb_wait_planner_add_region", _i, _vp, _vp, C.c_size_t)
_sig("nhb_wait_planner_launch", _i, _vp, C.POINTER(_vp), C.POINTER(C.c_size_t), _i, C.POINTER(_vp), C.POINTER(C.c_size_t), _i, _i, C.POINTER(_i), C.POINTER(_i))
_sig("nhb_wait_planner_wait_all", _i, _vp)
_sig("nhb_wait_planner_seq", C.c_longlong, _vp)
_sig("nhb_wait_planner_capture_begin", None, _vp)
_sig("nhb_wait_planner_capture_end", _i, _vp)
_sig("nhb_wait_planner_replayed", _i, _vp, _i)
_sig("nhb_symm_free", _i, _vp, _vp)
_sig("nhb_weight_upload_q8_0", _i, _vp, _vp, _i64, _i64, C.POINTER(_vp))
_sig("nhb_weight_free", _i, _vp, _vp)
_sig("nhb_weight_info_get", _i, _vp, C.POINTER(WeightInfo))
_sig("nhb_weight_download_q8_0", _i, _vp, _vp, _vp)
_sig("nhb_mul_mat", _i, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i, _i)
_sig("nhb_mul_mat_batch", _i, _vp, C.POINTER(MulMatOp), _i, _i, _i)
_sig("nhb_mul_mat_host", _i, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i, _i)
_sig("nhb_mul_mat_block_dots", _i, _vp, _vp, _vp, _i64, _i64, _vp)
_sig("nhb_quantize_q8_0", _i, _vp, _vp, _i64, _i64, _i64, _vp, _vp)
_sig("nhb_graph_begin", _i, _vp)
_sig("nhb_graph_end", _i, _vp, C.POINTER(_vp))
_sig("nhb_graph_launch", _i, _vp, _vp)
_sig("nhb_graph_free", _i, _vp, _vp)
_sig("nhb_comm_unique_id", _i, _vp)
_sig("nhb_comm_init", _i, _vp, _vp)
_sig("nhb_all_gather", _i, _vp, _vp, _i64, _i64, _i64)
_sig("nhb_mul_mat_q8_0_noalloc", _i, _vp, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _i64, _vp)
_sig("nhb_noalloc_max_bytes", _i64)
_sig("nhb_noalloc_last_error", C.c_char_p)
_sig("nhb_all_gather_batch", _i, _vp, C.POINTER(_vp), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64), _i)
_sig("nhb_mul_mat_swiglu_add", _i, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64)
_sig("nhb_mul_mat_add", _i, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64)
_sig("nhb_swiglu", _i, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64)
_sig("nhb_get_rows_q8_0", _i, _vp, _vp, _vp, _i64, _vp, _i64)
_sig("nhb_last_token_logits", _i, _vp, _vp, _vp, _i64, _i64, _vp, C.c_float, _i, _vp)
_sig("nhb_weight_save", _i, _vp, _vp, C.c_char_p)
_sig("nhb_weight_load", _i, _vp, C.c_char_p, _i64, _i64, C.POINTER(_vp))
_sig("nhb_chain_create", _i, _vp, C.POINTER(MulMatOp), C.POINTER(_i), _i, C.POINTER(_vp))
_sig("nhb_chain_launch", _i, _vp, _vp)
_sig("nhb_chain_free", _i, _vp, _vp)


def _ld(t) -> int:
    """Leading dimension of a 2-D tensor; a single row may carry any stride (numpy's relaxed strides), which means nothing."""
    return t.stride(0) if t.shape[0] > 1 else max(int(t.stride(0)), int(t.shape[1]), 1)


def _tensor_from_ptr(ptr: int, nbytes: int, device: int, dtype):
    """A torch view of device memory this library owns (no copy; the caller keeps the allocation alive)."""
    import torch

    class _Cai:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}

    t = torch.as_tensor(_Cai(), device=f"cuda:{device}")
    return t.view(dtype)


class NhbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"nihilus_b200 error {code}: {msg}")
        self.code = code


def last_error(ctx=None) -> str:
    s = lib.nhb_last_error(ctx)
    return s.decode() if s else ""


def _check(rc: int, ctx=None):
    if rc != OK:
        raise NhbError(rc, last_error(ctx))


def shard_rows(N: int, world: int, rank: int) -> tuple[int, int]:
    a, b = _i64(), _i64()
    _check(lib.nhb_shard_rows(N, world, rank, C.byref(a), C.byref(b)))
    return a.value, b.value


def place_rows(N: int, K: int, world: int, rank: int, replicate_below_bytes: int = 0) -> tuple[int, int]:
    a, b = _i64(), _i64()
    _check(lib.nhb_place_rows(N, K, world, rank, replicate_below_bytes, C.byref(a), C.byref(b)))
    return a.value, b.value


def gemm_tile_plan(rows: int, M: int, sms: int = 148) -> dict:
    sw, nt, lt, ct = _i(), _i(), _i(), _i()
    _check(lib.nhb_gemm_tile_plan(rows, M, sms, C.byref(sw), C.byref(nt), C.byref(lt), C.byref(ct)))
    return {"swapped": bool(sw.value), "tile_cols": nt.value, "lane_tiles": lt.value, "col_tiles": ct.value}


def repack_host(blocks: np.ndarray, n0: int = 0, n1: int | None = None):
    """uint8 [N, K/32, 34] -> (int8 [rows, K], uint16 [rows, K/32]) on the host (no GPU)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    N, nb, _ = blocks.shape
    n1 = N if n1 is None else n1
    q = np.empty((max(n1 - n0, 0), nb * 32), dtype=np.int8)
    d = np.empty((max(n1 - n0, 0), nb), dtype=np.uint16)
    _check(lib.nhb_repack_q8_0_host(blocks.ctypes.data, N, nb * 32, n0, n1, q.ctypes.data, d.ctypes.data))
    return q, d


def unpack_host(q: np.ndarray, d: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.int8)
    d = np.ascontiguousarray(d, dtype=np.uint16)
    rows, K = q.shape
    out = np.empty((rows, K // 32, 34), dtype=np.uint8)
    _check(lib.nhb_unpack_q8_0_host(q.ctypes.data, d.ctypes.data, rows, K, out.ctypes.data))
    return out


class Weight:
    def __init__(self, ctx: "Context", handle: int):
        self.ctx = ctx
        self.handle = handle
        info = WeightInfo()
        _check(lib.nhb_weight_info_get(handle, C.byref(info)))
        self.N, self.K, self.n0, self.n1 = info.N, info.K, info.n0, info.n1
        self.q_ptr, self.d_ptr, self.bytes_q8 = info.q, info.d, info.bytes_q8

    def save(self, path: str):
        """This shard's repacked planes as a cache file (nhb_weight_save)."""
        _check(lib.nhb_weight_save(self.ctx.handle, self.handle, os.fsencode(path)), self.ctx.handle)

    def download(self) -> np.ndarray:
        out = np.empty((self.n1 - self.n0, self.K // 32, 34), dtype=np.uint8)
        _check(lib.nhb_weight_download_q8_0(self.ctx.handle, self.handle, out.ctypes.data), self.ctx.handle)
        return out

    def free(self):
        if self.handle:
            lib.nhb_weight_free(self.ctx.handle, self.handle)
            self.handle = None


class Gguf:
    """A mapped GGUF model file (nhb_gguf_*): tensor table, scalar metadata, Q8_0 upload by tensor name."""

    def __init__(self, path: str):
        h = _vp()
        rc = lib.nhb_gguf_open(os.fsencode(path), C.byref(h))
        if rc != 0:
            raise NhbError(rc, (lib.nhb_gguf_last_error() or b"").decode())
        self.handle = h.value

    def close(self):
        if self.handle:
            lib.nhb_gguf_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __len__(self):
        return int(lib.nhb_gguf_tensor_count(self.handle))

    def tensor(self, key):
        """key: index or name -> dict(name, dims, type, bytes, offset)."""
        idx = key if isinstance(key, int) else int(lib.nhb_gguf_find(self.handle, key.encode()))
        t = GgufTensor()
        if idx < 0 or lib.nhb_gguf_tensor_get(self.handle, idx, C.byref(t)) != 0:
            raise KeyError(key)
        return {"name": t.name.decode(), "dims": tuple(t.dims[: max(t.n_dims, 1)]), "type": t.type, "bytes": t.bytes, "offset": t.offset,
                "data": t.data}

    def number(self, key: str):
        v = C.c_double()
        if lib.nhb_gguf_get_number(self.handle, key.encode(), C.byref(v)) != 0:
            raise KeyError(key)
        return v.value

    def string(self, key: str):
        v = lib.nhb_gguf_get_string(self.handle, key.encode())
        if v is None:
            raise KeyError(key)
        return v.decode()

    def read_f32(self, name: str) -> np.ndarray:
        t = self.tensor(name)
        out = np.empty(t["bytes"] // 4, dtype=np.float32)
        _check(lib.nhb_gguf_read_f32(self.handle, name.encode(), out.ctypes.data, out.size))
        return out.reshape(tuple(reversed(t["dims"])))

    def upload_q8_0(self, ctx: "Context", name: str) -> "Weight":
        h = _vp()
        _check(lib.nhb_gguf_upload_q8_0(ctx.handle, self.handle, name.encode(), C.byref(h)), ctx.handle)
        return Weight(ctx, h.value)


class Graph:
    def __init__(self, ctx: "Context", handle: int):
        self.ctx, self.handle = ctx, handle

    def launch(self):
        _check(lib.nhb_graph_launch(self.ctx.handle, self.handle), self.ctx.handle)

    def free(self):
        if self.handle:
            lib.nhb_graph_free(self.ctx.handle, self.handle)
            self.handle = None


class Chain:
    """A token's sequence of dependent stages as one persistent kernel (nhb_chain_*)."""

    def __init__(self, ctx: "Context", handle: int, keep):
        self.ctx, self.handle, self._keep = ctx, handle, keep  # the tensors the chain names stay alive with it

    def launch(self):
        _check(lib.nhb_chain_launch(self.ctx.handle, self.handle), self.ctx.handle)

    def free(self):
        if self.handle:
            lib.nhb_chain_free(self.ctx.handle, self.handle)
            self.handle = None
            self._keep = None


class Context:
    """One GPU, one row shard (rank of world)."""

    def __init__(self, device: int = 0, rank: int = 0, world: int = 1):
        h = _vp()
        _check(lib.nhb_ctx_create(C.byref(h), device, rank, world))
        self.handle = h.value
        self.device, self.rank, self.world = device, rank, world

    def close(self):
        if self.handle:
            lib.nhb_ctx_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def set_stream(self, cuda_stream: int | None):
        _check(lib.nhb_ctx_set_stream(self.handle, cuda_stream), self.handle)

    def use_torch_stream(self):
        """Run on torch's current stream, so tensors made by torch and kernels launched here are ordered."""
        import torch

        # torch reports its default stream as handle 0, which nhb_ctx_set_stream reads as "the context's own
        # stream"; 1 is cudaStreamLegacy, the same default stream named explicitly
        self.set_stream(torch.cuda.current_stream().cuda_stream or 1)

    def set_option(self, name: str, value: int):
        _check(lib.nhb_ctx_set_option(self.handle, name.encode(), value), self.handle)

    def sync(self):
        _check(lib.nhb_sync(self.handle), self.handle)

    @property
    def launches(self) -> int:
        return int(lib.nhb_ctx_launch_count(self.handle))

    def upload(self, blocks: np.ndarray) -> Weight:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        N, nb, bb = blocks.shape
        assert bb == 34
        h = _vp()
        _check(lib.nhb_weight_upload_q8_0(self.handle, blocks.ctypes.data, N, nb * 32, C.byref(h)), self.handle)
        return Weight(self, h.value)

    def load_weight(self, path: str, N: int, K: int) -> Weight:
        """A weight from its cache file (nhb_weight_load): the planes go straight to the device."""
        h = _vp()
        _check(lib.nhb_weight_load(self.handle, os.fsencode(path), N, K, C.byref(h)), self.handle)
        return Weight(self, h.value)

    def get_rows(self, table: Weight, token_ids, y=None):
        """Token-embedding gather: token_ids torch cuda int32 [M] -> f32 [M, K]."""
        import torch

        M = token_ids.shape[0]
        if y is None:
            y = torch.zeros((M, table.K), dtype=torch.float32, device=token_ids.device)
        _check(lib.nhb_get_rows_q8_0(self.handle, table.handle, token_ids.data_ptr(), M, y.data_ptr(), _ld(y) if M else table.K), self.handle)
        return y

    def last_token_logits(self, w: Weight, hidden, norm_w, eps: float, sqrt_mode: int = SQRT_IEEE):
        import torch

        seq = hidden.shape[0]
        out = torch.zeros((1, w.N), dtype=torch.float32, device=hidden.device)
        _check(lib.nhb_last_token_logits(self.handle, w.handle, hidden.data_ptr(), _ld(hidden), seq, norm_w.data_ptr(), eps, sqrt_mode, out.data_ptr()), self.handle)
        return out

    # ---- device-pointer level (torch tensors supply the memory) ----
    def mul_mat(self, w: Weight, x, y=None, act_mode: int = ACT_Q8, kernel: int = KERNEL_AUTO):
        """x: torch cuda f32 [M, K] (row stride allowed) -> y f32 [M, N] (this shard's columns written)."""
        import torch

        M = x.shape[0]
        if y is None:
            y = torch.zeros((M, w.N), dtype=torch.float32, device=x.device)
        _check(lib.nhb_mul_mat(self.handle, w.handle, x.data_ptr(), _ld(x) if M > 0 else w.K, y.data_ptr(),
                               _ld(y) if M > 0 else max(w.N, 1), M, act_mode, kernel), self.handle)
        return y

    def mul_mat_batch(self, ops, act_mode: int = ACT_Q8, kernel: int = KERNEL_AUTO):
        """ops: list of (Weight, x, y) torch tensors."""
        arr = (MulMatOp * len(ops))()
        for i, (w, x, y) in enumerate(ops):
            arr[i] = MulMatOp(w.handle, x.data_ptr(), _ld(x), y.data_ptr(), _ld(y), x.shape[0])
        _check(lib.nhb_mul_mat_batch(self.handle, arr, len(ops), act_mode, kernel), self.handle)

    def mul_mat_host(self, w: Weight, x: np.ndarray, y: np.ndarray | None = None, act_mode: int = ACT_Q8, kernel: int = KERNEL_AUTO,
                     sync: bool = True) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim == 1:
            x = x[None, :]
        M = x.shape[0]
        if y is None:
            y = np.zeros((M, w.N), dtype=np.float32)
        _check(lib.nhb_mul_mat_host(self.handle, w.handle, x.ctypes.data, x.shape[1], y.ctypes.data, max(w.N, 1), M, act_mode, kernel),
               self.handle)
        if sync:
            self.sync()
        return y

    def mul_mat_swiglu_add(self, w: Weight, gate, up, residual=None, y=None):
        """y = W . quantise(silu(gate) * up) [+ residual] (the FFN tail of a block)."""
        import torch

        M = gate.shape[0]
        if y is None:
            y = torch.zeros((M, w.N), dtype=torch.float32, device=gate.device)
        _check(lib.nhb_mul_mat_swiglu_add(self.handle, w.handle, gate.data_ptr(), up.data_ptr(), _ld(gate) if M else w.K,
                                          residual.data_ptr() if residual is not None else None, _ld(residual) if residual is not None and M else max(w.N, 1),
                                          y.data_ptr(), _ld(y) if M else max(w.N, 1), M), self.handle)
        return y

    def mul_mat_add(self, w: Weight, x, residual, y=None):
        """y = W . quantise(x) + residual (attn_output and the residual stream)."""
        import torch

        M = x.shape[0]
        if y is None:
            y = torch.zeros((M, w.N), dtype=torch.float32, device=x.device)
        _check(lib.nhb_mul_mat_add(self.handle, w.handle, x.data_ptr(), _ld(x) if M else w.K, residual.data_ptr(), _ld(residual) if M else max(w.N, 1),
                                   y.data_ptr(), _ld(y) if M else max(w.N, 1), M), self.handle)
        return y

    def swiglu(self, gate, up):
        import torch

        M, K = gate.shape
        h = torch.empty((M, K), dtype=torch.float32, device=gate.device)
        _check(lib.nhb_swiglu(self.handle, gate.data_ptr(), up.data_ptr(), _ld(gate) if M else K, h.data_ptr(), K, M, K), self.handle)
        return h

    def block_dots(self, w: Weight, x):
        import torch

        M = x.shape[0]
        out = torch.zeros((M, w.n1 - w.n0, w.K // 32), dtype=torch.int32, device=x.device)
        _check(lib.nhb_mul_mat_block_dots(self.handle, w.handle, x.data_ptr(), x.stride(0), M, out.data_ptr()), self.handle)
        return out

    def quantize(self, x):
        import torch

        M, K = x.shape
        q = torch.empty((M, K), dtype=torch.int8, device=x.device)
        d = torch.empty((M, K // 32), dtype=torch.float32, device=x.device)
        _check(lib.nhb_quantize_q8_0(self.handle, x.data_ptr(), x.stride(0), M, K, q.data_ptr(), d.data_ptr()), self.handle)
        return q, d

    # ---- rms_norm x norm-weight ----
    def rms_norm_mul(self, x, norm_w, eps: float, sqrt_mode: int = SQRT_IEEE, y=None):
        import torch

        M, K = x.shape
        if y is None:
            y = torch.empty((M, K), dtype=torch.float32, device=x.device)
        _check(lib.nhb_rms_norm_mul(self.handle, x.data_ptr(), x.stride(0) if M > 0 else K, norm_w.data_ptr(), eps, sqrt_mode, y.data_ptr(),
                                    y.stride(0) if M > 0 else K, M, K), self.handle)
        return y

    def rms_norm_mul_q8_0(self, x, norm_w, eps: float, sqrt_mode: int = SQRT_IEEE):
        """Returns the rows as 34-byte Q8_0 blocks: uint8 [M][K/32][34]."""
        import torch

        M, K = x.shape
        out = torch.empty((M, K // 32, 34), dtype=torch.uint8, device=x.device)
        _check(lib.nhb_rms_norm_mul_q8_0(self.handle, x.data_ptr(), x.stride(0) if M > 0 else K, norm_w.data_ptr(), eps, sqrt_mode,
                                         out.data_ptr(), M, K), self.handle)
        return out

    def rms_norm_mul_mat_batch(self, ops, norm_w, eps: float, sqrt_mode: int = SQRT_IEEE, kernel: int = KERNEL_AUTO):
        """ops: list of (Weight, x, y); x is the row before the norm, the same tensor in every op."""
        arr = (MulMatOp * len(ops))()
        for i, (w, x, y) in enumerate(ops):
            arr[i] = MulMatOp(w.handle, x.data_ptr(), _ld(x), y.data_ptr(), _ld(y), x.shape[0])
        _check(lib.nhb_rms_norm_mul_mat_batch(self.handle, arr, len(ops), norm_w.data_ptr(), eps, sqrt_mode, kernel), self.handle)

    def memcpy_h2d(self, dst_ptr: int, src_ptr: int, nbytes: int):
        _check(lib.nhb_memcpy_h2d(self.handle, dst_ptr, src_ptr, nbytes), self.handle)

    def memcpy_d2h(self, dst_ptr: int, src_ptr: int, nbytes: int):
        _check(lib.nhb_memcpy_d2h(self.handle, dst_ptr, src_ptr, nbytes), self.handle)

    def chain(self, stages) -> Chain:
        """stages: list of stages, each a list of (Weight, x, y); every stage may read the outputs of the one before."""
        flat = [op for st in stages for op in st]
        arr = (MulMatOp * max(len(flat), 1))()
        for i, (w, x, y) in enumerate(flat):
            arr[i] = MulMatOp(w.handle, x.data_ptr(), _ld(x), y.data_ptr(), _ld(y), x.shape[0])
        counts = (_i * max(len(stages), 1))(*[len(st) for st in stages])
        h = _vp()
        _check(lib.nhb_chain_create(self.handle, arr, counts, len(stages), C.byref(h)), self.handle)
        return Chain(self, h.value, flat)

    # ---- graphs ----
    def graph_begin(self):
        _check(lib.nhb_graph_begin(self.handle), self.handle)

    def graph_end(self) -> Graph:
        h = _vp()
        _check(lib.nhb_graph_end(self.handle, C.byref(h)), self.handle)
        return Graph(self, h.value)

    # ---- multi-GPU ----
    @staticmethod
    def comm_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        _check(lib.nhb_comm_unique_id(buf))
        return buf.raw

    def comm_init(self, uid: bytes):
        buf = C.create_string_buffer(uid, 128)
        _check(lib.nhb_comm_init(self.handle, buf), self.handle)

    def symm_empty(self, shape, dtype=None):
        """A zeroed torch tensor in symmetric memory (collective: same call, same order, on every rank)."""
        import torch

        dtype = dtype or torch.float32
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = max(n, 1) * torch.empty((), dtype=dtype).element_size()
        p = _vp()
        _check(lib.nhb_symm_alloc(self.handle, nbytes, C.byref(p)), self.handle)
        return _tensor_from_ptr(p.value, nbytes, self.device, dtype).view(*shape) if n else torch.empty(shape, dtype=dtype, device=f"cuda:{self.device}")

    def all_gather(self, y):
        M, N = y.shape
        _check(lib.nhb_all_gather(self.handle, y.data_ptr(), y.stride(0), M, N), self.handle)

    def all_gather_batch(self, ys):
        n = len(ys)
        ptrs = (_vp * n)(*[y.data_ptr() for y in ys])
        ld = (_i64 * n)(*[y.stride(0) for y in ys])
        ms = (_i64 * n)(*[y.shape[0] for y in ys])
        ns = (_i64 * n)(*[y.shape[1] for y in ys])
        _check(lib.nhb_all_gather_batch(self.handle, ptrs, ld, ms, ns, n), self.handle)


# ---- one process driving several GPUs: ctxs[i] is rank i of a world of len(ctxs) ----
def _handles(ctxs):
    return (_vp * len(ctxs))(*[c.handle for c in ctxs])


def symm_empty_local(ctxs, shape, dtype=None):
    """One zeroed torch tensor per context, the same symmetric allocation on every context's device."""
    import torch

    dtype = dtype or torch.float32
    n = 1
    for d in shape:
        n *= int(d)
    nbytes = max(n, 1) * torch.empty((), dtype=dtype).element_size()
    out = (_vp * len(ctxs))()
    _check(lib.nhb_symm_alloc_local(_handles(ctxs), len(ctxs), nbytes, out), ctxs[0].handle)
    return [_tensor_from_ptr(out[i], nbytes, c.device, dtype).view(*shape) for i, c in enumerate(ctxs)]


def all_gather_local(ctxs, ys):
    M, N = ys[0].shape
    ptrs = (_vp * len(ys))(*[y.data_ptr() for y in ys])
    _check(lib.nhb_all_gather_local(_handles(ctxs), len(ctxs), ptrs, ys[0].stride(0), M, N), ctxs[0].handle)


def sync_all(ctxs):
    _check(lib.nhb_sync_all(_handles(ctxs), len(ctxs)), ctxs[0].handle)


class WaitPlanner:
    """The wait decisions of the fused all-gather without a GPU (nhb_wait_planner_*): buffers are (address, bytes) pairs."""

    def __init__(self, peer_window: int = 4):
        self.handle = lib.nhb_wait_planner_create(peer_window)

    def add_region(self, base: int, nbytes: int):
        _check(lib.nhb_wait_planner_add_region(self.handle, base, nbytes))

    def launch(self, reads, writes, delivers: bool):
        """reads / writes: lists of (address, bytes).  Returns (waits, lag)."""
        ri = (_vp * max(len(reads), 1))(*[a for a, _ in reads])
        rb = (C.c_size_t * max(len(reads), 1))(*[b for _, b in reads])
        wi = (_vp * max(len(writes), 1))(*[a for a, _ in writes])
        wb = (C.c_size_t * max(len(writes), 1))(*[b for _, b in writes])
        waits, lag = _i(), _i()
        _check(lib.nhb_wait_planner_launch(self.handle, ri, rb, len(reads), wi, wb, len(writes), int(delivers), C.byref(waits), C.byref(lag)))
        return bool(waits.value), lag.value

    def wait_all(self) -> bool:
        return bool(lib.nhb_wait_planner_wait_all(self.handle))

    def capture_begin(self):
        lib.nhb_wait_planner_capture_begin(self.handle)

    def capture_end(self) -> int:
        return int(lib.nhb_wait_planner_capture_end(self.handle))

    def replayed(self, recording: int):
        _check(lib.nhb_wait_planner_replayed(self.handle, recording))

    @property
    def seq(self) -> int:
        return int(lib.nhb_wait_planner_seq(self.handle))

    def close(self):
        if self.handle:
            lib.nhb_wait_planner_destroy(self.handle)
            self.handle = None
