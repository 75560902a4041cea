"""The allocation-free entry point, nhb_mul_mat_q8_0_noalloc, against the regular nhb_mul_mat and the CPU oracle (needs a B200).

Collected last on purpose: a run that stops at the first failure has by then exercised every other test.

Who needs it: a host that may not allocate where it calls the operator -- an engine that carved up one device
arena at start-up and runs from a fixed memory plan, or a token loop that cannot
afford the device-wide synchronisation an allocation may bring.  The entry point takes raw device pointers
(weight planes, activations, outputs) and keeps its one temporary, the quantised activations, in a fixed
96 KiB array inside the library.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4  # same bound as the other parity tests: max|err| / max|ref|


def _bind(capi):
    fn = capi.lib.nhb_mul_mat_q8_0_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    err = capi.lib.nhb_noalloc_last_error
    err.restype = C.c_char_p
    err.argtypes = []
    return fn, err


def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row(capi, oracle):
    import torch

    from nihilus_b200 import synth
    from oracle import pyoracle as po

    fn, err = _bind(capi)
    ctx = capi.Context(0)
    ctx.use_torch_stream()
    try:
        for N, K, M in ((1024, 4096, 1), (300, 14336, 3), (77, 96, 4)):
            w = synth.make_weight(N, K, 5150 + N)
            h = ctx.upload(w)
            xs = [torch.from_numpy(synth.make_activation(M, K, 5200 + i)).cuda() for i in range(2)]
            want = []
            for x in xs:
                want.append(ctx.mul_mat(h, x).clone())
            ctx.sync()
            # two calls back to back on one stream, sharing the fixed scratch: the second must not see the first's data
            stream = torch.cuda.current_stream().cuda_stream
            got = [torch.full((M, N), float("nan"), device="cuda") for _ in xs]
            for x, y in zip(xs, got):
                rc = fn(h.q_ptr, h.d_ptr, N, K, x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), M, stream)
                assert rc == 0, err().decode()
            torch.cuda.synchronize()
            for y, ref in zip(got, want):
                ref = ref.cpu().numpy()
                rel = float(np.abs(y.cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-30))
                assert rel <= TOL, (N, K, M, rel, y.cpu().numpy()[0, :4], ref[0, :4])
            assert not torch.equal(got[0], got[1])
            # and against the CPU oracle, so that a fault shared with the regular entry point could not hide
            ref = oracle.mul_mat(po.Q8ACT_LANES, w, xs[1].cpu().numpy())
            assert float(np.abs(got[1].cpu().numpy() - ref).max() / np.abs(ref).max()) <= TOL
            h.free()
    finally:
        ctx.close()


def test_noalloc_rejects_what_does_not_fit_and_bad_arguments(capi):
    import torch

    fn, err = _bind(capi)
    q = torch.zeros(32 * 65536, dtype=torch.int8, device="cuda")
    d = torch.zeros(65536 // 32 * 32, dtype=torch.float16, device="cuda")
    x = torch.zeros((8, 65536), device="cuda")
    y = torch.zeros((8, 32), device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert capi.lib.nhb_noalloc_max_bytes() == 96 * 1024
    # M beyond 4, and M * (K + K/8) beyond the fixed array
    assert fn(q.data_ptr(), d.data_ptr(), 32, 4096, x.data_ptr(), 65536, y.data_ptr(), 32, 5, s) == capi.ERR_UNSUPPORTED
    assert "98304" in err().decode()
    assert fn(q.data_ptr(), d.data_ptr(), 32, 65536, x.data_ptr(), 65536, y.data_ptr(), 32, 2, s) == capi.ERR_UNSUPPORTED
    # malformed calls
    assert fn(q.data_ptr(), d.data_ptr(), 32, 100, x.data_ptr(), 65536, y.data_ptr(), 32, 1, s) == capi.ERR_ARG
    assert fn(None, d.data_ptr(), 32, 4096, x.data_ptr(), 65536, y.data_ptr(), 32, 1, s) == capi.ERR_ARG
    assert fn(q.data_ptr() + 16, d.data_ptr(), 32, 4096, x.data_ptr(), 65536, y.data_ptr(), 32, 1, s) == capi.ERR_ARG
    assert fn(q.data_ptr(), d.data_ptr(), 32, 4096, x.data_ptr(), 64, y.data_ptr(), 32, 1, s) == capi.ERR_ARG
    assert fn(q.data_ptr(), d.data_ptr(), 32, 4096, x.data_ptr(), 65536, y.data_ptr() + 2, 32, 1, s) == capi.ERR_ARG  # misaligned output
    # nothing to do is not an error
    assert fn(q.data_ptr(), d.data_ptr(), 0, 4096, x.data_ptr(), 65536, y.data_ptr(), 32, 1, s) == 0
    assert fn(q.data_ptr(), d.data_ptr(), 32, 4096, x.data_ptr(), 65536, y.data_ptr(), 32, 0, s) == 0
    torch.cuda.synchronize()
