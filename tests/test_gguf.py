"""GGUF reader in front of the upload: header, metadata, tensor table and placement against a writer that restates the
reference parser's format (CPU), then Q8_0 tensors uploaded from the mapped file and multiplied (gpu)."""
import os
import struct

import numpy as np
import pytest

from gguf_writer import GGML_F16, GGML_F32, GGML_Q8_0, T_ARRAY, T_BOOL, T_F32, T_STRING, T_U32, T_U64, write_gguf


def _model(tmp_path, alignment=32, **kw):
    from nihilus_b200 import synth

    wq = synth.make_weight(96, 256, 5)
    wk = synth.make_weight(40, 256, 6)
    norm = np.linspace(0.5, 1.5, 256, dtype=np.float32)
    emb = np.arange(2 * 3 * 64, dtype=np.float32).reshape(2, 3, 64)
    kvs = [
        ("general.architecture", T_STRING, "llama"),
        ("llama.block_count", T_U32, 1),
        ("llama.attention.layer_norm_rms_epsilon", T_F32, 1e-5),
        ("llama.context_length", T_U64, 8192),
        ("tokenizer.ggml.tokens", T_ARRAY, (T_STRING, ["<s>", "hello", "wor", "ld"])),
        ("tokenizer.ggml.token_type", T_ARRAY, (T_U32, [3, 1, 1, 1])),
        ("some.flag", T_BOOL, 1),
    ]
    tensors = [("blk.0.attn_q.weight", GGML_Q8_0, wq), ("blk.0.attn_norm.weight", GGML_F32, norm), ("blk.0.attn_k.weight", GGML_Q8_0, wk),
               ("extra.f32_3d", GGML_F32, emb)]
    path = str(tmp_path / "tiny.gguf")
    data_start = write_gguf(path, kvs, tensors, alignment=alignment, **kw)
    return path, data_start, {"wq": wq, "wk": wk, "norm": norm, "emb": emb}


@pytest.mark.parametrize("alignment", [32, 64, 4096])
def test_header_metadata_and_tensor_table(capi, tmp_path, alignment):
    path, data_start, ref = _model(tmp_path, alignment)
    raw = open(path, "rb").read()
    with capi.Gguf(path) as g:
        assert len(g) == 4
        assert g.string("general.architecture") == "llama"
        assert g.number("llama.block_count") == 1 and g.number("llama.context_length") == 8192 and g.number("some.flag") == 1
        assert abs(g.number("llama.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12
        with pytest.raises(KeyError):
            g.number("tokenizer.ggml.tokens")  # arrays are walked, not kept
        t = g.tensor("blk.0.attn_q.weight")
        assert t["dims"] == (256, 96) and t["type"] == 8 and t["bytes"] == 96 * 8 * 34
        assert t["offset"] == data_start and t["offset"] % alignment == 0
        assert raw[t["offset"]:t["offset"] + t["bytes"]] == ref["wq"].tobytes()
        tk = g.tensor("blk.0.attn_k.weight")
        assert tk["offset"] % alignment == 0 and raw[tk["offset"]:tk["offset"] + tk["bytes"]] == ref["wk"].tobytes()
        assert g.tensor(3)["name"] == "extra.f32_3d" and g.tensor(3)["dims"] == (64, 3, 2)
        assert (g.read_f32("blk.0.attn_norm.weight") == ref["norm"]).all()
        assert (g.read_f32("extra.f32_3d") == ref["emb"]).all()
        with pytest.raises(KeyError):
            g.tensor("blk.7.attn_q.weight")


def test_malformed_files_are_rejected(capi, tmp_path):
    path, _, _ = _model(tmp_path)
    good = open(path, "rb").read()

    def opens(data):
        p = str(tmp_path / "bad.gguf")
        with open(p, "wb") as f:
            f.write(data)
        try:
            capi.Gguf(p).close()
            return None
        except capi.NhbError as e:
            return str(e)

    assert opens(good) is None
    assert "magic" in opens(b"GGUX" + good[4:])
    assert "tensor count" in opens(good[:8] + struct.pack("<Q", 100001) + good[16:])
    assert "metadata count" in opens(good[:16] + struct.pack("<Q", 10001) + good[24:])
    assert opens(good[:40]) is not None  # truncated inside the metadata
    assert opens(good[:-100]) is not None  # tensor data cut short: the table no longer fits in front of the data
    assert "too small" in opens(good[:10])
    with pytest.raises(capi.NhbError):
        capi.Gguf(str(tmp_path / "does_not_exist.gguf"))
    # a tensor of a type this reader cannot size
    p2 = str(tmp_path / "k.gguf")
    write_gguf(p2, [], [("w", 12, np.zeros((4, 8), dtype=np.uint8))])
    with pytest.raises(capi.NhbError, match="type 12"):
        capi.Gguf(p2)
    # five dimensions
    p3 = str(tmp_path / "d5.gguf")
    write_gguf(p3, [], [("w", GGML_F32, np.zeros((1, 1, 1, 1, 4), dtype=np.float32))])
    with pytest.raises(capi.NhbError, match="4 dimensions"):
        capi.Gguf(p3)


def test_a_tensor_size_that_wraps_64_bits_is_rejected(capi, tmp_path):
    """Every dimension may be up to 2^32, so blocks x type size x rows can wrap: a q8_0 tensor of [2^32, 4042322161]
    would come out as 2^28 bytes and pass every inside-the-file check."""
    dims = [1 << 32, 4042322161]
    assert (dims[0] // 32 * 34 * dims[1]) % (1 << 64) == 1 << 28
    name = b"blk.0.attn_q.weight"
    head = struct.pack("<IIQQ", 0x46554747, 3, 1, 0)
    head += struct.pack("<Q", len(name)) + name + struct.pack("<I", 2) + struct.pack("<QQ", *dims) + struct.pack("<IQ", 8, 0)
    head += b"\0" * ((-len(head)) % 32)
    p = str(tmp_path / "wrap.gguf")
    with open(p, "wb") as f:
        f.write(head + b"\0" * (1 << 28))
    with pytest.raises(capi.NhbError, match="64 bits"):
        capi.Gguf(p)


def test_f16_and_upload_argument_checks(capi, tmp_path):
    p = str(tmp_path / "h.gguf")
    write_gguf(p, [], [("h", GGML_F16, np.ones((3, 32), dtype=np.float16))])
    with capi.Gguf(p) as g:
        assert g.tensor("h")["bytes"] == 3 * 32 * 2
        assert capi.lib.nhb_gguf_upload_q8_0(None, g.handle, b"h", None) != 0  # no context: rejected before any GPU call


@pytest.mark.gpu
def test_upload_from_gguf_and_multiply(capi, oracle, tmp_path):
    import torch

    from oracle import pyoracle as po

    path, _, ref = _model(tmp_path, 64)
    ctx = capi.Context(0)
    ctx.use_torch_stream()
    with capi.Gguf(path) as g:
        hq, hk = g.upload_q8_0(ctx, "blk.0.attn_q.weight"), g.upload_q8_0(ctx, "blk.0.attn_k.weight")
        nw = torch.from_numpy(g.read_f32("blk.0.attn_norm.weight")).cuda()
        eps = float(np.float32(g.number("llama.attention.layer_norm_rms_epsilon")))
        with pytest.raises(capi.NhbError):
            g.upload_q8_0(ctx, "blk.0.attn_norm.weight")  # f32, not a Q8_0 matrix
    # the mapping is gone; the device copies are not
    assert (hq.N, hq.K, hk.N, hk.K) == (96, 256, 40, 256)
    assert (hq.download() == ref["wq"]).all() and (hk.download() == ref["wk"]).all()
    x = (np.random.default_rng(4).standard_normal((2, 256)) * 2).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    yq, yk = torch.zeros((2, 96), device="cuda"), torch.zeros((2, 40), device="cuda")
    ctx.rms_norm_mul_mat_batch([(hq, xd, yq), (hk, xd, yk)], nw, eps)
    ctx.sync()
    normed = oracle.rms_norm_mul(x, ref["norm"], eps, 0)
    for w, y in ((ref["wq"], yq), (ref["wk"], yk)):
        r = oracle.mul_mat(po.Q8ACT_LANES, w, normed)
        assert np.abs(y.cpu().numpy() - r).max() <= 1e-4 * np.abs(r).max()
    hq.free()
    hk.free()
    ctx.close()
