"""A minimal GGUF writer for the tests: the on-disk format the reference's parser reads
(include/nihilus-incl/infra/model_parser.hpp:635-671, 855-940), restated from its reader.  Test infrastructure only."""
import struct

import numpy as np

T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 = range(13)
GGML_F32, GGML_F16, GGML_Q8_0 = 0, 1, 8


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _value(vtype: int, v) -> bytes:
    fmt = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<B", T_U64: "<Q", T_I64: "<q",
           T_F64: "<d"}
    if vtype in fmt:
        return struct.pack(fmt[vtype], v)
    if vtype == T_STRING:
        return _s(v)
    if vtype == T_ARRAY:
        etype, items = v
        return struct.pack("<IQ", etype, len(items)) + b"".join(_value(etype, it) for it in items)
    raise ValueError(vtype)


def write_gguf(path, kvs, tensors, alignment=32, magic=0x46554747, version=3, pad_tail=0):
    """kvs: list of (key, type, value); tensors: list of (name, ggml_type, array) where a Q8_0 array is uint8
    [N][K/32][34] (dims written as [K, N]) and an f32 array is float32 of any rank (dims written innermost first)."""
    kvs = list(kvs)
    if alignment != 32:
        kvs.append(("general.alignment", T_U32, alignment))
    head = struct.pack("<IIQQ", magic, version, len(tensors), len(kvs))
    for key, vtype, v in kvs:
        head += _s(key) + struct.pack("<I", vtype) + _value(vtype, v)
    infos, blobs, off = b"", [], 0
    for name, gtype, arr in tensors:
        if gtype == GGML_Q8_0:
            n, nb, bb = arr.shape
            assert bb == 34
            dims = [nb * 32, n]
        else:
            dims = list(reversed(arr.shape))
        off = (off + alignment - 1) // alignment * alignment
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", gtype, off)
        data = np.ascontiguousarray(arr).tobytes()
        blobs.append((off, data))
        off += len(data)
    data_len = off
    body = bytearray(data_len)
    for o, d in blobs:
        body[o:o + len(d)] = d
    head += infos
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad + bytes(body) + b"\0" * pad_tail)
    return len(head) + pad  # offset of the data section
