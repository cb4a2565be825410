"""Weights read straight out of a GGUF file by the native layer. The test writes a small GGUF v3 file itself (header,
metadata of several value types including an array and general.alignment, three tensors) and checks the parsed table on
the CPU, then the uploaded weights on a GPU."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from sharplight_b200 import native as N
from sharplight_b200 import synth


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, tensors, alignment=64, version=3):
    """tensors: list of (name, ggml_type, dims innermost first, raw bytes)."""
    kv = [(_s("general.architecture") + struct.pack("<I", 8) + _s("llama")),
          (_s("general.alignment") + struct.pack("<II", 4, alignment)),
          (_s("tokenizer.scores") + struct.pack("<IIQ", 9, 6, 3) + struct.pack("<3f", 0.5, 1.5, 2.5)),
          (_s("tokenizer.tokens") + struct.pack("<IIQ", 9, 8, 2) + _s("a") + _s("bc")),
          (_s("llama.block_count") + struct.pack("<IQ", 10, 7))]
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kv)) + b"".join(kv)
    infos, data, off = b"", b"", 0
    for name, ttype, dims, raw in tensors:
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ttype, off)
        data += raw + b"\0" * (-len(raw) % alignment)
        off += len(raw) + (-len(raw) % alignment)
    pos = len(head) + len(infos)
    with open(path, "wb") as f:
        f.write(head + infos + b"\0" * (-pos % alignment) + data)


@pytest.fixture
def gguf_file(tmp_path):
    w1 = synth.weight_blocks("Q4_K", 48, 512, seed=1)
    w2 = synth.weight_blocks("Q8_0", 20, 96, seed=2)
    w3 = synth.weight_blocks("Q5_0", 24, 128, seed=3)
    norm = np.arange(96, dtype=np.float32).tobytes()
    path = str(tmp_path / "tiny.gguf")
    write_gguf(path, [("blk.0.ffn_down.weight", 12, [512, 48], w1.tobytes()), ("output_norm.weight", 0, [96], norm),
                      ("blk.0.attn_q.weight", 8, [96, 20], w2.tobytes()), ("blk.0.attn_k.weight", 6, [128, 24], w3.tobytes())])
    return path, w1, w2


def _open(lib, path):
    h = C.c_void_p()
    assert lib.slc_gguf_open(path.encode(), C.byref(h)) == N.OK, lib.slc_gguf_last_error()
    return h


def _info(lib, h, index):
    name = C.create_string_buffer(256)
    fmt, rank, n, k, b = C.c_int32(), C.c_int32(), C.c_int64(), C.c_int64(), C.c_int64()
    assert lib.slc_gguf_tensor_info(h, index, name, 256, C.byref(fmt), C.byref(rank), C.byref(n), C.byref(k), C.byref(b)) == N.OK
    return name.value.decode(), fmt.value, rank.value, n.value, k.value, b.value


def test_gguf_table_is_parsed(gguf_file):
    path, w1, w2 = gguf_file
    lib = N.load()
    h = _open(lib, path)
    try:
        count = C.c_int64()
        assert lib.slc_gguf_tensor_count(h, C.byref(count)) == N.OK and count.value == 4
        assert _info(lib, h, 0) == ("blk.0.ffn_down.weight", 12, 2, 48, 512, w1.size)
        assert _info(lib, h, 1) == ("output_norm.weight", 0, 1, 1, 96, 0)          # f32, 1-D: not a served weight
        assert _info(lib, h, 2) == ("blk.0.attn_q.weight", 8, 2, 20, 96, w2.size)
        assert _info(lib, h, 3) == ("blk.0.attn_k.weight", 6, 2, 24, 128, 24 * 4 * 22)   # Q5_0: served through the Q8_0 layout
        idx = C.c_int64()
        assert lib.slc_gguf_find(h, b"blk.0.attn_q.weight", C.byref(idx)) == N.OK and idx.value == 2
        assert lib.slc_gguf_find(h, b"nope", C.byref(idx)) != N.OK and idx.value == -1
        tiny = C.create_string_buffer(4)
        assert lib.slc_gguf_tensor_info(h, 0, tiny, 4, None, None, None, None, None) == N.ERR_BUFFER_TOO_SMALL
    finally:
        lib.slc_gguf_close(h)


def test_gguf_rejects_bad_files(tmp_path, gguf_file):
    lib = N.load()
    h = C.c_void_p()
    assert lib.slc_gguf_open(str(tmp_path / "missing.gguf").encode(), C.byref(h)) != N.OK
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    assert lib.slc_gguf_open(str(bad).encode(), C.byref(h)) != N.OK and b"magic" in lib.slc_gguf_last_error()
    v9 = tmp_path / "v9.gguf"
    write_gguf(str(v9), [], version=9)
    assert lib.slc_gguf_open(str(v9).encode(), C.byref(h)) == N.ERR_UNSUPPORTED
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(open(gguf_file[0], "rb").read()[:150])
    assert lib.slc_gguf_open(str(cut).encode(), C.byref(h)) != N.OK and b"truncated" in lib.slc_gguf_last_error()


@pytest.mark.gpu
def test_gguf_upload_equals_upload_of_the_same_blocks(cuda_device, gguf_file):
    from sharplight_b200 import MatMulOp
    from sharplight_b200.provider import DeviceWeight
    path, w1, w2 = gguf_file
    lib = N.load()
    h = _open(lib, path)
    try:
        for index, (type_name, n, k, blocks) in ((0, ("Q4_K", 48, 512, w1)), (2, ("Q8_0", 20, 96, w2))):
            wh = C.c_void_p()
            assert lib.slc_weight_upload_gguf(cuda_device.handle, h, index, C.byref(wh)) == N.OK, lib.slc_gguf_last_error()
            w = DeviceWeight(cuda_device, {"Q4_K": 12, "Q8_0": 8}[type_name], n, k, wh.value)
            ref = cuda_device.upload_weight(type_name, (n, k), blocks)
            x = synth.activations(3, k, seed=5)
            a, b = MatMulOp(cuda_device, w, 3), MatMulOp(cuda_device, ref, 3)
            try:
                assert np.array_equal(w.download(), blocks)
                assert np.array_equal(a.run(x).view(np.uint32), b.run(x).view(np.uint32))
            finally:
                a.dispose(); b.dispose(); w.dispose(); ref.dispose()
        # the Q5_0 tensor: converted at upload, results equal to an upload of the same blocks
        wh = C.c_void_p()
        assert lib.slc_weight_upload_gguf(cuda_device.handle, h, 3, C.byref(wh)) == N.OK, lib.slc_gguf_last_error()
        w = DeviceWeight(cuda_device, N.FMT_Q5_0, 24, 128, wh.value)
        ref = cuda_device.upload_weight("Q5_0", (24, 128), synth.weight_blocks("Q5_0", 24, 128, seed=3))
        x = synth.activations(3, 128, seed=5)
        a, b = MatMulOp(cuda_device, w, 3), MatMulOp(cuda_device, ref, 3)
        try:
            assert np.array_equal(a.run(x).view(np.uint32), b.run(x).view(np.uint32))
        finally:
            a.dispose(); b.dispose(); w.dispose(); ref.dispose()
        wh = C.c_void_p()
        assert lib.slc_weight_upload_gguf(cuda_device.handle, h, 1, C.byref(wh)) == N.ERR_UNSUPPORTED      # the f32 norm vector
    finally:
        lib.slc_gguf_close(h)
