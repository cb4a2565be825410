"""Extracts the golden vectors of the quantized-MatMul path from the reference's own test fixtures.

Run where the reference tree is available: its root is the first argument (or the SHARPLIGHT_REFERENCE environment
variable). It reads
  tests/Sharplight.Cpu.Tests/Fixtures/ggml_quant_ext.bin  (record layout: GgmlDequantTests.cs:26-48)
  tests/Sharplight.Cpu.Tests/Fixtures/ggml_quant.bin      (record layout: QuantTests.cs:16-43)
and writes, beside this script, ``ggml_golden.npz`` with the records of ggml types 2 (Q4_0), 6 (Q5_0), 8 (Q8_0), 12 (Q4_K), 13 (Q5_K), 20 (IQ4_NL) and
14 (Q6_K): raw blocks, the floats ggml's own decoder produced, and (second file) the f32 source the blocks were
quantized from. Nothing is recomputed here: the arrays are byte-for-byte slices of the fixture files.
"""
from __future__ import annotations

import os
import struct
import sys

import numpy as np

TYPES = {2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 10: (256, 84), 11: (256, 110),
         12: (256, 144), 13: (256, 176), 14: (256, 210), 16: (256, 66), 17: (256, 74), 18: (256, 98),
         19: (256, 50), 20: (32, 18), 21: (256, 110), 22: (256, 82), 23: (256, 136), 29: (256, 56),
         34: (256, 54), 35: (256, 66), 39: (32, 17), 40: (64, 36)}
KEEP = (2, 6, 8, 12, 13, 14, 20)


def read_ext(path):
    data = open(path, "rb").read()
    (count,) = struct.unpack_from("<i", data, 0)
    off = 4
    out = []
    for i in range(count):
        tid, rows, cols = struct.unpack_from("<iii", data, off)
        off += 12
        bs, bb = TYPES[tid]
        nbytes = rows * cols // bs * bb
        blocks = np.frombuffer(data, np.uint8, nbytes, off).copy()
        off += nbytes
        expected = np.frombuffer(data, "<f4", rows * cols, off).copy()
        off += rows * cols * 4
        out.append((i, tid, rows, cols, blocks, expected))
    assert off == len(data), (off, len(data))
    return out


def read_src(path):
    data = open(path, "rb").read()
    (count,) = struct.unpack_from("<i", data, 0)
    off = 4
    out = []
    for i in range(count):
        tid, rows, cols = struct.unpack_from("<iii", data, off)
        off += 12
        bs, bb = TYPES[tid]
        src = np.frombuffer(data, "<f4", rows * cols, off).copy()
        off += rows * cols * 4
        nbytes = rows * cols // bs * bb
        blocks = np.frombuffer(data, np.uint8, nbytes, off).copy()
        off += nbytes
        deq = np.frombuffer(data, "<f4", rows * cols, off).copy()
        off += rows * cols * 4
        out.append((i, tid, rows, cols, src, blocks, deq))
    assert off == len(data), (off, len(data))
    return out


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SHARPLIGHT_REFERENCE")
    if not root:
        raise SystemExit("usage: make_golden.py <root of the Sharplight tree>")
    fx = os.path.join(root, "tests", "Sharplight.Cpu.Tests", "Fixtures")
    here = os.path.dirname(os.path.abspath(__file__))
    arrays = {}
    names = []
    for i, tid, rows, cols, blocks, expected in read_ext(os.path.join(fx, "ggml_quant_ext.bin")):
        if tid not in KEEP:
            continue
        kind = "ggml" if i % 2 == 0 else "random"   # GgmlDequantTests.cs:56: even records are ggml-quantized
        name = f"ext_{tid}_{kind}"
        names.append(name)
        arrays[name + "_shape"] = np.array([tid, rows, cols], np.int32)
        arrays[name + "_blocks"] = blocks
        arrays[name + "_expected"] = expected
    for i, tid, rows, cols, src, blocks, deq in read_src(os.path.join(fx, "ggml_quant.bin")):
        if tid not in KEEP:
            continue
        name = f"src_{tid}"
        names.append(name)
        arrays[name + "_shape"] = np.array([tid, rows, cols], np.int32)
        arrays[name + "_source"] = src
        arrays[name + "_blocks"] = blocks
        arrays[name + "_expected"] = deq
    arrays["names"] = np.array(names)
    out = os.path.join(here, "ggml_golden.npz")
    np.savez_compressed(out, **arrays)
    print("wrote", out, os.path.getsize(out), "bytes;", len(names), "records:", " ".join(names))


if __name__ == "__main__":
    main()
