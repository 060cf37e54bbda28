"""The .rax payload reader against containers laid out as
runtime/include/buddy/runtime/core/ModelManifest.h:124-310 describes them
(the reference ships no packaged .rax fixture, so the bytes are written here
from that description).  No GPU needed."""
import ctypes as C
import struct

import numpy as np
import pytest

from buddy_mlir_b200 import _lib


def make_rax(path, blobs, manifest=b"\x10\x00\x00\x00RAX0" + b"m" * 56, corrupt=None):
    """[manifest][payload blobs][index][footer]; blobs: [(kind, name, bytes)]."""
    out = bytearray(manifest)
    payload_offset = len(out)
    entries = []
    for kind, name, data in blobs:
        entries.append((kind, name.encode(), len(out), len(data)))
        out += data
    payload_size = len(out) - payload_offset
    index_offset = len(out)
    idx = bytearray(b"RAXIDX01" + struct.pack("<II", 1, len(entries)))
    for kind, name, off, size in entries:
        idx += struct.pack("<HHIQQ", kind, 0, len(name), off, size) + name
    out += idx
    footer = bytearray(b"RAXPAY01" + struct.pack("<QQQQQQ", len(manifest), payload_offset, payload_size,
                                                 index_offset, len(idx), 0) + b"\0" * 8)
    assert len(footer) == 64
    if corrupt == "payload_offset":
        footer[16:24] = struct.pack("<Q", payload_offset + 8)
    out += footer
    open(path, "wb").write(out)


def test_payload_entries_are_found_and_read(tmp_path):
    lib = _lib.load()
    f32 = np.arange(100, dtype=np.float32)
    i8 = np.arange(-50, 50, dtype=np.int8)
    p = tmp_path / "model.rax"
    make_rax(p, [(1, "kernels/forward.so", b"\x7fELF" + b"\0" * 60),
                 (2, "weights/arg0-w8a32-f32.data", f32.tobytes()),
                 (2, "weights/arg0-w8a32-i8.data", i8.tobytes())])
    h = C.c_void_p()
    _lib.check(lib.b200_rax_open(str(p).encode(), C.byref(h)))
    assert lib.b200_rax_count(h) == 3 and lib.b200_rax_manifest_bytes(h) == 64
    name = C.create_string_buffer(256)
    kind, off, size = C.c_int(), C.c_uint64(), C.c_uint64()
    _lib.check(lib.b200_rax_entry(h, 1, name, 256, C.byref(kind), C.byref(off), C.byref(size)))
    assert name.value == b"weights/arg0-w8a32-f32.data" and kind.value == 2 and size.value == 400
    i = lib.b200_rax_find(h, b"-i8.data")
    assert i == 2
    got = np.zeros(100, dtype=np.int8)
    _lib.check(lib.b200_rax_read(h, i, got.ctypes.data, got.nbytes))
    assert np.array_equal(got, i8)
    got32 = np.zeros(100, dtype=np.float32)
    _lib.check(lib.b200_rax_read(h, lib.b200_rax_find(h, b"-f32.data"), got32.ctypes.data, got32.nbytes))
    assert np.array_equal(got32, f32)
    assert lib.b200_rax_read(h, i, got.ctypes.data, 99) != 0          # size must match
    assert lib.b200_rax_find(h, b"nothing") == -1
    lib.b200_rax_close(h)


def test_manifest_only_and_malformed_packages(tmp_path):
    lib = _lib.load()
    h = C.c_void_p()
    p = tmp_path / "plain.rax"
    open(p, "wb").write(b"\x10\x00\x00\x00RAX0" + b"x" * 100)           # no payload footer
    _lib.check(lib.b200_rax_open(str(p).encode(), C.byref(h)))
    assert lib.b200_rax_count(h) == 0 and lib.b200_rax_manifest_bytes(h) == 108
    lib.b200_rax_close(h)
    q = tmp_path / "bad.rax"
    open(q, "wb").write(b"not a package at all")
    assert lib.b200_rax_open(str(q).encode(), C.byref(h)) == -1
    r = tmp_path / "bad2.rax"
    make_rax(r, [(2, "w.data", b"1234")], corrupt="payload_offset")
    assert lib.b200_rax_open(str(r).encode(), C.byref(h)) == -1
    assert b"payload" in lib.b200_last_error()
