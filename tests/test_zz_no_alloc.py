"""The allocation-free attention entry point against the ordinary one.

Some callers of this library cannot allocate device memory at decode time
(all of it was handed to a memory planner up front, or a device-stalling
cudaMalloc is not allowed inside their loop).  For them the library carries
its own split-partial scratch in a fixed array; this test drives that entry
point through the C ABI, twice in a row, and expects what b200_gqa_decode
computes with caller-owned scratch and what the CPU checker computes from the
same inputs; it also watches the free device memory across the calls.  It
lives in a file that pytest collects last, and it passes both on its own and
after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import _lib

pytestmark = pytest.mark.gpu


def _run(lib, static, q, K, V, pos, splits):
    import torch
    QH, D = q.shape
    KH, L, _ = K.shape
    dq, dk, dv = (torch.from_numpy(a).cuda() for a in (q, K, V))
    out = torch.zeros((QH, D), dtype=torch.float32, device="cuda")
    dpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    if static:
        rc = lib.b200_gqa_decode_static(p(dq), p(dk), p(dv), p(out), QH, KH, D, L, splits, p(dpos), st)
    else:
        n = lib.b200_gqa_scratch_floats(QH, D, splits)
        scratch = torch.zeros(n, dtype=torch.float32, device="cuda")
        rc = lib.b200_gqa_decode(p(dq), p(dk), p(dv), p(out), p(scratch), QH, KH, D, L, splits, p(dpos), st)
    _lib.check(rc)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_static_scratch_attention_matches_twice_in_a_row():
    lib = _lib.load()
    rng = np.random.default_rng(123)
    # two different shapes back to back: the second call finds the first call's
    # leftovers in the shared array
    for QH, KH, D, L, pos, splits in ((12, 2, 128, 1024, 1000, 16), (32, 8, 128, 512, 300, 8)):
        q = rng.standard_normal((QH, D)).astype(np.float32)
        K = rng.standard_normal((KH, L, D)).astype(np.float32)
        V = rng.standard_normal((KH, L, D)).astype(np.float32)
        want = _run(lib, False, q, K, V, pos, splits)
        checker = orc.gqa_decode(q, K, V, pos)
        for _ in range(2):
            got = _run(lib, True, q, K, V, pos, splits)
            # same kernel, same inputs: the tolerance of the attention parity tests (1e-5) is ample
            assert np.abs(got - want).max() / np.abs(want).max() < 1e-5
            assert np.abs(got - checker).max() / np.abs(checker).max() < 1e-5


def test_static_scratch_entry_allocates_nothing():
    import torch
    lib = _lib.load()
    rng = np.random.default_rng(7)
    QH, KH, D, L, pos, splits = 12, 2, 128, 256, 200, 8
    q = rng.standard_normal((QH, D)).astype(np.float32)
    K = rng.standard_normal((KH, L, D)).astype(np.float32)
    V = rng.standard_normal((KH, L, D)).astype(np.float32)
    dq, dk, dv = (torch.from_numpy(a).cuda() for a in (q, K, V))
    out = torch.zeros((QH, D), dtype=torch.float32, device="cuda")
    dpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda: _lib.check(lib.b200_gqa_decode_static(p(dq), p(dk), p(dv), p(out), QH, KH, D, L, splits, p(dpos), st))
    call()                      # the first call on a device looks up the array's address
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    want = orc.gqa_decode(q, K, V, pos)
    got = out.cpu().numpy()
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-5


def test_static_scratch_rejects_oversized_shapes():
    import torch
    lib = _lib.load()
    cap = 64 * 32 * 130 + 64  # B200_GQA_STATIC_SCRATCH_FLOATS
    assert lib.b200_gqa_scratch_floats(64, 128, 32) <= cap
    assert lib.b200_gqa_scratch_floats(128, 128, 32) > cap
    dummy = torch.zeros(16, dtype=torch.float32, device="cuda")
    dpos = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    rc = lib.b200_gqa_decode_static(p(dummy), p(dummy), p(dummy), p(dummy), 128, 16, 128, 64, 32, p(dpos), None)
    assert rc == -5
    assert b"built-in array" in lib.b200_last_error()


def test_static_scratch_rejects_bad_arguments_before_any_device_work():
    import torch
    lib = _lib.load()
    dummy = torch.zeros(16, dtype=torch.float32, device="cuda")
    dpos = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    before = lib.b200_launch_count()
    # the largest accepted shape puts the arrival counters at the very end of the
    # array; more kv heads than query heads must be refused on the host
    assert lib.b200_gqa_decode_static(p(dummy), p(dummy), p(dummy), p(dummy), 64, 128, 128, 64, 32, p(dpos), None) == -1
    assert lib.b200_gqa_decode_static(p(dummy), p(dummy), p(dummy), p(dummy), 12, 5, 128, 64, 8, p(dpos), None) == -1
    assert lib.b200_gqa_decode_static(p(dummy), p(dummy), p(dummy), p(dummy), 12, 2, 96, 64, 8, p(dpos), None) == -1
    assert lib.b200_gqa_decode_static(None, p(dummy), p(dummy), p(dummy), 12, 2, 128, 64, 8, p(dpos), None) == -1
    assert lib.b200_launch_count() == before
    torch.cuda.synchronize()
