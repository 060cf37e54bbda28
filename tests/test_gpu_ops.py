"""Parity of every kernel with the CPU restatement, through the C ABI.
Integer / byte / index work is compared bit for bit; floating point within
the tolerances written at each assert."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import _lib, memref, synthetic, TINY_QWEN3

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")

# f32 GEMV: same products, different summation order (lanes + shuffle tree vs
# sequential k).  Bound used everywhere below: 2e-5 of the row's magnitude scale.
F32_TOL = 2e-5


def rel(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() /
                 max(np.abs(b.astype(np.float64)).max(), 1e-30))


@pytest.fixture(autouse=True)
def _fresh_cache():
    yield
    memref.release_cached_weights()


# ---- the reference's own known answers, through its own ABI -------------------
def test_known_answers_through_memref_abi():
    k = np.load(os.path.join(G, "known_answers.npz"))
    y = memref.buddy_gemv_w8_f32(k["w8_A"], k["w8_W"], k["w8_scale"])
    assert np.array_equal(y, k["w8_expect"])
    y = memref.buddy_gemv_w4_f16(k["w4_A"], k["w4_P"], k["w4_scale"])
    assert np.array_equal(y, k["w4_expect"])
    # prefill example: rows [8,8,8,8]; decode and prefill agree on exact inputs
    y = memref.buddy_gemv_w8_f32(k["pf_A"], k["pf_W"], k["pf_scale"])
    assert np.array_equal(y, k["pf_expect"])


def test_matmul_f32_symbol_handles_strides_and_many_rows():
    rng = np.random.default_rng(0)
    A = rng.standard_normal((40, 2 * 96)).astype(np.float32)[:, ::2]   # non-unit stride
    B = rng.standard_normal((96, 50)).astype(np.float32)
    y = memref.buddy_matmul_f32(A, B)
    ref = orc.gemv_f32(np.ascontiguousarray(A), B)
    assert y.shape == (40, 50) and rel(y, ref) < F32_TOL


def test_matmul_f32_sees_new_contents_at_the_same_address():
    """B of buddy_matmul_f32 is any matmul operand (an activation, a reused
    scratch buffer): a second call with other values at the same address must
    use them.  No cache reset in between."""
    rng = np.random.default_rng(1)
    A = rng.standard_normal((3, 64)).astype(np.float32)
    B = rng.standard_normal((64, 48)).astype(np.float32)
    y1 = memref.buddy_matmul_f32(A, B)
    assert rel(y1, orc.gemv_f32(A, B)) < F32_TOL
    B[...] = rng.standard_normal((64, 48)).astype(np.float32)       # same buffer, new contents
    y2 = memref.buddy_matmul_f32(A, B)
    assert rel(y2, orc.gemv_f32(A, B)) < F32_TOL
    # a transposed view of a square matrix at the same address is another operand
    S = rng.standard_normal((64, 64)).astype(np.float32)
    assert rel(memref.buddy_matmul_f32(A, S), orc.gemv_f32(A, S)) < F32_TOL
    assert rel(memref.buddy_matmul_f32(A, S.T), orc.gemv_f32(A, np.ascontiguousarray(S.T))) < F32_TOL


def test_quantised_weight_cache_notices_rewrites_and_views():
    rng = np.random.default_rng(2)
    K, N = 64, 64
    x = rng.standard_normal((1, K)).astype(np.float32)
    Q = rng.integers(-127, 128, (K, N)).astype(np.int8)
    s = rng.uniform(0.001, 0.01, (1, N)).astype(np.float32)
    assert rel(memref.buddy_gemv_w8_f32(x, Q, s), orc.gemv_w8_f32(x, Q, s[0])) < F32_TOL
    assert rel(memref.buddy_gemv_w8_f32(x, Q, s), orc.gemv_w8_f32(x, Q, s[0])) < F32_TOL   # cache hit
    Q[...] = rng.integers(-127, 128, (K, N)).astype(np.int8)        # rewritten in place
    assert rel(memref.buddy_gemv_w8_f32(x, Q, s), orc.gemv_w8_f32(x, Q, s[0])) < F32_TOL
    s[...] = rng.uniform(0.001, 0.01, (1, N)).astype(np.float32)
    assert rel(memref.buddy_gemv_w8_f32(x, Q, s), orc.gemv_w8_f32(x, Q, s[0])) < F32_TOL
    assert rel(memref.buddy_gemv_w8_f32(x, Q.T, s), orc.gemv_w8_f32(x, np.ascontiguousarray(Q.T), s[0])) < F32_TOL


# ---- committed fixtures -----------------------------------------------------------
def test_gemv_fixtures():
    g = np.load(os.path.join(G, "ops_golden.npz"))
    for tag in "abc":
        y = memref.buddy_gemv_w8_f32(g[f"w8{tag}_x"], g[f"w8{tag}_Q"], g[f"w8{tag}_s"][None, :])
        assert rel(y, g[f"w8{tag}_y"]) < F32_TOL
        y = memref.buddy_matmul_f32(g[f"w8{tag}_x"], g[f"f{tag}_B"])
        assert rel(y, g[f"f{tag}_y"]) < F32_TOL
    # int4 f16: the reference accumulates in f16, the kernel in f32 -> 2e-2
    y = memref.buddy_gemv_w4_f16(g["w4_x"], g["w4_P"], g["w4_s"][None, :])
    assert rel(y.astype(np.float32), g["w4_y"].astype(np.float32)) < 2e-2
    y = memref.buddy_gemv_w4g_f32(g["w4g_x"], g["g_P"].view(np.int8), g["g_s"])
    assert rel(y, g["w4g_y"]) < F32_TOL


def test_small_op_fixtures():
    g = np.load(os.path.join(G, "ops_golden.npz"))
    y = memref.buddy_rmsnorm_f32(g["rn_x"][None, :], g["rn_w"], 1e-6)
    assert rel(y[0], g["rn_y"]) < 1e-6
    y = memref.buddy_silu_mul_f32(g["sm_g"][None, :], g["sm_u"][None, :])
    assert rel(y[0], g["sm_y"]) < 1e-6
    y = memref.buddy_rope_f32(g["rp_x"][None, :, None, :], g["rp_inv"], 613)
    # cos/sin of arguments up to 613 rad: device and libm differ by a few ulp
    assert rel(y[0, :, 0, :], g["rp_y"]) < 1e-5


@pytest.mark.parametrize("valid_len", [9, 37, 613, 1024])
def test_attention_fixture(valid_len):
    g = np.load(os.path.join(G, "ops_golden.npz"))
    K, V = g["at_K"].astype(np.float32), g["at_V"].astype(np.float32)
    out = memref.buddy_gqa_decode_f32(g["at_q"][None, :, None, :], K[None], V[None], valid_len - 1)
    assert rel(out[0, :, 0, :], g[f"at_out_{valid_len}"]) < 1e-5


# ---- bit-exact integer work -----------------------------------------------------------
def test_quantiser_bit_exact():
    from gpu_util import dev, ptr, stream, sync
    import torch
    lib = _lib.load()
    rng = np.random.default_rng(21)
    for K, N in ((96, 40), (1536, 256), (200, 1000)):
        W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        W[:, 1] = 0
        W[0, 2] = W[:, 2].max() * 2        # values exactly at +/- qmax
        d_w = dev(W)
        for bits in (8, 4):
            q = torch.empty((K, N), dtype=torch.int8, device="cuda")
            s = torch.empty(N, dtype=torch.float32, device="cuda")
            _lib.check(lib.b200_quantize_per_channel(ptr(d_w), K, N, bits, ptr(q), ptr(s), stream()))
            sync()
            Q, S = orc.quantize_per_channel(W, bits)
            assert np.array_equal(q.cpu().numpy(), Q)
            assert np.array_equal(s.cpu().numpy(), S)
    K, N, Gs = 512, 64, 128
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    W[:128, 0] = 0
    P = torch.empty((K, N // 2), dtype=torch.uint8, device="cuda")
    S = torch.empty((K // Gs, N), dtype=torch.float16, device="cuda")
    _lib.check(lib.b200_quantize_w4_group(ptr(dev(W)), K, N, Gs, ptr(P), ptr(S), stream()))
    sync()
    Po, So = orc.quantize_w4_group(W, Gs)
    assert np.array_equal(P.cpu().numpy(), Po)
    assert np.array_equal(S.cpu().numpy().view(np.uint16), So.view(np.uint16))


def test_nibble_pack_unpack_bit_exact():
    from gpu_util import dev, ptr, stream, sync
    import torch
    lib = _lib.load()
    rng = np.random.default_rng(2)
    flat = rng.integers(-8, 8, 2 * 5000).astype(np.int8)
    d = dev(flat)
    p = torch.empty(5000, dtype=torch.int8, device="cuda")
    _lib.check(lib.b200_pack_int4(ptr(d), flat.size, ptr(p), stream()))
    u = torch.empty(10000, dtype=torch.int8, device="cuda")
    _lib.check(lib.b200_unpack_int4(ptr(p), 5000, ptr(u), stream()))
    sync()
    assert np.array_equal(p.cpu().numpy(), orc.pack_int4(flat))
    assert np.array_equal(u.cpu().numpy(), orc.unpack_int4(orc.pack_int4(flat)))
    assert np.array_equal(u.cpu().numpy(), flat)
    # empty input is a no-op, odd counts are rejected
    assert lib.b200_pack_int4(ptr(d), 0, ptr(p), stream()) == 0
    assert lib.b200_pack_int4(ptr(d), 3, ptr(p), stream()) == -1


@pytest.mark.parametrize("kind", [_lib.W_I8, _lib.W_U4, _lib.W_F32])
@pytest.mark.parametrize("K,N", [(8, 8), (100, 34), (1536, 96), (8960, 16), (4160, 6)])
def test_repack_round_trip_bit_exact(kind, K, N):
    """reference layout -> packed device rows -> reference layout, and every
    packed byte sits where b200_packed_offset says."""
    from gpu_util import dev, ptr, stream, sync, packed_weight
    import torch
    lib = _lib.load()
    rng = np.random.default_rng(K * 31 + N)
    if kind == _lib.W_I8:
        ref = rng.integers(-128, 128, (K, N)).astype(np.int8)
    elif kind == _lib.W_U4:
        ref = orc.pack_int4(rng.integers(-8, 8, (K, N)).astype(np.int8)).reshape(K, N // 2)
    else:
        ref = rng.standard_normal((K, N)).astype(np.float32)
    signed = 1 if kind == _lib.W_U4 else 0
    packed = packed_weight(kind, ref, K, N, signed)
    back = torch.empty(ref.size * ref.itemsize, dtype=torch.uint8, device="cuda")
    _lib.check(lib.b200_unpack_weight(kind, ptr(packed), K, N, signed, ptr(back), stream()))
    sync()
    assert np.array_equal(back.cpu().numpy().view(ref.dtype).reshape(ref.shape), ref)
    # spot-check the layout contract on the host
    rb = lib.b200_packed_row_bytes(kind, K)
    rows = packed.cpu().numpy().reshape(N, rb)
    nib = C.c_int(0)
    vals = orc.unpack_int4(ref).reshape(K, N) if kind == _lib.W_U4 else ref
    for n in (0, N - 1):
        for k in range(0, K, max(1, K // 37)):
            off = lib.b200_packed_offset(kind, K, k, C.byref(nib))
            if kind == _lib.W_I8:
                assert rows[n, off].view(np.int8) == vals[k, n]
            elif kind == _lib.W_U4:
                code = (rows[n, off] >> 4) if nib.value else (rows[n, off] & 0xF)
                assert int(code) - 8 == int(vals[k, n])
            else:
                assert rows[n, off:off + 4].view(np.float32)[0] == vals[k, n]


# ---- GEMV sweep on device pointers ----------------------------------------------------
SHAPES = [(1536, 1536), (8960, 1536), (1536, 8960), (4096, 4096)]   # (N, K)


@pytest.mark.parametrize("N,K", SHAPES + [(151936, 1536), (14336, 4096)])
@pytest.mark.parametrize("M", [1, 16])
def test_gemv_w8_sweep(N, K, M):
    from gpu_util import dev, packed_weight, gemv
    if M == 16 and N > 20000:
        pytest.skip("one large-N case per kind is enough for the CPU checker's time")
    rng = np.random.default_rng(N + K + M)
    x = rng.standard_normal((M, K)).astype(np.float32)
    Q = rng.integers(-127, 128, (K, N)).astype(np.int8)
    s = rng.uniform(0.001, 0.01, N).astype(np.float32)
    w = packed_weight(_lib.W_I8, Q, K, N)
    y = gemv(_lib.W_I8, w, dev(s), K, N, dev(x)).cpu().numpy()
    assert rel(y, orc.gemv_w8_f32(x, Q, s)) < F32_TOL


@pytest.mark.parametrize("N,K", SHAPES + [(151936, 1536), (14336, 4096), (4096, 12288)])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 5])
def test_gemv_w4_group128_sweep(N, K, M):
    from gpu_util import dev, packed_weight, packed_scales, gemv
    if M not in (1, 16) and N * K > 4096 * 4096:
        pytest.skip("the large shapes are checked at M = 1 and M = 16")
    rng = np.random.default_rng(N * 3 + K + M)
    x = rng.standard_normal((M, K)).astype(np.float32)
    P = rng.integers(0, 256, (K, N // 2)).astype(np.uint8)          # nibbles uniform in [0,15]
    s = rng.uniform(0.001, 0.01, (K // 128, N)).astype(np.float16)
    w = packed_weight(_lib.W_U4, P, K, N, 0)
    sc = packed_scales(s, _lib.F16, K // 128, N)
    y = gemv(_lib.W_U4, w, sc, K, N, dev(x), group=128, scale_dtype=_lib.F16).cpu().numpy()
    assert rel(y, orc.gemv_w4g_f32(x, P, s, 128)) < F32_TOL


@pytest.mark.parametrize("N,K", [(1536, 1536), (256, 1536), (1536, 8960)])
@pytest.mark.parametrize("M", [1, 3])
def test_gemv_f32_sweep(N, K, M):
    from gpu_util import dev, packed_weight, gemv
    rng = np.random.default_rng(N + 7 * K + M)
    x = rng.standard_normal((M, K)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    y = gemv(_lib.W_F32, packed_weight(_lib.W_F32, B, K, N), None, K, N, dev(x)).cpu().numpy()
    assert rel(y, orc.gemv_f32(x, B)) < F32_TOL


def test_gemv_bf16_and_f16_activations():
    from gpu_util import dev, packed_weight, gemv
    import torch
    rng = np.random.default_rng(4)
    K, N = 1536, 512
    Q = rng.integers(-127, 128, (K, N)).astype(np.int8)
    s = rng.uniform(0.001, 0.01, N).astype(np.float32)
    w = packed_weight(_lib.W_I8, Q, K, N)
    for tdt, code in ((torch.bfloat16, _lib.BF16), (torch.float16, _lib.F16)):
        xt = torch.from_numpy(rng.standard_normal((4, K)).astype(np.float32)).to(tdt).cuda()
        y = gemv(_lib.W_I8, w, dev(s), K, N, xt, x_dtype=code).cpu().numpy()
        ref = orc.gemv_w8_f32(xt.float().cpu().numpy(), Q, s)
        assert rel(y, ref) < F32_TOL


def test_gemv_fused_prologue_and_epilogues():
    """RMSNorm prologue, bias, residual, accumulate and the SiLU-gate epilogue
    equal the separate ops of the CPU restatement."""
    from gpu_util import dev, packed_weight, gemv
    rng = np.random.default_rng(9)
    K, F = 1536, 640
    x = rng.standard_normal((1, K)).astype(np.float32)
    nw = (1 + 0.02 * rng.standard_normal(K)).astype(np.float32)
    Qg = rng.integers(-127, 128, (K, F)).astype(np.int8)
    Qu = rng.integers(-127, 128, (K, F)).astype(np.int8)
    sg = rng.uniform(0.0005, 0.002, F).astype(np.float32)
    su = rng.uniform(0.0005, 0.002, F).astype(np.float32)
    h = orc.rmsnorm(x[0], nw, 1e-6)[None, :]
    ref = orc.silu_mul(orc.gemv_w8_f32(h, Qg, sg)[0], orc.gemv_w8_f32(h, Qu, su)[0])
    inter = np.empty((K, 2 * F), np.int8)
    inter[:, 0::2], inter[:, 1::2] = Qg, Qu
    si = np.empty(2 * F, np.float32)
    si[0::2], si[1::2] = sg, su
    w = packed_weight(_lib.W_I8, inter, K, 2 * F)
    y = gemv(_lib.W_I8, w, dev(si), K, 2 * F, dev(x), norm_w=dev(nw), silu=True).cpu().numpy()
    assert y.shape == (1, F) and rel(y[0], ref) < 5e-5
    # bias + residual (x1 = x + o) and C += semantics
    N = 96
    Q = rng.integers(-127, 128, (K, N)).astype(np.int8)
    s = rng.uniform(0.001, 0.01, N).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    r = rng.standard_normal((1, N)).astype(np.float32)
    w = packed_weight(_lib.W_I8, Q, K, N)
    base = orc.gemv_w8_f32(x, Q, s)
    y = gemv(_lib.W_I8, w, dev(s), K, N, dev(x), bias=dev(b), residual=dev(r)).cpu().numpy()
    assert rel(y, r + (b + base)) < F32_TOL
    y0 = dev(r.copy())
    y = gemv(_lib.W_I8, w, dev(s), K, N, dev(x), accumulate=True, y0=y0).cpu().numpy()
    assert rel(y, orc.gemv_w8_f32(x, Q, s, y0=r)) < F32_TOL


def test_gemv_rejects_bad_arguments():
    from gpu_util import dev, packed_weight, stream
    lib = _lib.load()
    K, N = 64, 8
    w = packed_weight(_lib.W_I8, np.zeros((K, N), np.int8), K, N)
    x = dev(np.zeros((17, K), np.float32))
    y = dev(np.zeros((17, N), np.float32))
    wd = _lib.Weight(_lib.W_I8, 0, K, N, w.data_ptr(), None, 0, 0, None)
    a = _lib.GemvArgs(x.data_ptr(), 0, 0, 0, 0, y.data_ptr(), None, None, 0.0, 17, 0, 0)
    assert lib.b200_gemv(C.byref(wd), C.byref(a), stream()) == -1      # no scales
    wd.scale = x.data_ptr()
    assert lib.b200_gemv(C.byref(wd), C.byref(a), stream()) == -1      # M > 16
    assert b"M=17" in lib.b200_last_error()


# ---- attention, argmax, KV overflow on device pointers -----------------------------
@pytest.mark.parametrize("QH,KH,D,L,pos", [(12, 2, 128, 1024, 1023), (12, 2, 128, 1024, 0),
                                          (32, 8, 128, 4096, 4000), (8, 2, 64, 128, 77),
                                          (4, 4, 128, 64, 63), (6, 2, 64, 48, 20)])
def test_gqa_decode_shapes(QH, KH, D, L, pos):
    rng = np.random.default_rng(QH + L + pos)
    q = rng.standard_normal((QH, D)).astype(np.float32)
    K = rng.standard_normal((KH, L, D)).astype(np.float32)
    V = rng.standard_normal((KH, L, D)).astype(np.float32)
    out = memref.buddy_gqa_decode_f32(q[None, :, None, :], K[None], V[None], pos)
    assert rel(out[0, :, 0, :], orc.gqa_decode(q, K, V, pos)) < 1e-5


def test_gqa_decode_is_deterministic():
    rng = np.random.default_rng(1)
    q = rng.standard_normal((12, 128)).astype(np.float32)
    K = rng.standard_normal((2, 1024, 128)).astype(np.float32)
    V = rng.standard_normal((2, 1024, 128)).astype(np.float32)
    a = memref.buddy_gqa_decode_f32(q[None, :, None, :], K[None], V[None], 900)
    b = memref.buddy_gqa_decode_f32(q[None, :, None, :], K[None], V[None], 900)
    assert np.array_equal(a, b)


def test_argmax_first_ties():
    from gpu_util import dev, ptr, stream, sync
    import torch
    lib = _lib.load()
    rng = np.random.default_rng(8)
    scratch = torch.zeros(2048, dtype=torch.float32, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    cases = [np.array([0, 3, 3, 1], np.float32), rng.integers(0, 3, 151936).astype(np.float32),
             np.full(5000, -1.5, np.float32), rng.standard_normal(151936).astype(np.float32)]
    v = rng.standard_normal(151936).astype(np.float32)
    v[[7, 150000]] = 9.0
    cases.append(v)
    for v in cases:
        _lib.check(lib.b200_argmax_first(ptr(dev(v)), v.size, ptr(out), ptr(scratch), stream()))
        sync()
        assert int(out.item()) == orc.argmax_first(v) == int(np.argmax(v))


@pytest.mark.parametrize("position,keep", [(64, 16), (64, 0), (64, 63), (63, 16)])
def test_kv_overflow_bit_exact(position, keep):
    from gpu_util import dev, ptr, stream, sync
    import torch
    lib = _lib.load()
    rng = np.random.default_rng(13)
    nb, H, L, D = 4, 2, 64, 128
    host = [rng.standard_normal((H, L, D)).astype(np.float32) for _ in range(nb)]
    d = [dev(h) for h in host]
    table = torch.tensor([t.data_ptr() for t in d], dtype=torch.int64, device="cuda")
    newp = C.c_int(-5)
    _lib.check(lib.b200_kv_overflow(ptr(table), nb, H, L, D, position, keep, 10000.0,
                                    C.byref(newp), stream()))
    sync()
    want = orc.kv_overflow(host, H, L, D, position, keep, 10000.0)
    assert newp.value == want
    for t, h in zip(d, host):
        assert np.array_equal(t.cpu().numpy(), h)
