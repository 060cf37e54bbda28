"""ctypes binding of the CPU checker in oracle/ (test infrastructure)."""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(ROOT, "oracle", "_build", "libbuddy_oracle.so")
_REF_SO = os.path.join(ROOT, "oracle", "_ref", "libbuddy_ref_host.so")

LIN_F32, LIN_W8, LIN_W4G, LIN_W4, LIN_W8H, LIN_W8Q = 0, 1, 2, 3, 4, 5


class OrcLinear(C.Structure):
    _fields_ = [("kind", C.c_int32), ("group", C.c_int32), ("K", C.c_int64),
                ("N", C.c_int64), ("w", C.c_void_p), ("scale", C.c_void_p),
                ("bias", C.c_void_p)]


class OrcLayer(C.Structure):
    _fields_ = [("in_norm", C.c_void_p), ("post_norm", C.c_void_p),
                ("q_norm", C.c_void_p), ("k_norm", C.c_void_p)] + \
               [(n, OrcLinear) for n in ("q", "k", "v", "o", "gate", "up", "down")]


class OrcModel(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("hidden", "n_layers", "q_heads", "kv_heads",
                                          "head_dim", "ffn", "vocab", "max_len")] + \
               [("eps", C.c_float), ("embed", C.c_void_p), ("inv_freq", C.c_void_p),
                ("layers", C.POINTER(OrcLayer)), ("final_norm", C.c_void_p),
                ("lm_head", OrcLinear)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(_SO)
        _lib.orc_argmax_first.restype = C.c_int64
        _lib.orc_kv_overflow.restype = C.c_int64
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def ref_host():
    """buddy-mlir's own Sampler.h / KVCacheManager.h compiled from source, or
    None where the reference tree was never available to build it."""
    if not os.path.exists(_REF_SO):
        return None
    r = C.CDLL(_REF_SO)
    r.ref_greedy_sample.restype = C.c_int
    r.ref_kv_overflow.restype = C.c_int64
    return r


def _p(a):
    return C.c_void_p(a.ctypes.data)


def i64(v):
    return C.c_int64(int(v))


def quantize_per_channel(W, bits=8):
    W = np.ascontiguousarray(W, dtype=np.float32)
    K, N = W.shape
    Q = np.empty((K, N), dtype=np.int8)
    s = np.empty(N, dtype=np.float32)
    lib().orc_quantize_per_channel(_p(W), i64(K), i64(N), C.c_int(bits), _p(Q), _p(s))
    return Q, s


def quantize_per_channel_half(W, bits=8):
    """The quantiser as the reference runs it for its f16-activation variants (w8a16, w4a16):
    the module is converted to half before the graphs are traced
    (tools/buddy-codegen/import_model.py:118-145), so absmax, scale = absmax / qmax and
    round(w / scale) are half-precision operations (:830-850; each computed in f32 and rounded
    to half, as torch does on the CPU).  The clamp at 1e-10 rounds to zero in half and does
    nothing.  W [K,N] f32 -> (Q [K,N] int8, scale [N] f16)."""
    Wh = np.asarray(W, dtype=np.float32).astype(np.float16)
    qmax = np.float32(127.0 if bits == 8 else 7.0)
    amax = np.abs(Wh).max(axis=0, keepdims=True)
    scale = (amax.astype(np.float32) / qmax).astype(np.float16)
    ratio = (Wh.astype(np.float32) / scale.astype(np.float32)).astype(np.float16)
    lo, hi = (-128, 127) if bits == 8 else (-8, 7)
    Q = np.clip(np.rint(ratio.astype(np.float32)), lo, hi).astype(np.int8)
    return Q, scale.reshape(-1)


def pack_int4(flat):
    flat = np.ascontiguousarray(flat, dtype=np.int8).reshape(-1)
    out = np.empty(flat.size // 2, dtype=np.int8)
    lib().orc_pack_int4(_p(flat), i64(flat.size), _p(out))
    return out


def unpack_int4(packed):
    packed = np.ascontiguousarray(packed, dtype=np.int8).reshape(-1)
    out = np.empty(packed.size * 2, dtype=np.int8)
    lib().orc_unpack_int4(_p(packed), i64(packed.size), _p(out))
    return out


def quantize_w4_group(W, G):
    W = np.ascontiguousarray(W, dtype=np.float32)
    K, N = W.shape
    P = np.empty((K, N // 2), dtype=np.uint8)
    s = np.empty((K // G, N), dtype=np.float16)
    lib().orc_quantize_w4_group(_p(W), i64(K), i64(N), i64(G), _p(P), _p(s))
    return P, s


def gemv_w8_f32(x, Q, scale, y0=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    N = Q.shape[1]
    y = np.zeros((M, N), dtype=np.float32) if y0 is None else y0.copy()
    Q = np.ascontiguousarray(Q, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    lib().orc_gemv_w8_f32(_p(x), _p(Q), _p(scale), _p(y), i64(M), i64(K), i64(N))
    return y


def gemv_w8_f16(x, Q, scale):
    x = np.ascontiguousarray(x, dtype=np.float16)
    M, K = x.shape
    N = Q.shape[1]
    y = np.zeros((M, N), dtype=np.float16)
    Q = np.ascontiguousarray(Q, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float16).reshape(-1)
    lib().orc_gemv_w8_f16(_p(x), _p(Q), _p(scale), _p(y), i64(M), i64(K), i64(N))
    return y


def gemv_w4_f16(x, P, scale):
    x = np.ascontiguousarray(x, dtype=np.float16)
    M, K = x.shape
    N = P.shape[1] * 2
    y = np.zeros((M, N), dtype=np.float16)
    P = np.ascontiguousarray(P, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float16).reshape(-1)
    lib().orc_gemv_w4_f16(_p(x), _p(P), _p(scale), _p(y), i64(M), i64(K), i64(N))
    return y


def gemv_f32(x, B, y0=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    N = B.shape[1]
    y = np.zeros((M, N), dtype=np.float32) if y0 is None else y0.copy()
    B = np.ascontiguousarray(B, dtype=np.float32)
    lib().orc_gemv_f32(_p(x), _p(B), _p(y), i64(M), i64(K), i64(N))
    return y


def gemv_w4g_f32(x, P, scale, G):
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    N = P.shape[1] * 2
    y = np.zeros((M, N), dtype=np.float32)
    P = np.ascontiguousarray(P).view(np.uint8)
    scale = np.ascontiguousarray(scale, dtype=np.float16)
    lib().orc_gemv_w4g_f32(_p(x), _p(P), _p(scale), _p(y), i64(M), i64(K), i64(N), i64(G))
    return y


def pack_panels_f32(B, V):
    B = np.ascontiguousarray(B, dtype=np.float32)
    K, N = B.shape
    out = np.empty(K * N, dtype=np.float32)
    lib().orc_pack_panels_f32(_p(B), i64(K), i64(N), i64(V), _p(out))
    return out


def gemv_f32_packed(x, packed, K, N, V):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    y = np.zeros(N, dtype=np.float32)
    lib().orc_gemv_f32_packed(_p(x), _p(packed), _p(y), i64(K), i64(N), i64(V))
    return y


def gemm_w8_prefill_f32(A, Q, scale, C0):
    A = np.ascontiguousarray(A, dtype=np.float32)
    M, K = A.shape
    N = Q.shape[1]
    out = np.ascontiguousarray(C0, dtype=np.float32).copy()
    Q = np.ascontiguousarray(Q, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    lib().orc_gemm_w8_prefill_f32(_p(A), _p(Q), _p(scale), _p(out), i64(M), i64(K), i64(N))
    return out


def matmul_w8a8(A, Q, scale, bias=None):
    A = np.ascontiguousarray(A, dtype=np.float32)
    M, K = A.shape
    N = Q.shape[1]
    out = np.zeros((M, N), dtype=np.float32)
    Q = np.ascontiguousarray(Q, dtype=np.int8)
    scale = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().orc_matmul_w8a8(_p(A), _p(Q), _p(scale), None if b is None else _p(b), _p(out), i64(M), i64(K), i64(N))
    return out


def rmsnorm(x, w, eps):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    w = np.ascontiguousarray(w, dtype=np.float32)
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), _p(y), i64(x.size), C.c_float(eps))
    return y


def rope(v, inv_freq, pos):
    v = np.ascontiguousarray(v, dtype=np.float32).copy()
    heads, D = v.shape
    inv_freq = np.ascontiguousarray(inv_freq, dtype=np.float32)
    lib().orc_rope(_p(v), i64(heads), i64(D), _p(inv_freq), i64(pos))
    return v


def silu_mul(g, u):
    g = np.ascontiguousarray(g, dtype=np.float32).reshape(-1)
    u = np.ascontiguousarray(u, dtype=np.float32).reshape(-1)
    y = np.empty_like(g)
    lib().orc_silu_mul(_p(g), _p(u), _p(y), i64(g.size))
    return y


def argmax_first(v):
    v = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
    return int(lib().orc_argmax_first(_p(v), i64(v.size)))


def gqa_decode(q, Kc, Vc, pos):
    q = np.ascontiguousarray(q, dtype=np.float32)
    Kc = np.ascontiguousarray(Kc, dtype=np.float32)
    Vc = np.ascontiguousarray(Vc, dtype=np.float32)
    QH, D = q.shape
    KH, L, _ = Kc.shape
    out = np.empty_like(q)
    lib().orc_gqa_decode(_p(q), _p(Kc), _p(Vc), _p(out), i64(QH), i64(KH), i64(L), i64(D), i64(pos))
    return out


def _kv_ptr_array(kv):
    arr = (C.c_void_p * len(kv))(*[a.ctypes.data for a in kv])
    return arr


def kv_overflow(kv, kv_heads, max_len, D, position, keep, theta, use_ref=False):
    """In-place on the list of [kv_heads,max_len,D] arrays; returns new position."""
    arr = _kv_ptr_array(kv)
    fn = ref_host().ref_kv_overflow if use_ref else lib().orc_kv_overflow
    return int(fn(arr, i64(len(kv)), i64(kv_heads), i64(max_len), i64(D), i64(position),
                  i64(keep), C.c_float(theta)))


class OracleModel:
    """orc_decode_step over {(name, layer): array} tensors in the reference's
    [K,N] layout.  linears: name -> kind in ('f32', 'w8', 'w4g') decides how
    each projection is represented; quantised tensors are produced by the
    checker's own quantiser unless `quantised` supplies them."""

    def __init__(self, cfg, views, kinds=None, group=128, quantised=None):
        self.cfg = cfg
        self.keep = []
        kinds = kinds or {}
        quantised = quantised or {}

        def hold(a, dtype=None):
            a = np.ascontiguousarray(a, dtype=dtype)
            self.keep.append(a)
            return a

        def lin(name, layer, bias_name=None):
            W = views[(name, layer)]
            K, N = W.shape
            kind = kinds.get(name, "f32")
            L = OrcLinear()
            L.K, L.N, L.group = K, N, 0
            if kind == "f32":
                L.kind = LIN_F32
                L.w = hold(W, np.float32).ctypes.data
            elif kind in ("w8", "w8q"):     # w8q: the reference's w8a8, int8 activations as well
                Q, s = quantised.get((name, layer)) or quantize_per_channel(W, 8)
                L.kind = LIN_W8 if kind == "w8" else LIN_W8Q
                L.w = hold(Q, np.int8).ctypes.data
                L.scale = hold(s, np.float32).ctypes.data
            elif kind == "w4":      # the reference's w4a16: signed nibbles, per-channel f16 scale
                Q, sc = quantised.get((name, layer)) or quantize_per_channel(W, 4)
                L.kind = LIN_W4
                L.w = hold(pack_int4(np.ascontiguousarray(Q, dtype=np.int8).reshape(-1)).reshape(K, N // 2)).ctypes.data
                L.scale = hold(np.asarray(sc, dtype=np.float32).astype(np.float16)).ctypes.data
            elif kind == "w8h":     # the reference's w8a16: int8, per-channel f16 scale, f16 activations
                Q, sc = quantised.get((name, layer)) or quantize_per_channel(W, 8)
                L.kind = LIN_W8H
                L.w = hold(Q, np.int8).ctypes.data
                L.scale = hold(np.asarray(sc, dtype=np.float32).astype(np.float16)).ctypes.data
            elif kind == "w4g":
                P, s = quantised.get((name, layer)) or quantize_w4_group(W, group)
                L.kind, L.group = LIN_W4G, group
                L.w = hold(P).ctypes.data
                L.scale = hold(s, np.float16).ctypes.data
            else:
                raise ValueError(kind)
            if bias_name and (bias_name, layer) in views:
                L.bias = hold(views[(bias_name, layer)], np.float32).ctypes.data
            return L

        self.layers = (OrcLayer * cfg.n_layers)()
        for l in range(cfg.n_layers):
            Ly = self.layers[l]
            Ly.in_norm = hold(views[("in_norm", l)], np.float32).ctypes.data
            Ly.post_norm = hold(views[("post_norm", l)], np.float32).ctypes.data
            if cfg.qk_norm:
                Ly.q_norm = hold(views[("q_norm", l)], np.float32).ctypes.data
                Ly.k_norm = hold(views[("k_norm", l)], np.float32).ctypes.data
            Ly.q = lin("q", l, "q_bias")
            Ly.k = lin("k", l, "k_bias")
            Ly.v = lin("v", l, "v_bias")
            for n in ("o", "gate", "up", "down"):
                setattr(Ly, n, lin(n, l))
        m = OrcModel()
        m.hidden, m.n_layers, m.q_heads, m.kv_heads = cfg.hidden, cfg.n_layers, cfg.q_heads, cfg.kv_heads
        m.head_dim, m.ffn, m.vocab, m.max_len = cfg.head_dim, cfg.ffn, cfg.vocab, cfg.max_len
        m.eps = cfg.eps
        m.embed = hold(views[("embed", -1)], np.float32).ctypes.data
        m.inv_freq = hold(views[("inv_freq", -1)], np.float32).ctypes.data
        m.layers = self.layers
        m.final_norm = hold(views[("final_norm", -1)], np.float32).ctypes.data
        m.lm_head = lin("lm_head", -1)
        self.m = m
        self.kv = [np.zeros((cfg.kv_heads, cfg.max_len, cfg.head_dim), dtype=np.float32)
                   for _ in range(2 * cfg.n_layers)]
        self.kv_arr = _kv_ptr_array(self.kv)
        self.position = 0

    def prefill(self, tokens):
        """The prefill graph over len(tokens) rows from position 0: logits [rows, vocab]."""
        toks = np.ascontiguousarray(tokens, dtype=np.int64)
        logits = np.empty((len(toks), self.cfg.vocab), dtype=np.float32)
        lib().orc_prefill_rows(C.byref(self.m), toks.ctypes.data_as(C.c_void_p), i64(len(toks)), self.kv_arr, _p(logits))
        self.position = len(toks)
        return logits

    def decode(self, token, pos=None):
        pos = self.position if pos is None else pos
        logits = np.empty(self.cfg.vocab, dtype=np.float32)
        lib().orc_decode_step(C.byref(self.m), i64(token), i64(pos), self.kv_arr, _p(logits))
        self.position = pos + 1
        return logits
