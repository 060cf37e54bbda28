"""Seeded synthetic weights in buddy-mlir's flat-blob order.

Order of the f32 blob (frontend/Python/graph/graph.py:836-863 packs the params
in graph order; the frontend lists the module's parameters in the order the
traced graph first uses them and its buffers after them,
frontend/Python/frontend.py:922-933): embedding, per layer {input norm, Wq,
q bias, Wk, k bias, Wv, v bias, Wo, post-attention norm, Wgate, Wup, Wdown},
final norm, lm_head, inv_freq (the rotary buffer).  Every matmul weight is
[K,N] row-major (eliminate_weight_transpose.py:163-219).  This is the order
buddy-mlir's own importer (tools/buddy-codegen/import_model.py) produces for a
Qwen2 model with the transformers version it pins; tests/golden holds digests
of its blobs for the small model (make_reference_blobs.py).  The argument list
of the older examples/BuddyDeepSeekR1/subgraph0_decode_simplify.mlir:4 shows
another order (inv_freq second, bias before weight): files written by that
flow are not in this order.

For the w8a32 variant the same walk is split by dtype
(tools/buddy-codegen/import_model.py:818-887): o, gate, up, down and lm_head go
to the int8 blob, everything else to the float blob, followed by the scales in
original-weight order (quantize.py:577-589).

No real checkpoint is used anywhere: weights are N(0, 0.02) from a seeded
numpy generator, norm weights 1 + N(0, 0.02).
"""
import numpy as np

from .config import ModelConfig

QUANTISED_BY_REFERENCE = ("o", "gate", "up", "down", "lm_head")


def tensor_list(cfg: ModelConfig):
    """[(name, layer, shape)] in blob order."""
    H, QD, KD, F, V, D = cfg.hidden, cfg.q_dim, cfg.kv_dim, cfg.ffn, cfg.vocab, cfg.head_dim
    out = [("embed", -1, (V, H))]
    for l in range(cfg.n_layers):
        out.append(("in_norm", l, (H,)))
        # Qwen3: the head norms follow the projection they normalise (the importer's order for
        # transformers.Qwen3ForCausalLM: in norm, Wq, q norm, Wk, k norm, Wv, Wo, ...)
        out.append(("q", l, (H, QD)))
        if cfg.qkv_bias:
            out.append(("q_bias", l, (QD,)))
        if cfg.qk_norm:
            out.append(("q_norm", l, (D,)))
        out.append(("k", l, (H, KD)))
        if cfg.qkv_bias:
            out.append(("k_bias", l, (KD,)))
        if cfg.qk_norm:
            out.append(("k_norm", l, (D,)))
        out.append(("v", l, (H, KD)))
        if cfg.qkv_bias:
            out.append(("v_bias", l, (KD,)))
        out += [("o", l, (QD, H)), ("post_norm", l, (H,)), ("gate", l, (H, F)),
                ("up", l, (H, F)), ("down", l, (F, H))]
    out += [("final_norm", -1, (H,)), ("lm_head", -1, (H, V)), ("inv_freq", -1, (D // 2,))]
    return out


def blob_elements(cfg: ModelConfig):
    return sum(int(np.prod(s)) for _, _, s in tensor_list(cfg))


def inv_freq(cfg: ModelConfig):
    j = np.arange(0, cfg.head_dim, 2, dtype=np.float32) / np.float32(cfg.head_dim)
    return (np.float32(1.0) / np.power(np.float32(cfg.rope_theta), j)).astype(np.float32)


_CHUNK = 1 << 24


def _fill_normal(blob, seed):
    """blob[:] = N(0,1) from `seed`, in fixed 16 Mi-element chunks, each chunk
    from its own spawned PCG64 stream so the fill can use every host core and
    still depends on nothing but the seed."""
    from concurrent.futures import ThreadPoolExecutor
    import os
    n_chunks = (blob.size + _CHUNK - 1) // _CHUNK
    streams = np.random.SeedSequence(seed).spawn(n_chunks)

    def work(i):
        v = blob[i * _CHUNK:(i + 1) * _CHUNK]
        np.random.Generator(np.random.PCG64(streams[i])).standard_normal(
            v.size, dtype=np.float32, out=v)
    with ThreadPoolExecutor(max_workers=min(32, os.cpu_count() or 1)) as ex:
        list(ex.map(work, range(n_chunks)))


def make_f32_blob(cfg: ModelConfig, seed: int):
    """Returns (blob, views): blob is one float32 array, views maps
    (name, layer) -> the tensor as a view into the blob."""
    blob = np.empty(blob_elements(cfg), dtype=np.float32)
    _fill_normal(blob, seed)
    blob *= np.float32(0.02)
    views, off = {}, 0
    for name, layer, shape in tensor_list(cfg):
        n = int(np.prod(shape))
        v = blob[off:off + n]
        if name == "inv_freq":
            v[:] = inv_freq(cfg)
        elif name.endswith("norm"):
            v += np.float32(1.0)
        views[(name, layer)] = v.reshape(shape)
        off += n
    return blob, views


def split_w8a32(cfg: ModelConfig, views, quantize):
    """Reference-faithful w8a32 blobs from the f32 tensors.

    quantize(W [K,N] f32) -> (Q [K,N] int8, scale [N] f32).
    Returns (float_blob, int8_blob)."""
    floats, ints, scales = [], [], []
    for name, layer, _ in tensor_list(cfg):
        t = views[(name, layer)]
        if name in QUANTISED_BY_REFERENCE:
            q, s = quantize(t)
            ints.append(np.ascontiguousarray(q).reshape(-1))
            scales.append(np.ascontiguousarray(s, dtype=np.float32).reshape(-1))
        else:
            floats.append(t.reshape(-1))
    return np.concatenate(floats + scales), np.concatenate(ints)


def split_w4a16(cfg: ModelConfig, views, quantize):
    """Reference-faithful w4a16 blobs (tools/buddy-codegen/import_model.py:800-887,
    gen_config.py:51-71): every float tensor and every scale as f16, the quantised
    tensors as signed nibbles, two per byte, low nibble first, in flat row-major
    element order.  quantize(W [K,N] f32) -> (Q [K,N] int8 in [-8,7], scale [N] f32).
    Returns (f16_blob, packed_int4_blob)."""
    floats, ints, scales = [], [], []
    for name, layer, _ in tensor_list(cfg):
        t = views[(name, layer)]
        if name in QUANTISED_BY_REFERENCE:
            q, s = quantize(t)
            flat = np.ascontiguousarray(q, dtype=np.int8).reshape(-1).view(np.uint8)
            ints.append(((flat[0::2] & 0x0F) | ((flat[1::2] & 0x0F) << 4)).astype(np.uint8).view(np.int8))
            scales.append(np.ascontiguousarray(s, dtype=np.float32).astype(np.float16).reshape(-1))
        else:
            floats.append(t.reshape(-1).astype(np.float16))
    return np.concatenate(floats + scales), np.concatenate(ints)


def pack_decode_blob(cfg: ModelConfig, blob, vecsize: int = 32):
    """The decode file of the packed-decode spec: the f32 blob with every matmul weight
    [K, N] stored as [N / V][K][V] (frontend/Python/graph/transform/pack_decode_weights.py:
    32-124: reshape(k, n // V, V).permute(1, 0, 2)), everything else unchanged."""
    out = np.array(blob, dtype=np.float32, copy=True)
    off = 0
    for name, _, shape in tensor_list(cfg):
        n = int(np.prod(shape))
        if name in ("q", "k", "v", "o", "gate", "up", "down", "lm_head"):
            K, N = shape
            assert N % vecsize == 0
            w = blob[off:off + n].reshape(K, N // vecsize, vecsize)
            out[off:off + n] = np.ascontiguousarray(w.transpose(1, 0, 2)).reshape(-1)
        off += n
    return out


def split_w8a16(cfg: ModelConfig, views, quantize):
    """Reference-faithful w8a16 blobs (tools/buddy-codegen/gen_config.py:51-71): the w8a32
    split with every float tensor and every scale as f16.  quantize(W [K,N] f32) ->
    (Q [K,N] int8, scale [N] f32).  Returns (f16_blob, int8_blob)."""
    fb, ib = split_w8a32(cfg, views, quantize)
    return fb.astype(np.float16), ib


def to_bf16(a):
    """f32 -> bfloat16 bits (uint16), round to nearest even: what the reference's bf16 files hold
    (the module is converted with .bfloat16() before tracing, tools/buddy-codegen/import_model.py:
    118-145; the writer then keeps the high halves of the already-rounded values, :700-707)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def from_bf16(bits):
    """bfloat16 bits (uint16) -> f32, exact."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def prompt_tokens(cfg: ModelConfig, seed: int, n: int = 32):
    return np.random.default_rng(seed).integers(0, cfg.vocab, size=n).astype(np.int64)
