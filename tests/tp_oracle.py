"""Tensor-parallel decode step on the CPU checker's ops (test infrastructure).

Sharding follows buddy-mlir's 2-rank example
(examples/BuddyTensorParallel/buddy-deepseek-r1-distributed.cpp:521-617,
import-deepseek-r1.py:163-185): q/k/v split by heads and gate/up by FFN
columns (column-parallel), o and down split along K (row-parallel) with a sum
over ranks after each, lm_head split over the vocabulary.  Weights are
quantised BEFORE they are cut, so sharding never changes a quantised value; a
row-parallel rank scales its partial sum by the (shared) per-channel scale
before the sum over ranks.
"""
import numpy as np

import oracle_lib as orc


class LocalComm:
    """All ranks in one process: collectives over a list of per-rank arrays."""

    def __init__(self, size):
        self.size = size

    def allreduce(self, parts):
        total = parts[0].copy()
        for p in parts[1:]:
            total = total + p          # fixed rank order
        return [total.copy() for _ in parts]

    def allgather(self, parts):
        full = np.concatenate(parts)
        return [full.copy() for _ in parts]


def _quant(W, kind, group):
    if kind == "f32":
        return ("f32", np.ascontiguousarray(W, dtype=np.float32), None)
    if kind == "w8":
        Q, s = orc.quantize_per_channel(W, 8)
        return ("w8", Q, s)
    P, s = orc.quantize_w4_group(W, group)
    return ("w4g", P, s)


def _cols(t, lo, hi):
    kind, w, s = t
    if kind == "f32":
        return (kind, np.ascontiguousarray(w[:, lo:hi]), None)
    if kind == "w8":
        return (kind, np.ascontiguousarray(w[:, lo:hi]), np.ascontiguousarray(s[lo:hi]))
    return (kind, np.ascontiguousarray(w[:, lo // 2:hi // 2]), np.ascontiguousarray(s[:, lo:hi]))


def _rows(t, lo, hi, group):
    kind, w, s = t
    if kind == "f32":
        return (kind, np.ascontiguousarray(w[lo:hi]), None)
    if kind == "w8":
        return (kind, np.ascontiguousarray(w[lo:hi]), s)
    return (kind, np.ascontiguousarray(w[lo:hi]), np.ascontiguousarray(s[lo // group:hi // group]))


def _gemv(t, x, group):
    kind, w, s = t
    x = np.ascontiguousarray(x, dtype=np.float32)[None, :]
    if kind == "f32":
        return orc.gemv_f32(x, w)[0]
    if kind == "w8":
        return orc.gemv_w8_f32(x, w, s)[0]
    return orc.gemv_w4g_f32(x, w, s, group)[0]


class TPRank:
    """One rank's shard of the model and its local KV cache."""

    def __init__(self, cfg, views, kinds, rank, size, group=128):
        self.cfg, self.rank, self.size, self.group = cfg, rank, size, group
        D = cfg.head_dim
        qh, kh, F, V = cfg.q_heads // size, cfg.kv_heads // size, cfg.ffn // size, cfg.vocab // size
        self.qh, self.kh = qh, kh
        q0, k0, f0, v0 = rank * qh * D, rank * kh * D, rank * F, rank * V
        self.layers = []
        kinds = kinds or {}
        for l in range(cfg.n_layers):
            L = {}
            for n, lo, hi in (("q", q0, q0 + qh * D), ("k", k0, k0 + kh * D), ("v", k0, k0 + kh * D),
                              ("gate", f0, f0 + F), ("up", f0, f0 + F)):
                L[n] = _cols(_quant(views[(n, l)], kinds.get(n, "f32"), group), lo, hi)
                if (n + "_bias", l) in views:
                    L[n + "_bias"] = views[(n + "_bias", l)][lo:hi]
            L["o"] = _rows(_quant(views[("o", l)], kinds.get("o", "f32"), group), q0, q0 + qh * D, group)
            L["down"] = _rows(_quant(views[("down", l)], kinds.get("down", "f32"), group), f0, f0 + F, group)
            for n in ("in_norm", "post_norm", "q_norm", "k_norm"):
                if (n, l) in views:
                    L[n] = views[(n, l)]
            self.layers.append(L)
        self.lm = _cols(_quant(views[("lm_head", -1)], kinds.get("lm_head", "f32"), group), v0, v0 + V)
        self.embed, self.final_norm = views[("embed", -1)], views[("final_norm", -1)]
        self.inv_freq = views[("inv_freq", -1)]
        self.kv = [np.zeros((kh, cfg.max_len, D), np.float32) for _ in range(2 * cfg.n_layers)]


def tp_decode_step(ranks, comm, token, pos):
    """Advance every rank by one token; returns the (replicated) logits."""
    cfg = ranks[0].cfg
    D, g = cfg.head_dim, ranks[0].group
    xs = [r.embed[token].copy() for r in ranks]
    for l in range(cfg.n_layers):
        parts = []
        for r, x in zip(ranks, xs):
            L = r.layers[l]
            h = orc.rmsnorm(x, L["in_norm"], cfg.eps)
            q, k, v = (_gemv(L[n], h, g) for n in ("q", "k", "v"))
            if "q_bias" in L:
                q, k, v = L["q_bias"] + q, L["k_bias"] + k, L["v_bias"] + v
            q, k = q.reshape(r.qh, D), k.reshape(r.kh, D)
            if "q_norm" in L:
                q = np.stack([orc.rmsnorm(t, L["q_norm"], cfg.eps) for t in q])
                k = np.stack([orc.rmsnorm(t, L["k_norm"], cfg.eps) for t in k])
            q, k = orc.rope(q, r.inv_freq, pos), orc.rope(k, r.inv_freq, pos)
            r.kv[2 * l][:, pos] = k
            r.kv[2 * l + 1][:, pos] = v.reshape(r.kh, D)
            att = orc.gqa_decode(q, r.kv[2 * l], r.kv[2 * l + 1], pos)
            parts.append(_gemv(L["o"], att.reshape(-1), g))
        summed = comm.allreduce(parts)
        xs = [x + o for x, o in zip(xs, summed)]
        parts = []
        for r, x in zip(ranks, xs):
            L = r.layers[l]
            h = orc.rmsnorm(x, L["post_norm"], cfg.eps)
            mid = orc.silu_mul(_gemv(L["gate"], h, g), _gemv(L["up"], h, g))
            parts.append(_gemv(L["down"], mid, g))
        summed = comm.allreduce(parts)
        xs = [x + d for x, d in zip(xs, summed)]
    shards = [_gemv(r.lm, orc.rmsnorm(x, r.final_norm, cfg.eps), g) for r, x in zip(ranks, xs)]
    return comm.allgather(shards)[0]
