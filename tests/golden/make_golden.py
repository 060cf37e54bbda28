"""Generates the committed fixtures in this directory.  Run from the repo root:

    python tests/golden/make_golden.py

Needs `transformers` (5.5.0 here, the version buddy-mlir's requirements.txt
pins) for the HuggingFace cross-check; it does not need a GPU and does not
read the reference tree.  The HuggingFace Qwen2/Qwen3 modules are what
buddy-mlir traces (tools/buddy-codegen/import_model.py:118-204), so their
eager f32 logits on the same seeded weights are a second, independent
statement of the float decode graph.

Outputs
  hf_tiny_qwen2.npz / hf_tiny_qwen3.npz : token ids + HF eager logits per position
  ops_golden.npz : seeded op-level inputs and the CPU restatement's outputs
  known_answers.npz : the inputs/outputs of buddy-mlir's runnable examples
      examples/BuddyMatmul/dequant-matmul-vectorization-decode.mlir:93-133
      examples/BuddyMatmul/int4-dequant-matmul-vectorization-decode.mlir:160-206
      examples/BuddyMatmul/dequant-matmul-vectorization-blis-prefill.mlir:113-115
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle_lib as orc  # noqa: E402
from buddy_mlir_b200 import TINY_QWEN2, TINY_QWEN3, synthetic  # noqa: E402

SEED_W, SEED_P = 1234, 99


def hf_logits(cfg, views, tokens):
    import torch
    import transformers
    common = dict(hidden_size=cfg.hidden, intermediate_size=cfg.ffn,
                  num_hidden_layers=cfg.n_layers, num_attention_heads=cfg.q_heads,
                  num_key_value_heads=cfg.kv_heads, vocab_size=cfg.vocab,
                  max_position_embeddings=cfg.max_len, rms_norm_eps=cfg.eps,
                  rope_theta=cfg.rope_theta, tie_word_embeddings=False,
                  head_dim=cfg.head_dim, attn_implementation="eager")
    if cfg.qk_norm:
        hc = transformers.Qwen3Config(**common, attention_bias=False)
        model = transformers.Qwen3ForCausalLM(hc)
    else:
        hc = transformers.Qwen2Config(**common)
        model = transformers.Qwen2ForCausalLM(hc)
    model = model.float().eval()
    sd = {}
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    sd["model.embed_tokens.weight"] = t(views[("embed", -1)])
    sd["model.norm.weight"] = t(views[("final_norm", -1)])
    sd["lm_head.weight"] = t(views[("lm_head", -1)].T)
    for l in range(cfg.n_layers):
        p = f"model.layers.{l}."
        sd[p + "input_layernorm.weight"] = t(views[("in_norm", l)])
        sd[p + "post_attention_layernorm.weight"] = t(views[("post_norm", l)])
        for n in ("q", "k", "v", "o"):
            sd[p + f"self_attn.{n}_proj.weight"] = t(views[(n, l)].T)
        if cfg.qkv_bias:
            for n in ("q", "k", "v"):
                sd[p + f"self_attn.{n}_proj.bias"] = t(views[(f"{n}_bias", l)])
        if cfg.qk_norm:
            sd[p + "self_attn.q_norm.weight"] = t(views[("q_norm", l)])
            sd[p + "self_attn.k_norm.weight"] = t(views[("k_norm", l)])
        for n in ("gate", "up", "down"):
            sd[p + f"mlp.{n}_proj.weight"] = t(views[(n, l)].T)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in m or "inv_freq" in m for m in missing), missing
    with torch.no_grad():
        out = model(torch.from_numpy(tokens[None, :].astype(np.int64)))
    return out.logits[0].numpy().astype(np.float32)


def make_hf(cfg, path):
    blob, views = synthetic.make_f32_blob(cfg, SEED_W)
    tokens = synthetic.prompt_tokens(cfg, SEED_P, 12)
    logits = hf_logits(cfg, views, tokens)
    om = orc.OracleModel(cfg, views)
    worst = 0.0
    for i, tkn in enumerate(tokens):
        lo = om.decode(int(tkn))
        rel = np.abs(lo - logits[i]).max() / np.abs(logits[i]).max()
        worst = max(worst, rel)
    print(f"{cfg.name}: CPU restatement vs HuggingFace eager, max rel err {worst:.3e}")
    assert worst < 1e-4
    np.savez_compressed(path, tokens=tokens, logits=logits, seed_w=SEED_W, seed_p=SEED_P)


def make_known_answers(path):
    d = {}
    d["w8_A"] = np.ones((1, 8), np.float32)
    W = np.zeros((8, 8), np.int8)
    W[:, :2] = 2
    d["w8_W"] = W
    d["w8_scale"] = np.full((1, 8), 0.5, np.float32)
    d["w8_expect"] = np.array([[8, 8, 0, 0, 0, 0, 0, 0]], np.float32)
    d["w4_A"] = np.ones((1, 4), np.float16)
    d["w4_P"] = np.full((4, 2), 2, np.int8)
    d["w4_scale"] = np.ones((1, 4), np.float16)
    d["w4_expect"] = np.array([[8, 0, 8, 0]], np.float16)
    d["pf_A"] = np.ones((4, 4), np.float32)
    d["pf_W"] = np.full((4, 4), 2, np.int8)
    d["pf_scale"] = np.ones((1, 4), np.float32)
    d["pf_expect"] = np.full((4, 4), 8, np.float32)
    np.savez_compressed(path, **d)


def make_ops(path):
    rng = np.random.default_rng(7)
    d = {}
    # quantiser + packing (bit-exact rows)
    W = (rng.standard_normal((96, 40)) * 0.02).astype(np.float32)
    W[:, 3] = 0.0  # an all-zero column exercises the 1e-10 clamp
    d["q_W"] = W
    d["q8_Q"], d["q8_s"] = orc.quantize_per_channel(W, 8)
    d["q4_Q"], d["q4_s"] = orc.quantize_per_channel(W, 4)
    d["q4_P"] = orc.pack_int4(d["q4_Q"]).reshape(96, 20)
    Wg = (rng.standard_normal((256, 24)) * 0.02).astype(np.float32)
    d["g_W"] = Wg
    d["g_P"], d["g_s"] = orc.quantize_w4_group(Wg, 128)
    # GEMVs, ragged shapes on purpose
    for tag, (M, K, N) in {"a": (1, 200, 70), "b": (3, 1536, 96), "c": (16, 96, 34)}.items():
        x = rng.standard_normal((M, K)).astype(np.float32)
        Q = rng.integers(-127, 128, (K, N)).astype(np.int8)
        s = rng.uniform(0.001, 0.01, N).astype(np.float32)
        d[f"w8{tag}_x"], d[f"w8{tag}_Q"], d[f"w8{tag}_s"] = x, Q, s
        d[f"w8{tag}_y"] = orc.gemv_w8_f32(x, Q, s)
        B = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
        d[f"f{tag}_B"] = B
        d[f"f{tag}_y"] = orc.gemv_f32(x, B)
    x = rng.standard_normal((2, 256)).astype(np.float16)
    Qs = rng.integers(-8, 8, (256, 48)).astype(np.int8)
    P = orc.pack_int4(Qs).reshape(256, 24)
    s = rng.uniform(0.001, 0.01, 48).astype(np.float16)
    d["w4_x"], d["w4_P"], d["w4_s"] = x, P, s
    d["w4_y"] = orc.gemv_w4_f16(x, P, s)
    x = rng.standard_normal((2, 256)).astype(np.float32)
    d["w4g_x"] = x
    d["w4g_y"] = orc.gemv_w4g_f32(x, d["g_P"], d["g_s"], 128)
    # small ops
    xv = rng.standard_normal(1536).astype(np.float32)
    wv = (1 + 0.02 * rng.standard_normal(1536)).astype(np.float32)
    d["rn_x"], d["rn_w"], d["rn_y"] = xv, wv, orc.rmsnorm(xv, wv, 1e-6)
    qh = rng.standard_normal((12, 128)).astype(np.float32)
    inv = synthetic.inv_freq(TINY_QWEN3)
    d["rp_x"], d["rp_inv"], d["rp_y"] = qh, inv, orc.rope(qh, inv, 613)
    g, u = rng.standard_normal(300).astype(np.float32) * 3, rng.standard_normal(300).astype(np.float32)
    d["sm_g"], d["sm_u"], d["sm_y"] = g, u, orc.silu_mul(g, u)
    # attention at the valid lengths buddy-mlir's own numpy check used
    # (frontend/Python/ops/tosa.py:14075-14080): 9 / 37 / 613 / 1024
    q = rng.standard_normal((12, 128)).astype(np.float32)
    Kc = rng.standard_normal((2, 1024, 128)).astype(np.float32)
    Vc = rng.standard_normal((2, 1024, 128)).astype(np.float32)
    d["at_q"], d["at_K"], d["at_V"] = q, Kc.astype(np.float16), Vc.astype(np.float16)
    Kc, Vc = d["at_K"].astype(np.float32), d["at_V"].astype(np.float32)
    for L in (9, 37, 613, 1024):
        d[f"at_out_{L}"] = orc.gqa_decode(q, Kc, Vc, L - 1)
    np.savez_compressed(path, **d)


if __name__ == "__main__":
    make_known_answers(os.path.join(HERE, "known_answers.npz"))
    make_ops(os.path.join(HERE, "ops_golden.npz"))
    make_hf(TINY_QWEN2, os.path.join(HERE, "hf_tiny_qwen2.npz"))
    make_hf(TINY_QWEN3, os.path.join(HERE, "hf_tiny_qwen3.npz"))
    print("fixtures written to", HERE)
