"""The CPU checker against everything that pins it: buddy-mlir's runnable
known-answer examples, its own host headers compiled from source, the
HuggingFace eager cross-check and the committed fixtures."""
import os

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import TINY_QWEN2, TINY_QWEN3, synthetic

G = os.path.join(os.path.dirname(__file__), "golden")


def test_known_answer_w8_decode():
    # examples/BuddyMatmul/dequant-matmul-vectorization-decode.mlir:93-133
    k = np.load(os.path.join(G, "known_answers.npz"))
    y = orc.gemv_w8_f32(k["w8_A"], k["w8_W"], k["w8_scale"])
    assert np.array_equal(y, k["w8_expect"])


def test_known_answer_w4_decode():
    # examples/BuddyMatmul/int4-dequant-matmul-vectorization-decode.mlir:160-206
    k = np.load(os.path.join(G, "known_answers.npz"))
    y = orc.gemv_w4_f16(k["w4_A"], k["w4_P"], k["w4_scale"])
    assert np.array_equal(y, k["w4_expect"])


def test_known_answer_w8_prefill():
    # examples/BuddyMatmul/dequant-matmul-vectorization-blis-prefill.mlir:113-115
    k = np.load(os.path.join(G, "known_answers.npz"))
    y = orc.gemm_w8_prefill_f32(k["pf_A"], k["pf_W"], k["pf_scale"], np.zeros((4, 4), np.float32))
    assert np.array_equal(y, k["pf_expect"])


def test_nibble_rules():
    # import_model.py:810-815 and ops/tosa.py:12158-12203
    vals = np.arange(-8, 8, dtype=np.int8)
    flat = np.stack(np.meshgrid(vals, vals, indexing="ij"), -1).reshape(-1)
    packed = orc.pack_int4(flat)
    lo, hi = flat[0::2], flat[1::2]
    assert np.array_equal(packed.view(np.uint8), (lo.view(np.uint8) & 0xF) | ((hi.view(np.uint8) & 0xF) << 4))
    assert np.array_equal(orc.unpack_int4(packed), flat)


def test_quantiser_matches_torch_statement():
    # import_model.py:830-850 restated with torch, the library the reference uses
    import torch
    rng = np.random.default_rng(3)
    W = (rng.standard_normal((64, 24)) * 0.02).astype(np.float32)
    W[:, 5] = 0
    t = torch.from_numpy(W)
    for bits, qmax, lo, hi in ((8, 127.0, -128, 127), (4, 7.0, -8, 7)):
        amax = t.abs().amax(dim=[0], keepdim=True)
        scale = (amax / qmax).clamp(min=1e-10)
        q = torch.clamp(torch.round(t / scale), lo, hi).to(torch.int8)
        Q, s = orc.quantize_per_channel(W, bits)
        assert np.array_equal(Q, q.numpy())
        assert np.array_equal(s, scale.numpy().reshape(-1))


def test_panel_packing_address_math():
    # tests/Conversion/matmul-vectorization-decode-packed.mlir:18-28:
    # flat offset = nIdx*K + k*V + v with nIdx = n0 (a multiple of V)
    K, N, V = 64, 128, 32
    B = np.arange(K * N, dtype=np.float32).reshape(K, N)
    p = orc.pack_panels_f32(B, V)
    for n in (0, 31, 32, 100, 127):
        for k in (0, 1, 63):
            n0 = n // V * V
            assert p[n0 * K + k * V + n % V] == B[k, n]
    x = np.random.default_rng(0).standard_normal(K).astype(np.float32)
    assert np.array_equal(orc.gemv_f32_packed(x, p, K, N, V), orc.gemv_f32(x[None], B)[0])


def test_greedy_tie_rule_against_reference_sampler():
    ref = orc.ref_host()
    rng = np.random.default_rng(5)
    cases = [np.array([0, 3, 3, 1], np.float32)]
    for _ in range(20):
        v = rng.integers(0, 4, 257).astype(np.float32)
        cases.append(v)
    for v in cases:
        mine = orc.argmax_first(v)
        assert mine == int(np.argmax(v))
        if ref is not None:
            assert mine == ref.ref_greedy_sample(orc._p(v), orc.i64(v.size))
    assert orc.argmax_first(cases[0]) == 1


@pytest.mark.skipif(orc.ref_host() is None, reason="oracle/_ref was never built (no reference tree)")
@pytest.mark.parametrize("position,keep", [(64, 16), (64, 0), (64, 63), (80, 16), (63, 16)])
def test_kv_overflow_against_reference_headers(position, keep):
    # KVCacheManager.h:151-273 driven as in gen_session.py:1471-1506
    rng = np.random.default_rng(11)
    nb, H, L, D = 4, 2, 64, 128
    base = [rng.standard_normal((H, L, D)).astype(np.float32) for _ in range(nb)]
    a = [b.copy() for b in base]
    b = [b.copy() for b in base]
    pa = orc.kv_overflow(a, H, L, D, position, keep, 10000.0)
    pb = orc.kv_overflow(b, H, L, D, position, keep, 10000.0, use_ref=True)
    assert pa == pb
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


@pytest.mark.parametrize("valid_len", [9, 37, 613, 1024])
def test_attention_equals_two_pass_softmax(valid_len):
    # the equivalence buddy-mlir checked by hand (ops/tosa.py:14075-14080)
    g = np.load(os.path.join(G, "ops_golden.npz"))
    q = g["at_q"]
    K, V = g["at_K"].astype(np.float32), g["at_V"].astype(np.float32)
    out = orc.gqa_decode(q, K, V, valid_len - 1)
    assert np.array_equal(out, g[f"at_out_{valid_len}"])
    for h in range(q.shape[0]):
        s = (K[h // 6, :valid_len].astype(np.float64) @ q[h].astype(np.float64)) / np.sqrt(128.0)
        p = np.exp(s - s.max())
        ref = (p / p.sum()) @ V[h // 6, :valid_len].astype(np.float64)
        assert np.abs(out[h] - ref).max() < 2e-6


def test_ops_fixture_regression():
    g = np.load(os.path.join(G, "ops_golden.npz"))
    Q, s = orc.quantize_per_channel(g["q_W"], 8)
    assert np.array_equal(Q, g["q8_Q"]) and np.array_equal(s, g["q8_s"])
    assert s[3] == np.float32(1e-10)
    Q4, s4 = orc.quantize_per_channel(g["q_W"], 4)
    assert np.array_equal(Q4, g["q4_Q"]) and np.array_equal(orc.pack_int4(Q4).reshape(96, 20), g["q4_P"])
    P, gs = orc.quantize_w4_group(g["g_W"], 128)
    assert np.array_equal(P, g["g_P"]) and np.array_equal(gs, g["g_s"])
    for tag in "abc":
        assert np.array_equal(orc.gemv_w8_f32(g[f"w8{tag}_x"], g[f"w8{tag}_Q"], g[f"w8{tag}_s"]), g[f"w8{tag}_y"])
        assert np.array_equal(orc.gemv_f32(g[f"w8{tag}_x"], g[f"f{tag}_B"]), g[f"f{tag}_y"])
    assert np.array_equal(orc.gemv_w4_f16(g["w4_x"], g["w4_P"], g["w4_s"]), g["w4_y"])
    assert np.array_equal(orc.gemv_w4g_f32(g["w4g_x"], g["g_P"], g["g_s"], 128), g["w4g_y"])
    assert np.array_equal(orc.rmsnorm(g["rn_x"], g["rn_w"], 1e-6), g["rn_y"])
    assert np.array_equal(orc.rope(g["rp_x"], g["rp_inv"], 613), g["rp_y"])
    assert np.array_equal(orc.silu_mul(g["sm_g"], g["sm_u"]), g["sm_y"])


def test_w8_gemv_is_dequantised_matmul():
    g = np.load(os.path.join(G, "ops_golden.npz"))
    x, Q, s = g["w8b_x"], g["w8b_Q"], g["w8b_s"]
    ref = (x.astype(np.float64) @ Q.astype(np.float64)) * s.astype(np.float64)
    assert np.abs(g["w8b_y"] - ref).max() / np.abs(ref).max() < 1e-5


@pytest.mark.parametrize("cfg,name", [(TINY_QWEN2, "hf_tiny_qwen2.npz"), (TINY_QWEN3, "hf_tiny_qwen3.npz")])
def test_model_against_huggingface_fixture(cfg, name):
    f = np.load(os.path.join(G, name))
    _, views = synthetic.make_f32_blob(cfg, int(f["seed_w"]))
    om = orc.OracleModel(cfg, views)
    for i, t in enumerate(f["tokens"]):
        lo = om.decode(int(t))
        assert np.abs(lo - f["logits"][i]).max() / np.abs(f["logits"][i]).max() < 1e-4
        assert int(np.argmax(lo)) == int(np.argmax(f["logits"][i]))


def test_w8a8_restatement_matches_a_stepwise_numpy_evaluation():
    """frontend/Python/ops/linalg.py:12728-12846 written out once more with numpy f32 scalars:
    scale = max(absmax * (1/127), 1e-10), q = clip(rint(x * (1/scale))), exact integer matmul,
    float(acc) * (scale * wscale[n])."""
    rng = np.random.default_rng(12)
    A = (rng.standard_normal((5, 96)) * 2).astype(np.float32)
    Q = rng.integers(-128, 128, (96, 40)).astype(np.int8)
    ws = (rng.random(40).astype(np.float32) + np.float32(0.25)) * np.float32(0.02)
    bias = rng.standard_normal(40).astype(np.float32)
    f = np.float32
    scale = max(f(np.abs(A).max()) * (f(1.0) / f(127.0)), f(1e-10))
    inv = f(1.0) / f(scale)
    q = np.clip(np.rint(A * inv), -128, 127).astype(np.int32)       # np.rint: ties to even
    acc = q @ Q.astype(np.int32)
    want = acc.astype(np.float32) * (f(scale) * ws)[None, :]
    assert np.array_equal(orc.matmul_w8a8(A, Q, ws), want)
    assert np.array_equal(orc.matmul_w8a8(A, Q, ws, bias), want + bias[None, :])
    # ties: x * inv exactly halfway rounds to the even integer
    A2 = np.zeros((1, 64), dtype=np.float32)
    A2[0, 0], A2[0, 1], A2[0, 2] = 127.0, 2.5, 3.5
    s2 = max(f(127.0) * (f(1.0) / f(127.0)), f(1e-10))
    if f(2.5) * (f(1.0) / s2) == f(2.5):                               # only when the scale is exactly 1
        got = orc.matmul_w8a8(A2, np.eye(64, dtype=np.int8), np.ones(64, dtype=np.float32))
        assert got[0, 1] == f(2.0) * s2 and got[0, 2] == f(4.0) * s2


def test_prefill_rows_is_the_decode_graph_row_by_row_except_for_tensor_wide_scales():
    """orc_prefill_rows: bit-identical to decode steps for float and weight-only projections;
    a w8a8 projection takes its activation scale over all rows, so one row equals the decode
    step and many rows differ from it by quantisation noise only."""
    from buddy_mlir_b200 import TINY_QWEN2, synthetic
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 21)
    toks = [int(t) for t in synthetic.prompt_tokens(cfg, 3, 9)]
    for kinds in ({}, {n: "w8" for n in synthetic.QUANTISED_BY_REFERENCE}):
        a, b = orc.OracleModel(cfg, views, kinds=kinds), orc.OracleModel(cfg, views, kinds=kinds)
        rows = a.prefill(toks)
        for i, t in enumerate(toks):
            assert np.array_equal(rows[i], b.decode(t))
        for ka, kb in zip(a.kv, b.kv):
            assert np.array_equal(ka, kb)
    q = {n: "w8q" for n in synthetic.QUANTISED_BY_REFERENCE}
    a, b = orc.OracleModel(cfg, views, kinds=q), orc.OracleModel(cfg, views, kinds=q)
    assert np.array_equal(a.prefill(toks[:1])[0], b.decode(toks[0]))
    a, b = orc.OracleModel(cfg, views, kinds=q), orc.OracleModel(cfg, views, kinds=q)
    rows = a.prefill(toks)
    steps = np.stack([b.decode(t) for t in toks])
    assert not np.array_equal(rows, steps)
    w8 = orc.OracleModel(cfg, views, kinds={n: "w8" for n in synthetic.QUANTISED_BY_REFERENCE}).prefill(toks)
    for x in (rows, steps):     # int8 activations: within a few percent of the weight-only model
        assert np.abs(x - w8).max() < 0.1 * np.abs(w8).max()


def test_blobs_equal_what_the_reference_importer_writes():
    """tests/golden/reference_importer_tiny_qwen2.npz holds digests of the weight files that
    buddy-mlir's own importer (tools/buddy-codegen/import_model.py: TorchDynamo trace,
    eliminate_transpose, the quantisation passes, extract_*_weights) produced for the small
    Qwen2 model with the seeded weights: the tensor order, the [K,N] layout, which tensors are
    quantised, the quantiser's codes and scales, the nibble packing and the position of the
    scales must all be the same here, for every variant, bit for bit."""
    import hashlib
    from buddy_mlir_b200 import TINY_QWEN2 as cfg, synthetic
    f = np.load(os.path.join(G, "reference_importer_tiny_qwen2.npz"))
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    assert [f"{n}:{l}" for n, l, _ in synthetic.tensor_list(cfg)] == list(f["order"])
    from buddy_mlir_b200 import TINY_QWEN3
    assert [f"{n}:{l}" for n, l, _ in synthetic.tensor_list(TINY_QWEN3)] == list(f["qwen3_order"])
    assert sorted({str(n).split(":")[0] for n in f["quantised"]}) == sorted(synthetic.QUANTISED_BY_REFERENCE)
    blob, views = synthetic.make_f32_blob(cfg, int(f["seed_w"]))
    # the rotary buffer is the one tensor the HuggingFace module computes for itself
    assert np.allclose(views[("inv_freq", -1)], f["inv_freq"], rtol=1e-6, atol=0)
    views[("inv_freq", -1)][:] = f["inv_freq"]
    assert blob.size == int(f["f32_params_size"]) and sha(blob) == str(f["f32_params_sha256"])
    # the 16-bit files of the same walk, and the panel-packed decode file of the packed-decode spec
    assert sha(blob.astype(np.float16)) == str(f["f16_params_sha256"])
    assert sha(synthetic.to_bf16(blob)) == str(f["bf16_params_sha256"])
    assert np.array_equal(synthetic.from_bf16(synthetic.to_bf16(blob)).view(np.uint32) & 0xFFFF, np.zeros(blob.size, np.uint32))
    assert sha(synthetic.pack_decode_blob(cfg, blob)) == str(f["f32_decode_packed_sha256"])
    q8 = lambda W: orc.quantize_per_channel(W, 8)
    fb, ib = synthetic.split_w8a32(cfg, views, q8)
    assert np.array_equal(fb[-f["w8a32_scales"].size:], f["w8a32_scales"])
    for variant in ("w8a32", "w8a8"):       # the same files, another graph
        assert sha(fb) == str(f[f"{variant}_f32_params_sha256"])
        assert sha(ib) == str(f[f"{variant}_i8_params_sha256"])
    # f16-activation variants: the reference quantises the half module in half precision
    fb, ib = synthetic.split_w8a16(cfg, views, lambda W: orc.quantize_per_channel_half(W, 8))
    assert fb.dtype == np.float16 and sha(fb) == str(f["w8a16_f16_params_sha256"])
    assert sha(ib) == str(f["w8a16_i8_params_sha256"])
    fb, ib = synthetic.split_w4a16(cfg, views, lambda W: orc.quantize_per_channel_half(W, 4))
    assert fb.dtype == np.float16 and sha(fb) == str(f["w4a16_f16_params_sha256"])
    assert ib.size == int(f["w4a16_i4_params_size"]) and sha(ib) == str(f["w4a16_i4_params_sha256"])


def test_entry_abi_is_the_signature_of_the_reference_traced_graphs():
    """The same fixture holds the inputs and outputs of the prefill and decode graphs as
    buddy-mlir's importer traced them for the small model: what the compiled model's
    _mlir_ciface_forward_prefill / _mlir_ciface_forward_decode take after the weight blobs and
    what their result structs hold.  The generated shim must declare exactly that: tokens
    [1, max_len]; per call token [1,1], position [1], then the K and V cache of layer 0 and, for
    every further layer, a one-element counter followed by its K and V cache; results in the
    same order (position + 1, caches, counters + 1) with the logits last."""
    import re
    from buddy_mlir_b200 import TINY_QWEN2 as cfg, gen_model_entry
    f = np.load(os.path.join(G, "reference_importer_tiny_qwen2.npz"))
    kv = f"1x{cfg.kv_heads}x{cfg.max_len}x{cfg.head_dim}:float32"
    assert list(f["prefill_inputs"]) == [f"1x{cfg.max_len}:int64"]
    assert [s.rsplit(":", 1)[0] for s in f["prefill_outputs"]] == [kv] * (2 * cfg.n_layers) + [f"1x{cfg.max_len}x{cfg.vocab}:float32"]
    want_in = ["1x1:int64", "1:int64", kv, kv]
    for _ in range(cfg.n_layers - 1):
        want_in += ["1:int64", kv, kv]
    assert list(f["decode_inputs"]) == want_in
    outs = [s.rsplit(":", 1) for s in f["decode_outputs"]]
    assert [o[0] for o in outs] == want_in[1:] + [f"1x1x{cfg.vocab}:float32"]
    assert [o[1] for o in outs if o[0] == "1:int64"] == ["AddOp"] * cfg.n_layers      # counters come back + 1
    # the shim's declaration of the same
    src = gen_model_entry.source(cfg, "f32")
    sig = re.search(r"_mlir_ciface_forward_decode\(DecodeABI \*result,(.*?)\) \{", src, re.S).group(1)
    params = [p.strip().split()[0] for p in sig.split(",")]
    kinds = {"b200_memref_i64_2": "1x1:int64", "b200_memref_i64_1": "1:int64", "b200_memref_f32_4": kv}
    assert params[0] == "b200_memref_f32_1" and [kinds[p] for p in params[1:]] == want_in
    abi = re.search(r"struct DecodeABI \{(.*?)\};", src, re.S).group(1)
    fields = []
    for line in abi.strip().splitlines():
        typ, names = line.strip().rstrip(";").split(None, 1)
        fields += [typ] * len(names.split(","))
    assert [kinds.get(t, t) for t in fields] == want_in[1:] + ["b200_memref_f32_3"]


def test_w8a8_graphs_quantise_the_projections_and_tensors_this_library_does():
    """What buddy-mlir's w8a8 pass leaves in the traced graphs of the small model (same fixture):
    o, gate, up, down of every layer and the lm_head are integer matmuls, q / k / v stay float;
    the activation each of them quantises with ONE scale is the whole [max_len, K] tensor in the
    prefill graph (the lm_head included, every row) and the single row in the decode graph --
    the two cases b200_model_set_activation_int8 implements."""
    from buddy_mlir_b200 import TINY_QWEN2 as cfg, synthetic
    f = np.load(os.path.join(G, "reference_importer_tiny_qwen2.npz"))
    K = {"o": cfg.q_dim, "gate": cfg.hidden, "up": cfg.hidden, "down": cfg.ffn, "lm_head": cfg.hidden}
    for phase, rows in (("prefill", cfg.max_len), ("decode", 1)):
        got = sorted(str(s) for s in f[f"w8a8_{phase}_ops"])
        want = [f"QuantizedMatmulOp:{n}:{l}:{rows}x{K[n]}" for n in ("o", "gate", "up", "down") for l in range(cfg.n_layers)]
        want.append(f"QuantizedMatmulOp:lm_head:-1:{rows}x{K['lm_head']}")
        assert got == sorted(want)
    assert {s.split(":")[1] for s in f["w8a8_prefill_ops"]} == set(synthetic.QUANTISED_BY_REFERENCE)
