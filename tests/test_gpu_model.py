"""Whole-decode-step parity: logits within the stated tolerances of the CPU
restatement (max relative error 1e-3 for f32 and int8 weight-only, 2e-2 for
int4) and identical greedy tokens, on small shapes against the committed
HuggingFace fixtures and on the full 1.5B shapes against the live checker."""
import os

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import (DEEPSEEK_R1_1P5B, TINY_MEGA, TINY_QWEN2, TINY_QWEN3, _lib, synthetic)
from buddy_mlir_b200.model_entry import EntrySession, TieredEntrySession
from buddy_mlir_b200.session import ModelSession, greedy_sample, run_generation

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
ALL_LINEAR = ("q", "k", "v", "o", "gate", "up", "down", "lm_head")


def maxrel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def margin(logits):
    top2 = np.partition(logits, -2)[-2:]
    return float(top2[1] - top2[0])


def check_stream(step_fn, om, tokens, tol, n_greedy=0):
    """Feed `tokens`, then n_greedy greedy steps; compare logits and argmax at
    every step.  Reports the smallest top-1/top-2 margin seen."""
    worst, min_margin = 0.0, 1e30
    tok = None
    seq = list(tokens)
    for i in range(len(tokens) + n_greedy):
        t = seq[i] if i < len(seq) else tok
        got = step_fn(int(t))
        want = om.decode(int(t))
        worst = max(worst, maxrel(got, want))
        min_margin = min(min_margin, margin(want))
        a, b = greedy_sample(got), greedy_sample(want)
        assert a == b, f"greedy token differs at step {i}: {a} vs {b} (margin {margin(want):.3e})"
        tok = b
    assert worst < tol, f"max relative logit error {worst:.3e} >= {tol}"
    return worst, min_margin


@pytest.mark.parametrize("cfg,name", [(TINY_QWEN2, "hf_tiny_qwen2.npz"), (TINY_QWEN3, "hf_tiny_qwen3.npz")])
def test_tiny_f32_against_huggingface_fixture(cfg, name):
    f = np.load(os.path.join(G, name))
    blob, views = synthetic.make_f32_blob(cfg, int(f["seed_w"]))
    s = ModelSession(cfg)
    if cfg.qk_norm:
        s.load_tensors(views)
    else:
        s.load_blobs("f32", blob)
    for i, t in enumerate(f["tokens"]):
        s.decode(int(t))
        assert maxrel(s.logits_data(), f["logits"][i]) < 1e-4
        assert greedy_sample(s.logits_data()) == int(np.argmax(f["logits"][i]))
    s.close()


def test_qwen3_blob_is_walked_in_the_importers_order():
    """A Qwen3 model (head norms, no biases) from its flat blob: the same logits as the same
    tensors loaded by name."""
    cfg = TINY_QWEN3
    blob, views = synthetic.make_f32_blob(cfg, 31)
    a, b = ModelSession(cfg), ModelSession(cfg)
    a.load_blobs("f32", blob)
    b.load_tensors(views)
    for t in synthetic.prompt_tokens(cfg, 4, 6):
        a.decode(int(t))
        b.decode(int(t))
        assert np.array_equal(a.logits_data(), b.logits_data())
    a.close()
    b.close()


def test_tiny_f32_greedy_and_device_loop():
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 5)
    om = orc.OracleModel(cfg, views)
    s = ModelSession(cfg)
    s.load_blobs("f32", blob)
    prompt = synthetic.prompt_tokens(cfg, 6, 8)

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    check_stream(step, om, prompt, 1e-3, n_greedy=40)
    # device-resident loop and device argmax give the same ids as the host loop
    host_ids, _ = run_generation(s, prompt, len(prompt) + 30)
    s.reset_position()
    s.prefill(prompt)
    first = greedy_sample(s.logits_data())
    dev_ids = s.generate(first, 30)
    assert [first] + [int(t) for t in dev_ids] == host_ids
    s.reset_position()
    for t in prompt[:-1]:
        s.decode(int(t))
    assert s.decode_greedy(int(prompt[-1])) == first
    assert s.kernels_per_step() > 0 and s.step_bytes(16) > 0
    s.close()


def test_tiny_w8a32_reference_blobs_through_model_entry():
    """The reference-faithful variant (o, gate, up, down, lm_head int8; q/k/v
    float) fed as the reference's two blobs through _mlir_ciface_forward_decode,
    with host KV buffers."""
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 77)
    fb, ib = synthetic.split_w8a32(cfg, views, lambda W: orc.quantize_per_channel(W, 8))
    kinds = {n: "w8" for n in synthetic.QUANTISED_BY_REFERENCE}
    om = orc.OracleModel(cfg, views, kinds=kinds)
    es = EntrySession(cfg, "w8a32", [fb, ib])
    prompt = synthetic.prompt_tokens(cfg, 3, 6)

    def step(t):
        es.decode(t, check_alias=True)
        return es.logits.copy()
    check_stream(step, om, prompt, 1e-3, n_greedy=20)
    # the host KV buffers hold what the reference's in-place write would hold
    for b in range(2 * cfg.n_layers):
        assert maxrel(es.kv[b][0, :, :26], om.kv[b][:, :26]) < 1e-4
    # position discontinuity: host edits its cache (as handleKVCacheOverflow
    # does) and jumps back; the entry must pick the host's data up again
    pos = 10
    for b in range(2 * cfg.n_layers):
        es.kv[b][0, :, :pos] *= np.float32(0.5)
        om.kv[b][:, :pos] *= np.float32(0.5)
    es.position_ = pos
    om.position = pos
    check_stream(step, om, prompt[:3], 1e-3)
    es.close()


def test_load_weights_from_the_reference_blob_files(tmp_path):
    """loadWeights from files named and laid out as the reference writes them
    (tools/buddy-codegen/gen_config.py:51-71: arg0-w8a32-f32.data + arg0-w8a32-i8.data)."""
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 78)
    fb, ib = synthetic.split_w8a32(cfg, views, lambda W: orc.quantize_per_channel(W, 8))
    fp, ip = tmp_path / "arg0-w8a32-f32.data", tmp_path / "arg0-w8a32-i8.data"
    fb.tofile(fp)
    ib.tofile(ip)
    om = orc.OracleModel(cfg, views, kinds={n: "w8" for n in synthetic.QUANTISED_BY_REFERENCE})
    s = ModelSession(cfg)
    s.load_weights([str(fp), str(ip)], "w8a32")

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    check_stream(step, om, synthetic.prompt_tokens(cfg, 2, 6), 1e-3, n_greedy=6)
    s.close()


@pytest.mark.parametrize("cfg,all_w8", [(TINY_QWEN2, False), (TINY_MEGA, True), (TINY_QWEN3, "w4")])
def test_repack_cache_round_trip(tmp_path, cfg, all_w8):
    """The packed device layout saved by one session and loaded by another gives
    bit-identical logits (same kernels, same bytes); a file written for another
    configuration, a truncated file and a late save are refused."""
    blob, views = synthetic.make_f32_blob(cfg, 79)
    fb, ib = synthetic.split_w8a32(cfg, views, lambda W: orc.quantize_per_channel(W, 8))
    path = tmp_path / "model.b2pack"
    a = ModelSession(cfg)
    if all_w8 == "w4":      # group-wise int4 with QK-norm vectors, from tensors
        a.load_tensors(views, quantize_to="w4", group=64, save_packed=path)
    else:
        a.load_blobs("w8a32", fb, ib, all_linear_w8=all_w8, save_packed=path)
    b = ModelSession(cfg)
    b.load_packed(path)
    assert a.uses_persistent_kernel() == b.uses_persistent_kernel()
    for t in synthetic.prompt_tokens(cfg, 3, 8):
        a.decode(int(t))
        b.decode(int(t))
        assert np.array_equal(a.logits_data(), b.logits_data())
    with pytest.raises(RuntimeError):            # finalize has freed the per-projection buffers
        _lib.check(a.lib.b200_model_save_packed(a._h, str(tmp_path / "late.b2pack").encode()))
    other = TINY_QWEN3 if cfg is not TINY_QWEN3 else TINY_QWEN2
    c = ModelSession(other)
    with pytest.raises(RuntimeError):
        _lib.check(c.lib.b200_model_load_packed(c._h, str(path).encode()))
    cut = tmp_path / "cut.b2pack"
    cut.write_bytes(path.read_bytes()[: path.stat().st_size // 2])
    d = ModelSession(cfg)
    with pytest.raises(RuntimeError):
        _lib.check(d.lib.b200_model_load_packed(d._h, str(cut).encode()))
    for s in (a, b, c, d):
        s.close()


def test_tiny_w4a16_reference_blobs():
    """The reference's int4 flavour (tools/buddy-codegen/gen_config.py:37-71): f16 blob +
    nibble-packed blob, signed per-channel int4 on o / gate / up / down / lm_head.  The
    reference accumulates these GEMVs in f16 (Int4DequantMatMulVectorizationDecode.cpp:
    359-430), this library in f32: logits within 2e-2, and the same greedy token wherever
    the checker's top-1 / top-2 margin is larger than that tolerance."""
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 79)
    fb, ib = synthetic.split_w4a16(cfg, views, lambda W: orc.quantize_per_channel(W, 4))
    assert fb.dtype == np.float16 and ib.dtype == np.int8
    # the checker sees what the blobs hold: f16-rounded float tensors
    rounded = {k: (v.astype(np.float16).astype(np.float32) if k[0] not in synthetic.QUANTISED_BY_REFERENCE else v)
               for k, v in views.items()}
    om = orc.OracleModel(cfg, rounded, kinds={n: "w4" for n in synthetic.QUANTISED_BY_REFERENCE})
    s = ModelSession(cfg)
    s.load_blobs("w4a16", fb, ib)
    worst, agree, total = 0.0, 0, 0
    tok = None
    for i, t in enumerate(list(synthetic.prompt_tokens(cfg, 5, 8)) + [None] * 24):
        t = tok if t is None else int(t)
        s.decode(t)
        want = om.decode(t)
        got = s.logits_data()
        worst = max(worst, maxrel(got, want))
        if margin(want) > 2e-2 * float(np.abs(want).max()):
            assert greedy_sample(got) == greedy_sample(want)
        agree += int(greedy_sample(got) == greedy_sample(want))
        total += 1
        tok = greedy_sample(want)
    assert worst < 2e-2, worst
    print(f"w4a16 tiny: max rel logit err {worst:.3e}, greedy agreement {agree}/{total}")
    s.close()


@pytest.mark.parametrize("through_entry", [False, True])
def test_tiny_w8a16_reference_blobs(through_entry):
    """The reference's w8a16 flavour (tools/buddy-codegen/gen_config.py:37-71): the w8a32 split
    with an f16 float blob and f16 scales, f16 activations / cache / logits.  The reference
    accumulates these GEMVs in f16, this library in f32: logits within 2e-2, the same greedy
    token wherever the checker's margin is larger than that; once through the device session,
    once through the model entries with a half cache."""
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 82)
    fb, ib = synthetic.split_w8a16(cfg, views, lambda W: orc.quantize_per_channel(W, 8))
    assert fb.dtype == np.float16 and ib.dtype == np.int8
    rounded = {k: (v.astype(np.float16).astype(np.float32) if k[0] not in synthetic.QUANTISED_BY_REFERENCE else v)
               for k, v in views.items()}
    om = orc.OracleModel(cfg, rounded, kinds={n: "w8h" for n in synthetic.QUANTISED_BY_REFERENCE})
    if through_entry:
        s = EntrySession(cfg, "w8a16", [fb, ib])
        step = lambda t: (s.decode(t), s.logits)[1]
    else:
        s = ModelSession(cfg)
        s.load_blobs("w8a16", fb, ib)
        step = lambda t: (s.decode(t), s.logits_data())[1]
    worst, tok = 0.0, None
    for t in list(synthetic.prompt_tokens(cfg, 6, 8)) + [None] * 16:
        t = tok if t is None else int(t)
        got = step(t)
        want = om.decode(t)
        worst = max(worst, maxrel(got, want))
        if margin(want) > 2e-2 * float(np.abs(want).max()):
            assert greedy_sample(got) == greedy_sample(want)
        tok = greedy_sample(want)
    assert worst < 2e-2, worst
    s.close()


def _w8a8_case(seed):
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, seed)
    fb, ib = synthetic.split_w8a32(cfg, views, lambda W: orc.quantize_per_channel(W, 8))
    om = orc.OracleModel(cfg, views, kinds={n: "w8q" for n in synthetic.QUANTISED_BY_REFERENCE})
    return cfg, fb, ib, om


# The w8a8 graphs round every activation to one of 255 levels.  The float operations before a
# projection (RMSNorm sums, exp, sin / cos) differ from the checker's by a few ulp, so a value
# within that distance of a rounding boundary (about 3e-5 of all values) falls to the other side
# and moves one term of one dot product by a level: 1 / (127 sqrt(K)) of the output's magnitude
# per flip, 5e-4 at K = 256, and the projections after it amplify that (their own roundings
# move).  Most runs see no flip and agree to 1e-7; on the CPU alone, the checker against itself
# with the embedding one ulp off reaches 1.0e-2 over twelve decode steps for one seed in three
# of this small model.  The bound is the checker's own quantisation noise (w8a8 against
# weight-only logits: 1.9e-2 to 2.6e-2 here) with a little room: what a wiring error would
# exceed and a rounding flip cannot.  Bit-exactness is established per projection
# (test_gpu_gemm.py); the greedy token is compared wherever the checker's margin is larger.
W8A8_TOL = 3e-2


def test_tiny_w8a8_device_session_prefill_and_decode():
    """models/deepseek_r1/specs/w8a8.json: the files of w8a32, int8 activations with one dynamic
    scale per activation tensor (all rows of the prefill, the one row of a decode step)."""
    cfg, fb, ib, om = _w8a8_case(86)
    s = ModelSession(cfg)
    s.load_blobs("w8a8", fb, ib)
    assert s.lib.b200_model_activation_int8(s._h) == 1
    prompt = [int(t) for t in synthetic.prompt_tokens(cfg, 8, 23)]
    got = s.prefill_rows(prompt, 0, all_rows=True)
    want = om.prefill(prompt)
    assert got.shape == want.shape and maxrel(got, want) < W8A8_TOL
    # the last row alone still sees the scale of all rows
    s2 = ModelSession(cfg)
    s2.load_blobs("w8a8", fb, ib)
    last = s2.prefill_rows(prompt, 0, all_rows=False)
    assert np.array_equal(np.asarray(last).reshape(-1), got[-1])
    s2.close()
    worst, tok = 0.0, greedy_sample(want[-1])
    for _ in range(12):
        s.decode(tok)
        w = om.decode(tok)
        worst = max(worst, maxrel(s.logits_data(), w))
        if margin(w) > W8A8_TOL * float(np.abs(w).max()):
            assert greedy_sample(s.logits_data()) == greedy_sample(w)
        tok = greedy_sample(w)
    assert worst < W8A8_TOL, worst
    # the device loop feeds its own token back: the same ids as single steps from the same state
    ids = s.generate(tok, 6)
    t = tok
    for i in range(6):
        w = om.decode(t)
        if margin(w) <= W8A8_TOL * float(np.abs(w).max()):
            break       # too close to call: the streams may part here
        assert int(ids[i]) == greedy_sample(w), i
        t = greedy_sample(w)
    print(f"w8a8 tiny: prefill max rel {maxrel(got, want):.2e}, decode max rel {worst:.2e}")
    s.close()


def test_w8a8_switch_leaves_no_residue_in_a_session_of_the_persistent_kernel():
    """The same session alternates between the float step (persistent kernel) and the int8 step
    (its own CUDA graph): after switching back, the float logits are bit for bit those of a
    session that never switched; the batched entry points refuse a w8a8 session."""
    from buddy_mlir_b200.session import BatchSession
    cfg = TINY_MEGA
    _, views = synthetic.make_f32_blob(cfg, 89)
    toks = [int(t) for t in synthetic.prompt_tokens(cfg, 10, 6)]

    def fresh():
        s = ModelSession(cfg)
        s.load_tensors(views, quantize_to="w8")
        assert s.uses_persistent_kernel()
        return s
    a = fresh()
    ref = []
    for t in toks:
        a.decode(t)
        ref.append(a.logits_data().copy())
    a.close()
    b = fresh()
    om = orc.OracleModel(cfg, views, kinds={n: "w8q" for n in ALL_LINEAR})
    b.set_activation_int8(True)
    for t in toks[:3]:
        b.decode(t)
        assert maxrel(b.logits_data(), om.decode(t)) < W8A8_TOL
    bs = BatchSession(b, max_seqs=2, page_size=16, n_pages=16, max_context=64)
    with pytest.raises(_lib.B200Error):
        bs.prefill(bs.add(), toks, want_logits=False)
    bs.close()
    b.set_activation_int8(False)
    b.reset_position()
    for i, t in enumerate(toks):
        b.decode(t)
        assert np.array_equal(b.logits_data(), ref[i]), i
    b.close()


def test_tiny_w8a8_through_the_model_entries():
    """The generated entry pair of the w8a8 spec: the prefill entry quantises over all max_len
    rows of the padded token container, as the reference's prefill graph does."""
    cfg, fb, ib, om = _w8a8_case(87)
    es = EntrySession(cfg, "w8a8", [fb, ib])
    prompt = [int(t) for t in synthetic.prompt_tokens(cfg, 9, 11)]
    logits = es.prefill(prompt, pad_id=0)
    want = om.prefill(prompt + [0] * (cfg.max_len - len(prompt)))
    assert maxrel(logits[:len(prompt)], want[:len(prompt)]) < W8A8_TOL
    om.position = len(prompt)
    tok = greedy_sample(want[len(prompt) - 1])
    for _ in range(8):
        es.decode(tok)
        w = om.decode(tok)
        assert maxrel(es.logits, w) < W8A8_TOL
        if margin(w) > W8A8_TOL * float(np.abs(w).max()):
            assert greedy_sample(es.logits) == greedy_sample(w)
        tok = greedy_sample(w)
    es.close()


def test_tiny_f16_blob_through_the_model_entries():
    """The reference's f16 flavour (tools/buddy-codegen/gen_config.py:37-71): one f16 blob,
    half cache and logits.  The device computes in f32 on the widened weights; the checker is
    the f32 restatement on the same f16-rounded tensors, 2e-2 (the reference's own f16
    arithmetic has no restatement here: parity of this variant is unpinned beyond that)."""
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 83)
    rounded = {k: v.astype(np.float16).astype(np.float32) for k, v in views.items()}
    om = orc.OracleModel(cfg, rounded)
    es = EntrySession(cfg, "f16", [blob.astype(np.float16)])
    prompt = synthetic.prompt_tokens(cfg, 7, 9)
    logits = es.prefill(prompt, pad_id=0)
    for t in prompt:
        want = om.decode(int(t))
    assert maxrel(logits[len(prompt) - 1], want) < 2e-2
    tok = greedy_sample(want)
    for _ in range(8):
        es.decode(tok)
        want = om.decode(tok)
        assert maxrel(es.logits, want) < 2e-2
        if margin(want) > 2e-2 * float(np.abs(want).max()):
            assert greedy_sample(es.logits) == greedy_sample(want)
        tok = greedy_sample(want)
    es.close()


def test_tiny_bf16_blob_through_the_model_entries():
    """The reference's bf16 flavour (tools/buddy-codegen/gen_config.py:40-44,54): one blob of
    bfloat16 values (the module converted with .bfloat16(), import_model.py:118-145, 700-707),
    bfloat16 cache and logits on the host.  The device computes in f32 on the widened weights
    and rounds at the boundary; the checker is the f32 restatement on the same rounded
    tensors, 2e-2 (bf16 keeps 8 bits: 4e-3 per value; the reference's own bf16 arithmetic has
    no restatement here: parity of this variant is unpinned beyond that)."""
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 88)
    high = synthetic.to_bf16(blob)
    rounded = {k: synthetic.from_bf16(synthetic.to_bf16(v)).reshape(v.shape) for k, v in views.items()}
    om = orc.OracleModel(cfg, rounded)
    es = EntrySession(cfg, "bf16", [high])
    prompt = synthetic.prompt_tokens(cfg, 7, 9)
    logits = es.prefill(prompt, pad_id=0)
    for t in prompt:
        want = om.decode(int(t))
    assert maxrel(logits[len(prompt) - 1], want) < 2e-2
    assert maxrel(es.kv_floats(0)[0, :, :len(prompt)], om.kv[0][:, :len(prompt)]) < 1e-2
    tok = greedy_sample(want)
    for _ in range(8):
        es.decode(tok)
        want = om.decode(tok)
        assert maxrel(es.logits, want) < 2e-2
        if margin(want) > 2e-2 * float(np.abs(want).max()):
            assert greedy_sample(es.logits) == greedy_sample(want)
        tok = greedy_sample(want)
    es.close()


def test_packed_decode_spec_plain_prefill_blob_and_panel_packed_decode_blob():
    """models/deepseek_r1/specs/f32_packed_decode.json: the prefill entry gets the plain f32
    blob, the decode entry the copy whose matmul weights sit in 32-column panels
    (pack_decode_weights.py:32-124, gen_session.py:1393).  Both are one model: the device
    session is built once, decode continues on the prefilled cache, logits equal the
    checker's; a decode blob of another model is not mistaken for it."""
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 84)
    packed = synthetic.pack_decode_blob(cfg, blob)
    assert not np.array_equal(packed, blob) and np.array_equal(np.sort(packed), np.sort(blob))
    om = orc.OracleModel(cfg, views)
    es = EntrySession(cfg, "f32", [blob], decode_blobs=[packed])
    prompt = synthetic.prompt_tokens(cfg, 12, 7)
    logits = es.prefill(prompt, pad_id=0)
    for t in prompt:
        want = om.decode(int(t))
    assert maxrel(logits[len(prompt) - 1], want) < 1e-3
    tok = greedy_sample(want)
    for _ in range(6):
        es.decode(tok, check_alias=True)
        want = om.decode(tok)
        assert maxrel(es.logits, want) < 1e-3 and greedy_sample(es.logits) == greedy_sample(want)
        tok = greedy_sample(want)
    assert _lib.load().b200_forward_session_builds() == 1
    es.close()
    # the panels of ANOTHER model: the decode entry must build its own session from them
    other, oviews = synthetic.make_f32_blob(cfg, 85)
    es = EntrySession(cfg, "f32", [blob], decode_blobs=[synthetic.pack_decode_blob(cfg, other)])
    es.prefill(prompt, pad_id=0)
    om2 = orc.OracleModel(cfg, oviews)
    for b in range(2 * cfg.n_layers):              # the cache the first model's prefill left on the host
        om2.kv[b][:, :len(prompt)] = es.kv_floats(b)[0, :, :len(prompt)]
    om2.position = len(prompt)
    es.decode(tok)
    assert maxrel(es.logits, om2.decode(tok)) < 1e-3
    assert _lib.load().b200_forward_session_builds() == 2
    es.close()


def test_tiered_cache_spec_entries_per_cache_size():
    """models/deepseek_r1/specs/f32_tiered_kv_cache.json: one prefill / decode symbol per cache
    size; the host moves its cache to a larger tier as the sequence grows (gen_session.py:
    303-800).  The prompt lands in the 32-row tier, decode crosses into the 64- and the 128-row
    tiers; logits equal the checker's all the way and the device session is built once."""
    from buddy_mlir_b200.gen_model_entry import TINY_TIERS
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 86)
    om = orc.OracleModel(cfg, views)
    es = TieredEntrySession(cfg, blob, TINY_TIERS)
    prompt = synthetic.prompt_tokens(cfg, 16, 27)
    logits = es.prefill(prompt, pad_id=0)
    assert logits.shape == (32, cfg.vocab) and es.slot == 0
    for t in prompt:
        want = om.decode(int(t))
    assert maxrel(logits[len(prompt) - 1], want) < 1e-3
    tok = greedy_sample(want)
    seen = set()
    for _ in range(45):                      # positions 27 .. 71: tiers 32 -> 64 -> 128
        es.decode(tok)
        seen.add(es.tiers[es.slot])
        want = om.decode(tok)
        assert maxrel(es.logits, want) < 1e-3 and greedy_sample(es.logits) == greedy_sample(want)
        tok = greedy_sample(want)
    assert seen == {32, 64, 128}
    assert _lib.load().b200_forward_session_builds() == 1
    es.close()


def test_w4a16_model_entries_with_half_cache_and_logits():
    """The w4a16 shim: f16 blob, nibble-packed blob, KV cache and logits as IEEE half
    (uint16) on the host, exactly the descriptor types the generated session uses for
    this variant (tools/buddy-codegen/gen_config.py:37-71).  Prefill, then decode steps;
    an overflow-style rewrite of the host cache is noticed through the rounded rows."""
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 80)
    fb, ib = synthetic.split_w4a16(cfg, views, lambda W: orc.quantize_per_channel(W, 4))
    rounded = {k: (v.astype(np.float16).astype(np.float32) if k[0] not in synthetic.QUANTISED_BY_REFERENCE else v)
               for k, v in views.items()}
    om = orc.OracleModel(cfg, rounded, kinds={n: "w4" for n in synthetic.QUANTISED_BY_REFERENCE})
    es = EntrySession(cfg, "w4a16", [fb, ib])
    assert es.kv[0].dtype == np.uint16
    prompt = synthetic.prompt_tokens(cfg, 11, 10)
    logits = es.prefill(prompt, pad_id=0)
    for t in prompt:
        want = om.decode(int(t))
    assert maxrel(logits[len(prompt) - 1], want) < 2e-2
    for b in range(2 * cfg.n_layers):
        assert maxrel(es.kv_floats(b)[0, :, :len(prompt)], om.kv[b][:, :len(prompt)]) < 2e-2
    tok = greedy_sample(want)
    for _ in range(6):
        es.decode(tok, check_alias=True)
        want = om.decode(tok)
        assert maxrel(es.logits, want) < 2e-2
        if margin(want) > 2e-2 * float(np.abs(want).max()):
            assert greedy_sample(es.logits) == greedy_sample(want)
        tok = greedy_sample(want)
    # the host rewrites its (half) cache, as handleKVCacheOverflow does: the next step must
    # take the rows from the host again -- here: zeroed history, so the logits change
    before = es.logits.copy()
    for k in es.kv:
        k[...] = 0
    es.position_ -= 1
    es.decode(tok)
    assert not np.array_equal(es.logits, before)
    es.close()


def test_model_entry_failure_leaves_zero_logits_and_a_sticky_status():
    """The entries return void: after a failure (here a position outside the cache) the
    caller still gets a logits buffer it can copy from, all zeros, and the status stays
    set until the session is reset."""
    cfg = TINY_QWEN2
    blob, _ = synthetic.make_f32_blob(cfg, 81)
    es = EntrySession(cfg, "f32", [blob])
    es.decode(3)
    es.position_ = cfg.max_len + 5
    with pytest.raises(RuntimeError):
        es.decode(3)
    assert np.array_equal(es.logits, np.zeros(cfg.vocab, dtype=np.float32))
    assert _lib.load().b200_forward_status() != 0
    es.close()
    assert _lib.load().b200_forward_status() == 0


def test_tiny_all_linear_w8_quantised_on_device():
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 8)
    om = orc.OracleModel(cfg, views, kinds={n: "w8" for n in ALL_LINEAR})
    s = ModelSession(cfg)
    s.load_blobs("f32", blob, all_linear_w8=True)

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    check_stream(step, om, synthetic.prompt_tokens(cfg, 4, 8), 1e-3, n_greedy=24)
    s.close()


@pytest.mark.parametrize("cfg", [TINY_QWEN2, TINY_QWEN3])
def test_tiny_w4_group128(cfg):
    blob, views = synthetic.make_f32_blob(cfg, 9)
    om = orc.OracleModel(cfg, views, kinds={n: "w4g" for n in ALL_LINEAR}, group=128)
    s = ModelSession(cfg)
    s.load_tensors(views, quantize_to="w4", group=128)

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    check_stream(step, om, synthetic.prompt_tokens(cfg, 4, 8), 2e-2, n_greedy=16)
    s.close()


def test_session_kv_overflow_matches_checker():
    cfg = TINY_QWEN2.with_(max_len=64)
    blob, views = synthetic.make_f32_blob(cfg, 12)
    om = orc.OracleModel(cfg, views)
    s = ModelSession(cfg)
    s.load_blobs("f32", blob)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, cfg.vocab, 64)
    for t in toks:
        s.decode(int(t))
        om.decode(int(t))
    assert s.position() == 64
    assert s.handle_kv_cache_overflow(cfg.max_len // 4, 10000.0)
    newp = orc.kv_overflow(om.kv, cfg.kv_heads, cfg.max_len, cfg.head_dim, 64, cfg.max_len // 4, 10000.0)
    assert s.position() == newp == 40
    om.position = newp
    for b in range(2 * cfg.n_layers):
        assert maxrel(s.kv_download(b), om.kv[b]) < 1e-5
    s.decode(7)
    assert maxrel(s.logits_data(), om.decode(7)) < 1e-3
    s.close()


@pytest.mark.parametrize("cfg", [TINY_MEGA, TINY_QWEN3])
def test_persistent_kernel_matches_checker_and_graph_path(cfg, monkeypatch):
    """Batch-1 int8 decode runs as one persistent kernel; it must agree with
    the CPU checker, with the multi-kernel graph path, and with itself."""
    blob, views = synthetic.make_f32_blob(cfg, 21)
    om = orc.OracleModel(cfg, views, kinds={n: "w8" for n in ALL_LINEAR})
    s = ModelSession(cfg)
    s.load_tensors(views, quantize_to="w8")
    assert s.uses_persistent_kernel() and s.kernels_per_step() == 1
    prompt = synthetic.prompt_tokens(cfg, 4, 8)

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    check_stream(step, om, prompt, 1e-3, n_greedy=40)
    for b in range(2 * cfg.n_layers):
        assert maxrel(s.kv_download(b)[:, :48], om.kv[b][:, :48]) < 1e-4
    # device loop == host loop, twice (determinism)
    host_ids, _ = run_generation(s, prompt, len(prompt) + 30)
    runs = []
    for _ in range(2):
        s.reset_position()
        s.prefill(prompt)
        first = greedy_sample(s.logits_data())
        runs.append([first] + [int(t) for t in s.generate(first, 30)])
    assert runs[0] == runs[1] == host_ids
    # the multi-kernel graph path on the same weights
    monkeypatch.setenv("BUDDY_B200_DECODE", "graph")
    g = ModelSession(cfg)
    g.load_tensors(views, quantize_to="w8")
    assert not g.uses_persistent_kernel() and g.kernels_per_step() > 1
    s.reset_position()
    for t in prompt:
        s.decode(int(t))
        g.decode(int(t))
        assert maxrel(s.logits_data(), g.logits_data()) < 1e-4
    s.close()
    g.close()


def test_persistent_kernel_crosses_the_wrap_of_its_tag_space():
    """The CTAs of the persistent kernel exchange activations under 32-bit tags numbered from
    the launch counter; the counter is preset just below the point where the tags wrap
    (2^32 / (8 * (layers + 3)) launches) and the steps across it must equal the checker's."""
    cfg = TINY_MEGA
    _, views = synthetic.make_f32_blob(cfg, 33)
    om = orc.OracleModel(cfg, views, kinds={n: "w8" for n in ALL_LINEAR})
    s = ModelSession(cfg)
    s.load_tensors(views, quantize_to="w8")
    assert s.uses_persistent_kernel()
    wrap = (1 << 32) // (8 * (cfg.n_layers + 3))
    _lib.check(s.lib.b200_model_set_launch_counter(s._h, wrap - 4))
    tok = 5
    for i in range(10):                      # launches wrap-4 .. wrap+5
        s.decode(tok)
        want = om.decode(tok)
        assert maxrel(s.logits_data(), want) < 1e-3, i
        assert greedy_sample(s.logits_data()) == greedy_sample(want)
        tok = greedy_sample(want)
    ids = s.generate(tok, 6)                 # and the multi-step launch path
    for t in ids:
        want = om.decode(tok)
        assert int(t) == greedy_sample(want)
        tok = int(t)
    s.close()


# ---- prefill: all prompt rows in one pass (dense GEMMs) --------------------------------------
@pytest.mark.parametrize("cfg,quant,n_prompt", [(TINY_MEGA, "w8", 40), (TINY_QWEN2, "w8", 40), (TINY_QWEN3, "w8", 40),
                                                (TINY_QWEN2, None, 40), (TINY_MEGA, "w8", 93), (TINY_QWEN2, "w8", 77),
                                                (TINY_QWEN3, None, 100)])
def test_dense_prefill_matches_checker_rows_and_cache(cfg, quant, n_prompt):
    """Every prompt row's logits and the KV rows left behind equal the checker's
    token-by-token pass; decode then continues from the prefilled cache.  Prompts
    of 64 rows and more take the attention kernel tiled over query rows (ragged
    last tile included), shorter ones the per-row kernel."""
    blob, views = synthetic.make_f32_blob(cfg, 51)
    kinds = {n: "w8" for n in ALL_LINEAR} if quant else None
    om = orc.OracleModel(cfg, views, kinds=kinds)
    s = ModelSession(cfg)
    s.load_tensors(views, quantize_to=quant)
    prompt = synthetic.prompt_tokens(cfg, 8, n_prompt)
    logits = s.prefill_rows(prompt, 0, all_rows=True)
    for i, t in enumerate(prompt):
        want = om.decode(int(t))
        assert maxrel(logits[i], want) < 1e-3, i
        assert greedy_sample(logits[i]) == greedy_sample(want)
    assert s.last_next_token == greedy_sample(logits[-1])
    for b in range(2 * cfg.n_layers):
        assert maxrel(s.kv_download(b)[:, :n_prompt], om.kv[b][:, :n_prompt]) < 1e-4
    # a second chunk on top of the first, then free-running decode
    more = synthetic.prompt_tokens(cfg, 9, 16)
    logits = s.prefill_rows(more, all_rows=False)
    for t in more:
        want = om.decode(int(t))
    assert maxrel(logits, want) < 1e-3

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    check_stream(step, om, [greedy_sample(want)], 1e-3, n_greedy=8)
    s.close()


# ---- full-size shapes -------------------------------------------------------------------
@pytest.fixture(scope="module")
def full_weights():
    return synthetic.make_f32_blob(DEEPSEEK_R1_1P5B, 20260101)


def test_1p5b_f32_logits_and_greedy_tokens(full_weights):
    """Config: DeepSeek-R1-Distill-Qwen-1.5B shapes, f32, 32 random prompt ids
    then greedy decode; logits within 1e-3, tokens identical."""
    cfg = DEEPSEEK_R1_1P5B
    blob, views = full_weights
    om = orc.OracleModel(cfg, views)
    s = ModelSession(cfg)
    s.load_blobs("f32", blob)

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    # 32 random prompt ids, then 128 free-running greedy steps compared with the
    # CPU checker step by step (the first 64 must be identical; all 128 are checked)
    worst, mm = check_stream(step, om, synthetic.prompt_tokens(cfg, 17, 32), 1e-3, n_greedy=128)
    print(f"1.5B f32: max rel logit err {worst:.3e}, smallest top-1/top-2 margin {mm:.3e}")
    s.close()


def test_1p5b_int8_all_linear_with_long_context(full_weights):
    """Config: int8 per-output-channel weight-only on every linear layer,
    f32 activations.  Greedy identity over prompt + generated tokens, then a
    step at context ~1000 over a seeded synthetic KV prefix."""
    cfg = DEEPSEEK_R1_1P5B
    blob, views = full_weights
    om = orc.OracleModel(cfg, views, kinds={n: "w8" for n in ALL_LINEAR})
    s = ModelSession(cfg)
    s.load_blobs("f32", blob, all_linear_w8=True)
    assert s.uses_persistent_kernel()

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    worst, mm = check_stream(step, om, synthetic.prompt_tokens(cfg, 17, 32), 1e-3, n_greedy=64)
    print(f"1.5B int8: max rel logit err {worst:.3e}, smallest margin {mm:.3e}")
    rng = np.random.default_rng(5)
    pos = 1000
    for b in range(2 * cfg.n_layers):
        pre = rng.standard_normal((cfg.kv_heads, pos, cfg.head_dim)).astype(np.float32)
        om.kv[b][:, :pos] = pre
        s.kv_upload(b, om.kv[b], 0, pos)
    s.position_ = pos
    om.position = pos
    check_stream(step, om, [11, 12, 13], 1e-3)
    assert s.position() == pos + 3
    # the last 64 of the 256 steps that grow the context to 1024: the device loop
    # (device argmax, no host round trip) against the checker's free-running ids
    pos = cfg.max_len - 64
    s.position_ = pos
    om.position = pos
    tok, want = 4242, []
    for _ in range(64):
        tok = greedy_sample(om.decode(int(tok)))
        want.append(tok)
    got = [int(t) for t in s.generate(4242, 64)]
    assert got == want
    assert s.position() == cfg.max_len
    # dense prefill of a 128-token prompt, then 16 greedy steps, against the checker
    om.position = 0
    prompt = synthetic.prompt_tokens(cfg, 23, 128)
    for t in prompt:
        want_last = om.decode(int(t))
    s.prefill(prompt, dense=True)
    assert maxrel(s.logits_data(), want_last) < 1e-3
    check_stream(step, om, [greedy_sample(want_last)], 1e-3, n_greedy=16)
    s.close()


def _one_ulp_off(views):
    """The same tensors with every embedding value one or two ulp larger."""
    v = dict(views)
    v[("embed", -1)] = (views[("embed", -1)] * np.float32(1 + 2e-7)).astype(np.float32)
    return v


def test_1p5b_w8a8_prefill_rows_and_decode_steps(full_weights):
    """The w8a8 arithmetic at the 1.5B shapes, every linear layer int8 (q/k/v with their bias are
    the QuantizedAddMMOp form): a 48-row prefill with one activation scale per projection over
    all rows, then decode steps of one row each.

    At these widths the w8a8 graphs are chaotic in the last bit: one activation that rounds to
    the other level perturbs the next projection's input by about 1e-3, which moves a few
    percent of ITS roundings, and after three or four projections the two computations round
    independently (the weight-only graphs move by 2e-6 under the same change).  On the CPU
    alone, the checker's logits for an embedding table one ulp off differ from its logits for
    the original by nothing when no rounding happens to flip, and otherwise by 1.5e-2 after one
    layer, 3e-2 after two and 1.2e-1 at full depth: the distance of two computations that round
    independently, which is at most the quantisation noise of each.  That noise (the w8a8
    checker against the weight-only checker on the same input) is the yardstick: the device
    must be within twice it, at two layers and at 28; the checker's own one-ulp distance is
    printed beside it."""
    kinds = {n: "w8q" for n in ALL_LINEAR}
    for cfg, views, blob in ((DEEPSEEK_R1_1P5B.with_(name="r1_two_layers", n_layers=2, vocab=32768), None, None),
                             (DEEPSEEK_R1_1P5B,) + tuple(reversed(full_weights))):
        if views is None:
            blob, views = synthetic.make_f32_blob(cfg, 77)
        quant = {k: orc.quantize_per_channel(W, 8) for k, W in views.items() if k[0] in ALL_LINEAR}
        om = orc.OracleModel(cfg, views, kinds=kinds, quantised=quant)
        prompt = [int(t) for t in synthetic.prompt_tokens(cfg, 19, 48)]
        want = om.prefill(prompt)
        itself = maxrel(orc.OracleModel(cfg, _one_ulp_off(views), kinds=kinds, quantised=quant).prefill(prompt), want)
        noise = maxrel(want, orc.OracleModel(cfg, views, kinds={n: "w8" for n in ALL_LINEAR}, quantised=quant).prefill(prompt))
        s = ModelSession(cfg)
        s.load_blobs("f32", blob, all_linear_w8=True)
        s.set_activation_int8(True)
        got = s.prefill_rows(prompt, 0, all_rows=True)
        rows = maxrel(got, want)
        tok, step = greedy_sample(want[-1]), 0.0
        for _ in range(4):
            s.decode(tok)
            w = om.decode(tok)
            step = max(step, maxrel(s.logits_data(), w))
            tok = greedy_sample(w)
        print(f"{cfg.name} w8a8: prefill max rel {rows:.3e}, decode {step:.3e}; quantisation noise of the checker "
              f"{noise:.3e}, the checker against itself one ulp off {itself:.3e}; {s.last_ms():.2f} ms for the last "
              f"decode step")
        assert rows < 2 * noise and step < 2 * noise, (rows, step, noise)
        s.close()


def test_qwen3_8b_shapes_int4_group128_at_context_4k():
    """Two layers of the Qwen3-8B shapes (hidden 4096, 32 q / 8 kv heads, FFN
    12288, QK-norm, vocab 151936), int4 group-128, three steps at context ~4090
    over a seeded cache prefix: logits within 2e-2 and the same argmax."""
    from buddy_mlir_b200 import QWEN3_8B
    cfg = QWEN3_8B.with_(name="qwen3_8b_2l", n_layers=2)
    blob, views = synthetic.make_f32_blob(cfg, 31)
    om = orc.OracleModel(cfg, views, kinds={n: "w4g" for n in ALL_LINEAR}, group=128)
    s = ModelSession(cfg)
    s.load_tensors(views, quantize_to="w4", group=128)
    rng = np.random.default_rng(6)
    pos = cfg.max_len - 6
    for b in range(2 * cfg.n_layers):
        om.kv[b][:, :pos] = rng.standard_normal((cfg.kv_heads, pos, cfg.head_dim)).astype(np.float32)
        s.kv_upload(b, om.kv[b], 0, pos)
    s.position_ = pos
    om.position = pos

    def step(t):
        s.decode(t)
        return s.logits_data().copy()
    worst, mm = check_stream(step, om, [101, 202, 303], 2e-2)
    print(f"8B-shape int4 g128 at ctx {pos}: max rel logit err {worst:.3e}, smallest margin {mm:.3e}")
    s.close()


# ---- the model entry pair, loaded the way the generated ModelSession loads it ------------
@pytest.mark.parametrize("cfg,variant", [(TINY_QWEN2, "f32"), (TINY_QWEN2, "w8a32")])
def test_prefill_then_decode_through_the_model_entries(cfg, variant):
    """dlopen(RTLD_LOCAL) of the shim, both symbols resolved, prefill of a
    padded prompt, then 16 greedy decode steps: logits and ids equal the
    checker's; the first decode uploads nothing (the cache stayed on the device)."""
    blob, views = synthetic.make_f32_blob(cfg, 41)
    if variant == "w8a32":
        fb, ib = synthetic.split_w8a32(cfg, views, lambda W: orc.quantize_per_channel(W, 8))
        blobs = [fb, ib]
        om = orc.OracleModel(cfg, views, kinds={n: "w8" for n in synthetic.QUANTISED_BY_REFERENCE})
    else:
        blobs = [blob]
        om = orc.OracleModel(cfg, views)
    es = EntrySession(cfg, variant, blobs)
    prompt = synthetic.prompt_tokens(cfg, 9, 12)
    pad = 7
    logits = es.prefill(prompt, pad_id=pad)
    assert logits.shape == (cfg.max_len, cfg.vocab)
    # every row the reference computes: the prompt rows and the pad rows behind them
    for i in range(cfg.max_len):
        want = om.decode(int(prompt[i]) if i < len(prompt) else pad)
        assert maxrel(logits[i], want) < 1e-3
        assert greedy_sample(logits[i]) == greedy_sample(want)
    for b in range(2 * cfg.n_layers):
        assert maxrel(es.kv[b][0], om.kv[b]) < 1e-4
    om.position = len(prompt)
    assert es.position_ == len(prompt)
    tok = greedy_sample(es.logits)
    for i in range(16):
        es.decode(tok, check_alias=True)
        want = om.decode(tok)
        assert maxrel(es.logits, want) < 1e-3
        assert greedy_sample(es.logits) == greedy_sample(want)
        tok = greedy_sample(want)
    es.close()


def test_prefill_entry_skips_pad_rows_on_request(monkeypatch):
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 43)
    om = orc.OracleModel(cfg, views)
    es = EntrySession(cfg, "f32", [blob])
    prompt = synthetic.prompt_tokens(cfg, 10, 9)
    monkeypatch.setenv("BUDDY_B200_PREFILL_PAD", "7")
    logits = es.prefill(prompt, pad_id=7)
    for i in range(len(prompt)):
        assert maxrel(logits[i], om.decode(int(prompt[i]))) < 1e-3
    assert not logits[len(prompt):].any()
    es.decode(5)
    assert maxrel(es.logits, om.decode(5)) < 1e-3
    es.close()


def test_model_entry_tells_sequences_with_aligned_positions_apart():
    """The reference entry is stateless.  A second sequence whose prompt is as
    long as the first one's final position, prefilled on the CPU into the same
    host buffers, must be decoded against ITS cache, not the previous one's."""
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 44)
    es = EntrySession(cfg, "f32", [blob])
    om = orc.OracleModel(cfg, views)
    for t in synthetic.prompt_tokens(cfg, 1, 10):
        es.decode(int(t))
        om.decode(int(t))
    assert es.position_ == 10
    # sequence two: ten other tokens, "prefilled" by the checker into the host buffers
    om2 = orc.OracleModel(cfg, views)
    for t in synthetic.prompt_tokens(cfg, 2, 10):
        om2.decode(int(t))
    for b in range(2 * cfg.n_layers):
        es.kv[b][0, :, :10] = om2.kv[b][:, :10]
    es.position_ = 10                     # same position as where sequence one stopped
    es.decode(33)
    assert maxrel(es.logits, om2.decode(33)) < 1e-3
    es.close()
