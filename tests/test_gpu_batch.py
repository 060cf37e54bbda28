"""Batched decode over the paged KV cache: every sequence of the batch against
the CPU restatement run on that sequence alone (contiguous cache).  Logits
within 1e-3, greedy tokens identical."""
import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import TINY_MEGA, TINY_QWEN2, TINY_QWEN3, _lib, synthetic
from buddy_mlir_b200.session import BatchSession, ModelSession, greedy_sample

pytestmark = pytest.mark.gpu
ALL_LINEAR = ("q", "k", "v", "o", "gate", "up", "down", "lm_head")


def maxrel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


@pytest.mark.parametrize("cfg,quant", [(TINY_MEGA, "w8"), (TINY_QWEN2, "w8"), (TINY_QWEN3, "w8"), (TINY_QWEN2, None)])
def test_batched_decode_matches_per_sequence_checker(cfg, quant):
    _, views = synthetic.make_f32_blob(cfg, 61)
    kinds = {n: "w8" for n in ALL_LINEAR} if quant else None
    s = ModelSession(cfg)
    s.load_tensors(views, quantize_to=quant)
    page = 8
    bs = BatchSession(s, max_seqs=6, page_size=page, n_pages=40, max_context=cfg.max_len)
    rng = np.random.default_rng(3)
    lengths = [3, 17, 8, 30, 1]                 # ragged prompts: pages fill unevenly
    shared = None
    oms, seqs, toks = [], [], []
    for i, n in enumerate(lengths):
        om = orc.OracleModel(cfg, views, kinds=kinds)
        prompt = rng.integers(0, cfg.vocab, n)
        for t in prompt:
            want = om.decode(int(t))
        q = bs.add()
        got, nxt = bs.prefill(q, prompt)
        assert maxrel(got, want) < 1e-3 and nxt == greedy_sample(want)
        assert bs.length(q) == n
        oms.append(om)
        seqs.append(q)
        toks.append(nxt)
    used = sum((n + page - 1) // page for n in lengths)
    assert bs.free_pages() == 40 - used
    for step in range(10):
        logits, nxt = bs.decode(seqs, toks)
        for i, om in enumerate(oms):
            want = om.decode(int(toks[i]))
            assert maxrel(logits[i], want) < 1e-3, (step, i)
            assert int(nxt[i]) == greedy_sample(want)
        toks = [int(t) for t in nxt]
    # a subset of the batch, in another order
    sub = [seqs[3], seqs[0]]
    logits, nxt = bs.decode(sub, [toks[3], toks[0]])
    assert maxrel(logits[0], oms[3].decode(toks[3])) < 1e-3
    assert maxrel(logits[1], oms[0].decode(toks[0])) < 1e-3
    # pages of a removed sequence are handed out again
    before = bs.free_pages()
    bs.remove(seqs[1])
    assert bs.free_pages() > before
    q = bs.add()
    om = orc.OracleModel(cfg, views, kinds=kinds)
    prompt = rng.integers(0, cfg.vocab, 21)
    for t in prompt:
        want = om.decode(int(t))
    got, _ = bs.prefill(q, prompt)
    assert maxrel(got, want) < 1e-3
    bs.close()
    s.close()


@pytest.mark.parametrize("cfg,chunks", [(TINY_MEGA, (70, 66, 5)), (TINY_QWEN2, (70, 40)), (TINY_QWEN3, (93, 20))])
def test_long_prefill_chunks_take_the_tiled_attention(cfg, chunks):
    """Chunks of 64 rows and more of one sequence run the attention tiled over
    query rows through the block table (first chunk from position 0, later ones on
    top of the pages already filled, ragged last tiles); decode then continues."""
    _, views = synthetic.make_f32_blob(cfg, 62)
    kinds = {n: "w8" for n in ALL_LINEAR}
    s = ModelSession(cfg)
    s.load_tensors(views, quantize_to="w8")
    bs = BatchSession(s, max_seqs=2, page_size=8, n_pages=40, max_context=cfg.max_len)
    om = orc.OracleModel(cfg, views, kinds=kinds)
    rng = np.random.default_rng(5)
    q = bs.add()
    for n in chunks:
        prompt = rng.integers(0, cfg.vocab, n)
        for t in prompt:
            want = om.decode(int(t))
        got, nxt = bs.prefill(q, prompt)
        assert maxrel(got, want) < 1e-3 and nxt == greedy_sample(want)
    tok = nxt
    for _ in range(6):
        logits, nx = bs.decode([q], [tok])
        want = om.decode(int(tok))
        assert maxrel(logits[0], want) < 1e-3 and int(nx[0]) == greedy_sample(want)
        tok = int(nx[0])
    bs.close()
    s.close()


def test_batch_limits_are_reported():
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 62)
    s = ModelSession(cfg)
    s.load_tensors(views, quantize_to="w8")
    bs = BatchSession(s, max_seqs=2, page_size=4, n_pages=3, max_context=16)
    a, b = bs.add(), bs.add()
    with pytest.raises(_lib.B200Error):
        bs.add()                                   # no sequence slot left
    bs.prefill(a, np.arange(8))                    # two pages
    with pytest.raises(_lib.B200Error):
        bs.prefill(b, np.arange(8))                # the pool has one page left
    with pytest.raises(_lib.B200Error):
        bs.prefill(a, np.arange(12))               # beyond max_context
    with pytest.raises(_lib.B200Error):
        bs.decode([a, a], [1, 2])                  # a sequence listed twice
    bs.close()
    s.close()
