"""The timed CPU baseline: the restatement behind buddy-mlir's own generation loop.
oracle/oracle_runner_plugin.cpp is a runner plugin (the ABI buddy-cli loads) whose
session runs the CPU restatement, driven by the reference's runGeneration + Sampler
compiled from the buddy-mlir tree; oracle/runner_host plays buddy-cli.  The ids must be
those of the restatement's own greedy loop, and the reference's statistics must come out."""
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import TINY_QWEN2, synthetic
from buddy_mlir_b200.session import greedy_sample

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "oracle", "_ref", "runner_host")
PLUGIN = os.path.join(ROOT, "oracle", "_ref", "libbuddy_oracle_runner.so")

pytestmark = pytest.mark.skipif(not (os.path.exists(HOST) and os.path.exists(PLUGIN)),
                                reason="built where a buddy-mlir checkout is present (oracle/Makefile)")


def run(tmp_path, blob, prompt, max_new, **env):
    path = tmp_path / "arg0.data"
    blob.tofile(path)
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("x\n")
    out = subprocess.run([HOST, PLUGIN, str(path), str(vocab), str(max_new), " ".join(str(int(t)) for t in prompt)],
                         env=dict(os.environ, ORC_RUNNER_MODEL="tiny_qwen2", **env),
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    ids = [l for l in out.stdout.splitlines() if l.startswith("[ids] ")][-1]
    stats = [l for l in out.stdout.splitlines() if l.startswith("[stats] ")][-1].split()
    return [int(x) for x in ids[len("[ids] "):].split()], dict(zip(stats[1::2], stats[2::2])), out.stderr


@pytest.mark.parametrize("w8", [False, True])
def test_reference_loop_over_the_restatement_gives_its_greedy_ids(tmp_path, w8):
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 92)
    kinds = {n: "w8" for n in ("q", "k", "v", "o", "gate", "up", "down", "lm_head")} if w8 else None
    om = orc.OracleModel(cfg, views, kinds=kinds)
    prompt = synthetic.prompt_tokens(cfg, 14, 9)
    for t in prompt:
        logits = om.decode(int(t))
    want = [greedy_sample(logits)]
    for _ in range(10):
        want.append(greedy_sample(om.decode(want[-1])))
    got, stats, err = run(tmp_path, blob, prompt, len(prompt) + 10, ORC_RUNNER_ALL_LINEAR_W8="1" if w8 else "0")
    assert got == want
    assert int(stats["tokens"]) == len(want) - 1 and float(stats["decode_s"]) > 0    # decode-loop steps
    assert "[Decode]" in err and "tokens/s" in err          # printStats of the reference


def test_seeded_cache_prefix_moves_the_timed_loop_to_a_long_context(tmp_path):
    cfg = TINY_QWEN2
    blob, _ = synthetic.make_f32_blob(cfg, 93)
    prompt = synthetic.prompt_tokens(cfg, 15, 2)
    a, _, _ = run(tmp_path, blob, prompt, len(prompt) + 4)
    b, _, _ = run(tmp_path, blob, prompt, len(prompt) + 4, ORC_RUNNER_KV_PREFIX="100,7")
    assert len(a) == len(b) == 5 and a != b                  # 100 rows of history change the logits
