"""The buddy-cli runner plugin: loaded the way buddy-cli loads a runner
(dlopen + buddy_create_inference_runner_v1, tools/buddy-cli/buddy-cli.cpp:195-252)
by a small host built from the reference's own headers, it runs the
reference's generation loop (runtime/llm/TextGeneration.cpp:157-277) over the
device session; the generated ids must be the CPU checker's greedy ids."""
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import TINY_QWEN2, synthetic
from buddy_mlir_b200.session import greedy_sample

pytestmark = pytest.mark.gpu


def margin(logits):
    top2 = np.partition(logits, -2)[-2:]
    return float(top2[1] - top2[0])
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "oracle", "_ref", "runner_host")
PLUGIN = os.path.join(ROOT, "buddy_mlir_b200", "libbuddy_b200_runner.so")


@pytest.mark.skipif(not (os.path.exists(HOST) and os.path.exists(PLUGIN)),
                    reason="the plugin and its host are built where a buddy-mlir checkout is present")
@pytest.mark.parametrize("variant", ["f32", "w8a32", "w8a8"])
def test_runner_plugin_generates_the_checkers_tokens(tmp_path, variant):
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 91)
    if variant in ("w8a32", "w8a8"):     # the same two files; w8a8 quantises the activations as well
        fb, ib = synthetic.split_w8a32(cfg, views, lambda W: orc.quantize_per_channel(W, 8))
        fpath, ipath = tmp_path / f"arg0-{variant}-f32.data", tmp_path / f"arg0-{variant}-i8.data"
        fb.tofile(fpath)
        ib.tofile(ipath)
        weights = f"{fpath},{ipath}"
        kind = "w8" if variant == "w8a32" else "w8q"
        om = orc.OracleModel(cfg, views, kinds={n: kind for n in synthetic.QUANTISED_BY_REFERENCE})
    else:
        fpath = tmp_path / "arg0.data"
        blob.tofile(fpath)
        weights = str(fpath)
        om = orc.OracleModel(cfg, views)
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("".join(f"t{i}\n" for i in range(cfg.vocab)))
    prompt = synthetic.prompt_tokens(cfg, 13, 20)
    max_new = len(prompt) + 12           # runGeneration: maxSteps = maxNewTokens - promptTokens
    # the checker's greedy continuation (the prefill graph: a w8a8 projection scales over all rows)
    logits = om.prefill([int(t) for t in prompt])[-1]
    want = [greedy_sample(logits)]
    sure = 1 if variant != "w8a8" or margin(logits) > 3e-2 * float(np.abs(logits).max()) else 0
    for _ in range(12):
        logits = om.decode(want[-1])
        want.append(greedy_sample(logits))
        # w8a8: a rounding flip may move the logits by up to the quantisation noise, so the ids are
        # compared up to the first step whose top-2 margin is smaller than that
        if sure == len(want) - 1 and (variant != "w8a8" or margin(logits) > 3e-2 * float(np.abs(logits).max())):
            sure = len(want)
    # the first run walks the blobs and writes the pack cache, the second one loads it
    cache = tmp_path / "weights.b2pack"
    env = dict(os.environ, BUDDY_B200_MODEL="tiny_qwen2", BUDDY_B200_PACK_CACHE=str(cache))
    if variant == "w8a8":
        env["BUDDY_B200_VARIANT"] = "w8a8"
    for run in range(2):
        out = subprocess.run([HOST, PLUGIN, weights, str(vocab), str(max_new), " ".join(str(int(t)) for t in prompt)],
                             env=env, capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, out.stderr[-2000:]
        line = [l for l in out.stdout.splitlines() if l.startswith("[ids] ")][-1]
        got = [int(x) for x in line[len("[ids] "):].split()]
        assert len(got) == len(want) and got[:sure] == want[:sure], run
        assert cache.exists() and "pack cache" not in out.stderr
