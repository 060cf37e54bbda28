"""Boundary B2 with the reference's own host code: the ModelSession that buddy-mlir's
gen_session.py generates for the small model (compiled unmodified into oracle/_ref/session_host
together with the reference's runGeneration and Sampler) dlopens the model-entry shim of this
library, resolves _mlir_ciface_forward_prefill / _mlir_ciface_forward_decode by name, reads the
weight file, runs its prefill over the padded token container and its decode loop through the
generated ABI structs.  The ids it generates must be the CPU checker's greedy ids."""
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import TINY_QWEN2, gen_model_entry, synthetic
from buddy_mlir_b200.session import greedy_sample

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "oracle", "_ref", "session_host")
SHIM = os.path.join(ROOT, "buddy_mlir_b200", gen_model_entry.shim_name(TINY_QWEN2, "f32", False))


@pytest.mark.skipif(not (os.path.exists(HOST) and os.path.exists(SHIM)),
                    reason="the generated session is built where a buddy-mlir checkout is present")
def test_generated_model_session_runs_over_the_shim(tmp_path):
    cfg = TINY_QWEN2
    blob, views = synthetic.make_f32_blob(cfg, 92)
    weights = tmp_path / "arg0.data"
    blob.tofile(weights)
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("".join(f"t{i}\n" for i in range(cfg.vocab)))
    prompt = synthetic.prompt_tokens(cfg, 14, 20)
    max_new = len(prompt) + 12           # runGeneration: maxSteps = maxNewTokens - promptTokens
    om = orc.OracleModel(cfg, views)
    for t in prompt:
        logits = om.decode(int(t))
    want = [greedy_sample(logits)]
    for _ in range(12):
        want.append(greedy_sample(om.decode(want[-1])))
    out = subprocess.run([HOST, SHIM, str(weights), str(vocab), str(max_new), "0", " ".join(str(int(t)) for t in prompt)],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "failed" not in out.stderr, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("[ids] ")][-1]
    got = [int(x) for x in line[len("[ids] "):].split()]
    assert got == want
