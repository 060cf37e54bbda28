"""Boundary B2 with the reference's own host code: the ModelSession that buddy-mlir's
gen_session.py generates for the small model (compiled unmodified into
oracle/_ref/session_host_<flavour> together with the reference's runGeneration and Sampler)
dlopens the model-entry shim of this library, resolves _mlir_ciface_forward_prefill /
_mlir_ciface_forward_decode by name (one pair per cache size for the tiered spec), reads the
weight files, runs its prefill over the padded token container and its decode loop through the
generated ABI structs.  The ids it generates must be the CPU checker's greedy ids.  Flavours
with f32 arithmetic only: their ids are comparable one to one."""
import os
import subprocess

import pytest

import oracle_lib as orc
from buddy_mlir_b200 import TINY_QWEN2, synthetic
from buddy_mlir_b200.session import greedy_sample
from test_session_hosts import ROOT, shim_of, weight_files

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("flavour", ["f32", "w8a32", "f32_tiered", "f32_packed"])
def test_generated_model_session_runs_over_the_shim(tmp_path, flavour):
    cfg = TINY_QWEN2
    host = os.path.join(ROOT, "oracle", "_ref", f"session_host_{flavour}")
    shim = shim_of(flavour, cfg)
    if not (os.path.exists(host) and os.path.exists(shim)):
        pytest.skip("the generated sessions are built where a buddy-mlir checkout is present")
    blob, views = synthetic.make_f32_blob(cfg, 92)
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("".join(f"t{i}\n" for i in range(cfg.vocab)))
    prompt = synthetic.prompt_tokens(cfg, 14, 20)
    n_new = 48                           # the tiered session moves from 32 rows to 64 and on to 128
    max_new = len(prompt) + n_new        # runGeneration: maxSteps = maxNewTokens - promptTokens
    kinds = {n: "w8" for n in synthetic.QUANTISED_BY_REFERENCE} if flavour == "w8a32" else None
    om = orc.OracleModel(cfg, views, kinds=kinds)
    for t in prompt:
        logits = om.decode(int(t))
    want = [greedy_sample(logits)]
    for _ in range(n_new):
        want.append(greedy_sample(om.decode(want[-1])))
    out = subprocess.run([host, shim, weight_files(flavour, cfg, blob, views, str(tmp_path)), str(vocab), str(max_new),
                          "0", " ".join(str(int(t)) for t in prompt)],
                         capture_output=True, text=True, timeout=300, env=dict(os.environ, MALLOC_CHECK_="3"))
    assert out.returncode == 0, out.stderr[-2000:]
    assert "failed" not in out.stderr, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("[ids] ")][-1]
    got = [int(x) for x in line[len("[ids] "):].split()]
    assert got == want
