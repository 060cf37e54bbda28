"""The ModelSession that buddy-mlir's gen_session.py generates, for every variant of
gen_config.py:37-71 and for the tiered-cache and packed-decode specs, compiled unmodified
behind the reference's runGeneration (oracle/_ref/session_host_<flavour>), over the matching
model-entry shim of this library -- on a machine WITHOUT a GPU.  The library then refuses
every call (it has no CPU path), the shim hands back zero logits and the reason, and the
reference's host code must come through all of it: dlopen, every dlsym it performs (one
symbol pair per cache size for the tiered spec), the weight files with the sizes the
generated code expects, the prefill and decode ABI structs with their ownership rules
(results the session frees, results that alias its state, results it passes in pre-allocated),
and its destructors.  glibc's heap checks are on (MALLOC_CHECK_=3): a double free or a write
past a result buffer aborts the host.  The numerical side of the same binaries is the GPU test
tests/test_gpu_session_host.py."""
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import TINY_QWEN2, gen_model_entry, synthetic

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FLAVOURS = ("f32", "f16", "bf16", "w8a32", "w8a8", "w8a16", "w4a16", "f32_tiered", "f32_packed")


def weight_files(flavour, cfg, blob, views, d):
    v = flavour.split("_")[0]
    half = lambda bits: (lambda W: orc.quantize_per_channel_half(W, bits))   # noqa: E731
    if v == "f32":
        arrs = [blob] + ([synthetic.pack_decode_blob(cfg, blob)] if flavour == "f32_packed" else [])
    elif v == "f16":
        arrs = [blob.astype(np.float16)]
    elif v == "bf16":
        arrs = [synthetic.to_bf16(blob)]
    elif v in ("w8a32", "w8a8"):
        arrs = list(synthetic.split_w8a32(cfg, views, lambda W: orc.quantize_per_channel(W, 8)))
    elif v == "w8a16":
        arrs = list(synthetic.split_w8a16(cfg, views, half(8)))
    else:
        arrs = list(synthetic.split_w4a16(cfg, views, half(4)))
    paths = []
    for i, a in enumerate(arrs):
        p = os.path.join(d, f"{flavour}_{i}.data")
        a.tofile(p)
        paths.append(p)
    return ",".join(paths)


def shim_of(flavour, cfg):
    v = flavour.split("_")[0]
    name = gen_model_entry.shim_name(cfg, v, False, flavour == "f32_packed",
                                     gen_model_entry.TINY_TIERS if flavour == "f32_tiered" else None)
    return os.path.join(ROOT, "buddy_mlir_b200", name)


@pytest.mark.parametrize("flavour", FLAVOURS)
def test_generated_session_comes_through_the_shim_without_a_gpu(tmp_path, flavour):
    import torch
    if torch.cuda.is_available():
        pytest.skip("with a GPU present the numerical test covers this path")
    cfg = TINY_QWEN2
    host = os.path.join(ROOT, "oracle", "_ref", f"session_host_{flavour}")
    shim = shim_of(flavour, cfg)
    if not (os.path.exists(host) and os.path.exists(shim)):
        pytest.skip("the generated sessions are built where a buddy-mlir checkout is present")
    blob, views = synthetic.make_f32_blob(cfg, 5)
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("".join(f"t{i}\n" for i in range(cfg.vocab)))
    # 40 prompt ids: the tiered session starts in its second cache size and moves up while decoding
    prompt = " ".join(str(int(t)) for t in synthetic.prompt_tokens(cfg, 3, 40))
    env = dict(os.environ, MALLOC_CHECK_="3", MALLOC_PERTURB_="165")
    out = subprocess.run([host, shim, weight_files(flavour, cfg, blob, views, str(tmp_path)), str(vocab), "70", "0", prompt],
                         capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, (out.returncode, out.stderr[-1500:])
    line = [l for l in out.stdout.splitlines() if l.startswith("[ids] ")][-1]
    ids = [int(x) for x in line[len("[ids] "):].split()]
    assert len(ids) == 70 - 40 + 1                       # the first token and 30 decode steps
    assert "no CUDA device" in out.stderr and ids == [0] * len(ids)


@pytest.mark.parametrize("flavour", ["f32", "w8a32", "w8a8", "f32_tiered", "f32_packed"])
def test_generated_session_over_the_same_shim_source_with_the_checkers_numbers(tmp_path, flavour):
    """The same generated sessions, the same shim SOURCE, but linked against
    oracle/oracle_forward_backend.cpp, which implements the b200_forward_* contract with the CPU
    restatement: the whole host side of the model entry -- the reference's session, its
    generation loop and sampler, and this library's shim with its result-ownership rules
    (allocated, aliased, filled in place; the tiered session moving its cache between sizes
    while it decodes) -- runs with real numbers on a machine without a GPU, and the ids must be
    the restatement's own greedy ids.  (w8a8: the prefill scales over all rows of the padded
    token container.)"""
    cfg = TINY_QWEN2
    host = os.path.join(ROOT, "oracle", "_ref", f"session_host_{flavour}")
    shim = os.path.join(ROOT, "oracle", "_build", "shims", os.path.basename(shim_of(flavour, cfg)))
    if not (os.path.exists(host) and os.path.exists(shim)):
        pytest.skip("the generated sessions are built where a buddy-mlir checkout is present")
    blob, views = synthetic.make_f32_blob(cfg, 93)
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("".join(f"t{i}\n" for i in range(cfg.vocab)))
    prompt = [int(t) for t in synthetic.prompt_tokens(cfg, 15, 20)]
    n_new = 48                     # the tiered session moves from 32 rows to 64 and on to 128
    kind = {"w8a32": "w8", "w8a8": "w8q"}.get(flavour)
    om = orc.OracleModel(cfg, views, kinds={n: kind for n in synthetic.QUANTISED_BY_REFERENCE} if kind else None)
    if flavour == "w8a8":          # one activation scale per projection over the whole padded container
        logits = om.prefill(prompt + [0] * (cfg.max_len - len(prompt)))[len(prompt) - 1]
        om.position = len(prompt)
    else:
        for t in prompt:
            logits = om.decode(t)
    want = [int(np.argmax(logits))]
    for _ in range(n_new):
        want.append(int(np.argmax(om.decode(want[-1]))))
    env = dict(os.environ, MALLOC_CHECK_="3", MALLOC_PERTURB_="165")
    out = subprocess.run([host, shim, weight_files(flavour, cfg, blob, views, str(tmp_path)), str(vocab),
                          str(len(prompt) + n_new), "0", " ".join(str(t) for t in prompt)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, (out.returncode, out.stderr[-1500:])
    assert "failed" not in out.stderr, out.stderr[-1500:]
    line = [l for l in out.stdout.splitlines() if l.startswith("[ids] ")][-1]
    assert [int(x) for x in line[len("[ids] "):].split()] == want
