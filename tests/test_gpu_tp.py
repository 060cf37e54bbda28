"""Tensor-parallel decode on 2 GPUs against the unsharded CPU checker.  Needs
two CUDA devices; skipped otherwise."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import numpy as np, torch, torch.distributed as dist
from buddy_mlir_b200 import TINY_QWEN3, _lib, synthetic
from buddy_mlir_b200.session import ModelSession
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")
lib = _lib.load()
uid = np.zeros(128, dtype=np.uint8)
if rank == 0:
    _lib.check(lib.b200_tp_unique_id(uid.ctypes.data))
box = [uid.tobytes()]
dist.broadcast_object_list(box, src=0)
uid = np.frombuffer(box[0], dtype=np.uint8).copy()
_lib.check(lib.b200_tp_init(uid.ctypes.data, rank, world))
cfg = TINY_QWEN3
kind = sys.argv[3]
_, views = synthetic.make_f32_blob(cfg, 31)
s = ModelSession(cfg, rank, world)
s.load_tensors(views, quantize_to=None if kind == "f32" else kind, group=128)
out = []
for tok in synthetic.prompt_tokens(cfg, 2, 6):
    s.decode(int(tok))
    out.append(s.logits_data().copy())
ids = s.generate(int(np.argmax(out[-1])), 8)
if rank == 0:
    np.savez(sys.argv[2], logits=np.stack(out), ids=ids, sum_kind=s.tp_sum_kind())
dist.barrier()
s.close()
lib.b200_tp_shutdown()
dist.destroy_process_group()
'''


def _two_gpus():
    try:
        import torch
        return torch.cuda.device_count() >= 2
    except Exception:
        return False


@pytest.mark.skipif(not _two_gpus(), reason="needs two CUDA devices")
@pytest.mark.parametrize("sum_path", ["peer", "nccl"])
@pytest.mark.parametrize("kind,tol", [("f32", 1e-3), ("w8", 1e-3), ("w4", 2e-2)])
def test_tp2_matches_unsharded_checker(tmp_path, kind, tol, sum_path):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as orc
    from buddy_mlir_b200 import TINY_QWEN3, synthetic
    with socket.socket() as so:
        so.bind(("127.0.0.1", 0))
        port = so.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    out = str(tmp_path / "out.npz")
    # NVLS off: a rank that dies with multicast-bound memory can fault its peers
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    # the sums of the row-parallel projections: peer stores from the GEMV epilogue (default) or NCCL
    env.pop("BUDDY_B200_TP_SUM", None)
    if sum_path == "nccl":
        env["BUDDY_B200_TP_SUM"] = "nccl"
    subprocess.check_call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                           "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port",
                           str(port), str(script), ROOT, out, kind], env=env, timeout=600)
    got = np.load(out)
    assert int(got["sum_kind"]) == (2 if sum_path == "peer" else 1)
    cfg = TINY_QWEN3
    _, views = synthetic.make_f32_blob(cfg, 31)
    okind = {"f32": "f32", "w8": "w8", "w4": "w4g"}[kind]
    full = orc.OracleModel(cfg, views, kinds={n: okind for n in
                                              ("q", "k", "v", "o", "gate", "up", "down", "lm_head")}, group=128)
    tok = None
    for i, t in enumerate(synthetic.prompt_tokens(cfg, 2, 6)):
        want = full.decode(int(t))
        assert np.abs(got["logits"][i] - want).max() / np.abs(want).max() < tol
        assert int(np.argmax(got["logits"][i])) == int(np.argmax(want))
        tok = int(np.argmax(want))
    for nxt in got["ids"]:
        want = full.decode(tok)
        assert int(nxt) == int(np.argmax(want))
        tok = int(nxt)
