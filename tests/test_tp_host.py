"""Tensor-parallel sharding logic on the CPU: the sharded decode step equals
the unsharded one, in one process and as two gloo ranks."""
import os
import socket
import sys

import numpy as np
import pytest

import oracle_lib as orc
import tp_oracle
from buddy_mlir_b200 import TINY_QWEN2, TINY_QWEN3, synthetic

ALL = ("q", "k", "v", "o", "gate", "up", "down", "lm_head")


@pytest.mark.parametrize("cfg,kind,tol", [(TINY_QWEN2, "f32", 1e-5), (TINY_QWEN2, "w8", 1e-5),
                                          (TINY_QWEN3, "w4g", 1e-5)])
def test_sharded_step_equals_unsharded(cfg, kind, tol):
    _, views = synthetic.make_f32_blob(cfg, 31)
    kinds = {n: kind for n in ALL}
    full = orc.OracleModel(cfg, views, kinds=kinds, group=128)
    ranks = [tp_oracle.TPRank(cfg, views, kinds, r, 2, group=128) for r in range(2)]
    comm = tp_oracle.LocalComm(2)
    for pos, tok in enumerate(synthetic.prompt_tokens(cfg, 2, 6)):
        want = full.decode(int(tok))
        got = tp_oracle.tp_decode_step(ranks, comm, int(tok), pos)
        assert np.abs(got - want).max() / np.abs(want).max() < tol
        assert int(np.argmax(got)) == int(np.argmax(want))


def _gloo_worker(rank, size, port, out_path):
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=size)

    class GlooComm:
        def allreduce(self, parts):
            t = torch.from_numpy(parts[0].copy())
            dist.all_reduce(t)
            return [t.numpy()]

        def allgather(self, parts):
            t = torch.from_numpy(parts[0].copy())
            outs = [torch.empty_like(t) for _ in range(size)]
            dist.all_gather(outs, t)
            return [np.concatenate([o.numpy() for o in outs])]

    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 31)
    kinds = {n: "w8" for n in ALL}
    me = tp_oracle.TPRank(cfg, views, kinds, rank, size)
    logits = []
    for pos, tok in enumerate(synthetic.prompt_tokens(cfg, 2, 4)):
        logits.append(tp_oracle.tp_decode_step([me], GlooComm(), int(tok), pos))
    if rank == 0:
        np.save(out_path, np.stack(logits))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "logits.npy")
    mp.spawn(_gloo_worker, args=(2, port, out), nprocs=2, join=True)
    got = np.load(out)
    cfg = TINY_QWEN2
    _, views = synthetic.make_f32_blob(cfg, 31)
    full = orc.OracleModel(cfg, views, kinds={n: "w8" for n in ALL})
    for pos, tok in enumerate(synthetic.prompt_tokens(cfg, 2, 4)):
        want = full.decode(int(tok))
        assert np.abs(got[pos] - want).max() / np.abs(want).max() < 1e-5
        assert int(np.argmax(got[pos])) == int(np.argmax(want))
