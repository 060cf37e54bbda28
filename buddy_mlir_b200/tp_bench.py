"""Tensor-parallel decode bench (bench.py --gpus N, N > 1): the Qwen3-8B
architecture with int4 group-128 weights, context 4096, one rank per GPU.

Sharding follows buddy-mlir's tensor-parallel example
(examples/BuddyTensorParallel/buddy-deepseek-r1-distributed.cpp:521-617):
column-parallel q/k/v/gate/up, row-parallel o/down with a sum over ranks after
each (NCCL all-reduce over NVLink instead of MPI_Sendrecv), vocab-sharded
lm_head (all-gather of the logits shards).  Strong scaling: the model is
fixed, every rank holds 1/N of the weights and of the KV heads.
"""
import ctypes as C
import json
import os
import time

import numpy as np

from . import _lib
from .config import QWEN3_8B
from .session import ModelSession
from .synthetic import tensor_list, inv_freq

METRIC = "decode tokens/s (bs=1, ctx 4k, tensor parallel)"


class TiledWeights:
    """{(name, layer): f32 tensor} generated on demand: one seeded N(0, 0.02)
    block per tensor shape class, tiled (timing does not depend on the values;
    holding 30 GB of distinct random floats per rank would)."""

    def __init__(self, cfg, seed):
        self.cfg = cfg
        self.shapes = {(n, l): s for n, l, s in tensor_list(cfg)}
        rng = np.random.default_rng(seed)
        self.block = (rng.standard_normal(1 << 22).astype(np.float32) * np.float32(0.02))

    def __contains__(self, key):
        return key in self.shapes

    def __getitem__(self, key):
        name, layer = key
        shape = self.shapes[key]
        n = int(np.prod(shape))
        if name == "inv_freq":
            return inv_freq(self.cfg)
        reps = (n + self.block.size - 1) // self.block.size
        start = (hash((name, max(layer, 0))) % 4099) * 7
        a = np.tile(self.block, reps + 1)[start:start + n].copy()
        if name.endswith("norm"):
            a += np.float32(1.0)
        return a.reshape(shape)


def _time_generate(s, steps, warmup, start, dist):
    import torch
    s.position_ = start
    tok = 11
    ids = s.generate(tok, warmup)
    tok = int(ids[-1])
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    s.generate(tok, steps)
    ms = torch.tensor([s.last_ms()], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    torch.cuda.synchronize()
    return float(ms.item())


def run(args):
    import torch
    import torch.distributed as dist
    from bench import ClockSampler, peaks
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    # no in-switch (multicast) reductions: the library's own sums are plain peer stores, and a
    # rank that dies with memory bound to a multicast object can take its peers down
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if world > 1:
        dist.init_process_group("nccl")
    lib = _lib.load()
    cfg = QWEN3_8B
    steps, warmup = args.steps, args.warmup
    start = cfg.max_len - steps - warmup
    if start < 0:
        raise SystemExit("--steps + --warmup must be <= 4096")
    weights = TiledWeights(cfg, 20260101)

    def build(tp_rank, tp_size):
        s = ModelSession(cfg, tp_rank, tp_size)
        s.load_tensors(weights, quantize_to="w4", group=128)
        rng = np.random.default_rng(5)
        pre = np.zeros((cfg.kv_heads, cfg.max_len, cfg.head_dim), dtype=np.float32)
        pre[:, :start] = rng.standard_normal((cfg.kv_heads, start, cfg.head_dim)).astype(np.float32)
        for b in range(2 * cfg.n_layers):
            s.kv_upload(b, pre, 0, start)
        return s

    # reference point inside the same run: the unsharded model on rank 0 alone
    tp1 = None
    if rank == 0:
        s1 = build(0, 1)
        tp1_ms = _time_generate(s1, steps, warmup, start, None)
        tp1 = steps / (tp1_ms / 1000.0)
        s1.close()
    if world > 1:
        dist.barrier()
        uid = np.zeros(128, dtype=np.uint8)
        if rank == 0:
            _lib.check(lib.b200_tp_unique_id(uid.ctypes.data))
        box = [uid.tobytes()]
        dist.broadcast_object_list(box, src=0)
        uid = np.frombuffer(box[0], dtype=np.uint8).copy()
        _lib.check(lib.b200_tp_init(uid.ctypes.data, rank, world))
    s = build(rank, world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.b200_launch_count()
    ms = _time_generate(s, steps, warmup, start, dist if world > 1 else None)
    launches = lib.b200_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    value = steps / (ms / 1000.0)
    # end to end: logits to host memory and host argmax every step (rank 0 drives)
    s.position_ = start
    tok = 11
    for _ in range(warmup):
        s.decode(tok)
        tok = int(np.argmax(s.logits_data()))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        s.decode(tok)
        tok = int(np.argmax(s.logits_data()))
    torch.cuda.synchronize()
    e2e_dt = torch.tensor([time.perf_counter() - t0], device="cuda")
    if world > 1:
        dist.all_reduce(e2e_dt, op=dist.ReduceOp.MAX)
    step_bytes = s.step_bytes(cfg.max_len - steps // 2)
    if rank == 0:
        hbm, which = peaks()
        achieved = step_bytes / (ms / steps) / 1e6
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None,
                "dtype": "f32 activations, int4 group-128 weights", "data": "synthetic",
                "config": {"workload": "qwen3-8b architecture, int4 group-128 (zero-point 8, f16 scales) "
                                       "weight-only, f32 activations and KV, batch 1, greedy decode",
                           "context": f"{start + warmup}..{cfg.max_len}", "tp": world,
                           "tp1_tokens_per_s_same_run": tp1,
                           "collectives": ("2 sums of 16 KB per layer by peer stores from the GEMV epilogue over NVLink "
                                           "(tagged pairs, no collective library) + 1 NCCL all-gather of logits")
                                          if s.tp_sum_kind() == 2 else
                                          "2 NCCL all-reduce of 16 KB per layer + 1 all-gather of logits",
                           "l2": "inputs larger than L2 (3.9 GB of weights per step across ranks)",
                           "weights": "seeded N(0,0.02) block, tiled"},
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                             "frac": achieved / hbm, "traffic": None, "peak_source": which,
                             "kernel": "per-rank decode step (CUDA graph replay), bytes per rank",
                             "bytes_per_step_per_rank": step_bytes},
                "e2e": {"value": steps / float(e2e_dt.item()), "unit": "tokens/s",
                        "h2d_bytes_per_step": 16 * world, "d2h_bytes_per_step": cfg.vocab * 4 * world},
                "gpu_launches": int(launches) * world, "kernels_per_step": int(launches // steps),
                "clocks": clocks}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()   # nobody unmaps its staging buffer while a peer may still store into it
    s.close()
    if world > 1:
        lib.b200_tp_shutdown()
        dist.barrier()
        dist.destroy_process_group()
