"""Tensor-parallel decode bench (bench.py --gpus N, N > 1; this file sits beside
bench.py and is not part of the package): the Qwen3-8B architecture with int4
group-128 weights, context 4096, one rank per GPU.

Sharding follows buddy-mlir's tensor-parallel example
(examples/BuddyTensorParallel/buddy-deepseek-r1-distributed.cpp:521-617):
column-parallel q/k/v/gate/up, row-parallel o/down with a sum over ranks after
each (NCCL all-reduce over NVLink instead of MPI_Sendrecv), vocab-sharded
lm_head (all-gather of the logits shards).  Strong scaling: the model is
fixed, every rank holds 1/N of the weights and of the KV heads.

Outside the timed region the same run checks the sharded path against the CPU
checker: two layers of the same shapes (hidden 4096, 32 q / 8 kv heads, FFN
12288, QK-norm, vocab 151936; int4 group-128) are sharded over the N ranks,
four steps are decoded, and rank 0 compares logits and argmax with the
unsharded checker ("parity" in the JSON line; a mismatch exits non-zero).

`run_reference` is `bench.py --impl reference --gpus N`: the CPU checker on
the same Qwen3-8B int4 configuration, all host threads, rank 0 only.
"""
import ctypes as C
import json
import os
import time

import numpy as np

import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from buddy_mlir_b200 import _lib  # noqa: E402
from buddy_mlir_b200.config import QWEN3_8B  # noqa: E402
from buddy_mlir_b200.session import ModelSession  # noqa: E402
from buddy_mlir_b200.synthetic import tensor_list, inv_freq, make_f32_blob  # noqa: E402

ALL_LINEAR = ("q", "k", "v", "o", "gate", "up", "down", "lm_head")
PARITY_TOL = 2e-2   # max relative logit error, int4 (the tolerance of the int4 model tests)

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


def workload_config(cfg, start, warmup, world):
    return {"workload": "qwen3-8b architecture, int4 group-128 (zero-point 8, f16 scales) "
                        "weight-only, f32 activations, f32 KV cache (294,912 B per position), "
                        "batch 1, greedy decode",
            "context": f"{start + warmup}..{cfg.max_len}", "tp": world,
            "l2": "inputs larger than L2 (3.9 GB of weights per step across ranks)",
            "weights": "seeded N(0,0.02) block, tiled"}


def parity_leg(lib, rank, world, dist):
    """Two layers of the Qwen3-8B shapes sharded over the ranks, four steps near
    the end of a seeded 4k cache, against the unsharded CPU checker on rank 0."""
    import torch
    cfg = QWEN3_8B.with_(name="qwen3_8b_2l", n_layers=2)
    _, views = make_f32_blob(cfg, 31)
    s = ModelSession(cfg, rank, world)
    s.load_tensors(views, quantize_to="w4", group=128)
    pos = cfg.max_len - 8
    rng = np.random.default_rng(6)
    pre = [rng.standard_normal((cfg.kv_heads, pos, cfg.head_dim)).astype(np.float32)
           for _ in range(2 * cfg.n_layers)]
    full = np.zeros((cfg.kv_heads, cfg.max_len, cfg.head_dim), dtype=np.float32)
    for b in range(2 * cfg.n_layers):
        full[:, :pos] = pre[b]
        s.kv_upload(b, full, 0, pos)
    om = None
    if rank == 0:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as orc
        om = orc.OracleModel(cfg, views, kinds={n: "w4g" for n in ALL_LINEAR}, group=128)
        for b in range(2 * cfg.n_layers):
            om.kv[b][:, :pos] = pre[b]
        om.position = pos
    s.position_ = pos
    tok, worst, equal = 101, 0.0, True
    for _ in range(4):
        s.decode(tok)
        got = s.logits_data()
        if rank == 0:
            want = om.decode(tok)
            worst = max(worst, float(np.abs(got - want).max() / np.abs(want).max()))
            equal = equal and int(np.argmax(got)) == int(np.argmax(want))
            tok = int(np.argmax(want))
        if world > 1:
            t = torch.tensor([tok], device="cuda")
            dist.broadcast(t, src=0)
            tok = int(t.item())
    kind = s.tp_sum_kind()
    if world > 1:
        dist.barrier()
    s.close()
    return {"max_rel": worst, "tokens_equal": bool(equal), "tp_sum_kind": kind, "tolerance": PARITY_TOL,
            "model": "2 layers of the qwen3-8b shapes, int4 group-128, 4 steps at context 4088..4091, "
                     "against the unsharded CPU checker"}


def run_reference(args):
    """bench.py --impl reference --gpus N (N > 1): the CPU checker on the Qwen3-8B int4
    configuration, every host thread, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)   # torchrun exports 1
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as orc
    cfg = QWEN3_8B
    steps, warmup = args.steps, args.warmup
    start = cfg.max_len - steps - warmup
    if start < 0:
        raise SystemExit("--steps + --warmup must be <= 4096")
    om = orc.OracleModel(cfg, TiledWeights(cfg, 20260101), kinds={n: "w4g" for n in ALL_LINEAR}, group=128)
    rng = np.random.default_rng(5)
    pre = rng.standard_normal((cfg.kv_heads, start, cfg.head_dim)).astype(np.float32)
    for b in range(2 * cfg.n_layers):
        om.kv[b][:, :start] = pre
    om.position = start
    tok = 11
    for _ in range(warmup):
        tok = int(np.argmax(om.decode(tok)))
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = int(np.argmax(om.decode(tok)))
    dt = time.perf_counter() - t0
    v = steps / dt
    cores = orc.lib().orc_num_threads()
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": 1000.0 * dt / steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 activations, int4 group-128 weights",
        "data": "synthetic", "config": workload_config(cfg, start, warmup, args.gpus),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} decode steps, context {start + warmup}..{cfg.max_len}"},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def run(args, ClockSampler, peaks):
    import torch
    import torch.distributed as dist
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

    # parity of the sharded path, outside the timed region (needs the communicator: below)
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
    parity = parity_leg(lib, rank, world, dist)
    s = build(rank, world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.b200_launch_count()
    ms = _time_generate(s, steps, warmup, start, dist if world > 1 else None)
    launches = lib.b200_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    value = steps / (ms / 1000.0)
    # end to end: the host drives every step through the public call (token id in, greedy
    # token id back to host memory); the logits stay sharded on the devices
    s.position_ = start
    tok = 11
    for _ in range(warmup):
        tok = s.decode_greedy(tok)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = s.decode_greedy(tok)
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
                "config": dict(workload_config(cfg, start, warmup, world),
                               tp1_tokens_per_s_same_run=tp1,
                               collectives=("2 sums of 16 KB per layer by peer stores from the GEMV epilogue over NVLink "
                                            "(tagged pairs, no collective library) + one (value, index) pair per rank "
                                            "for the greedy token, also by peer stores")
                               if s.tp_sum_kind() == 2 else
                               "2 NCCL all-reduce of 16 KB per layer + 1 all-gather of logits"),
                "parity": parity,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                             "frac": achieved / hbm, "traffic": None, "peak_source": which,
                             "kernel": "per-rank decode step (CUDA graph replay), bytes per rank",
                             "bytes_per_step_per_rank": step_bytes},
                "e2e": {"value": steps / float(e2e_dt.item()), "unit": "tokens/s",
                        "h2d_bytes_per_step": 16 * world, "d2h_bytes_per_step": 32 * world,
                        "result": "greedy token id per step (device argmax over the vocabulary shards)"},
                "gpu_launches": int(launches) * world, "kernels_per_step": int(launches // steps),
                "clocks": clocks}
        print(json.dumps(line))
    bad = rank == 0 and not (parity["tokens_equal"] and parity["max_rel"] < PARITY_TOL)
    if world > 1:
        dist.barrier()   # nobody unmaps its staging buffer while a peer may still store into it
    s.close()
    if world > 1:
        lib.b200_tp_shutdown()
        dist.barrier()
        dist.destroy_process_group()
    if bad:
        raise SystemExit(f"tensor-parallel parity failed: {parity}")
