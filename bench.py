#!/usr/bin/env python
"""Decode-throughput bench of the buddy-mlir decode hot path on B200.

    python bench.py --gpus 1 --steps 256 --warmup 8
    python bench.py --impl reference --steps 64 --warmup 3

N = 1 workload (the configuration the headline metric is quoted on): the
DeepSeek-R1-Distill-Qwen-1.5B architecture with int8 per-output-channel
weight-only quantisation of every linear layer, f32 activations, batch 1,
greedy decode with the KV context growing to 1024 over the timed steps.  A
"step" is one decode token.  Weights are seeded N(0, 0.02); KV rows before the
first timed position are seeded N(0, 1) (no checkpoint, no dataset).

N > 1 workload: the Qwen3-8B architecture with int4 group-128 weights,
context 4096, tensor-parallel over the N GPUs (column-parallel q/k/v/gate/up,
row-parallel o/down with a sum over NVLink peer stores after each, vocab-sharded
lm_head): strong scaling, one rank per GPU; the line carries a `parity` object
(the sharded model against the unsharded CPU checker).

`value` is tokens/s with everything resident in HBM (the device-resident
greedy loop, CUDA events on the session's stream).  `e2e` is the same metric
through the reference-facing entry `_mlir_ciface_forward_decode` with HOST
buffers: token in, logits and the new KV rows back to host memory every step,
greedy argmax on the host as buddy-mlir's runGeneration does.

`--impl reference` times the CPU restatement of buddy-mlir's generated decode
code (oracle/, OpenMP over the same 32-column tiles) on the host cores, same
configuration, driven and timed by buddy-mlir's own runGeneration + Sampler when
the prebuilt runner is present (oracle/_ref); the reference's compiled path
itself cannot be produced without its LLVM toolchain.

Beside the metric, outside the timed region, the N = 1 line reports
`gemv_isolated` (the GEMV sweep) and `dense_path` (the same model's prefill of
2048 tokens, batched decode of 64 sequences over the paged cache, and the
gate|up GEMM at 1024 rows on the tcgen05 path); `--gemv-only`, `--gemm-only`
and `--batch-only` print those alone; `--w8a8-only` prints the w8a8 numbers alone.
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

SEED_W, SEED_KV, SEED_P = 20260101, 5, 17
ALL_LINEAR = ("q", "k", "v", "o", "gate", "up", "down", "lm_head")
METRIC = "decode tokens/s (bs=1, ctx 1k)"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=5)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_step_kernel launch (ncu, full-size
# 1.5B int8 model at context ~1000), and the git blob hash of the kernel source it was captured
# from.  The figure is only reported while the source is still that one.
TRAFFIC = {"bytes": 1717368176, "kernel_source": "buddy_mlir_b200/csrc/mega.cu",
           "git_blob": "fbdb80c4ec6f5ae66337f7c5b248aeed4b7800a5",
           "capture": "ncu --set full --clock-control none -k regex:decode_step -c 1, bench.py --resident-only"}


def git_blob_hash(path):
    import hashlib
    data = open(path, "rb").read()
    return hashlib.sha1(b"blob %d\0" % len(data) + data).hexdigest()


def measured_traffic(persistent):
    if not persistent:
        return None, None
    src = os.path.join(ROOT, TRAFFIC["kernel_source"])
    if not os.path.exists(src) or git_blob_hash(src) != TRAFFIC["git_blob"]:
        return None, "stale: the kernel source changed since the ncu capture"
    return TRAFFIC["bytes"], f"ncu capture of {TRAFFIC['kernel_source']} at git blob {TRAFFIC['git_blob'][:12]}"


def kv_prefix(cfg, n_pos, buffer):
    rng = np.random.default_rng([SEED_KV, buffer])
    a = np.zeros((cfg.kv_heads, cfg.max_len, cfg.head_dim), dtype=np.float32)
    a[:, :n_pos] = rng.standard_normal((cfg.kv_heads, n_pos, cfg.head_dim)).astype(np.float32)
    return a


def plan_positions(cfg, steps, warmup):
    if steps + warmup > cfg.max_len:
        raise SystemExit(f"--steps + --warmup must be <= {cfg.max_len}")
    return cfg.max_len - steps - warmup


# ------------------------------------------------------------------------------
REF_HOST = os.path.join(ROOT, "oracle", "_ref", "runner_host")
REF_LOOP = os.path.join(ROOT, "oracle", "_ref", "libbuddy_oracle_runner.so")


def reference_loop(blob, start, steps, warm):
    """The CPU restatement behind buddy-mlir's own generation loop (runGeneration + Sampler,
    compiled from the reference tree into oracle/_ref/libbuddy_oracle_runner.so and loaded the
    way buddy-cli loads a runner): tokens/s as the reference measures them
    (runtime/llm/TextGeneration.cpp:135-152).  The cache is seeded up to `start`, `warm` prompt
    tokens run as the (untimed) prefill, `steps` decode steps are timed.  None when the
    prebuilt runner is absent or the blob cannot be written."""
    import subprocess
    import tempfile
    if not (os.path.exists(REF_HOST) and os.path.exists(REF_LOOP)):
        return None
    try:
        # the blob file lives in memory-backed storage when there is room for it
        shm = "/dev/shm"
        base = None
        try:
            st = os.statvfs(shm)
            if st.f_bavail * st.f_frsize > blob.nbytes + (1 << 30):
                base = shm
        except OSError:
            pass
        with tempfile.TemporaryDirectory(dir=base) as d:
            path = os.path.join(d, "arg0.data")
            blob.tofile(path)
            vocab = os.path.join(d, "vocab.txt")
            open(vocab, "w").write("x\n")
            env = dict(os.environ, ORC_RUNNER_MODEL="deepseek_r1_1p5b", ORC_RUNNER_ALL_LINEAR_W8="1",
                       ORC_RUNNER_KV_PREFIX=f"{start},{SEED_KV}", OMP_NUM_THREADS=str(os.cpu_count() or 1))
            prompt = " ".join(str(11 + i) for i in range(max(1, warm)))
            out = subprocess.run([REF_HOST, REF_LOOP, path, vocab, str(max(1, warm) + steps), prompt],
                                 env=env, capture_output=True, text=True, timeout=900)
        if out.returncode != 0:
            return None
        st = [l for l in out.stdout.splitlines() if l.startswith("[stats] ")][-1].split()
        st = dict(zip(st[1::2], st[2::2]))
        n, dt = int(st["tokens"]), float(st["decode_s"])
        if n < 1 or dt <= 0:
            return None
        return {"tokens_per_s": n / dt, "steps": n, "decode_s": dt, "threads": int(st["threads"])}
    except Exception:
        return None


def cpu_baseline(cfg, blob, views, start, budget_s=12.0, max_steps=64, warm=2):
    """The CPU restatement (oracle/) on the host cores: a bounded sample of the
    same workload, timed by the reference's own generation loop when the prebuilt
    runner is there, else by a plain loop over the restatement's decode step."""
    start = max(0, min(start, cfg.max_len - warm - max_steps))   # the sample must fit the cache
    r = reference_loop(blob, start, max_steps, warm)
    if r is not None:
        return {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["threads"], "kind": "port",
                "loop": "buddy-mlir runGeneration + Sampler (runtime/llm/TextGeneration.cpp), its own clock",
                "sample": f"{r['steps']} decode steps of the same int8 1.5B model from context {start + warm} "
                          f"({r['decode_s']:.1f} s, after {warm} untimed prompt rows)"}
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as orc
    om = orc.OracleModel(cfg, views, kinds={n: "w8" for n in ALL_LINEAR})
    for b in range(2 * cfg.n_layers):
        om.kv[b][:] = kv_prefix(cfg, start, b)
    om.position = start
    tok = 11
    for _ in range(warm):
        tok = int(np.argmax(om.decode(tok)))
    t0, n = time.perf_counter(), 0
    while n < max_steps and time.perf_counter() - t0 < budget_s and om.position < cfg.max_len:
        tok = int(np.argmax(om.decode(tok)))
        n += 1
    dt = time.perf_counter() - t0
    return {"value": n / dt, "unit": "tokens/s", "cores": orc.lib().orc_num_threads(),
            "kind": "port", "loop": "python loop over orc_decode_step",
            "sample": f"{n} decode steps of the same int8 1.5B model from context {start + warm} "
                      f"({dt:.1f} s, after {warm} warm-up steps)"}


def run_reference(args):
    """--impl reference: the CPU restatement timed alone, same config."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    os.environ.setdefault("OMP_NUM_THREADS", str(os.cpu_count() or 1))
    from buddy_mlir_b200 import DEEPSEEK_R1_1P5B as cfg, synthetic
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as orc
    blob, views = synthetic.make_f32_blob(cfg, SEED_W)
    start = plan_positions(cfg, args.steps, args.warmup)
    loop = "python loop over orc_decode_step"
    r = reference_loop(blob, start, args.steps, args.warmup)
    if r is not None and r["steps"] == args.steps:
        dt = r["decode_s"]
        loop = "buddy-mlir runGeneration + Sampler (runtime/llm/TextGeneration.cpp), its own clock"
    else:
        om = orc.OracleModel(cfg, views, kinds={n: "w8" for n in ALL_LINEAR})
        for b in range(2 * cfg.n_layers):
            om.kv[b][:] = kv_prefix(cfg, start, b)
        om.position = start
        tok = 11
        for _ in range(args.warmup):
            tok = int(np.argmax(om.decode(tok)))
        t0 = time.perf_counter()
        for _ in range(args.steps):
            tok = int(np.argmax(om.decode(tok)))
        dt = time.perf_counter() - t0
    v = args.steps / dt
    cores = orc.lib().orc_num_threads()
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * dt / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations, int8 weights",
            "data": "synthetic",
            "config": workload_config(cfg, start, args),
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "loop": loop,
                             "sample": f"{args.steps} decode steps, context {start + args.warmup}..{cfg.max_len}"},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def workload_config(cfg, start, args):
    return {"workload": "deepseek-r1-distill-qwen-1.5b architecture, int8 per-output-channel weight-only "
                        "(all linear layers), f32 activations, batch 1, greedy decode",
            "context": f"{start + args.warmup}..{cfg.max_len}", "l2": "inputs larger than L2 (1.55 GB of weights per step)",
            "weights": "seeded N(0,0.02)", "kv_prefix": "seeded N(0,1)"}


GEMV_SHAPES = {
    # name: (weight kind, N, K, group)
    "gate_up": ("i8", 17920, 1536, 0), "down": ("i8", 1536, 8960, 0), "o": ("i8", 1536, 1536, 0),
    "lm_head": ("i8", 151936, 1536, 0),
    "u4_qkv_8b": ("u4", 6144, 4096, 128), "u4_gate_up_8b": ("u4", 24576, 4096, 128),
    "u4_down_8b": ("u4", 4096, 12288, 128), "u4_lm_head_8b": ("u4", 151936, 4096, 128),
}


def gemv_microbench(lib, only=None):
    """Isolated M = 1 GEMV launches (b200_gemv) over weights that do not fit L2,
    CUDA events on the launching (current) stream.  int8 per-channel shapes of
    the 1.5B model and int4 group-128 shapes of the 8B model."""
    import ctypes as C
    import torch
    from buddy_mlir_b200 import _lib
    out = {}
    hbm, _ = peaks()
    for name, (kind, N, K, group) in GEMV_SHAPES.items():
        if only and name != only:
            continue
        nbytes = N * K if kind == "i8" else N * K // 2
        copies = max(2, int(400e6 // nbytes) + 1)
        ws = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(copies)]
        ng = K // group if group else 1
        sc = (torch.rand(N * ng, device="cuda") * 0.01).half() if group else torch.rand(N, device="cuda") * 0.01
        x = torch.randn(1, K, device="cuda")
        y = torch.zeros(1, N, device="cuda")
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

        def launch(i):
            w = _lib.Weight(_lib.W_I8 if kind == "i8" else _lib.W_U4, group, K, N, ws[i % copies].data_ptr(),
                            sc.data_ptr(), _lib.F16 if group else _lib.F32, 0, None)
            a = _lib.GemvArgs(x.data_ptr(), 0, 0, 0, 0, y.data_ptr(), None, None, 0.0, 1, 0, 0)
            _lib.check(lib.b200_gemv(C.byref(w), C.byref(a), st))
        for i in range(copies):
            launch(i)
        torch.cuda.synchronize()
        reps = 4 * copies
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            launch(i)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1000.0 / reps
        gbs = (nbytes + N * ng * (2 if group else 4) + 4 * K + 4 * N) / us / 1e3
        out[name] = {"N": N, "K": K, "weights": "int8 per-channel" if kind == "i8" else "int4 group-128",
                     "us": round(us, 2), "GB/s": round(gbs, 1), "frac": round(gbs / hbm, 3)}
    return out


GEMM_SHAPES = {
    # name: (M, N, K): the 1.5B model's projections at the reference's prefill length and at batch 64
    "qkv_m1024": (1024, 2048, 1536), "o_m1024": (1024, 1536, 1536), "gate_up_m1024": (1024, 17920, 1536),
    "down_m1024": (1024, 1536, 8960), "lm_head_m1024": (1024, 151936, 1536),
    "gate_up_m64": (64, 17920, 1536), "down_m64": (64, 1536, 8960), "lm_head_m64": (64, 151936, 1536),
}


def gemm_microbench(lib, only=None):
    """Isolated b200_gemm_w8 launches (tcgen05 path): activation split + GEMM kernel, CUDA events
    on the launching stream, int8 weights that do not fit L2 rotated between launches.
    TFLOP/s counts 2*M*N*K once (every tile is multiplied twice on the tensor cores, once per
    bf16 term of the f32 activations, so the tensor pipe does twice that)."""
    import ctypes as C
    import torch
    from buddy_mlir_b200 import _lib
    d = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    peak = float(d.get("bf16_tflops_sustained", 1400.0))
    out = {}
    for name, (M, N, K) in GEMM_SHAPES.items():
        if only and name != only:
            continue
        copies = max(2, int(300e6 // (N * K)) + 1)
        ws_ = [torch.randint(0, 255, (N * K,), dtype=torch.uint8, device="cuda") for _ in range(copies)]
        sc = torch.rand(N, device="cuda") * 0.01
        A = torch.randn(M, K, device="cuda")
        Cd = torch.zeros(M, N, device="cuda")
        nb = lib.b200_gemm_w8_workspace_bytes(M, K)
        ws = torch.zeros(nb, dtype=torch.uint8, device="cuda")
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

        def launch(i):
            w = _lib.Weight(_lib.W_I8, 0, K, N, ws_[i % copies].data_ptr(), sc.data_ptr(), _lib.F32, 0, None)
            _lib.check(lib.b200_gemm_w8(C.byref(w), A.data_ptr(), M, K, Cd.data_ptr(), N, None, 0, None, 0.0, 0,
                                        ws.data_ptr(), nb, st))
        for i in range(3):
            launch(i)
        torch.cuda.synchronize()
        reps = max(4, 2 * copies)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            launch(i)
        e1.record()
        torch.cuda.synchronize()
        _lib.check(lib.b200_gemm_w8_status(ws.data_ptr(), st))
        us = e0.elapsed_time(e1) * 1000.0 / reps
        tf = 2.0 * M * N * K / us / 1e6
        out[name] = {"M": M, "N": N, "K": K, "us": round(us, 1), "TFLOP/s": round(tf, 1),
                     "frac_of_bf16_sustained": round(tf / peak, 3), "tensor_pipe_frac": round(2 * tf / peak, 3)}
        # the same shape as W8A8 (int8 activations, integer tensor cores): quantiser + GEMM
        nb8 = lib.b200_gemm_w8a8_workspace_bytes(M, K)
        ws8 = torch.zeros(nb8, dtype=torch.uint8, device="cuda")

        def launch8(i):
            w = _lib.Weight(_lib.W_I8, 0, K, N, ws_[i % copies].data_ptr(), sc.data_ptr(), _lib.F32, 0, None)
            _lib.check(lib.b200_gemm_w8a8(C.byref(w), A.data_ptr(), M, K, Cd.data_ptr(), N, ws8.data_ptr(), nb8, st))
        for i in range(3):
            launch8(i)
        torch.cuda.synchronize()
        e0.record()
        for i in range(reps):
            launch8(i)
        e1.record()
        torch.cuda.synchronize()
        _lib.check(lib.b200_gemm_w8_status(ws8.data_ptr(), st))
        us8 = e0.elapsed_time(e1) * 1000.0 / reps
        out[name]["w8a8_us"] = round(us8, 1)
        out[name]["w8a8_TOP/s"] = round(2.0 * M * N * K / us8 / 1e6, 1)
    return {"shapes": out, "peak_tflops": peak,
            "note": "frac = algorithmic 2MNK / time / measured sustained bf16 peak; the tensor pipe does twice the "
                    "algorithmic work (two bf16 terms per f32 activation); w8a8_* = the same shape with int8 "
                    "activations on the integer tensor-core path (no measured int8 peak on this pool: absolute only)"}


def run_gemm_only(args):
    import torch
    from buddy_mlir_b200 import _lib
    lib = _lib.load()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    print(json.dumps({"gemm_isolated": gemm_microbench(lib, args.gemm_shape)}))


def batch_numbers(blob, steps, warmup):
    """Batched decode + prefill of the 1.5B int8 model (dense tcgen05 GEMM path): 64 sequences
    with seeded lengths uniform in [128, 2048] in the paged KV cache, a 2048-token prefill, then
    `steps` decode steps of the whole batch."""
    import torch
    from buddy_mlir_b200 import DEEPSEEK_R1_1P5B as cfg
    from buddy_mlir_b200.session import BatchSession, ModelSession
    s = ModelSession(cfg)
    s.load_blobs("f32", blob, all_linear_w8=True)
    B, page = 64, 16
    rng = np.random.default_rng(SEED_P)
    lengths = rng.integers(128, 2049, B)
    n_pages = int(sum((int(n) + steps + warmup + page - 1) // page + 1 for n in lengths)) + 2048 // page + 8
    bs = BatchSession(s, max_seqs=B + 1, page_size=page, n_pages=n_pages, max_context=2048 + steps + warmup + 16)
    # one 2048-token prefill, timed (after a warm-up pass of the same size on a scratch sequence)
    scratch = bs.add()
    bs.prefill(scratch, rng.integers(0, cfg.vocab, 2048), want_logits=False)
    bs.remove(scratch)
    scratch = bs.add()
    # profiler range (ncu --profile-from-start off): the timed prefill and, below, the last decode step
    torch.cuda.profiler.start()
    bs.prefill(scratch, rng.integers(0, cfg.vocab, 2048), want_logits=False)
    torch.cuda.profiler.stop()
    prefill_ms = bs.last_ms()
    bs.remove(scratch)
    seqs, toks = [], []
    for n in lengths:
        q = bs.add()
        _, nxt = bs.prefill(q, rng.integers(0, cfg.vocab, int(n)), want_logits=False)
        seqs.append(q)
        toks.append(nxt)
    for _ in range(warmup):
        _, nxt = bs.decode(seqs, toks, want_logits=False)
        toks = [int(t) for t in nxt]
    ms = []
    for i in range(steps):
        if i == steps - 1:
            torch.cuda.profiler.start()
        _, nxt = bs.decode(seqs, toks, want_logits=False)
        ms.append(bs.last_ms())
        toks = [int(t) for t in nxt]
    torch.cuda.profiler.stop()
    step_ms = float(np.mean(ms))
    flops = 2.0 * (1310195712 + 233373696)       # per token: the linear layers and the lm_head
    out = {"batched_decode": {"sequences": B, "lengths": "uniform [128, 2048], seeded", "page_size": page,
                              "ms_per_step": step_ms, "tokens_per_s": B / (step_ms / 1000.0),
                              "steps": steps, "weights": "int8 per-channel, every linear layer"},
           "prefill_2048": {"ms": prefill_ms, "tokens_per_s": 2048 / (prefill_ms / 1000.0),
                            "linear_TFLOP/s": 2048 * flops / (prefill_ms / 1000.0) / 1e12},
           "model": "deepseek-r1-distill-qwen-1.5b architecture, seeded weights"}
    bs.close()
    out["w8a8"] = w8a8_numbers(s, rng)
    s.close()
    return out


def w8a8_numbers(s, rng):
    """The session's weights under the arithmetic of the w8a8 graphs (int8 activations, one
    dynamic scale per activation tensor): a max_len-row prefill on the integer tensor cores and
    decode steps of one row (dp4a GEMV per projection, a CUDA graph)."""
    import torch
    cfg = s.cfg
    s.set_activation_int8(True)
    toks = rng.integers(0, cfg.vocab, cfg.max_len)
    s.prefill_rows(toks, 0, all_rows=False)
    s.prefill_rows(toks, 0, all_rows=False)
    q_prefill_ms = s.last_ms()
    s.prefill_rows(toks[:512], 0, all_rows=False)
    s.generate(int(toks[0]), 8)
    s.generate(int(toks[1]), 32)
    q_step_ms = s.last_ms() / 32
    torch.cuda.profiler.start()      # two more steps as a profiler range of their own
    s.generate(int(toks[2]), 2)
    torch.cuda.profiler.stop()
    s.set_activation_int8(False)
    weight_bytes = 1310195712 + 233373696       # int8 linear layers + lm_head, read once per step
    return {"prefill_1024": {"ms": q_prefill_ms, "tokens_per_s": cfg.max_len / (q_prefill_ms / 1000.0)},
            "decode": {"ms_per_step": q_step_ms, "tokens_per_s": 1000.0 / q_step_ms, "context": "520..552",
                       "weight_GB/s": weight_bytes / (q_step_ms / 1000.0) / 1e9,
                       "path": "CUDA graph: one dp4a GEMV per projection, the row quantised inside it"}}


def run_w8a8_only(args):
    """--w8a8-only: the w8a8 numbers of the 1.5B int8 model alone (one JSON line; a small
    device footprint, which keeps a profiler capture of its kernels short)."""
    import torch
    from buddy_mlir_b200 import DEEPSEEK_R1_1P5B as cfg, _lib, synthetic
    from buddy_mlir_b200.session import ModelSession
    _lib.load()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    blob, _ = synthetic.make_f32_blob(cfg, SEED_W)
    s = ModelSession(cfg)
    s.load_blobs("f32", blob, all_linear_w8=True)
    print(json.dumps({"w8a8": w8a8_numbers(s, np.random.default_rng(SEED_P)),
                      "model": "deepseek-r1-distill-qwen-1.5b architecture, seeded weights, every linear layer int8"}))
    s.close()


def run_batch_only(args):
    """--batch-only: the batched decode + prefill numbers alone (one JSON line)."""
    import torch
    from buddy_mlir_b200 import DEEPSEEK_R1_1P5B as cfg, _lib, synthetic
    _lib.load()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    blob, _ = synthetic.make_f32_blob(cfg, SEED_W)
    print(json.dumps(batch_numbers(blob, args.steps, args.warmup)))


def run_gemv_only(args):
    """--gemv-only: just the isolated GEMV sweep (one JSON line); --gemv-shape picks one shape,
    which keeps a profiler capture of that kernel small."""
    import torch
    from buddy_mlir_b200 import _lib
    lib = _lib.load()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    print(json.dumps({"gemv_isolated": gemv_microbench(lib, args.gemv_shape)}))


def run_single(args):
    import torch
    from buddy_mlir_b200 import DEEPSEEK_R1_1P5B as cfg, _lib, synthetic
    from buddy_mlir_b200.model_entry import EntrySession
    from buddy_mlir_b200.session import ModelSession
    lib = _lib.load()          # raises if the CUDA library is missing: no fallback
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    steps, warmup = args.steps, args.warmup
    start = plan_positions(cfg, steps, warmup)
    t_setup = time.perf_counter()
    blob, views = synthetic.make_f32_blob(cfg, SEED_W)

    # ---- resident-in-HBM number ------------------------------------------------
    s = ModelSession(cfg)
    s.load_blobs("f32", blob, all_linear_w8=True)
    for b in range(2 * cfg.n_layers):
        s.kv_upload(b, kv_prefix(cfg, start, b), 0, start)
    persistent = s.uses_persistent_kernel()
    s.position_ = start
    tok = 11
    warm_ids = s.generate(tok, warmup) if warmup > 0 else [tok]
    tok = int(warm_ids[-1])
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    launches0 = lib.b200_launch_count()
    ids = s.generate(tok, steps)
    ms = s.last_ms()
    launches = lib.b200_launch_count() - launches0
    clocks = sampler.stop()
    value = steps / (ms / 1000.0)
    ctx_mid = cfg.max_len - steps // 2
    step_bytes = s.step_bytes(ctx_mid)
    hbm, which = peaks()
    achieved = step_bytes / (ms / steps) / 1e6        # GB/s
    traffic, traffic_source = measured_traffic(persistent)
    gemv = None if args.resident_only else gemv_microbench(lib)
    s.close()
    if args.resident_only:
        # profiling runs: only the resident-in-HBM leg, so a capture stays small
        print(json.dumps({"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": 1,
                          "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
                          "resident_only": True, "gpu_launches": int(launches),
                          "bytes_per_step": step_bytes, "clocks": clocks}))
        return

    # ---- end to end through the model entry, host buffers --------------------------
    es = EntrySession(cfg, "f32", [blob], all_linear_w8=True)
    for b in range(2 * cfg.n_layers):
        es.kv[b][0] = kv_prefix(cfg, start, b)
    es.position_ = start
    tok = 11
    for _ in range(warmup):
        es.decode(tok)
        tok = int(np.argmax(es.logits))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_ids = []
    for _ in range(steps):
        es.decode(tok)
        tok = int(np.argmax(es.logits))
        e2e_ids.append(tok)
    torch.cuda.synchronize()
    e2e_dt = time.perf_counter() - t0
    es.close()
    same = bool(np.array_equal(np.asarray(e2e_ids), np.asarray(ids)))
    d2h = cfg.vocab * 4 + 2 * cfg.n_layers * cfg.kv_heads * cfg.head_dim * 4
    setup_s = time.perf_counter() - t_setup

    # the dense path beside the headline (config 5 of the same model): not part of the metric
    dense = None
    if not args.resident_only:
        dense = batch_numbers(blob, 16, 3)
        dense["gemm_gate_up_m1024"] = gemm_microbench(lib, "gate_up_m1024")["shapes"]["gate_up_m1024"]
        # time to first token through the reference's ABI: _mlir_ciface_forward_prefill computes all
        # max_len rows, as the reference's prefill graph does, and returns [1, max_len, vocab] logits
        # and the KV buffers in host memory
        es = EntrySession(cfg, "f32", [blob], all_linear_w8=True)
        prompt = synthetic.prompt_tokens(cfg, SEED_P, 32)
        es.prefill(prompt)
        es.prefill(prompt)
        dense["entry_prefill"] = {"ms": 1000.0 * es.last_prefill_call_s, "rows": cfg.max_len,
                                  "d2h_bytes": cfg.max_len * cfg.vocab * 4 +
                                  2 * cfg.n_layers * cfg.kv_heads * cfg.max_len * cfg.head_dim * 4,
                                  "call": "_mlir_ciface_forward_prefill, host buffers, all max_len rows"}
        es.close()
    base = cpu_baseline(cfg, blob, views, start)
    line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 activations, int8 weights",
            "data": "synthetic", "config": workload_config(cfg, start, args),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                         "frac": achieved / hbm, "traffic": traffic, "traffic_source": traffic_source,
                         "peak_source": which,
                         "kernel": "decode_step_kernel (one persistent launch per token)" if persistent else "whole decode step (CUDA graph replay)",
                         "bytes_per_step": step_bytes, "frac_of_8TBs_nominal": achieved / 8000.0},
            "gemv_isolated": gemv,
            "dense_path": dense,
            "cpu_baseline": base,
            "e2e": {"value": steps / e2e_dt, "unit": "tokens/s", "h2d_bytes_per_step": 16,
                    "d2h_bytes_per_step": d2h, "tokens_match_resident_run": same},
            "gpu_launches": int(launches), "kernels_per_step": int(launches // steps),
            "clocks": clocks, "setup_s": round(setup_s, 1)}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--gemv-only", action="store_true", help="run only the isolated GEMV sweep")
    ap.add_argument("--gemv-shape", default=None, help="with --gemv-only: one shape of GEMV_SHAPES")
    ap.add_argument("--gemm-only", action="store_true", help="run only the isolated dense-GEMM sweep (tcgen05 path)")
    ap.add_argument("--batch-only", action="store_true", help="batched decode (64 sequences, paged KV) + a 2048-token prefill")
    ap.add_argument("--w8a8-only", action="store_true", help="the w8a8 arithmetic on the 1.5B int8 model: prefill and decode")
    ap.add_argument("--gemm-shape", default=None, help="with --gemm-only: one shape of GEMM_SHAPES")
    ap.add_argument("--resident-only", action="store_true",
                    help="skip the isolated-GEMV, end-to-end and CPU legs (for profiler captures)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
            import bench_tp
            return bench_tp.run_reference(args)
        return run_reference(args)
    if args.gemv_only:
        return run_gemv_only(args)
    if args.gemm_only:
        return run_gemm_only(args)
    if args.batch_only:
        return run_batch_only(args)
    if args.w8a8_only:
        return run_w8a8_only(args)
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return run_single(args)
    import bench_tp
    return bench_tp.run(args, ClockSampler, peaks)


if __name__ == "__main__":
    main()
