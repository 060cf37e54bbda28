"""The dense weight-only GEMM (tcgen05 path) against the CPU restatement of
buddy-mlir's prefill matmul, through the C ABI.  Tolerance 1e-3 of the
output's magnitude (the tolerance stated for f32 logits); observed errors are
near 1e-5 (two bf16 terms per activation, exact int8 weights, f32
accumulation)."""
import os

import numpy as np
import pytest

import oracle_lib as orc
from buddy_mlir_b200 import _lib

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
TOL = 1e-3


def rel(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() /
                 max(np.abs(b.astype(np.float64)).max(), 1e-30))


def test_prefill_known_answer_rows_of_eight():
    """examples/BuddyMatmul/dequant-matmul-vectorization-blis-prefill.mlir:113-115:
    A = ones[4x4], W = 2, scale = 1 -> rows [8, 8, 8, 8].  K is padded with zeros to
    the 64 the tensor-core tile needs (a zero column adds nothing)."""
    from gpu_util import dev, packed_weight, gemm_w8
    k = np.load(os.path.join(G, "known_answers.npz"))
    A = np.zeros((4, 64), np.float32)
    A[:, :4] = k["pf_A"]
    W = np.zeros((64, 4), np.int8)
    W[:4] = k["pf_W"]
    w = packed_weight(_lib.W_I8, W, 64, 4)
    y = gemm_w8(w, dev(k["pf_scale"].reshape(-1)), 64, 4, dev(A)).cpu().numpy()
    assert np.array_equal(y, k["pf_expect"])


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (1, 256, 128), (64, 1536, 1536), (200, 2048, 1536),
                                   (1024, 1536, 8960), (1024, 17920, 1536), (100, 3000, 1536),
                                   (513, 700, 1600), (300, 2500, 2048)])
def test_gemm_w8_matches_prefill_restatement(M, N, K):
    from gpu_util import dev, packed_weight, gemm_w8
    if M * N * K > 3e9:
        M_chk = 96          # the checker runs these rows (the GPU still computes all of them)
    else:
        M_chk = M
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    Q = rng.integers(-127, 128, (K, N)).astype(np.int8)
    s = rng.uniform(0.001, 0.01, N).astype(np.float32)
    w = packed_weight(_lib.W_I8, Q, K, N)
    y = gemm_w8(w, dev(s), K, N, dev(A)).cpu().numpy()
    rows = np.linspace(0, M - 1, M_chk).astype(int)
    want = orc.gemm_w8_prefill_f32(A[rows], Q, s, np.zeros((len(rows), N), np.float32))
    assert rel(y[rows], want) < TOL
    print(f"gemm {M}x{N}x{K}: max rel err {rel(y[rows], want):.2e}")


@pytest.mark.parametrize("M,K,N", [(70, 1536, 512), (600, 1600, 768)])
def test_gemm_w8_fused_norm_bias_residual_and_silu_pairs(M, K, N):
    """Few rows: the converting kernel (split over K); many rows: the dense kernel with the
    warp-per-row activation split, a K that ends in a partial block of the packed rows."""
    from gpu_util import dev, packed_weight, gemm_w8
    rng = np.random.default_rng(5)
    A = rng.standard_normal((M, K)).astype(np.float32)
    Q = rng.integers(-127, 128, (K, N)).astype(np.int8)
    s = rng.uniform(0.001, 0.01, N).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    R = rng.standard_normal((M, N)).astype(np.float32)
    nw = (1 + 0.02 * rng.standard_normal(K)).astype(np.float32)
    w = packed_weight(_lib.W_I8, Q, K, N)
    h = np.stack([orc.rmsnorm(A[i], nw, 1e-6) for i in range(M)])
    base = orc.gemm_w8_prefill_f32(h, Q, s, np.zeros((M, N), np.float32))
    y = gemm_w8(w, dev(s), K, N, dev(A), bias=dev(b), residual=dev(R), norm_w=dev(nw)).cpu().numpy()
    assert rel(y, R + (base + b)) < TOL
    # gate/up pairs interleaved by row: out[:, j] = silu(row 2j) * row 2j+1
    g = orc.gemm_w8_prefill_f32(A, Q, s, np.zeros((M, N), np.float32))
    want = np.stack([orc.silu_mul(g[i, 0::2], g[i, 1::2]) for i in range(M)])
    y = gemm_w8(w, dev(s), K, N, dev(A), silu=True).cpu().numpy()
    assert y.shape == (M, N // 2) and rel(y, want) < TOL


# ---- W8A8: int8 x int8 on the integer tensor cores (QuantizedMatmulOp) ------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (7, 130, 128), (64, 1536, 1536), (200, 1000, 576), (1024, 2048, 1536)])
def test_matmul_w8a8_is_bit_identical_to_the_restatement(M, N, K):
    """frontend/Python/ops/linalg.py:12728-12846: dynamic per-tensor int8 activations, exact
    integer contraction, one f32 rescale.  Integer work: bit-exact, ragged M and N included."""
    from buddy_mlir_b200 import memref
    rng = np.random.default_rng(M * 31 + N)
    A = (rng.standard_normal((M, K)) * 3).astype(np.float32)
    A[0, 0] = 11.5                                   # the tensor's absmax, away from the mean
    Q = rng.integers(-128, 128, (K, N)).astype(np.int8)
    scale = (rng.random((1, N)).astype(np.float32) + 0.5) * np.float32(0.01)
    want = orc.matmul_w8a8(A, Q, scale)
    got = memref.buddy_matmul_w8a8_f32(A, Q, scale)
    assert got.shape == (M, N)
    assert np.array_equal(got, want)


@pytest.mark.gpu
def test_matmul_w8a8_all_zero_activations_and_bad_k():
    from buddy_mlir_b200 import memref
    Q = np.ones((64, 128), dtype=np.int8)
    scale = np.ones((1, 128), dtype=np.float32)
    got = memref.buddy_matmul_w8a8_f32(np.zeros((3, 64), dtype=np.float32), Q, scale)
    assert np.array_equal(got, np.zeros((3, 128), dtype=np.float32))      # scale clamps at 1e-10, q = 0
    with pytest.raises(RuntimeError):
        memref.buddy_matmul_w8a8_f32(np.zeros((3, 40), dtype=np.float32), np.ones((40, 128), dtype=np.int8), scale)
