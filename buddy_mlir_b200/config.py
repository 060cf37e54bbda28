"""Model shapes of the decode path (the configs buddy-mlir's specs bake into
its generated ModelSession: tools/buddy-codegen/gen_session.py:156-180,
models/deepseek_r1/specs/*.json)."""
from dataclasses import dataclass, replace

from ._lib import ModelConfigC


@dataclass(frozen=True)
class ModelConfig:
    name: str
    hidden: int
    n_layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    max_len: int
    eps: float = 1e-6
    rope_theta: float = 1e4
    qkv_bias: bool = True   # Qwen2
    qk_norm: bool = False   # Qwen3

    def to_c(self, tp_rank=0, tp_size=1):
        return ModelConfigC(self.hidden, self.n_layers, self.q_heads, self.kv_heads,
                            self.head_dim, self.ffn, self.vocab, self.max_len,
                            self.eps, self.rope_theta, int(self.qkv_bias),
                            int(self.qk_norm), tp_rank, tp_size)

    def with_(self, **kw):
        return replace(self, **kw)

    @property
    def q_dim(self):
        return self.q_heads * self.head_dim

    @property
    def kv_dim(self):
        return self.kv_heads * self.head_dim


# DeepSeek-R1-Distill-Qwen-1.5B (Qwen2 architecture), max_token_len 1024 as in
# models/deepseek_r1/specs/f32.json.
DEEPSEEK_R1_1P5B = ModelConfig("deepseek_r1_1p5b", 1536, 28, 12, 2, 128, 8960,
                               151936, 1024)
# Qwen3-8B architecture (QK-RMSNorm, no qkv bias), context 4096.
QWEN3_8B = ModelConfig("qwen3_8b", 4096, 36, 32, 8, 128, 12288, 151936, 4096,
                       rope_theta=1e6, qkv_bias=False, qk_norm=True)
# Small shapes for tests (same structure, seconds on a CPU).
TINY_QWEN2 = ModelConfig("tiny_qwen2", 256, 2, 4, 2, 64, 512, 1024, 128)
TINY_QWEN3 = ModelConfig("tiny_qwen3", 256, 2, 8, 2, 128, 512, 1024, 128,
                         qkv_bias=False, qk_norm=True)
# Small shapes that still reach both row modes of the persistent decode kernel
# (K = 512 and 1536 warp-per-row; K = 2112 shared rows with a ragged last block).
TINY_MEGA = ModelConfig("tiny_mega", 512, 2, 12, 2, 128, 2112, 2048, 256)
