"""buddy_mlir_b200: hand-written sm_100a kernels for buddy-mlir's LLM decode
path behind its runtime C ABI.  The CUDA library is the product; this package
is the thin host side (ctypes binding, MemRef descriptors, session mirror)."""
from . import _lib
from .config import (DEEPSEEK_R1_1P5B, QWEN3_8B, TINY_MEGA, TINY_QWEN2,
                     TINY_QWEN3, ModelConfig)

__all__ = ["_lib", "ModelConfig", "DEEPSEEK_R1_1P5B", "QWEN3_8B", "TINY_QWEN2",
           "TINY_QWEN3", "TINY_MEGA"]
