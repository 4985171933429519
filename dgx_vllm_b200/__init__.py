"""B200-native (sm_100a) NVFP4 hot path: quantizer, dense block-scaled GEMM, 2:4-sparse MoE GEMV,
grouped MoE GEMM -- drop-in replacements for the ops Avarok-Cybersecurity/dgx-vllm wires into vLLM."""
from . import _lib  # noqa: F401
from . import sparse_fp4_v7  # noqa: F401
from .ops import cutlass_scaled_fp4_mm, scaled_fp4_quant  # noqa: F401

__all__ = ["sparse_fp4_v7", "scaled_fp4_quant", "cutlass_scaled_fp4_mm"]
