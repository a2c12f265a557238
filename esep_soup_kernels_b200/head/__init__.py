"""Fused LM head (lm_head matmul + cross-entropy + entropy + argmax) for B200.

Mirrors the public names of the reference's ``solution/head/__init__.py:6-9`` for the op itself
(``fused_linear_ce``, ``warmup``); the reference's ``patch`` (trainer wiring) is caller glue and
not part of this package. Importing this package loads libesep_head.so and fails if it cannot.
"""

from . import _lib

_lib.load()

from .op import (CHUNK_ROWS, G_SCALE, VOCAB, FusedLinearCE, fused_linear_ce,  # noqa: E402
                 fused_linear_ce_with_metrics, last_device_status, warmup)
from .step import HeadStep, HeadWeight, causal_lm_head_step, step_metrics, step_sums  # noqa: E402
from .norm import final_norm_backward, final_norm_forward, fused_norm_linear_ce  # noqa: E402
from .weight import Fp16Fixup, embedding_forward16, share_fp16_weight  # noqa: E402

__all__ = ["fused_linear_ce", "fused_linear_ce_with_metrics", "warmup", "FusedLinearCE",
           "last_device_status", "HeadStep", "HeadWeight", "causal_lm_head_step", "step_metrics",
           "step_sums",
           "final_norm_forward", "final_norm_backward", "fused_norm_linear_ce",
           "Fp16Fixup", "embedding_forward16", "share_fp16_weight",
           "CHUNK_ROWS", "G_SCALE", "VOCAB"]
