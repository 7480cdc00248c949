"""Dense bf16 flash-attention forward for NVIDIA B200 (sm_100a).

Drop-in for the `forward` entry point of the reference package of the same
name (moonmath_attention/__init__.py:11-31, moonmath_attention/_kernel.py:14-82):

>>> import torch
>>> import moonmath_attention as ma
>>> q = torch.randn(1, 4, 1024, 128, dtype=torch.bfloat16, device="cuda")
>>> k = torch.randn(1, 4, 1024, 128, dtype=torch.bfloat16, device="cuda")
>>> v = torch.randn(1, 4, 1024, 128, dtype=torch.bfloat16, device="cuda")
>>> out = ma.forward(q, k, v)         # torch.bfloat16, same shape

`forward_lite` / `LiteAttention` (moonmath_attention/lite.py of the reference) skip key blocks between
denoising steps; `mla_decode_a16w8*` (moonmath_attention/mla.py of the reference) are the MLA absorbed-decode
operators over an fp8 KV cache.  The package talks to the CUDA kernels
through a ctypes binding of libmoonmath_attention_sm100.so; importing it fails
if that library has not been built.
"""

from ._kernel import forward, forward_lite, last_status, plan_tail, workspace_bytes
from .lite import LiteAttention
from .mla import (
    mla_decode_a16w8,
    mla_decode_a16w8_multiq,
    mla_decode_a16w8_multiq_paged_dev,
    mla_decode_a16w8_multiq_plan_parts_q,
    mla_decode_a16w8_paged_dev,
    mla_decode_a16w8_plan_parts,
    mla_decode_a16w8_plan_parts_capped,
    mla_decode_a16w8_plan_parts_q,
)
from . import _abi as abi

__all__ = [
    "forward", "forward_lite", "LiteAttention", "plan_tail", "workspace_bytes", "last_status", "abi",
    "mla_decode_a16w8", "mla_decode_a16w8_paged_dev", "mla_decode_a16w8_plan_parts",
    "mla_decode_a16w8_plan_parts_capped", "mla_decode_a16w8_plan_parts_q", "mla_decode_a16w8_multiq",
    "mla_decode_a16w8_multiq_paged_dev", "mla_decode_a16w8_multiq_plan_parts_q",
]
