"""The vocabulary projection of a decode step (the reference's ``lm_head`` op, monolith/nn/lm_head.py:50-60): BF16 logits of at
most 8 rows from the hidden states and the [vocab, hidden] weight, the final RMSNorm fused on the input. The logits are what
``sample`` / ``argmax`` / ``verify`` take next on the same stream."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib


def lm_head(hidden: torch.Tensor, weight: torch.Tensor, norm_weight: Optional[torch.Tensor] = None, *, eps: float = 1e-6, one_plus: bool = True,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``bf16(x @ weightᵀ)`` with FP32 accumulation; ``x = hidden`` or, with ``norm_weight``, ``bf16(rms_norm(hidden) * (1 + norm_weight))``
    (``one_plus=False``: ``* norm_weight``), as monolith/nn/oracle.py:20-32 defines both. ``hidden`` [rows <= 8, H] and ``weight`` [V, H]
    bfloat16 CUDA tensors with unit stride along H; returns [rows, V] bfloat16."""
    if hidden.dim() != 2 or weight.dim() != 2 or hidden.shape[1] != weight.shape[1]:
        raise ValueError("lm_head: hidden [rows, H] and weight [V, H]")
    if hidden.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not hidden.is_cuda or weight.device != hidden.device:
        raise ValueError("lm_head: bfloat16 CUDA tensors on one device")
    rows, H = hidden.shape
    V = weight.shape[0]
    if rows > 8:
        raise ValueError("lm_head: at most 8 rows (a decode step)")
    if hidden.stride(1) != 1:
        hidden = hidden.contiguous()
    if weight.stride(1) != 1:
        raise ValueError("lm_head: the weight's rows must be contiguous")
    if norm_weight is not None:
        if norm_weight.shape != (H,) or norm_weight.dtype != torch.bfloat16 or norm_weight.device != hidden.device:
            raise ValueError("lm_head: norm_weight [H] bfloat16 on the same device")
        norm_weight = norm_weight.contiguous()
    logits = out if out is not None else torch.empty(rows, V, dtype=torch.bfloat16, device=hidden.device)
    if logits.shape != (rows, V) or logits.dtype != torch.bfloat16 or logits.stride(1) != 1 or logits.device != hidden.device:
        raise ValueError("lm_head: out must be [rows, V] bfloat16 on the same device")
    a = _lib.HeadArgs()
    a.struct_size = C.sizeof(_lib.HeadArgs)
    a.rows, a.hidden, a.hidden_stride = rows, hidden.data_ptr(), hidden.stride(0) if rows > 1 else H
    a.weight, a.weight_stride, a.hidden_dim, a.vocab = weight.data_ptr(), weight.stride(0) if V > 1 else H, H, V
    a.norm_weight = norm_weight.data_ptr() if norm_weight is not None else None
    a.eps, a.one_plus = float(eps), 1 if one_plus else 0
    a.logits, a.logits_stride = logits.data_ptr(), logits.stride(0) if rows > 1 else V
    a.stream = torch.cuda.current_stream(hidden.device).cuda_stream
    with torch.cuda.device(hidden.device):
        _lib.check(_lib.lib().lm_head(C.byref(a)), "lm_head")
    return logits
