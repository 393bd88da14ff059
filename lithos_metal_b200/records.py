"""The reference's binary parameter records, decoded into this library's arguments.

lithos-metal's emit code hands its sampling and step-closing kernels small little-endian records (``SampleParams``,
``SelectParams``, ``AcceptParams``: monolith/kernels.py:756-768, 814-825, 831-835; the structs are declared in
kernels/common/sample.metal:14-16 and kernels/common/spec_ops.metal). A binding that replaces those dispatches receives the
same bytes; these functions turn them into the keyword arguments of :func:`lithos_metal_b200.sample`,
:func:`lithos_metal_b200.verify_select` and :func:`lithos_metal_b200.accept_scan`. Pure Python: no device is touched.
"""
from __future__ import annotations

import struct
from typing import Any, Dict

from .sampler import SamplingParams

SAMPLE_RECORD = struct.Struct("<IIIIIfffIIII")      # vocab, t_active, n_sg, n_spans, top_k, temperature, top_p, min_p, seed_lo, seed_hi, step, flags
SELECT_RECORD = struct.Struct("<IfII16fIIII")       # gamma, threshold, t_max, mode, cost[16], log_cap, ctx_cap, lm, pad
ACCEPT_RECORD = struct.Struct("<IiIIIIII")          # ring_cap, eos, log_cap, ctx_cap, lm, pad x 3


def sample_args_from_record(record: bytes) -> Dict[str, Any]:
    """``SampleParams`` -> ``dict(params=SamplingParams(...), step=, rows=, vocab=)``. The flag bits say which thresholds are on
    (1 top_k, 2 top_p, 4 min_p, 8 top-p inside top-k); a knob whose bit is clear is passed as off, whatever its field holds."""
    if len(record) != SAMPLE_RECORD.size:
        raise ValueError(f"SampleParams is {SAMPLE_RECORD.size} bytes, got {len(record)}")
    vocab, t_active, _n_sg, _n_spans, top_k, temperature, top_p, min_p, seed_lo, seed_hi, step, flags = SAMPLE_RECORD.unpack(record)
    if not temperature > 0.0:
        raise ValueError("SampleParams: temperature must be positive (the greedy path has its own record)")
    params = SamplingParams(temperature=temperature, top_k=top_k if flags & 1 else 0, top_p=top_p if flags & 2 else 0.0,
                            min_p=min_p if flags & 4 else 0.0, seed=(seed_hi << 32) | seed_lo, topp_in_topk=bool(flags & 8), draw="gumbel")
    return {"params": params, "step": step, "rows": t_active, "vocab": vocab}


def select_args_from_record(record: bytes) -> Dict[str, Any]:
    """``SelectParams`` -> the keyword arguments of ``verify_select`` (``t_max`` = the rows of the step program)."""
    if len(record) != SELECT_RECORD.size:
        raise ValueError(f"SelectParams is {SELECT_RECORD.size} bytes, got {len(record)}")
    f = SELECT_RECORD.unpack(record)
    gamma, threshold, t_max, mode = f[0], f[1], f[2], f[3]
    cost, (log_cap, ctx_cap, lm, _pad) = list(f[4:20]), f[20:24]
    return {"gamma": gamma, "threshold": threshold, "t_max": t_max, "mode": mode, "cost": cost if mode == 1 else None, "log_cap": log_cap,
            "ctx_cap": ctx_cap, "lm": bool(lm)}


def accept_args_from_record(record: bytes) -> Dict[str, Any]:
    """``AcceptParams`` -> ``dict(ring_cap=, eos=, log_cap=, ctx_cap=, lm=)`` (``eos`` = -1: the stop tokens are a compiled-in list,
    monolith/kernels.py:729-741, which the caller passes as ``eos=[...]``)."""
    if len(record) != ACCEPT_RECORD.size:
        raise ValueError(f"AcceptParams is {ACCEPT_RECORD.size} bytes, got {len(record)}")
    ring_cap, eos, log_cap, ctx_cap, lm, *_pad = ACCEPT_RECORD.unpack(record)
    return {"ring_cap": ring_cap, "eos": eos, "log_cap": log_cap, "ctx_cap": ctx_cap, "lm": bool(lm)}
