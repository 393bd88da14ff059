"""numpy restatement of the reference's lm_head op, TEST INFRASTRUCTURE ONLY.

monolith/nn/lm_head.py:50-60 lowers ``lm_head`` (inputs: hidden rows, weight [vocab, hidden], optionally the final norm's weight;
output BF16 logits); its semantics are monolith/nn/oracle.py:20-32: ``linear`` = ``x @ wᵀ`` with FP32 accumulation and one rounding
to BF16, ``rms_norm`` = ``x * rsqrt(mean(x²) + eps)`` in FP32, times ``1 + w`` (or ``w``), rounded to the input dtype. The sums are
formed in binary64 here, so a logit can differ from an FP32-accumulated one by one BF16 unit in the last place where the sum
falls next to a rounding boundary; the tests allow exactly that. Pinned by ``tests/golden`` section ``lm_head`` (outputs of
the reference's own two functions on seeded inputs).
"""
from __future__ import annotations

from typing import Optional

import numpy as np


def _f32(codes: np.ndarray) -> np.ndarray:
    return (np.asarray(codes, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def rms_norm(x_codes: np.ndarray, w_codes: np.ndarray, eps: float, one_plus: bool = True) -> np.ndarray:
    """oracle.py:25-32 on BF16 codes: the normalised rows as BF16 codes."""
    x = _f32(x_codes).astype(np.float64)
    y = (x / np.sqrt((x * x).mean(-1, keepdims=True) + np.float64(np.float32(eps)))).astype(np.float32)
    w = _f32(w_codes)
    scale = (np.float32(1.0) + w) if one_plus else w
    return _bf16(y * scale)


def lm_head(x_codes: np.ndarray, w_codes: np.ndarray, norm_codes: Optional[np.ndarray] = None, eps: float = 1e-6, one_plus: bool = True) -> np.ndarray:
    """Logits [rows, vocab] as BF16 codes (oracle.py:20-22 behind the optional norm)."""
    if norm_codes is not None:
        x_codes = rms_norm(x_codes, norm_codes, eps, one_plus)
    acc = _f32(x_codes).astype(np.float64) @ _f32(w_codes).astype(np.float64).T
    return _bf16(acc.astype(np.float32))


def ulp_distance(a_codes: np.ndarray, b_codes: np.ndarray) -> np.ndarray:
    """Distance in BF16 units in the last place between two arrays of BF16 codes (monotone integer keys)."""
    def key(c):
        c = np.asarray(c, dtype=np.uint16).astype(np.int32)
        return np.where(c & 0x8000, -(c & 0x7FFF), c)                      # sign-magnitude to a signed integer line (-0 and +0 meet at 0)
    return np.abs(key(a_codes) - key(b_codes))


def close(got_codes: np.ndarray, want_codes: np.ndarray, share: float = 0.99) -> bool:
    """The tolerance of the lm_head tests: every logit within one BF16 unit in the last place of the other -- or, for sums that cancel
    to (nearly) nothing, within 1e-3 absolutely -- and at least `share` of them equal."""
    d = ulp_distance(got_codes, want_codes)
    near = np.abs(_f32(got_codes).astype(np.float64) - _f32(want_codes).astype(np.float64)) <= 1e-3
    return bool(np.all((d <= 1) | near)) and float((d == 0).mean()) >= share
