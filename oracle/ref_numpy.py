"""numpy restatement of the reference's sampler oracle (monolith/nn/sampling_ref.py), TEST INFRASTRUCTURE ONLY.

Same definitions, same dtypes at every step; the one deliberate difference is that the per-distinct-value counts
come from ``np.unique(return_counts=True)`` instead of one ``(v == x).sum()`` per distinct value (sampling_ref.py:30),
which gives identical numbers in O(V log V) instead of O(distinct x V). Used to cross-check ``lm_oracle.c`` and as a
second CPU timing ("numpy port") beside the C port.
"""
from __future__ import annotations

import numpy as np

_M64 = (1 << 64) - 1


def thresholds(logits, *, temperature=1.0, top_k=0, top_p=0.0, min_p=0.0, topp_in_topk=False) -> float:
    """sampling_ref.py:20-38."""
    v = np.asarray(logits, dtype=np.float32)
    taus = []
    if top_k > 0:
        taus.append(float(np.partition(v, v.size - min(top_k, v.size))[v.size - min(top_k, v.size)]))
    if 0.0 < top_p < 1.0:
        vals, counts = np.unique(v, return_counts=True)
        vals, counts = vals[::-1], counts[::-1].astype(np.float64)
        cum = np.cumsum(counts * np.exp((vals.astype(np.float64) - vals[0]) / temperature))
        total = cum[vals >= taus[0]][-1] if topp_in_topk and top_k > 0 else cum[-1]
        taus.append(float(vals[int(np.argmax(cum >= top_p * total))]))
    if min_p > 0.0:
        taus.append(float(v.max() + temperature * np.log(min_p)))
    return max(taus) if taus else -np.inf


def uniform01(seed: int, step: int, t: int, idx) -> np.ndarray:
    """sampling_ref.py:41-51 (the 23-bit uniform of the splitmix64 hash), computed on Python-int-free uint64 arrays."""
    with np.errstate(over="ignore"):
        i = np.asarray(idx, dtype=np.uint64)
        x = np.uint64(seed & _M64) + np.uint64(step) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(t) * np.uint64(0xC2B2AE3D27D4EB4F) \
            + i * np.uint64(0x165667B19E3779F9)
        x ^= x >> np.uint64(30); x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27); x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    u = ((x >> np.uint64(41)) & np.uint64(0x7FFFFF)).astype(np.float32)
    return (u + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def gumbel_noise(seed: int, step: int, t: int, idx) -> np.ndarray:
    """sampling_ref.py:52."""
    return -np.log(-np.log(uniform01(seed, step, t, idx))).astype(np.float32)


def sample(logits, *, seed, step, t=0, temperature=1.0, top_k=0, top_p=0.0, min_p=0.0, topp_in_topk=False) -> int:
    """sampling_ref.py:55-62."""
    v = np.asarray(logits, dtype=np.float32)
    tau = thresholds(v, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, topp_in_topk=topp_in_topk)
    keys = v * np.float32(1.0 / temperature) + gumbel_noise(seed, step, t, np.arange(v.size))
    keys = np.where(v >= np.float32(tau), keys, -np.inf).astype(np.float32)
    return int(np.argmax(keys))


def warped_probabilities(logits, *, temperature=1.0, top_k=0, top_p=0.0, min_p=0.0) -> np.ndarray:
    """sampling_ref.py:65-71."""
    v = np.asarray(logits, dtype=np.float64)
    tau = thresholds(v.astype(np.float32), temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p)
    p = np.exp(np.where(v >= tau, (v - v.max()) / temperature, -np.inf))
    return p / p.sum()
