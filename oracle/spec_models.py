"""Pure-Python models of the speculative round's two scalar control kernels. TEST INFRASTRUCTURE ONLY.

``accept_scan`` follows kernels/common/spec_ops.metal:148-195 (its Python model in the reference's tests is
tests/kernels/test_draft_ops.py:319-356); ``verify_select`` follows spec_ops.metal:108-146 with the parameter
record of monolith/kernels.py:814-825; ``advance`` follows kernels/common/advance.metal:15-37. States are plain dicts
with the field names of monolith/core/step_state.py:38-62.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple


def accept_scan(state: Dict, tokens: Sequence[int], ring_cap: int, eos: int, ctx_cap: int = 0, lm: bool = False) -> Tuple[Dict, List[Tuple[int, int]], int]:
    """Returns (new state, ring writes [(slot, value)], log entry or -1)."""
    s = dict(state)
    s["pending_tokens"] = list(state["pending_tokens"])
    writes: List[Tuple[int, int]] = []
    if s["done"]:
        return s, writes, -1
    t = s["t_this_step"]
    if s["prefill_left"] > 0:
        log = (t << 16) | 0xFFFF
        s["position"] += t
        s["step"] += 1
        s["n_inject"] = t
        s["checkpoint_index"] = t
        s["n_chain"] = 0
        if ctx_cap and s["position"] >= ctx_cap:
            s["error"], s["done"] = 2, 1
        return s, writes, log
    L = s["verify_len"]
    base = t - 1 - L
    acc = 0
    while acc < L and tokens[base + acc] == s["pending_tokens"][base + acc + 1]:
        acc += 1
    bonus = tokens[base + acc]
    head = s["ring_head"]
    if head + acc + 1 - s["ring_tail"] > ring_cap:
        s["error"], s["done"] = 1, 1
        return s, writes, -1
    committed, last, stop = 0, bonus, False
    for k in range(acc + 1):
        tok = s["pending_tokens"][base + k + 1] if k < acc else bonus
        writes.append((head % ring_cap, ((head + 1) << 32) | (tok & 0xFFFFFFFF)))
        head += 1
        committed += 1
        last = tok
        if eos >= 0 and tok == eos:
            stop = True
            break
    log = (committed << 16) | (L << 8) | acc
    s["ring_head"] = head
    if s["stop_at"] and head >= s["stop_at"]:
        stop = True
    s["accepted"] = acc
    s["anchor"] = last
    s["position"] += base + committed
    s["step"] += 1
    s["verify_len"] = 0
    s["t_this_step"] = 1
    s["n_inject"] = s["checkpoint_index"] = base + committed
    s["n_chain"] = 1
    if lm:
        s["n_inject"] = s["position"] - s["drafter_ctx_len"] if s["position"] > s["drafter_ctx_len"] else 0
    if stop:
        s["done"] = 1
    if ctx_cap and s["position"] >= ctx_cap:
        s["error"], s["done"] = 2, 1
    return s, writes, log


def verify_select(state: Dict, drafts: Sequence[int], conf: Sequence[float], *, gamma: int, threshold: float, t_max: int, mode: int = 0,
                  cost: Sequence[float] = (), ctx_cap: int = 0, lm: bool = False) -> Dict:
    import numpy as np

    f32 = np.float32
    s = dict(state)
    for k in ("pending_tokens", "draft_tokens", "confidence"):
        s[k] = list(state[k])
    if s["done"]:
        return s
    if lm:
        s["drafter_ctx_len"] = s["position"] + (0 if s["prefill_left"] > 0 else gamma)
    else:
        s["drafter_ctx_len"] = s["drafter_ctx_len"] + s["n_inject"]
    s["n_inject"] = 0
    if s["prefill_left"] > 0:
        return s
    for k in range(gamma):
        s["draft_tokens"][k] = int(drafts[k])
        s["confidence"][k] = float(f32(conf[k]))
    L = 0
    lmax = min(gamma, t_max - 1)
    if ctx_cap:
        if s["position"] >= ctx_cap:
            s["error"], s["done"] = 2, 1
            return s
        lmax = min(lmax, ctx_cap - s["position"] - 1)
    if mode == 2:
        L = min(int(max(f32(threshold), f32(0.0))), lmax)
    elif mode == 1:
        c = [f32(x) for x in cost] + [f32(1.0)] * (16 - len(cost))
        a, expect, best = f32(1.0), f32(1.0), f32(1.0) / c[0]
        for l in range(1, lmax + 1):
            a = f32(a * f32(conf[l - 1]))
            expect = f32(expect + a)
            score = f32(expect / c[l])
            if score > best:
                best, L = score, l
    elif threshold <= 0.0:
        L = lmax
    else:
        while L < lmax and f32(conf[L]) >= f32(threshold):
            L += 1
    s["gamma"] = gamma
    s["verify_len"] = L
    s["pending_tokens"][0] = s["anchor"]
    for k in range(L):
        s["pending_tokens"][k + 1] = int(drafts[k])
    s["t_this_step"] = 1 + L
    return s


def advance(state: Dict, tokens: Sequence[int], ring_cap: int, eos: int, ctx_cap: int = 0) -> Tuple[Dict, List[Tuple[int, int]]]:
    s = dict(state)
    s["pending_tokens"] = list(state["pending_tokens"])
    writes: List[Tuple[int, int]] = []
    if s["done"]:
        return s, writes
    t = s["t_this_step"]
    if s["prefill_left"] > 0:
        s["position"] += t
        s["step"] += 1
        if ctx_cap and s["position"] >= ctx_cap:
            s["error"], s["done"] = 2, 1
        return s, writes
    tok = tokens[t - 1]
    head = s["ring_head"]
    if head - s["ring_tail"] >= ring_cap:
        s["error"], s["done"] = 1, 1
        return s, writes
    writes.append((head % ring_cap, ((head + 1) << 32) | (tok & 0xFFFFFFFF)))
    s["ring_head"] = head + 1
    if s["stop_at"] and s["ring_head"] >= s["stop_at"]:
        s["done"] = 1
    s["pending_tokens"][0] = tok
    s["position"] += t
    s["step"] += 1
    s["t_this_step"] = 1
    if eos >= 0 and tok == eos:
        s["done"] = 1
    if ctx_cap and s["position"] >= ctx_cap:
        s["error"], s["done"] = 2, 1
    return s, writes
