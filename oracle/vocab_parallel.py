"""numpy model of the vocab-parallel sampler's two steps. TEST INFRASTRUCTURE ONLY.

The reference has no multi-GPU path (it is single-device); the vocab-parallel mode is new. Its definition: the result
must equal the single-GPU sampler's result on the concatenated vocabulary, bit for bit. Each shard reports, per
row, its maximum, its FP64 softmass relative to that maximum, and every logit at or above its own k-th largest
(`local_record`); every rank then merges all shards' records identically (`merge_records`). The byte layout of a
record is the one the CUDA library writes, so the host-side exchange can be tested on CPU ranks with these functions
standing in for the kernels.
"""
from __future__ import annotations

import struct
from typing import Sequence, Tuple

import numpy as np

from . import lib as _lib, widen
import ctypes as C

HEADER = 32            # float vmax, float pad, double mass, int32 n, uint32 status, 8 bytes pad
STATUS_OVERFLOW = 32


def record_bytes(cap: int) -> int:
    return HEADER + 8 * cap


def candidate_cap(top_k: int) -> int:
    return (top_k + 64 + 7) // 8 * 8


def local_record(z_shard: np.ndarray, shard_start: int, *, temperature: float, top_k: int, cap: int) -> bytes:
    """One row of one shard -> its record."""
    z = np.asarray(z_shard, dtype=np.float32)
    vmax = np.float32(z.max())
    mass = float(np.exp((z.astype(np.float64) - float(vmax)) / float(np.float32(temperature))).sum()) if vmax > -np.inf else 0.0
    k = min(top_k, z.size)
    tau_local = np.partition(z, z.size - k)[z.size - k]
    if tau_local > -np.inf:
        idx = np.nonzero(z >= tau_local)[0]
    else:                                                                  # fewer than top_k logits above -inf: those, and the first -inf logit for the rest
        idx = np.concatenate([np.nonzero(z > -np.inf)[0], np.nonzero(z == -np.inf)[0][:1]])
    status = 0
    if idx.size > cap:
        status, idx = STATUS_OVERFLOW, idx[:cap]
    vals = np.zeros(cap, np.float32)
    ids = np.full(cap, -1, np.int32)
    vals[:idx.size] = z[idx]
    ids[:idx.size] = idx + shard_start
    return struct.pack("<ffdiI8x", float(vmax), 0.0, mass, int(idx.size), status) + vals.tobytes() + ids.tobytes()


def unpack_record(rec: bytes, cap: int):
    vmax, _, mass, n, status = struct.unpack_from("<ffdiI", rec, 0)
    vals = np.frombuffer(rec, np.float32, cap, HEADER)[:n]
    ids = np.frombuffer(rec, np.int32, cap, HEADER + 4 * cap)[:n]
    return np.float32(vmax), mass, n, status, vals, ids


def merge_records(records: Sequence[bytes], cap: int, *, temperature: float, top_k: int, top_p: float = 0.0, min_p: float = 0.0,
                  topp_in_topk: bool = False, draw: str = "inverse_cdf", u: float = 0.0, seed: int = 0, step: int = 0, t: int = 0) -> Tuple[int, float, int]:
    """All shards' records of one row -> (token, tau, status)."""
    T32 = np.float32(temperature)
    T = float(T32)
    parts = [unpack_record(r, cap) for r in records]
    status = 0
    for p in parts:
        status |= p[3]
    if status & STATUS_OVERFLOW:
        return -1, float("-inf"), status
    vals = np.concatenate([p[4] for p in parts]).astype(np.float32)
    ids = np.concatenate([p[5] for p in parts]).astype(np.int64)
    order = np.lexsort((ids, -vals.astype(np.float64)))                 # value descending, index ascending
    vals, ids = vals[order], ids[order]
    vmax = np.float32(max(p[0] for p in parts))
    z_total = 0.0
    for p in parts:                                                      # fixed order: shard 0, 1, ...
        z_total += p[1] * np.exp((float(p[0]) - float(vmax)) / T)
    n = vals.size
    tau = -np.inf
    tau_k = np.float32(-np.inf)
    if top_k > 0:
        tau_k = vals[min(top_k, n) - 1]
        tau = float(tau_k)
    if 0.0 < top_p < 1.0:
        m = np.exp((vals.astype(np.float64) - float(vmax)) / T)
        cum = np.cumsum(m)
        total = cum[vals >= tau_k][-1] if (topp_in_topk and top_k > 0) else z_total
        target = float(np.float32(top_p)) * total
        run_end = np.append(vals[1:] != vals[:-1], True)
        hit = np.nonzero(run_end & (cum >= target))[0]
        if hit.size:
            tau = max(tau, float(vals[hit[0]]))
    if min_p > 0.0:
        tau = max(tau, float(vmax) + T * np.log(float(np.float32(min_p))))
    tau_f = np.float32(tau)
    kept = vals >= tau_f
    L = _lib()
    if draw == "inverse_cdf":
        c = L.lmo_exp2_scale(T32)
        kid = ids[kept]
        w = np.array([L.lmo_weight_q40(float(v), float(vmax), c) for v in vals[kept]], dtype=object)
        o = np.lexsort((kid, -vals[kept].astype(np.float64)))          # descending logit, equal logits by ascending index
        total = int(sum(w))
        if total == 0:
            return -1, float(tau_f), status
        target = L.lmo_cdf_target(np.float32(u), total)
        cum = 0
        for j in o:
            cum += int(w[j])
            if cum > target:
                return int(kid[j]), float(tau_f), status
        return -1, float(tau_f), status
    inv_t = np.float32(1.0 / T)
    best, tok = None, -1
    for v, i in zip(vals[kept], ids[kept]):
        key = np.float32(np.float32(v * inv_t) + np.float32(L.lmo_gumbel(seed & (2**64 - 1), step, t, int(i))))
        if best is None or key > best or (key == best and i < tok):
            best, tok = key, int(i)
    return tok, float(tau_f), status
