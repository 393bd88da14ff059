"""CPU oracle for the generation-control path. TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import this package; the
shipped package ``lithos_metal_b200`` never does. The arithmetic lives in ``lm_oracle.c`` (each function cites the
reference file:line it restates); this module is its ctypes binding plus array plumbing. ``ref_numpy`` holds a
numpy restatement of ``monolith/nn/sampling_ref.py`` in the reference's own formulation, used to cross-check the
C code against the golden vectors and to time "the reference as shipped".
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence, Tuple

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(_build.build())
        f32p, i32p, f64p, u64p = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_double), C.POINTER(C.c_uint64)
        _lib.lmo_thresholds.restype = C.c_float
        _lib.lmo_thresholds.argtypes = [f32p, C.c_int64, C.c_double, C.c_int32, C.c_double, C.c_double, C.c_int32, f32p, f64p, C.POINTER(C.c_int64)]
        _lib.lmo_uniform01.restype = C.c_float
        _lib.lmo_uniform01.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]
        _lib.lmo_gumbel.restype = C.c_float
        _lib.lmo_gumbel.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]
        _lib.lmo_sample_gumbel.restype = C.c_int32
        _lib.lmo_sample_gumbel.argtypes = [f32p, C.c_int64, C.c_float, C.c_double, C.c_uint64, C.c_uint32, C.c_uint32, f32p]
        _lib.lmo_warped_probs.restype = None
        _lib.lmo_warped_probs.argtypes = [f32p, C.c_int64, C.c_float, C.c_double, f64p]
        _lib.lmo_argmax.restype = C.c_int32
        _lib.lmo_argmax.argtypes = [f32p, C.c_int64]
        _lib.lmo_apply_penalties.restype = None
        _lib.lmo_apply_penalties.argtypes = [f32p, C.c_int64, i32p, C.c_int64, C.c_float, C.c_float]
        _lib.lmo_spec_exp2.restype = C.c_float
        _lib.lmo_spec_exp2.argtypes = [C.c_float]
        _lib.lmo_exp2_scale.restype = C.c_float
        _lib.lmo_exp2_scale.argtypes = [C.c_float]
        _lib.lmo_weight_q40.restype = C.c_uint64
        _lib.lmo_weight_q40.argtypes = [C.c_float, C.c_float, C.c_float]
        _lib.lmo_cdf_target.restype = C.c_uint64
        _lib.lmo_cdf_target.argtypes = [C.c_float, C.c_uint64]
        _lib.lmo_sample_invcdf.restype = C.c_int32
        _lib.lmo_sample_invcdf.argtypes = [f32p, C.c_int64, C.c_float, C.c_float, C.c_float, u64p]
        _lib.lmo_sample_invcdf_index.restype = C.c_int32
        _lib.lmo_sample_invcdf_index.argtypes = [f32p, C.c_int64, C.c_float, C.c_float, C.c_float, u64p]
        _lib.lmo_accept_greedy.restype = C.c_int32
        _lib.lmo_accept_greedy.argtypes = [i32p, i32p, C.c_int32, i32p]
        _lib.lmo_confidence.restype = None
        _lib.lmo_confidence.argtypes = [C.POINTER(C.c_uint16), C.POINTER(C.c_uint16), f32p, C.c_float, f32p, C.c_int32, C.c_int32, C.c_int32, f32p]
        _lib.lmo_draft_q.restype = C.c_int32
        _lib.lmo_draft_q.argtypes = [f32p, C.c_int64, C.c_float, C.c_uint64, C.c_uint32, C.c_uint32, f32p, C.POINTER(C.c_uint64), f32p, f32p]
        _lib.lmo_draft_probs.restype = None
        _lib.lmo_draft_probs.argtypes = [f32p, C.c_int64, C.c_float, C.c_float, C.c_uint64, f32p]
        _lib.lmo_verify_stochastic.restype = C.c_int32
        _lib.lmo_verify_stochastic.argtypes = [f32p, C.c_int64, C.c_int32, f32p, C.c_float, i32p, f32p, f32p, C.c_float, i32p, f32p]
        _lib.lmo_verify_gumbel.restype = C.c_int32
        _lib.lmo_verify_gumbel.argtypes = [f32p, C.c_int64, C.c_int32, f32p, C.c_float, i32p, f32p, f32p, C.c_uint64, C.c_uint32, C.c_uint32, i32p, f32p]
        _lib.lmo_sample_batch.restype = None
        _lib.lmo_sample_batch.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, f32p, C.c_float, i32p, C.c_int32, f32p, C.c_float,
                                          f32p, C.c_float, C.c_int32, i32p, C.c_int64, C.c_int64, C.c_float, C.c_float, C.c_int32, f32p,
                                          C.c_uint64, C.c_uint32, C.c_int64, i32p, f32p, f32p, C.c_int32]
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: Optional[np.ndarray], ty):
    return None if a is None else a.ctypes.data_as(C.POINTER(ty))


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even BF16 codes (uint16) of a float32 array (monolith/formats/fp.py:111-117)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def widen(logits: np.ndarray) -> np.ndarray:
    """FP32 view of a logits array given as BF16 codes (uint16) or float32."""
    return bf16_to_f32(logits) if logits.dtype == np.uint16 else _f32(logits)


def apply_penalties(z: np.ndarray, history, repetition_penalty: float = 1.0, presence_penalty: float = 0.0) -> np.ndarray:
    out = _f32(z).copy()
    h = np.ascontiguousarray(history, dtype=np.int32)
    lib().lmo_apply_penalties(_p(out, C.c_float), out.size, _p(h, C.c_int32), h.size, repetition_penalty, presence_penalty)
    return out


def argmax(z: np.ndarray) -> int:
    z = _f32(z)
    return int(lib().lmo_argmax(_p(z, C.c_float), z.size))


def thresholds(z: np.ndarray, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, min_p: float = 0.0,
               topp_in_topk: bool = False, stats: bool = False):
    """tau of one row (sampling_ref.thresholds); with ``stats`` also (vmax, kept mass, kept count)."""
    z = _f32(z)
    vmax, mass, cnt = C.c_float(), C.c_double(), C.c_int64()
    tau = lib().lmo_thresholds(_p(z, C.c_float), z.size, float(temperature), int(top_k), float(top_p), float(min_p), int(topp_in_topk),
                               C.byref(vmax), C.byref(mass), C.byref(cnt))
    return (float(tau), float(vmax.value), float(mass.value), int(cnt.value)) if stats else float(tau)


def uniform01(seed: int, step: int, t: int, i: int) -> float:
    return float(lib().lmo_uniform01(seed & (2**64 - 1), step, t, i))


def sample_gumbel(z: np.ndarray, *, seed: int, step: int, t: int = 0, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0,
                  min_p: float = 0.0, topp_in_topk: bool = False) -> Tuple[int, float]:
    """(token, best-minus-second key gap) of the reference's Gumbel-max draw (sampling_ref.sample)."""
    z = _f32(z)
    tau = thresholds(z, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, topp_in_topk=topp_in_topk)
    gap = C.c_float()
    tok = lib().lmo_sample_gumbel(_p(z, C.c_float), z.size, tau, float(temperature), seed & (2**64 - 1), step, t, C.byref(gap))
    return int(tok), float(gap.value)


def warped_probabilities(z: np.ndarray, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, min_p: float = 0.0,
                         topp_in_topk: bool = False) -> np.ndarray:
    z = _f32(z)
    tau = thresholds(z, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, topp_in_topk=topp_in_topk)
    out = np.empty(z.size, dtype=np.float64)
    lib().lmo_warped_probs(_p(z, C.c_float), z.size, tau, float(temperature), _p(out, C.c_double))
    return out


def sample_invcdf(z: np.ndarray, u: float, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, min_p: float = 0.0,
                  topp_in_topk: bool = False) -> int:
    z = _f32(z)
    tau = thresholds(z, temperature=float(np.float32(temperature)), top_k=top_k, top_p=float(np.float32(top_p)), min_p=float(np.float32(min_p)),
                     topp_in_topk=topp_in_topk)
    return int(lib().lmo_sample_invcdf(_p(z, C.c_float), z.size, tau, np.float32(temperature), np.float32(u), None))


def sample_invcdf_index_order(z: np.ndarray, u: float, *, temperature: float = 1.0, tau: float = -np.inf) -> int:
    """The inverse-CDF draw over {z >= tau} in ascending index order: what the verify step does when it draws from a row's own softmax."""
    z = _f32(z)
    return int(lib().lmo_sample_invcdf_index(_p(z, C.c_float), z.size, np.float32(tau), np.float32(temperature), np.float32(u), None))


def sample_batch(logits: np.ndarray, *, temperature, top_k=0, top_p=0.0, min_p=0.0, topp_in_topk=False, history=None,
                 repetition_penalty: float = 1.0, presence_penalty: float = 0.0, draw: str = "inverse_cdf", uniforms=None, seed: int = 0,
                 step: int = 0, row_offset: int = 0, n_threads: int = 1):
    """Every row of ``logits`` [rows, V] (uint16 BF16 codes or float32) through the full row pipeline: penalties,
    thresholds, draw. Knobs are scalars or per-row arrays. Returns (tokens int32, tau float32, stats float32 [rows, 2])."""
    logits = np.ascontiguousarray(logits)
    assert logits.ndim == 2 and logits.dtype in (np.uint16, np.float32)
    rows, vocab = logits.shape

    def knob(x, ty):
        a = np.asarray(x)
        return (None, ty(a)) if a.ndim == 0 else (np.ascontiguousarray(a, dtype=ty), ty(0))

    t_a, t_s = knob(temperature, np.float32)
    k_a, k_s = knob(top_k, np.int32)
    p_a, p_s = knob(top_p, np.float32)
    m_a, m_s = knob(min_p, np.float32)
    h = None if history is None else np.ascontiguousarray(history, dtype=np.int32)
    u = None if uniforms is None else np.ascontiguousarray(uniforms, dtype=np.float32)
    tok = np.empty(rows, dtype=np.int32)
    tau = np.empty(rows, dtype=np.float32)
    stats = np.zeros((rows, 2), dtype=np.float32)
    lib().lmo_sample_batch(logits.ctypes.data, 0 if logits.dtype == np.uint16 else 1, rows, vocab, vocab, _p(t_a, C.c_float), float(t_s),
                           _p(k_a, C.c_int32), int(k_s), _p(p_a, C.c_float), float(p_s), _p(m_a, C.c_float), float(m_s), int(topp_in_topk),
                           _p(h, C.c_int32), 0 if h is None else h.shape[1], 0 if h is None else h.shape[1], repetition_penalty, presence_penalty,
                           {"gumbel": 0, "inverse_cdf": 1}[draw], _p(u, C.c_float), seed & (2**64 - 1), step, row_offset, _p(tok, C.c_int32),
                           _p(tau, C.c_float), _p(stats, C.c_float), n_threads)
    return tok, tau, stats


def verify_greedy(target_logits: np.ndarray, draft_ids: Sequence[int]) -> Tuple[int, int, np.ndarray]:
    """(accept length, final token, the target's own pick per row) for greedy verification."""
    z = widen(target_logits)
    toks = np.array([argmax(z[r]) for r in range(z.shape[0])], dtype=np.int32)
    d = np.ascontiguousarray(draft_ids, dtype=np.int32)
    fin = C.c_int32()
    acc = lib().lmo_accept_greedy(_p(toks, C.c_int32), _p(d, C.c_int32), d.size, C.byref(fin))
    return int(acc), int(fin.value), toks


def confidence(hidden: np.ndarray, emb, w: np.ndarray, b: float, sts=None) -> np.ndarray:
    """conf [gamma] float32 of the DSpark confidence head; ``hidden`` [gamma, H] / ``emb`` [gamma, rank] as BF16 codes (uint16)."""
    h = np.ascontiguousarray(hidden, dtype=np.uint16)
    gamma, n_hidden = h.shape
    e = np.ascontiguousarray(emb, dtype=np.uint16) if emb is not None else np.zeros((gamma, 0), dtype=np.uint16)
    ww = _f32(w)
    out = np.zeros(gamma, dtype=np.float32)
    t = None if sts is None else _f32(sts)
    lib().lmo_confidence(_p(h, C.c_uint16), _p(e, C.c_uint16) if e.size else None, _p(ww, C.c_float), np.float32(b),
                         None if t is None else _p(t, C.c_float), gamma, n_hidden, e.shape[1], _p(out, C.c_float))
    return out


def draft_q(logits_row: np.ndarray, *, temperature: float, seed: int, step: int, position: int):
    """(token, vmax, integer mass, lse, gap between the two best Gumbel keys) of the drafter's draw at draft ``position``."""
    z = np.ascontiguousarray(widen(logits_row)).reshape(-1)
    vmax, lse, gap, mass = C.c_float(), C.c_float(), C.c_float(), C.c_uint64()
    tok = lib().lmo_draft_q(_p(z, C.c_float), z.shape[0], np.float32(temperature), seed, step, position, C.byref(vmax), C.byref(mass), C.byref(lse),
                            C.byref(gap))
    return int(tok), float(vmax.value), int(mass.value), float(lse.value), float(gap.value)


def draft_probs(logits_row: np.ndarray, *, temperature: float, vmax: float, mass: int) -> np.ndarray:
    """q(v) of one drafter row from its logits and statistics, float32 [V]."""
    z = np.ascontiguousarray(widen(logits_row)).reshape(-1)
    out = np.zeros(z.shape[0], dtype=np.float32)
    lib().lmo_draft_probs(_p(z, C.c_float), z.shape[0], np.float32(temperature), np.float32(vmax), mass, _p(out, C.c_float))
    return out


def verify_gumbel(target_logits: np.ndarray, draft_ids, draft_probs: np.ndarray, *, seed: int, step: int, temperature: float = 1.0, tau=None,
                  u_accept=None, row0: int = 0) -> Tuple[int, int, float]:
    """(accept length, final token, gap between the two best keys of the deciding draw) for stochastic verification with the
    reference's own randomness: accept stream 3000 + r (unless u_accept is given), Gumbel-max residual draw on stream 4000."""
    z = np.ascontiguousarray(widen(target_logits))
    n = len(draft_ids)
    assert z.shape[0] == n + 1
    d = np.ascontiguousarray(draft_ids, dtype=np.int32)
    q = _f32(draft_probs)
    ta = np.full(n + 1, -np.inf, dtype=np.float32) if tau is None else _f32(tau)
    ua = None if u_accept is None else _f32(u_accept)
    fin, gap = C.c_int32(), C.c_float()
    acc = lib().lmo_verify_gumbel(_p(z, C.c_float), z.shape[1], n, _p(ta, C.c_float), np.float32(temperature), _p(d, C.c_int32), _p(q, C.c_float),
                                  _p(ua, C.c_float) if ua is not None else None, int(seed) & (2**64 - 1), int(step), int(row0), C.byref(fin), C.byref(gap))
    return int(acc), int(fin.value), float(gap.value)


def verify_stochastic(target_logits: np.ndarray, draft_ids, draft_probs: np.ndarray, u_accept, u_final: float, *, temperature: float = 1.0,
                      tau=None) -> Tuple[int, int, np.ndarray]:
    """(accept length, final token, p(draft) per row) for stochastic verification with injected uniforms."""
    z = np.ascontiguousarray(widen(target_logits))
    n = len(draft_ids)
    assert z.shape[0] == n + 1
    d = np.ascontiguousarray(draft_ids, dtype=np.int32)
    q = _f32(draft_probs)
    ua = _f32(u_accept)
    ta = np.full(n + 1, -np.inf, dtype=np.float32) if tau is None else _f32(tau)
    fin = C.c_int32()
    pd = np.zeros(n, dtype=np.float32)
    acc = lib().lmo_verify_stochastic(_p(z, C.c_float), z.shape[1], n, _p(ta, C.c_float), np.float32(temperature), _p(d, C.c_int32),
                                      _p(q, C.c_float), _p(ua, C.c_float), np.float32(u_final), C.byref(fin), _p(pd, C.c_float))
    return int(acc), int(fin.value), pd
