"""StepState — the binary contract of GPU-resident generation control — and the scalar kernels that close a step.

``StepStateLayout`` mirrors ``monolith/core/step_state.py:28-119`` (same field order, offsets, padding, ``pack`` / ``unpack``), so a
state buffer written by either side reads the same. ``accept_scan``, ``verify_select`` and ``advance`` launch the CUDA
counterparts of the reference's ``accept_scan`` / ``verify_select`` (kernels/common/spec_ops.metal:108-195) and ``advance``
(kernels/common/advance.metal:15-37) on such a buffer; ``confidence`` is the DSpark confidence head that produces the
``conf`` vector ``verify_select`` reads (kernels/common/spec_ops.metal:85-106, ``conf_params`` monolith/kernels.py:802-808); parameters follow ``accept_params`` / ``select_params`` / ``advance_params``
(monolith/kernels.py:748-752, 814-835).
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import Dict, List, Mapping, Optional, Sequence, Union

import torch

from . import _lib

_FIELDS = [  # (name, struct code, count: int or "t" (t_max) or "g" (max(gamma_max, 1)))
    ("step", "I", 1), ("position", "I", 1), ("kv_len", "I", 1), ("t_this_step", "I", 1), ("pending_tokens", "i", "t"),
    ("rng_lo", "I", 1), ("rng_hi", "I", 1), ("anchor", "i", 1), ("gamma", "I", 1), ("draft_tokens", "i", "g"), ("confidence", "f", "g"),
    ("verify_len", "I", 1), ("accepted", "I", 1), ("checkpoint_index", "I", 1), ("drafter_ctx_len", "I", 1), ("done", "I", 1), ("error", "I", 1),
    ("ring_head", "I", 1), ("ring_tail", "I", 1), ("prefill_left", "I", 1), ("n_inject", "I", 1), ("stop_at", "I", 1), ("n_chain", "I", 1),
]

ERROR_RING_OVERFLOW, ERROR_CONTEXT_FULL, ERROR_BARRIER_TIMEOUT = 1, 2, 3


class StepStateLayout:
    """Field offsets of StepState for a given ``t_max`` / ``gamma_max``; 4-byte fields, total padded to 16 bytes."""

    def __init__(self, t_max: int = 8, gamma_max: int = 7) -> None:
        if t_max < 1 or gamma_max < 0 or t_max < gamma_max + 1:
            raise ValueError(f"StepStateLayout: need t_max >= gamma_max + 1 >= 1, got t_max={t_max}, gamma_max={gamma_max}")
        self.t_max, self.gamma_max = t_max, gamma_max
        g = max(gamma_max, 1)
        self.counts: Dict[str, int] = {}
        self.codes: Dict[str, str] = {}
        self.offsets: Dict[str, int] = {}
        off = 0
        for name, code, count in _FIELDS:
            n = t_max if count == "t" else g if count == "g" else count
            self.counts[name], self.codes[name], self.offsets[name] = n, code, off
            off += 4 * n
        self.size = (off + 15) // 16 * 16
        assert self.size == _lib.lib().lm_step_state_bytes(t_max, gamma_max)

    def offset(self, name: str) -> int:
        return self.offsets[name]

    def pack(self, values: Mapping[str, object]) -> bytes:
        buf = bytearray(self.size)
        for name, code, _ in _FIELDS:
            n = self.counts[name]
            raw = values.get(name, [] if n > 1 else 0)
            seq = list(raw) if n > 1 else [raw]
            if len(seq) > n:
                raise ValueError(f"StepState.{name}: {len(seq)} values for {n} slots")
            seq = seq + [0] * (n - len(seq))
            struct.pack_into("<" + code * n, buf, self.offsets[name], *seq)
        return bytes(buf)

    def unpack(self, data: bytes) -> Dict[str, object]:
        if len(data) < self.size:
            raise ValueError(f"StepState.unpack: need {self.size} bytes, got {len(data)}")
        out: Dict[str, object] = {}
        for name, code, _ in _FIELDS:
            n = self.counts[name]
            vals = struct.unpack_from("<" + code * n, data, self.offsets[name])
            out[name] = list(vals) if n > 1 else vals[0]
        return out

    def to_device(self, values: Mapping[str, object], device="cuda") -> torch.Tensor:
        return torch.frombuffer(bytearray(self.pack(values)), dtype=torch.uint8).to(device)

    def from_device(self, state: torch.Tensor) -> Dict[str, object]:
        return self.unpack(bytes(state.cpu().numpy().tobytes()))


def _args(layout: StepStateLayout, state: torch.Tensor, eos: Union[int, Sequence[int]], keep: List) -> "_lib.StepArgs":
    if state.dtype != torch.uint8 or not state.is_cuda or state.numel() < layout.size or not state.is_contiguous():
        raise ValueError("state must be a contiguous uint8 CUDA tensor of the layout's size")
    a = _lib.StepArgs()
    a.struct_size = C.sizeof(_lib.StepArgs)
    a.t_max, a.gamma_max, a.step_state = layout.t_max, layout.gamma_max, state.data_ptr()
    if isinstance(eos, int):
        a.eos = eos
    else:                                                     # a finite stop-token set (kernels.py:729-741); empty disables
        if any(type(t) is not int or not 0 <= t < 2**31 for t in eos):
            raise ValueError("EOS must be an integer or a sequence of nonnegative int32 token IDs")
        a.eos = -1
        if len(eos):
            lst = torch.tensor(sorted(set(eos)), dtype=torch.int32, device=state.device)
            keep.append(lst)
            a.eos_list, a.n_eos = lst.data_ptr(), lst.numel()
    a.stream = torch.cuda.current_stream(state.device).cuda_stream
    return a


def accept_scan(layout: StepStateLayout, state: torch.Tensor, tokens: torch.Tensor, ring: torch.Tensor, *, eos: Union[int, Sequence[int]] = -1,
                log: Optional[torch.Tensor] = None, ctx_cap: int = 0, lm: bool = False) -> None:
    """Greedy verify + commit on the device: ``tokens`` int32 [t], ``ring`` int64 [ring_cap] (slots ``(seq << 32) | token``),
    ``log`` optional int32 [log_cap]. In place on ``state`` / ``ring`` / ``log``; asynchronous."""
    keep: List = []
    a = _args(layout, state, eos, keep)
    if tokens.dtype != torch.int32 or ring.dtype != torch.int64 or not tokens.is_cuda or not ring.is_cuda:
        raise ValueError("tokens must be int32 and ring int64 CUDA tensors")
    a.tokens, a.ring, a.ring_cap = tokens.data_ptr(), ring.data_ptr(), ring.numel()
    if log is not None:
        a.log, a.log_cap = log.data_ptr(), log.numel()
    a.ctx_cap, a.lm = ctx_cap, int(lm)
    with torch.cuda.device(state.device):
        _lib.check(_lib.lib().lm_accept_scan(C.byref(a)), "lm_accept_scan")


def verify_select(layout: StepStateLayout, state: torch.Tensor, drafts: torch.Tensor, conf: torch.Tensor, *, gamma: int, threshold: float,
                  mode: int = 0, cost: Optional[Sequence[float]] = None, conf_log: Optional[torch.Tensor] = None, ctx_cap: int = 0, lm: bool = False,
                  t_max: Optional[int] = None) -> None:
    """Stage the next round: mode 0 = confident prefix (``threshold``), 1 = cost-aware (``cost[l]`` relative to ``cost[0] = 1``),
    2 = fixed length (``threshold`` = L). ``drafts`` int32 [gamma], ``conf`` float32 [gamma]; ``t_max`` = rows of the step program
    when smaller than the layout's (L is clamped to ``t_max - 1``)."""
    c = list(cost or [])
    if mode == 1 and (len(c) < 1 or len(c) > 16 or abs(c[0] - 1.0) > 1e-6 or any(x <= 0 for x in c)):
        raise ValueError("select_params: the cost rule needs 1..16 positive costs relative to cost[0] = 1")
    keep: List = []
    a = _args(layout, state, -1, keep)
    if drafts.dtype != torch.int32 or conf.dtype != torch.float32 or not drafts.is_cuda or not conf.is_cuda:
        raise ValueError("drafts must be int32 and conf float32 CUDA tensors")
    a.drafts, a.conf, a.gamma, a.threshold, a.mode = drafts.data_ptr(), conf.data_ptr(), gamma, float(threshold), mode
    c = c + [1.0] * (16 - len(c))
    a.cost = (C.c_float * 16)(*c)
    if conf_log is not None:
        a.conf_log, a.conf_log_cap = conf_log.data_ptr(), conf_log.numel() // 16
    a.ctx_cap, a.lm, a.t_limit = ctx_cap, int(lm), 0 if t_max is None else int(t_max)
    with torch.cuda.device(state.device):
        _lib.check(_lib.lib().lm_verify_select(C.byref(a)), "lm_verify_select")


def advance(layout: StepStateLayout, state: torch.Tensor, tokens: torch.Tensor, ring: torch.Tensor, *, eos: Union[int, Sequence[int]] = -1,
            ctx_cap: int = 0) -> None:
    """Close a plain decode step: publish the last row's token to the ring, advance the state."""
    keep: List = []
    a = _args(layout, state, eos, keep)
    a.tokens, a.ring, a.ring_cap, a.ctx_cap = tokens.data_ptr(), ring.data_ptr(), ring.numel(), ctx_cap
    with torch.cuda.device(state.device):
        _lib.check(_lib.lib().lm_advance(C.byref(a)), "lm_advance")


def confidence(hidden: torch.Tensor, emb: Optional[torch.Tensor], w: torch.Tensor, b: torch.Tensor, *, gamma: Optional[int] = None,
               sts: Optional[Sequence[float]] = None, out: Optional[torch.Tensor] = None, layout: Optional[StepStateLayout] = None,
               state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``conf[k] = sigmoid(bf16(bf16(w . [hidden_k ; emb_k]) + b) / sts[k])`` for ``k < gamma`` (default: every row of ``hidden``).

    ``hidden`` [rows, H] bfloat16, ``emb`` [rows, rank] bfloat16 or None, ``w`` [H + rank] float32, ``b`` [1] float32, ``sts`` up
    to 16 positive calibration temperatures (missing ones are 1). Returns float32 [rows]; positions >= gamma keep what ``out``
    held (zeros for a fresh tensor). With ``layout`` / ``state`` nothing is written once the state is done."""
    if hidden.dtype != torch.bfloat16 or not hidden.is_cuda or hidden.dim() != 2 or not hidden.is_contiguous():
        raise ValueError("hidden must be a contiguous bfloat16 CUDA tensor [rows, H]")
    rows, n_hidden = int(hidden.shape[0]), int(hidden.shape[1])
    gamma = rows if gamma is None else int(gamma)
    if not 0 <= gamma <= min(rows, 16):
        raise ValueError("gamma must lie in 0..min(rows, 16)")
    rank = 0
    if emb is not None:
        if emb.dtype != torch.bfloat16 or not emb.is_cuda or emb.dim() != 2 or emb.shape[0] < gamma or not emb.is_contiguous():
            raise ValueError("emb must be a contiguous bfloat16 CUDA tensor [rows, rank]")
        rank = int(emb.shape[1])
    t = [float(x) for x in (sts or [])]
    if len(t) > 16 or any(x <= 0 for x in t):
        raise ValueError("conf_params: up to 16 positive STS temperatures")
    dev = hidden.device
    w = w.to(device=dev, dtype=torch.float32).contiguous()
    b = b.to(device=dev, dtype=torch.float32).reshape(1).contiguous()
    if w.numel() != n_hidden + rank:
        raise ValueError("w must hold hidden + rank weights")
    conf = torch.zeros(rows, dtype=torch.float32, device=dev) if out is None else out
    a = _lib.ConfidenceArgs()
    a.struct_size = C.sizeof(_lib.ConfidenceArgs)
    a.gamma, a.hidden, a.rank = gamma, n_hidden, rank
    a.hidden_rows, a.emb_rows, a.w, a.b, a.out_conf = hidden.data_ptr(), (emb.data_ptr() if rank else None), w.data_ptr(), b.data_ptr(), conf.data_ptr()
    keep = [w, b]
    if t:
        ts = torch.tensor(t + [1.0] * (16 - len(t)), dtype=torch.float32, device=dev)
        keep.append(ts)
        a.sts = ts.data_ptr()
    if state is not None:
        a.step_state, a.t_max, a.gamma_max = state.data_ptr(), layout.t_max, layout.gamma_max
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().lm_confidence(C.byref(a)), "lm_confidence")
    return conf
