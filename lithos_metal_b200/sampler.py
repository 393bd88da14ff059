"""Host side of the generation-control path: the reference's sampler front ends on top of the CUDA library.

Mirrors ``monolith/nn/sampler.py`` (``GreedySampler``, ``StochasticSampler``: same constructor arguments, same
``forward`` signatures, same ``ValueError`` for a non-positive temperature) and the functions of
``monolith/nn/sampling_ref.py`` (``thresholds``, ``sample``, ``warped_probabilities``: same keyword arguments), and
adds what the B200 path offers beyond them: per-row knobs, repetition / presence penalties, FP32 logits, and the
inverse-CDF draw from caller-supplied uniforms. PyTorch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple, Union

import numpy as np
import torch

from . import _lib

Knob = Union[float, int, torch.Tensor]


@dataclass
class SamplingParams:
    """The request knobs of the reference (``Session(...)`` keyword arguments, monolith/generate.py:81-90, and the
    ChatRequest fields, monolith/serving/protocol.py:80-83) plus the penalties and the draw mode."""
    temperature: Knob = 0.0            # 0 = greedy
    top_k: Knob = 0                    # 0 = off
    top_p: Knob = 0.0                  # on iff 0 < p < 1
    min_p: Knob = 0.0                  # 0 = off
    seed: int = 0
    topp_in_topk: bool = False         # top-p over the top-k set (the reference sets it under draft_sampling="sample")
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    draw: str = "gumbel"               # "gumbel" (the reference's counter-based Gumbel-max) or "inverse_cdf" (injected uniforms)
    exact_only: bool = False           # skip the candidate kernel for rows with a top_k (same results; for cross-checks)
    grid_limit: int = 0                # at most this many thread blocks (0 = one per SM); leaves SMs free for other streams


@dataclass
class SampleOutput:
    tokens: torch.Tensor               # int32 [rows]
    tau: Optional[torch.Tensor] = None     # float32 [rows]
    stats: Optional[torch.Tensor] = None   # float32 [rows, 2]: (max logit, kept softmax mass)
    probs: Optional[torch.Tensor] = None   # float32 [rows, vocab]
    status: Optional[torch.Tensor] = None  # int32 [rows] status bits
    vmax: Optional[torch.Tensor] = None    # float32 [rows]: the row's maximum logit (after penalties)
    mass: Optional[torch.Tensor] = None    # int64 [rows]: the kept set's fixed-point mass (with vmax: what the verify step can take over)


_workspaces: Dict[Tuple[int, str, int], torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int, kind: str = "sample") -> torch.Tensor:
    """A zero-filled scratch buffer per (device, kind, CUDA stream), grown on demand. The kernels keep live counters in their
    workspace and leave it clean, so calls that can overlap on the GPU must not share one: every stream gets its own, and a
    stream's calls are ordered. A buffer that is outgrown is handed back to the allocator only after the stream's pending work
    (``record_stream``)."""
    stream = torch.cuda.current_stream(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), kind, stream.cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            ws.record_stream(stream)
        with torch.cuda.stream(stream):
            ws = torch.zeros(max(nbytes, 4096), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _state_fields(step_state) -> Tuple[int, int, int, torch.Tensor]:
    """(pointer, t_max, gamma_max, keep-alive) of a ``(StepStateLayout, state tensor)`` pair."""
    layout, state = step_state
    if not state.is_cuda or state.dtype != torch.uint8 or state.numel() < layout.size or not state.is_contiguous():
        raise ValueError("step_state: (StepStateLayout, contiguous uint8 CUDA tensor of layout.size bytes)")
    return state.data_ptr(), int(layout.t_max), int(layout.gamma_max), state


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    if t.dtype == torch.float32:
        return _lib.DTYPE_F32
    raise TypeError(f"logits must be bfloat16 or float32, got {t.dtype}")


def _check_logits(logits: torch.Tensor) -> torch.Tensor:
    if not isinstance(logits, torch.Tensor) or not logits.is_cuda:
        raise RuntimeError("lithos_metal_b200 runs on CUDA tensors only (there is no CPU path)")
    if logits.dim() != 2:
        raise ValueError("logits must be [rows, vocab]")
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    return logits


def _row_stride(t: torch.Tensor) -> int:
    """Elements between consecutive rows (a single-row view may carry any stride: it is never used)."""
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _knob(x: Knob, rows: int, dtype: torch.dtype, device: torch.device, name: str):
    """(device pointer or None, scalar, keep-alive tensor) for a scalar or per-row knob."""
    if isinstance(x, torch.Tensor):
        if x.numel() != rows:
            raise ValueError(f"{name}: expected {rows} per-row values, got {x.numel()}")
        t = x.to(device=device, dtype=dtype).contiguous()
        return t.data_ptr(), 0, t
    return None, x, None


def sample(logits: torch.Tensor, params: Optional[SamplingParams] = None, *, history: Optional[torch.Tensor] = None,
           uniforms: Optional[torch.Tensor] = None, step: int = 0, row_offset: int = 0, return_tau: bool = False, return_stats: bool = False,
           return_probs: bool = False, return_status: bool = False, out: Optional[torch.Tensor] = None, step_state=None, return_vmax: bool = False,
           **knobs: Any) -> SampleOutput:
    """One sampling step over every row of ``logits`` [rows, vocab] (bfloat16 or float32, CUDA).

    ``params`` (or the same fields as keyword arguments) hold scalar knobs or per-row tensors. ``history`` [rows, n]
    int32 token ids enables the penalties; ``uniforms`` [rows] float32 feeds the inverse-CDF draw; ``row_offset`` is
    the global index of row 0 (the Gumbel stream id of row r is ``row_offset + r``). ``step_state`` = ``(StepStateLayout,
    state tensor)`` hands the noise seed, the step and the number of active rows to the device-side state, as the reference's
    kernels read them (rows beyond ``t_this_step`` and a finished state leave ``out`` untouched): a captured CUDA graph then
    draws fresh noise on every replay. Asynchronous on the current stream; nothing is copied to the host.
    """
    p = params if params is not None else SamplingParams(**knobs)
    if params is not None and knobs:
        raise TypeError("pass either params or knob keyword arguments, not both")
    logits = _check_logits(logits)
    rows, vocab = logits.shape
    dev = logits.device
    if p.draw not in ("gumbel", "inverse_cdf"):
        raise ValueError("draw must be 'gumbel' or 'inverse_cdf'")
    if not isinstance(p.temperature, torch.Tensor) and not p.temperature >= 0:
        raise ValueError("temperature must be >= 0 (0 selects greedy)")
    if not p.repetition_penalty > 0:
        raise ValueError("repetition_penalty must be positive")
    a = _lib.SampleArgs()
    a.struct_size = C.sizeof(_lib.SampleArgs)
    a.dtype = _dtype_code(logits)
    a.logits, a.rows, a.vocab, a.row_stride = logits.data_ptr(), rows, vocab, _row_stride(logits)
    keep = []
    ptr, s, t = _knob(p.temperature, rows, torch.float32, dev, "temperature"); a.temperature, a.temperature_s = ptr, float(s); keep.append(t)
    ptr, s, t = _knob(p.top_k, rows, torch.int32, dev, "top_k"); a.top_k, a.top_k_s = ptr, int(s); keep.append(t)
    ptr, s, t = _knob(p.top_p, rows, torch.float32, dev, "top_p"); a.top_p, a.top_p_s = ptr, float(s); keep.append(t)
    ptr, s, t = _knob(p.min_p, rows, torch.float32, dev, "min_p"); a.min_p, a.min_p_s = ptr, float(s); keep.append(t)
    a.flags = (_lib.FLAG_TOPP_IN_TOPK if p.topp_in_topk else 0) | (_lib.FLAG_EXACT_ONLY if p.exact_only else 0) | ((int(p.grid_limit) & 0xFF) << 8)
    a.draw = _lib.DRAW_GUMBEL if p.draw == "gumbel" else _lib.DRAW_INVERSE_CDF
    if history is not None:
        if history.dim() != 2 or history.shape[0] != rows:
            raise ValueError("history must be [rows, n]")
        history = history.to(device=dev, dtype=torch.int32)
        if history.stride(1) != 1:
            history = history.contiguous()
        a.history, a.hist_len, a.hist_stride = history.data_ptr(), history.shape[1], _row_stride(history)
    a.repetition_penalty, a.presence_penalty = float(p.repetition_penalty), float(p.presence_penalty)
    stochastic = isinstance(p.temperature, torch.Tensor) or p.temperature > 0
    if p.draw == "inverse_cdf" and stochastic:
        if uniforms is None:
            raise ValueError("draw='inverse_cdf' needs uniforms [rows]")
        uniforms = uniforms.to(device=dev, dtype=torch.float32).contiguous()
        if uniforms.numel() != rows:
            raise ValueError("uniforms must hold one value per row")
        a.uniforms = uniforms.data_ptr()
    a.seed, a.step, a.row_offset = int(p.seed) & (2**64 - 1), int(step) & 0xFFFFFFFF, int(row_offset)
    if step_state is not None:
        a.step_state, a.t_max, a.gamma_max, st_keep = _state_fields(step_state)
        keep.append(st_keep)
    tokens = out if out is not None else torch.empty(rows, dtype=torch.int32, device=dev)
    if tokens.dtype != torch.int32 or tokens.numel() != rows or not tokens.is_contiguous():
        raise ValueError("out must be a contiguous int32 tensor with one entry per row")
    res = SampleOutput(tokens)
    a.out_tokens = tokens.data_ptr()
    if return_tau:
        res.tau = torch.empty(rows, dtype=torch.float32, device=dev); a.out_tau = res.tau.data_ptr()
    if return_stats:
        res.stats = torch.empty(rows, 2, dtype=torch.float32, device=dev); a.out_stats = res.stats.data_ptr()
    if return_probs:
        res.probs = torch.empty(rows, vocab, dtype=torch.float32, device=dev); a.out_probs, a.probs_stride = res.probs.data_ptr(), vocab
    if return_status:
        res.status = torch.empty(rows, dtype=torch.int32, device=dev); a.out_status = res.status.data_ptr()
    if return_vmax:
        res.vmax = torch.empty(rows, dtype=torch.float32, device=dev); a.out_vmax = res.vmax.data_ptr()
        res.mass = torch.empty(rows, dtype=torch.int64, device=dev); a.out_mass = res.mass.data_ptr()
    L = _lib.lib()
    ws = _workspace(dev, L.lm_workspace_bytes(rows, vocab))
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        _lib.check(L.lm_sample(C.byref(a)), "lm_sample")
    return res


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy pick of every row: int32 [rows], ties -> lowest index."""
    logits = _check_logits(logits)
    rows, vocab = logits.shape
    tokens = out if out is not None else torch.empty(rows, dtype=torch.int32, device=logits.device)
    L = _lib.lib()
    ws = _workspace(logits.device, L.lm_workspace_bytes(rows, vocab))
    with torch.cuda.device(logits.device):
        _lib.check(L.lm_argmax(logits.data_ptr(), _dtype_code(logits), rows, vocab, _row_stride(logits), tokens.data_ptr(), ws.data_ptr(), ws.numel(),
                               torch.cuda.current_stream(logits.device).cuda_stream), "lm_argmax")
    return tokens


class GreedySampler:
    """``monolith.nn.sampler.GreedySampler``: ``forward(logits [T, V]) -> int64 [T]``, argmax of the logits widened
    to float32, ties -> lowest index."""

    def __init__(self, prefix: str = "") -> None:
        self.prefix = prefix

    def forward(self, logits: torch.Tensor) -> torch.Tensor:
        return argmax(logits).to(torch.int64)

    __call__ = forward


class StochasticSampler:
    """``monolith.nn.sampler.StochasticSampler``: temperature, top-k, top-p and min-p thresholds and the Gumbel-max
    draw keyed by (seed, step, position, index); ``forward(logits [T, V], step=0) -> int64 [T]``."""

    def __init__(self, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, min_p: float = 0.0, seed: int = 0, *, prefix: str = "",
                 topp_in_topk: bool = False) -> None:
        if temperature <= 0:
            raise ValueError("StochasticSampler: temperature must be positive; use GreedySampler for greedy decoding")
        self.prefix = prefix
        self.temperature, self.top_k, self.top_p, self.min_p, self.seed = float(temperature), int(top_k), float(top_p), float(min_p), int(seed)
        self.topp_in_topk = bool(topp_in_topk)

    def params(self) -> SamplingParams:
        return SamplingParams(self.temperature, self.top_k, self.top_p, self.min_p, self.seed, self.topp_in_topk, draw="gumbel")

    def forward(self, logits: torch.Tensor, step: int = 0) -> torch.Tensor:
        return sample(logits, self.params(), step=step).tokens.to(torch.int64)

    __call__ = forward


# ---- the functions of monolith/nn/sampling_ref.py, computed on the GPU for one row ---------------------------------

def _row(logits) -> torch.Tensor:
    t = torch.as_tensor(np.asarray(logits, dtype=np.float32)) if not isinstance(logits, torch.Tensor) else logits
    t = t.reshape(1, -1)
    return t if t.is_cuda else t.cuda()


def thresholds(logits, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, min_p: float = 0.0, topp_in_topk: bool = False) -> float:
    """``sampling_ref.thresholds``: the logit threshold tau of one row (-inf if nothing is enabled)."""
    r = sample(_row(logits), SamplingParams(temperature, top_k, top_p, min_p, 0, topp_in_topk), return_tau=True)
    return float(r.tau[0])


def sample_row(logits, *, seed: int, step: int, t: int = 0, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, min_p: float = 0.0,
               topp_in_topk: bool = False) -> int:
    """``sampling_ref.sample``: the token drawn for one position (Gumbel-max, stream id ``t``)."""
    r = sample(_row(logits), SamplingParams(temperature, top_k, top_p, min_p, seed, topp_in_topk), step=step, row_offset=t)
    return int(r.tokens[0])


def warped_probabilities(logits, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, min_p: float = 0.0) -> np.ndarray:
    """``sampling_ref.warped_probabilities``: the distribution the draws follow (float32 here, float64 there)."""
    r = sample(_row(logits), SamplingParams(temperature, top_k, top_p, min_p), return_probs=True)
    return r.probs[0].cpu().numpy()
