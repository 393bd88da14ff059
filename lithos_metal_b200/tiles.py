"""Sampling from logits that arrive tile by tile: the host side of the lm_tile_* entry points.

The reference's vocabulary projection writes its logits [T, V] to memory and the sampler reads them back
(lm_head_forward, monolith/nn/lm_head.py:50-60; the sampler dispatches, monolith/kernels.py:720-775). A projection that
produces its output in column tiles hands each tile to :meth:`TileSampler.consume` instead and asks for the tokens at the end;
the full tensor never has to exist. The tokens are the ones :func:`lithos_metal_b200.sample` returns for the same logits,
history and knobs; rows this path does not take (stochastic rows without a top_k, undecidable boundaries) come back as token -1
with ``STATUS_TILE_DECLINED`` and the caller samples those from materialised logits.
"""
import ctypes as C
from typing import Optional

import torch

from . import _lib
from .sampler import SampleOutput, SamplingParams, _dtype_code, _knob, _row_stride, _state_fields


class TileSampler:
    """State for one sampling step over ``rows`` rows of a ``vocab``-wide projection whose logits arrive in column tiles.

    ``params`` holds the same knobs as :func:`sample`; ``temperature`` and ``top_k`` are needed while the tiles arrive, the
    rest at :meth:`finish`. ``history`` [rows, n] int32 token ids (with the penalties of ``params``) is noted by :meth:`begin`
    and applied to the logits as they arrive. The state (about 64 KiB per row, plus vocab / 8 bytes per row with a history)
    lives on ``device`` and is reused by :meth:`begin`.
    """

    def __init__(self, rows: int, vocab: int, params: SamplingParams, device: Optional[torch.device] = None,
                 history: Optional[torch.Tensor] = None) -> None:
        self.rows, self.vocab, self.params = int(rows), int(vocab), params
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if not params.repetition_penalty > 0:
            raise ValueError("repetition_penalty must be positive")
        self._pen = history is not None and history.shape[1] > 0 and not (params.repetition_penalty == 1.0 and params.presence_penalty == 0.0)
        L = _lib.lib()
        self._state = torch.empty(max(L.lm_tile_state_bytes(self.rows, self.vocab, 1 if self._pen else 0), 256), dtype=torch.uint8, device=self.device)
        self._t = _knob(params.temperature, self.rows, torch.float32, self.device, "temperature")
        self._k = _knob(params.top_k, self.rows, torch.int32, self.device, "top_k")
        self._history = None
        self.begin(history)

    def _args(self) -> "_lib.TileArgs":
        a = _lib.TileArgs()
        a.struct_size = C.sizeof(_lib.TileArgs)
        a.rows, a.vocab = self.rows, self.vocab
        a.temperature, a.temperature_s = self._t[0], float(self._t[1])
        a.top_k, a.top_k_s = self._k[0], int(self._k[1])
        a.state, a.state_bytes = self._state.data_ptr(), self._state.numel()
        a.stream = torch.cuda.current_stream(self.device).cuda_stream
        a.repetition_penalty, a.presence_penalty = float(self.params.repetition_penalty), float(self.params.presence_penalty)
        if self._history is not None:
            a.history, a.hist_len, a.hist_stride = self._history.data_ptr(), self._history.shape[1], _row_stride(self._history)
        return a

    def begin(self, history: Optional[torch.Tensor] = None) -> None:
        """Forget every tile seen so far and note the step's token history (stream-ordered). A sampler built without a history
        cannot be given one later (its state has no room for the ids)."""
        if history is not None and self._pen:
            if history.dim() != 2 or history.shape[0] != self.rows:
                raise ValueError("history must be [rows, n]")
            history = history.to(device=self.device, dtype=torch.int32)
            self._history = history if history.stride(1) == 1 else history.contiguous()
        elif history is not None and not (self.params.repetition_penalty == 1.0 and self.params.presence_penalty == 0.0) and history.shape[1] > 0:
            raise ValueError("this TileSampler was built without a history")
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lm_tile_begin(C.byref(self._args())), "lm_tile_begin")

    def consume(self, tile: torch.Tensor, col0: int) -> None:
        """Take ``tile`` [rows, cols] (bfloat16 or float32, CUDA, unit stride along columns) = the logits of columns
        ``col0 .. col0 + cols``. At most ``TILE_MAX_COLS`` columns per call; every column exactly once, in any order."""
        if tile.dim() != 2 or tile.shape[0] != self.rows or tile.stride(1) != 1 or not tile.is_cuda:
            raise ValueError("tile must be a CUDA tensor [rows, cols] with unit stride along columns")
        a = self._args()
        a.dtype = _dtype_code(tile)
        a.tile, a.tile_stride = tile.data_ptr(), _row_stride(tile)
        a.col0, a.cols = int(col0), tile.shape[1]
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lm_tile_consume(C.byref(a)), "lm_tile_consume")

    def finish(self, *, uniforms: Optional[torch.Tensor] = None, step: int = 0, row_offset: int = 0, return_tau: bool = False,
               return_status: bool = True, out: Optional[torch.Tensor] = None, step_state=None, return_vmax: bool = False) -> SampleOutput:
        """The tokens of the rows, as :func:`sample` would return them for the assembled logits; -1 with
        ``STATUS_TILE_DECLINED`` for rows to be sampled from materialised logits."""
        p, rows, dev = self.params, self.rows, self.device
        a = _lib.SampleArgs()
        a.struct_size = C.sizeof(_lib.SampleArgs)
        a.dtype, a.rows, a.vocab, a.row_stride = _lib.DTYPE_BF16, rows, self.vocab, self.vocab
        keep = []
        a.temperature, a.temperature_s = self._t[0], float(self._t[1])
        a.top_k, a.top_k_s = self._k[0], int(self._k[1])
        ptr, s, t = _knob(p.top_p, rows, torch.float32, dev, "top_p"); a.top_p, a.top_p_s = ptr, float(s); keep.append(t)
        ptr, s, t = _knob(p.min_p, rows, torch.float32, dev, "min_p"); a.min_p, a.min_p_s = ptr, float(s); keep.append(t)
        a.flags = _lib.FLAG_TOPP_IN_TOPK if p.topp_in_topk else 0
        a.draw = _lib.DRAW_GUMBEL if p.draw == "gumbel" else _lib.DRAW_INVERSE_CDF
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
        if return_status:
            res.status = torch.empty(rows, dtype=torch.int32, device=dev); a.out_status = res.status.data_ptr()
        if return_vmax:
            res.vmax = torch.empty(rows, dtype=torch.float32, device=dev); a.out_vmax = res.vmax.data_ptr()
            res.mass = torch.empty(rows, dtype=torch.int64, device=dev); a.out_mass = res.mass.data_ptr()
        a.stream = torch.cuda.current_stream(dev).cuda_stream
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().lm_tile_finish(C.byref(a), self._state.data_ptr(), self._state.numel()), "lm_tile_finish")
        return res
