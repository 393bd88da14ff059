"""Multi-GPU layer of the generation-control path. One process per GPU (``torch.distributed``).

The reference is single-device, so both modes are new; each is defined by "same result as one GPU":

* row-sharded batches (``shard_rows``, ``sample_row_sharded``): rows are independent, every rank samples a contiguous block
  of rows with ``row_offset`` = its first global row, so Gumbel streams and tokens do not depend on the split. No
  collective on the data path.
* vocab-parallel sampling (``VocabParallelSampler``): every rank holds a contiguous shard of each row's vocabulary; per
  step it computes small records per row (maximum, FP64 softmass, top-k candidates of the shard, or of each piece the shard
  is cut into), all-gathers the records (the only exchange: a few KB per row and rank, NCCL over NVLink), and merges them
  identically on every rank. The kept set must lie inside the top-k candidates, so ``top_k >= 1`` is required. With
  ``exchange="peer"`` there is no collective: the records stay in memory that the peers have mapped (symmetric memory), a barrier
  over the ranks orders the local steps before the merges, and every merge reads the peers' records in place (the results of a call
  are then overwritten by the next call's).

The compute steps go through a backend object so that the exchange logic can be exercised on CPU ranks (gloo) with a
stand-in backend; the default backend is the CUDA library and nothing else ships.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .sampler import SampleOutput, SamplingParams, _check_logits, _dtype_code, _knob, _row_stride, sample


def shard_rows(total_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """(first row, row count) of ``rank``'s contiguous block; the remainder goes to the first ranks."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the group")
    base, extra = divmod(total_rows, world)
    return rank * base + min(rank, extra), base + (1 if rank < extra else 0)


def shard_vocab(vocab: int, rank: int, world: int) -> Tuple[int, int]:
    """(first index, width) of ``rank``'s contiguous vocabulary shard."""
    return shard_rows(vocab, rank, world)


def sample_row_sharded(local_logits: torch.Tensor, params: SamplingParams, *, first_row: int, history: Optional[torch.Tensor] = None,
                       uniforms: Optional[torch.Tensor] = None, step: int = 0, **kw) -> SampleOutput:
    """This rank's rows of a row-sharded batch: ``lm_sample`` with the global index of its first row. Per-row knobs,
    history and uniforms are this rank's slices."""
    return sample(local_logits, params, history=history, uniforms=uniforms, step=step, row_offset=first_row, **kw)


class CudaVocabBackend:
    """The two kernels of the vocab-parallel mode through the C ABI."""

    def candidate_cap(self, top_k: int) -> int:
        return int(_lib.lib().lm_vocab_candidate_cap(int(top_k)))

    def record_bytes(self, cap: int) -> int:
        return int(_lib.lib().lm_vocab_record_bytes(cap))

    def pieces(self, shards: int, cap: int, width: int, rows: int = 1) -> int:
        """Records per row that the local step leaves for a shard of ``width`` logits when ``shards`` GPUs take part in a call of ``rows`` rows."""
        return int(_lib.lib().lm_vocab_pieces(int(shards), int(cap), int(width), int(rows)))

    def _fill(self, a, p: SamplingParams, rows: int, dev, keep):
        ptr, s, t = _knob(p.temperature, rows, torch.float32, dev, "temperature"); a.temperature, a.temperature_s = ptr, float(s); keep.append(t)
        ptr, s, t = _knob(p.top_k, rows, torch.int32, dev, "top_k"); a.top_k, a.top_k_s = ptr, int(s); keep.append(t)
        ptr, s, t = _knob(p.top_p, rows, torch.float32, dev, "top_p"); a.top_p, a.top_p_s = ptr, float(s); keep.append(t)
        ptr, s, t = _knob(p.min_p, rows, torch.float32, dev, "min_p"); a.min_p, a.min_p_s = ptr, float(s); keep.append(t)

    def local(self, logits: torch.Tensor, shard_start: int, p: SamplingParams, cap: int, shards: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """This GPU's records, [pieces * rows, record bytes]: the shard is cut into as many pieces (each with a record per row) as
        the merge still takes together with the other ``shards - 1`` GPUs' pieces, so that the local step spreads over the GPU."""
        logits = _check_logits(logits)
        rows, width = logits.shape
        pieces = self.pieces(shards, cap, width, rows)
        rec = out if out is not None else torch.empty(pieces * rows, self.record_bytes(cap), dtype=torch.uint8, device=logits.device)
        if rec.shape != (pieces * rows, self.record_bytes(cap)) or rec.dtype != torch.uint8 or not rec.is_contiguous():
            raise ValueError("local: out must be a contiguous uint8 tensor [pieces * rows, record bytes]")
        a = _lib.VocabArgs()
        a.struct_size = C.sizeof(_lib.VocabArgs)
        a.dtype, a.logits, a.rows, a.vocab_local, a.row_stride, a.shard_start = _dtype_code(logits), logits.data_ptr(), rows, width, _row_stride(logits), shard_start
        a.cap, a.records, a.pieces = cap, rec.data_ptr(), pieces
        keep = []
        self._fill(a, p, rows, logits.device, keep)
        a.stream = torch.cuda.current_stream(logits.device).cuda_stream
        with torch.cuda.device(logits.device):
            _lib.check(_lib.lib().lm_vocab_local(C.byref(a)), "lm_vocab_local")
        return rec

    def merge(self, gathered: Optional[torch.Tensor], p: SamplingParams, cap: int, uniforms: Optional[torch.Tensor], step: int, row_offset: int, out=None,
              in_place=None):
        """``gathered`` [shards, rows, record bytes], or ``in_place`` = (device pointer to one 64-bit address per GPU, GPUs, pieces, rows,
        device): the records read where their GPUs left them (own memory and peer mappings) instead of a gathered copy."""
        a = _lib.VocabArgs()
        a.struct_size = C.sizeof(_lib.VocabArgs)
        if in_place is not None:
            ptrs, gpus, pieces, rows, dev = in_place
            a.rows, a.shards, a.cap, a.record_ptrs, a.pieces = rows, gpus * pieces, cap, int(ptrs), pieces
        else:
            shards, rows, _ = gathered.shape
            dev = gathered.device
            a.rows, a.shards, a.cap, a.records = rows, shards, cap, gathered.data_ptr()
        keep = []
        self._fill(a, p, rows, dev, keep)
        a.flags = _lib.FLAG_TOPP_IN_TOPK if p.topp_in_topk else 0
        a.draw = _lib.DRAW_GUMBEL if p.draw == "gumbel" else _lib.DRAW_INVERSE_CDF
        if uniforms is not None:
            uniforms = uniforms.to(device=dev, dtype=torch.float32).contiguous()
            a.uniforms = uniforms.data_ptr()
        a.seed, a.step, a.row_offset = int(p.seed) & (2**64 - 1), int(step) & 0xFFFFFFFF, int(row_offset)
        if out is not None:
            tokens, tau, status = out                                      # [rows] int32 / float32 / int32 on the records' device
        else:
            tokens = torch.empty(rows, dtype=torch.int32, device=dev)
            tau = torch.empty(rows, dtype=torch.float32, device=dev)
            status = torch.empty(rows, dtype=torch.int32, device=dev)
        a.out_tokens, a.out_tau, a.out_status = tokens.data_ptr(), tau.data_ptr(), status.data_ptr()
        a.stream = torch.cuda.current_stream(dev).cuda_stream
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().lm_vocab_merge(C.byref(a)), "lm_vocab_merge")
        return tokens, tau, status


class VocabParallelSampler:
    """Sampling with the vocabulary split over the ranks of ``group`` (shard order = rank order).

    ``sample(local_logits [rows, width of this rank's shard])`` returns the same tokens on every rank, equal to what a
    single GPU draws from the concatenated rows. ``params.top_k`` must be >= 1 everywhere; penalties are not supported
    in this mode.
    """

    def __init__(self, params: SamplingParams, vocab: int, group=None, backend=None, rank: Optional[int] = None, world: Optional[int] = None,
                 reuse_buffers: bool = False, exchange: str = "all_gather"):
        """``reuse_buffers``: keep the record, gather and result tensors between calls of the same shape (a decode loop: no allocation per
        step; a call's results are then overwritten by the next call's)."""
        self.params, self.vocab, self.group = params, int(vocab), group
        self._reuse, self._buffers = bool(reuse_buffers), {}
        # exchange = "peer": no collective at all. Every rank leaves its records in a buffer that its peers have mapped (symmetric
        # memory over NVLink), a barrier over the ranks on the stream orders the local steps before the merges, and every rank's merge
        # reads the peers' records in place. Two buffers in turn: a rank two steps ahead would need to pass a barrier that the rank
        # still reading has not reached. Falls back to the all-gather where symmetric memory cannot be set up.
        if exchange not in ("all_gather", "peer"):
            raise ValueError("exchange is 'all_gather' or 'peer'")
        self._exchange, self._peer, self._turn = exchange, {}, 0
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.backend = backend if backend is not None else CudaVocabBackend()
        if params.repetition_penalty != 1.0 or params.presence_penalty != 0.0:
            raise ValueError("vocab-parallel sampling does not take penalties")
        if not isinstance(params.temperature, torch.Tensor) and not params.temperature > 0:
            raise ValueError("vocab-parallel sampling needs temperature > 0 (greedy: use argmax per shard and a max-reduce)")
        k = params.top_k
        k_max = int(k.max()) if isinstance(k, torch.Tensor) else int(k)
        k_min = int(k.min()) if isinstance(k, torch.Tensor) else int(k)
        if k_min < 1:
            raise ValueError("vocab-parallel sampling needs top_k >= 1 on every row")
        self.cap = self.backend.candidate_cap(k_max)
        limit = (_lib.VOCAB_MAX_CANDIDATES // 1024) * (1024 // self.world) if self.world <= 64 else 0
        if self.cap > limit:
            raise ValueError(f"top_k {k_max} over {self.world} shards needs {self.cap} candidates per shard and row; the merge takes {limit}")
        self.shard_start, self.shard_width = shard_vocab(self.vocab, self.rank, self.world)
        # When the local step cuts the shard into pieces, a piece's record needs room for twice the top_k only (its bound lets a few
        # logits more than top_k through), not for top_k + 64: smaller records, a smaller all-gather.
        pieces_of = getattr(self.backend, "pieces", None)
        if pieces_of is not None and pieces_of(self.world, self.cap, self.shard_width) > 1:
            self.cap = min(self.cap, max(16, (2 * k_max + 7) // 8 * 8))

    def _peer_buffers(self, rows: int, dev):
        """Two record buffers of this rank that the peers have mapped, their handles, result tensors, pieces; None if that cannot be had."""
        key = (rows, dev)
        if key not in self._peer:
            made = None
            try:
                import torch.distributed._symmetric_memory as symm
                group = self.group if self.group is not None else dist.group.WORLD
                pieces = self.backend.pieces(self.world, self.cap, self.shard_width, rows)
                nbytes = pieces * rows * self.backend.record_bytes(self.cap)
                recs, handles = [], []
                for _ in range(2):
                    flat = symm.empty(nbytes, dtype=torch.uint8, device=dev)
                    handles.append(symm.rendezvous(flat, group))
                    recs.append(flat.view(pieces * rows, -1))
                out = (torch.empty(rows, dtype=torch.int32, device=dev), torch.empty(rows, dtype=torch.float32, device=dev),
                       torch.empty(rows, dtype=torch.int32, device=dev))
                made = (recs, handles, out, pieces)
            except Exception:                                                 # no symmetric memory here: the all-gather it is
                made = None
            self._peer[key] = made
        return self._peer[key]

    def sample(self, local_logits: torch.Tensor, uniforms: Optional[torch.Tensor] = None, step: int = 0, row_offset: int = 0) -> SampleOutput:
        if local_logits.shape[1] != self.shard_width:
            raise ValueError(f"this rank's shard is {self.shard_width} wide, got {local_logits.shape[1]}")
        if self.params.draw == "inverse_cdf" and uniforms is None:
            raise ValueError("draw='inverse_cdf' needs uniforms [rows]")
        rows = local_logits.shape[0]
        if self._exchange == "peer" and self.world > 1 and local_logits.is_cuda:
            peer = self._peer_buffers(rows, local_logits.device)
            if peer is not None:
                recs, handles, out, pieces = peer
                i = self._turn
                self._turn ^= 1
                self.backend.local(local_logits, self.shard_start, self.params, self.cap, self.world, out=recs[i])
                handles[i].barrier(channel=0)                                  # every rank's records of this step are written
                tokens, tau, status = self.backend.merge(None, self.params, self.cap, uniforms, step, row_offset, out=out,
                                                         in_place=(handles[i].buffer_ptrs_dev, self.world, pieces, rows, local_logits.device))
                return SampleOutput(tokens, tau=tau, status=status)
        kept = self._buffers.get((rows, local_logits.device)) if self._reuse else None
        if kept is None:
            rec = self.backend.local(local_logits, self.shard_start, self.params, self.cap, self.world)   # [pieces * rows, record bytes]
            flat = torch.empty(self.world * rec.shape[0], rec.shape[1], dtype=rec.dtype, device=rec.device)   # shard-major: [shard][piece][row]
            out = None
            if self._reuse and rec.is_cuda:
                out = (torch.empty(rows, dtype=torch.int32, device=rec.device), torch.empty(rows, dtype=torch.float32, device=rec.device),
                       torch.empty(rows, dtype=torch.int32, device=rec.device))
                self._buffers[(rows, local_logits.device)] = (rec, flat, out)
        else:
            rec, flat, out = kept
            self.backend.local(local_logits, self.shard_start, self.params, self.cap, self.world, out=rec)
        if self.world > 1:
            dist.all_gather_into_tensor(flat, rec, group=self.group)           # the one exchange of the step
        else:
            flat.copy_(rec)
        gathered = flat.view(-1, rows, rec.shape[1])                           # every piece of every shard is a shard of the merge
        if out is not None:
            tokens, tau, status = self.backend.merge(gathered, self.params, self.cap, uniforms, step, row_offset, out=out)
        else:
            tokens, tau, status = self.backend.merge(gathered, self.params, self.cap, uniforms, step, row_offset)
        return SampleOutput(tokens, tau=tau, status=status)
