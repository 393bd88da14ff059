"""DSpark speculative verification on the GPU: one launch checks ``n`` drafted tokens against ``n + 1`` rows of
target logits. Stands in for the accept chain of a speculative round in the reference (greedy: the prefix match of
``accept_scan``, kernels/common/spec_ops.metal:162-165; sampled drafts: ``spec_q_accept`` and the residual draw,
kernels/common/sample.metal:279-347). ``draft_q`` is the drafter's side of such a round: the draw of draft k from the
drafter's logits plus the row statistics that let ``verify`` evaluate q_k later (``draft_q_partial`` / ``draft_q_final``,
kernels/common/sample.metal:212-269)."""
from __future__ import annotations

import ctypes as C
from typing import NamedTuple, Optional, Tuple

import torch

from . import _lib
from .sampler import _check_logits, _dtype_code, _row_stride, _state_fields, _workspace


class DraftQ(NamedTuple):
    """What the drafter keeps of its sampled drafts: tokens int32 [n], ``lse`` float32 [n] (log sum exp(z / T), the
    reference's q_lse), and the exact row statistics ``vmax`` float32 [n] / ``mass`` int64 [n] that ``verify`` evaluates
    q from; ``status`` int32 [n] (LM_STATUS_NEAR_TIE / LM_STATUS_NAN bits); ``q_logits`` the copy of the rows, if asked for."""
    tokens: torch.Tensor
    lse: torch.Tensor
    vmax: torch.Tensor
    mass: torch.Tensor
    status: torch.Tensor
    q_logits: Optional[torch.Tensor]


def draft_q(logits: torch.Tensor, *, temperature: float, seed: int = 0, step: int = 0, first_position: int = 0, copy_logits: bool = False,
            step_state=None) -> DraftQ:
    """The drafter's draw for draft positions ``first_position .. first_position + rows - 1``, one logits row each
    (``logits`` [rows, V] bfloat16/float32, rows <= 16): ``argmax_i(z_i * float32(1/T) + gumbel(seed, step, 2000 + position, i))``,
    the unfiltered softmax at ``temperature`` as the reference's drafter samples it. ``step_state`` = ``(StepStateLayout, state)``
    takes seed and step from the device-side state instead (nothing is written once it is done). Asynchronous on the current stream."""
    if not temperature > 0:
        raise ValueError("temperature must be positive")
    logits = _check_logits(logits)
    dev, rows, vocab = logits.device, int(logits.shape[0]), int(logits.shape[1])
    if not 1 <= rows <= _lib.MAX_DRAFT + 1:
        raise ValueError(f"1..{_lib.MAX_DRAFT + 1} rows")
    a = _lib.DraftQArgs()
    a.struct_size = C.sizeof(_lib.DraftQArgs)
    a.dtype, a.rows, a.first_position = _dtype_code(logits), rows, int(first_position)
    a.logits, a.vocab, a.row_stride = logits.data_ptr(), vocab, _row_stride(logits)
    a.temperature, a.seed, a.step = float(temperature), int(seed) & (2**64 - 1), int(step)
    tokens = torch.empty(rows, dtype=torch.int32, device=dev)
    lse, vmax = torch.empty(rows, dtype=torch.float32, device=dev), torch.empty(rows, dtype=torch.float32, device=dev)
    mass, status = torch.empty(rows, dtype=torch.int64, device=dev), torch.empty(rows, dtype=torch.int32, device=dev)
    a.out_tokens, a.out_lse, a.out_vmax, a.out_mass, a.out_status = tokens.data_ptr(), lse.data_ptr(), vmax.data_ptr(), mass.data_ptr(), status.data_ptr()
    q_logits = None
    if copy_logits:
        q_logits = torch.empty(rows, vocab, dtype=logits.dtype, device=dev)
        a.out_q_logits, a.q_logits_stride = q_logits.data_ptr(), vocab
    L = _lib.lib()
    ws = _workspace(dev, L.lm_verify_workspace_bytes(rows, vocab), "verify")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    if step_state is not None:
        a.step_state, a.t_max, a.gamma_max, _keep = _state_fields(step_state)
    with torch.cuda.device(dev):
        _lib.check(L.lm_draft_q(C.byref(a)), "lm_draft_q")
    return DraftQ(tokens, lse, vmax, mass, status, q_logits)


def verify(target_logits: torch.Tensor, draft_ids: Optional[torch.Tensor], draft_probs: Optional[torch.Tensor] = None, uniforms: Optional[torch.Tensor] = None,
           u_resample: Optional[torch.Tensor] = None, mode: str = "greedy", *, temperature: float = 1.0, tau: Optional[torch.Tensor] = None,
           return_p_draft: bool = False, draft_logits: Optional[torch.Tensor] = None, draft_stats: Optional[DraftQ] = None,
           commit: Optional[dict] = None, seed: int = 0, step: int = 0, residual_draw: str = "inverse_cdf", step_state=None,
           out: Optional[torch.Tensor] = None, wait_limit: int = 0, selftest: int = 0, target_vmax: Optional[torch.Tensor] = None,
           target_mass: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, ...]:
    """``(accept_len [1], final_token [1], tokens [n + 1])`` as int32 CUDA tensors (plus ``p_draft [n]`` on request).

    ``target_logits`` [n + 1, V] bfloat16/float32; ``draft_ids`` [n] int32; stochastic mode also takes the drafter's
    probabilities ``draft_probs`` [n, V] float32, the accept uniforms ``uniforms`` [n] and the resample uniform
    ``u_resample`` [1], all in [0, 1); ``tau`` [n + 1] optionally restricts every row to its kept set (``sample(...,
    return_tau=True)``). Instead of ``draft_probs`` the drafter's distribution may be given the way the reference keeps it:
    ``draft_logits`` [n, V] bfloat16 (the rows ``draft_q`` sampled from) with ``draft_stats`` = what ``draft_q`` returned
    for them at the same temperature. ``commit`` closes the round in the same launch: a dict with ``layout`` (StepStateLayout),
    ``state`` and ``ring`` tensors and optionally ``eos``, ``log``, ``ctx_cap``, ``lm`` — the arguments of ``accept_scan``, which
    then runs on the verified tokens inside the verify kernel (the state must describe this round: ``verify_len == n``,
    ``t_this_step == n + 1``). Without ``uniforms`` / ``u_resample`` the kernel takes the reference's counter-based noise of
    ``(seed, step)`` (accept stream 3000 + r, resample stream 4000); ``residual_draw="gumbel"`` selects the reference's
    Gumbel form of the final draw. ``step_state`` = ``(StepStateLayout, state)`` hands the round itself to the device-side state:
    verify length, drafts (``draft_ids`` may then be None: ``target_logits`` holds ``layout.t_max`` rows), seed and step are read
    there, and a finished state leaves the outputs untouched. ``out`` (int32 [rows + 2]) receives accept, final and the tokens.
    ``target_vmax`` (float32, one value per target row; stochastic mode) hands the kernel the exact row maxima the sampler already knows, as the
    reference's verify kernels get them, and spares the launch one exchange between its thread blocks; ``target_mass`` (int64, the kept sets'
    fixed-point masses for the same thresholds and temperature: ``sample(..., return_vmax=True).mass``) spares it the second.
    ``wait_limit`` / ``selftest`` exercise the kernel's bounded waits (tests only). Asynchronous on the current stream.
    """
    if mode not in ("greedy", "stochastic"):
        raise ValueError("mode must be 'greedy' or 'stochastic'")
    target_logits = _check_logits(target_logits)
    dev = target_logits.device
    if residual_draw not in ("inverse_cdf", "gumbel"):
        raise ValueError("residual_draw must be 'inverse_cdf' or 'gumbel'")
    n = int(draft_ids.numel()) if draft_ids is not None else int(target_logits.shape[0]) - 1
    if draft_ids is None and step_state is None:
        raise ValueError("draft_ids may only be omitted with a step_state")
    if target_logits.shape[0] != n + 1:
        raise ValueError("target_logits must have one row per draft plus the bonus row")
    if not 1 <= n <= _lib.MAX_DRAFT:
        raise ValueError(f"1..{_lib.MAX_DRAFT} drafts")
    a = _lib.VerifyArgs()
    a.struct_size = C.sizeof(_lib.VerifyArgs)
    a.mode = _lib.VERIFY_GREEDY if mode == "greedy" else _lib.VERIFY_STOCHASTIC
    a.dtype, a.n_draft = _dtype_code(target_logits), n
    a.target_logits, a.vocab, a.row_stride = target_logits.data_ptr(), target_logits.shape[1], _row_stride(target_logits)
    keep = []
    if draft_ids is not None:
        draft_ids = draft_ids.to(device=dev, dtype=torch.int32).contiguous()
        a.draft_ids = draft_ids.data_ptr()
        keep.append(draft_ids)
    a.seed, a.step = int(seed) & (2**64 - 1), int(step) & 0xFFFFFFFF
    a.residual_draw = _lib.RESIDUAL_GUMBEL if residual_draw == "gumbel" else _lib.RESIDUAL_INVERSE_CDF
    a.wait_limit, a.selftest = int(wait_limit), int(selftest)
    if target_vmax is not None:
        target_vmax = target_vmax.to(device=dev, dtype=torch.float32).contiguous()
        if target_vmax.numel() != target_logits.shape[0]:
            raise ValueError("target_vmax must hold one value per target row")
        a.target_vmax = target_vmax.data_ptr()
        if target_mass is not None:
            target_mass = target_mass.to(device=dev, dtype=torch.int64).contiguous()
            if target_mass.numel() != target_logits.shape[0]:
                raise ValueError("target_mass must hold one value per target row")
            a.target_mass = target_mass.data_ptr()
    if step_state is not None:
        a.step_state, a.t_max, a.gamma_max, st_keep = _state_fields(step_state)
        keep.append(st_keep)
    if mode == "stochastic":
        if draft_probs is None and (draft_logits is None or draft_stats is None):
            raise ValueError("stochastic verification needs draft_probs (or draft_logits + draft_stats)")
        if not temperature > 0:
            raise ValueError("temperature must be positive")
        if draft_probs is None:
            if draft_logits.shape != (n, target_logits.shape[1]) or draft_logits.dtype != torch.bfloat16 or not draft_logits.is_cuda:
                raise ValueError("draft_logits must be bfloat16 CUDA [n, V]")
            if draft_logits.stride(1) != 1:
                draft_logits = draft_logits.contiguous()
            q_vmax, q_mass = draft_stats.vmax[:n].contiguous(), draft_stats.mass[:n].contiguous()
            if q_vmax.numel() != n or q_mass.numel() != n:
                raise ValueError("draft_stats must hold one entry per draft")
            a.draft_logits, a.draft_logits_stride = draft_logits.data_ptr(), _row_stride(draft_logits)
            a.draft_vmax, a.draft_mass = q_vmax.data_ptr(), q_mass.data_ptr()
            keep += [draft_logits, q_vmax, q_mass]
        elif draft_probs.shape != (n, target_logits.shape[1]) or draft_probs.dtype != torch.float32 or not draft_probs.is_cuda:
            raise ValueError("draft_probs must be float32 CUDA [n, V]")
        elif draft_probs.stride(1) != 1:
            draft_probs = draft_probs.contiguous()
        if uniforms is not None:
            uniforms = uniforms.to(device=dev, dtype=torch.float32).contiguous()
            if uniforms.numel() != n:
                raise ValueError("uniforms must hold one value per draft")
            a.u_accept = uniforms.data_ptr()
        if u_resample is not None:
            u_resample = u_resample.to(device=dev, dtype=torch.float32).reshape(1).contiguous()
            a.u_final = u_resample.data_ptr()
        if draft_probs is not None:
            a.draft_probs, a.probs_stride = draft_probs.data_ptr(), _row_stride(draft_probs)
            keep.append(draft_probs)
        a.temperature = float(temperature)
        keep += [uniforms, u_resample]
        if tau is not None:
            tau = tau.to(device=dev, dtype=torch.float32).contiguous()
            if tau.numel() != n + 1:
                raise ValueError("tau must hold one value per row")
            a.tau = tau.data_ptr()
    if out is None:
        out = torch.empty(n + 3, dtype=torch.int32, device=dev)
    elif out.dtype != torch.int32 or out.numel() != n + 3 or not out.is_cuda or not out.is_contiguous():
        raise ValueError("out must be a contiguous int32 CUDA tensor with n + 3 entries")
    a.out_accept, a.out_final, a.out_tokens = out.data_ptr(), out.data_ptr() + 4, out.data_ptr() + 8
    p_draft = None
    if return_p_draft and mode == "stochastic":
        p_draft = torch.empty(n, dtype=torch.float32, device=dev)
        a.out_p_draft = p_draft.data_ptr()
    if commit is not None:
        from . import step_state as _ss
        c = _ss._args(commit["layout"], commit["state"], commit.get("eos", -1), keep)
        ring, log = commit["ring"], commit.get("log")
        if ring.dtype != torch.int64 or not ring.is_cuda:
            raise ValueError("ring must be an int64 CUDA tensor")
        c.ring, c.ring_cap = ring.data_ptr(), ring.numel()
        if log is not None:
            c.log, c.log_cap = log.data_ptr(), log.numel()
        c.ctx_cap, c.lm = int(commit.get("ctx_cap", 0)), int(bool(commit.get("lm", False)))
        keep.append(c)
        a.commit = C.addressof(c)
    L = _lib.lib()
    ws = _workspace(dev, L.lm_verify_workspace_bytes(n, target_logits.shape[1]), "verify")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        _lib.check(L.lm_verify(C.byref(a)), "lm_verify")
    res = (out[0:1], out[1:2], out[2:])
    return res + (p_draft,) if p_draft is not None else res
