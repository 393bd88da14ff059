"""ctypes binding of the CUDA library (C ABI in include/lithos_b200.h). There is no CPU fallback: if the shared
object is missing and cannot be built, importing the binding raises."""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

LM_OK = 0
DTYPE_BF16, DTYPE_F32 = 0, 1
DRAW_GUMBEL, DRAW_INVERSE_CDF = 0, 1
ABI_VERSION = 3                      # LM_ABI_VERSION of include/lithos_b200.h this binding was written against
FLAG_TOPP_IN_TOPK = 1
FLAG_EXACT_ONLY = 2
VERIFY_GREEDY, VERIFY_STOCHASTIC = 0, 1
RESIDUAL_INVERSE_CDF, RESIDUAL_GUMBEL = 0, 1
VERIFY_SELFTEST_WITHHOLD = 1
STATUS_GENERIC_PATH, STATUS_NAN, STATUS_NEAR_TIE, STATUS_TOPP_EDGE, STATUS_OVERFLOW = 1, 2, 4, 8, 32
STATUS_CANDIDATE_PATH = 64
STATUS_TILE_DECLINED = 128
STATUS_SLICED_PATH = 256
TILE_MAX_COLS = 2048
VOCAB_MAX_CANDIDATES = 8192
MAX_DRAFT = 15
MAX_VOCAB = 1048576
ARGMAX_STATIC_MAX_ROWS = 4096


class SampleArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("logits", C.c_void_p), ("rows", C.c_int64), ("vocab", C.c_int64),
        ("row_stride", C.c_int64),
        ("temperature", C.c_void_p), ("temperature_s", C.c_float), ("top_k", C.c_void_p), ("top_k_s", C.c_int32),
        ("top_p", C.c_void_p), ("top_p_s", C.c_float), ("min_p", C.c_void_p), ("min_p_s", C.c_float),
        ("flags", C.c_uint32), ("draw", C.c_int32),
        ("history", C.c_void_p), ("hist_len", C.c_int64), ("hist_stride", C.c_int64), ("repetition_penalty", C.c_float),
        ("presence_penalty", C.c_float),
        ("uniforms", C.c_void_p), ("seed", C.c_uint64), ("step", C.c_uint32), ("row_offset", C.c_int64),
        ("out_tokens", C.c_void_p), ("out_tau", C.c_void_p), ("out_stats", C.c_void_p), ("out_probs", C.c_void_p), ("probs_stride", C.c_int64),
        ("out_status", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
        ("step_state", C.c_void_p), ("t_max", C.c_int32), ("gamma_max", C.c_int32), ("out_vmax", C.c_void_p), ("out_mass", C.c_void_p),
    ]


class TileArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("tile", C.c_void_p), ("rows", C.c_int64), ("vocab", C.c_int64),
        ("tile_stride", C.c_int64), ("col0", C.c_int64), ("cols", C.c_int64),
        ("temperature", C.c_void_p), ("temperature_s", C.c_float), ("top_k", C.c_void_p), ("top_k_s", C.c_int32),
        ("state", C.c_void_p), ("state_bytes", C.c_size_t), ("stream", C.c_void_p),
        ("history", C.c_void_p), ("hist_len", C.c_int64), ("hist_stride", C.c_int64), ("repetition_penalty", C.c_float), ("presence_penalty", C.c_float),
    ]


class VerifyArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("mode", C.c_int32), ("dtype", C.c_int32), ("n_draft", C.c_int32), ("target_logits", C.c_void_p),
        ("vocab", C.c_int64), ("row_stride", C.c_int64), ("draft_ids", C.c_void_p), ("draft_probs", C.c_void_p), ("probs_stride", C.c_int64),
        ("temperature", C.c_float), ("tau", C.c_void_p), ("u_accept", C.c_void_p), ("u_final", C.c_void_p),
        ("out_accept", C.c_void_p), ("out_final", C.c_void_p), ("out_tokens", C.c_void_p), ("out_p_draft", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
        ("draft_logits", C.c_void_p), ("draft_logits_stride", C.c_int64), ("draft_vmax", C.c_void_p), ("draft_mass", C.c_void_p),
        ("commit", C.c_void_p),
        ("seed", C.c_uint64), ("step", C.c_uint32), ("residual_draw", C.c_int32),
        ("step_state", C.c_void_p), ("t_max", C.c_int32), ("gamma_max", C.c_int32), ("wait_limit", C.c_uint32), ("selftest", C.c_uint32),
        ("target_vmax", C.c_void_p), ("target_mass", C.c_void_p),
    ]


class DraftQArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("rows", C.c_int32), ("first_position", C.c_int32), ("logits", C.c_void_p),
        ("vocab", C.c_int64), ("row_stride", C.c_int64), ("temperature", C.c_float), ("seed", C.c_uint64), ("step", C.c_uint32),
        ("out_tokens", C.c_void_p), ("out_lse", C.c_void_p), ("out_vmax", C.c_void_p), ("out_mass", C.c_void_p), ("out_status", C.c_void_p),
        ("out_q_logits", C.c_void_p), ("q_logits_stride", C.c_int64), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
        ("step_state", C.c_void_p), ("t_max", C.c_int32), ("gamma_max", C.c_int32),
    ]


class ConfidenceArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("gamma", C.c_int32), ("hidden", C.c_int32), ("rank", C.c_int32), ("hidden_rows", C.c_void_p),
        ("emb_rows", C.c_void_p), ("w", C.c_void_p), ("b", C.c_void_p), ("sts", C.c_void_p), ("out_conf", C.c_void_p), ("step_state", C.c_void_p),
        ("t_max", C.c_int32), ("gamma_max", C.c_int32), ("stream", C.c_void_p),
    ]


class StepArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("t_max", C.c_int32), ("gamma_max", C.c_int32), ("step_state", C.c_void_p), ("tokens", C.c_void_p),
        ("ring", C.c_void_p), ("ring_cap", C.c_uint32), ("eos", C.c_int32), ("eos_list", C.c_void_p), ("n_eos", C.c_int32),
        ("log", C.c_void_p), ("log_cap", C.c_uint32), ("ctx_cap", C.c_uint32), ("lm", C.c_int32),
        ("drafts", C.c_void_p), ("conf", C.c_void_p), ("gamma", C.c_uint32), ("threshold", C.c_float), ("mode", C.c_uint32), ("cost", C.c_float * 16),
        ("conf_log", C.c_void_p), ("conf_log_cap", C.c_uint32), ("t_limit", C.c_uint32), ("stream", C.c_void_p),
    ]


class VocabArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("logits", C.c_void_p), ("rows", C.c_int64), ("vocab_local", C.c_int64),
        ("row_stride", C.c_int64), ("shard_start", C.c_int64), ("shards", C.c_int32), ("cap", C.c_int32),
        ("temperature", C.c_void_p), ("temperature_s", C.c_float), ("top_k", C.c_void_p), ("top_k_s", C.c_int32),
        ("top_p", C.c_void_p), ("top_p_s", C.c_float), ("min_p", C.c_void_p), ("min_p_s", C.c_float),
        ("flags", C.c_uint32), ("draw", C.c_int32), ("uniforms", C.c_void_p), ("seed", C.c_uint64), ("step", C.c_uint32), ("row_offset", C.c_int64),
        ("records", C.c_void_p), ("out_tokens", C.c_void_p), ("out_tau", C.c_void_p), ("out_status", C.c_void_p), ("stream", C.c_void_p),
        ("pieces", C.c_int32), ("pad_", C.c_int32), ("record_ptrs", C.c_void_p),
    ]


class HeadArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("rows", C.c_int32), ("hidden", C.c_void_p), ("hidden_stride", C.c_int64), ("weight", C.c_void_p),
        ("weight_stride", C.c_int64), ("hidden_dim", C.c_int64), ("vocab", C.c_int64), ("norm_weight", C.c_void_p), ("eps", C.c_float),
        ("one_plus", C.c_int32), ("logits", C.c_void_p), ("logits_stride", C.c_int64), ("stream", C.c_void_p),
    ]


EXPORTS = ["lm_head", "lm_accept_scan", "lm_verify_select", "lm_advance", "lm_step_state_bytes", "lm_sample", "lm_argmax", "lm_argmax_static", "lm_vocab_local", "lm_vocab_merge", "lm_vocab_record_bytes", "lm_vocab_candidate_cap", "lm_vocab_pieces", "lm_verify", "lm_draft_q", "lm_confidence", "lm_tile_state_bytes", "lm_tile_begin", "lm_tile_consume", "lm_tile_finish", "lm_workspace_bytes", "lm_verify_workspace_bytes", "lm_uniform01", "lm_abi_version",
           "lm_error_string", "lm_last_cuda_error", "lm_device_sm_count"]

_lib = None


def library_path() -> str:
    return _build.OUT


def lib():
    """The loaded library (built on first use if the in-tree shared object is missing or older than its sources)."""
    global _lib
    if _lib is None:
        path = _build.build() if os.environ.get("LITHOS_B200_NO_BUILD") != "1" else _build.OUT
        if not os.path.exists(path):
            raise RuntimeError(f"lithos_metal_b200: CUDA library {path} is missing; run `python -m lithos_metal_b200.build`")
        L = C.CDLL(path)
        L.lm_sample.restype = C.c_int
        L.lm_sample.argtypes = [C.POINTER(SampleArgs)]
        L.lm_verify.restype = C.c_int
        L.lm_verify.argtypes = [C.POINTER(VerifyArgs)]
        L.lm_tile_state_bytes.restype = C.c_size_t
        L.lm_tile_state_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int32]
        L.lm_tile_begin.restype = C.c_int
        L.lm_tile_begin.argtypes = [C.POINTER(TileArgs)]
        L.lm_tile_consume.restype = C.c_int
        L.lm_tile_consume.argtypes = [C.POINTER(TileArgs)]
        L.lm_tile_finish.restype = C.c_int
        L.lm_tile_finish.argtypes = [C.POINTER(SampleArgs), C.c_void_p, C.c_size_t]
        L.lm_confidence.restype = C.c_int
        L.lm_confidence.argtypes = [C.POINTER(ConfidenceArgs)]
        L.lm_draft_q.restype = C.c_int
        L.lm_draft_q.argtypes = [C.POINTER(DraftQArgs)]
        L.lm_argmax.restype = C.c_int
        L.lm_argmax.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.lm_argmax_static.restype = C.c_int
        L.lm_argmax_static.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        L.lm_vocab_local.restype = L.lm_vocab_merge.restype = C.c_int
        L.lm_vocab_local.argtypes = L.lm_vocab_merge.argtypes = [C.POINTER(VocabArgs)]
        L.lm_vocab_record_bytes.restype = C.c_size_t
        L.lm_vocab_record_bytes.argtypes = [C.c_int32]
        L.lm_vocab_candidate_cap.restype = C.c_int32
        L.lm_vocab_candidate_cap.argtypes = [C.c_int32]
        L.lm_head.restype = C.c_int
        L.lm_head.argtypes = [C.POINTER(HeadArgs)]
        L.lm_vocab_pieces.restype = C.c_int32
        L.lm_vocab_pieces.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_int64]
        for fn in (L.lm_accept_scan, L.lm_verify_select, L.lm_advance):
            fn.restype, fn.argtypes = C.c_int, [C.POINTER(StepArgs)]
        L.lm_step_state_bytes.restype = C.c_size_t
        L.lm_step_state_bytes.argtypes = [C.c_int32, C.c_int32]
        L.lm_workspace_bytes.restype = C.c_size_t
        L.lm_workspace_bytes.argtypes = [C.c_int64, C.c_int64]
        L.lm_verify_workspace_bytes.restype = C.c_size_t
        L.lm_verify_workspace_bytes.argtypes = [C.c_int32, C.c_int64]
        L.lm_uniform01.restype = C.c_float
        L.lm_uniform01.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]
        L.lm_abi_version.restype = C.c_int
        L.lm_error_string.restype = C.c_char_p
        L.lm_error_string.argtypes = [C.c_int]
        L.lm_last_cuda_error.restype = C.c_char_p
        L.lm_device_sm_count.restype = C.c_int
        if L.lm_abi_version() != ABI_VERSION:
            raise RuntimeError("lithos_metal_b200: ABI version mismatch between the binding and the shared object")
        _lib = L
    return _lib


class LithosError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != LM_OK:
        L = lib()
        detail = L.lm_last_cuda_error().decode() if rc == -3 else ""
        raise LithosError(f"{what}: {L.lm_error_string(rc).decode()} ({rc}){': ' + detail if detail else ''}")
