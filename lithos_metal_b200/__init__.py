"""B200-native generation control: sampling (penalties, temperature, top-k / top-p / min-p, greedy argmax, seeded
draws) and DSpark speculative verification, as hand-written sm_100a CUDA behind a C ABI (include/lithos_b200.h).

The Python names mirror the reference's sampler interface (monolith/nn/sampler.py, monolith/nn/sampling_ref.py).
"""
from .sampler import (GreedySampler, SampleOutput, SamplingParams, StochasticSampler, argmax, sample, sample_row, thresholds,
                      warped_probabilities)
from .verify import DraftQ, draft_q, verify
from .step_state import StepStateLayout, accept_scan, advance, confidence, verify_select
from .records import accept_args_from_record, sample_args_from_record, select_args_from_record
from .tiles import TileSampler
from .head import lm_head
from . import parallel

__all__ = ["TileSampler", "lm_head", "GreedySampler", "StochasticSampler", "SamplingParams", "SampleOutput", "sample", "argmax", "sample_row", "thresholds",
           "warped_probabilities", "verify", "draft_q", "DraftQ", "StepStateLayout", "accept_scan", "verify_select", "advance", "confidence", "parallel",
           "sample_args_from_record", "select_args_from_record", "accept_args_from_record"]
