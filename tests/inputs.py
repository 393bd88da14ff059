"""Seeded input generators shared by the tests (the recipes of the reference's tests and of the benchmark configs)."""
import numpy as np

import oracle

OPTION_SETS = {   # the six option sets of the reference's sampler test
    "plain": dict(temperature=1.0),
    "topk": dict(temperature=0.7, top_k=40),
    "topp": dict(temperature=1.0, top_p=0.9),
    "minp": dict(temperature=1.3, min_p=0.05),
    "all": dict(temperature=0.8, top_k=50, top_p=0.95, min_p=0.02),
    "topp-in-topk": dict(temperature=0.8, top_k=50, top_p=0.9, topp_in_topk=True),
}


def sampling_test_logits(vocab: int, opts: dict) -> np.ndarray:
    """BF16 codes [3, vocab] of N(0, 4^2), seeded by vocab + len(opts) like the reference's test."""
    rng = np.random.default_rng(vocab + len(opts))
    return oracle.f32_to_bf16((rng.standard_normal((3, vocab)) * 4.0).astype(np.float32))


def argmax_test_logits(vocab: int) -> np.ndarray:
    rng = np.random.default_rng(vocab)
    logits = rng.standard_normal((4, vocab)).astype(np.float32) * 4
    logits[0, vocab - 1] = 100.0
    logits[1, 5] = logits[1, 7] = 50.0
    logits[2] = -np.abs(logits[2]) - 1
    return oracle.f32_to_bf16(logits)


def config1():
    """One FP32 row, V = 151936, N(0, 2^2) with 8 spikes at +12 (seed 0); injected uniform from seed 1."""
    rng = np.random.default_rng(0)
    V = 151936
    z = (rng.standard_normal(V) * 2.0).astype(np.float32)
    spikes = rng.choice(V, size=8, replace=False)
    z[spikes] = 12.0
    u = np.float32(np.random.default_rng(1).random())
    return z[None, :], u


def config2(vocab: int = 151936, seed: int = 2):
    """DSpark step: target [8, V] BF16 codes, 7 draft ids, draft probs [7, V] = softmax(target[:7] + N(0, 0.5^2)), uniforms."""
    rng = np.random.default_rng(seed)
    target = oracle.f32_to_bf16((rng.standard_normal((8, vocab)) * 2.0).astype(np.float32))
    drafts = rng.integers(0, vocab, 7).astype(np.int32)
    noisy = oracle.bf16_to_f32(target[:7]) + (rng.standard_normal((7, vocab)) * 0.5).astype(np.float32)
    e = np.exp((noisy - noisy.max(-1, keepdims=True)).astype(np.float64))
    q = (e / e.sum(-1, keepdims=True)).astype(np.float32)
    u_accept = rng.random(7).astype(np.float32)
    u_final = np.float32(rng.random())
    return target, drafts, q, u_accept, u_final


def config3(rows: int = 256, vocab: int = 151936, hist_len: int = 2048, seed: int = 3):
    """Batched penalised sampling: BF16 N(0, 2^2) logits, per-row T ~ U[0.3, 1.5], top_k in {0, 20, 50, 1000},
    top_p ~ U[0.8, 1.0], history [rows, hist_len] uniform ids, uniforms [rows]."""
    rng = np.random.default_rng(seed)
    logits = oracle.f32_to_bf16((rng.standard_normal((rows, vocab), dtype=np.float32) * np.float32(2.0)))
    temperature = rng.uniform(0.3, 1.5, rows).astype(np.float32)
    top_k = rng.choice(np.array([0, 20, 50, 1000], dtype=np.int32), rows)
    top_p = rng.uniform(0.8, 1.0, rows).astype(np.float32)
    history = rng.integers(0, vocab, (rows, hist_len)).astype(np.int32)
    uniforms = rng.random(rows).astype(np.float32)
    return dict(logits=logits, temperature=temperature, top_k=top_k, top_p=top_p, history=history, uniforms=uniforms,
                repetition_penalty=1.1, presence_penalty=0.5)
