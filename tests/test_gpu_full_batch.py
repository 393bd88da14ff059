"""Whole batches against the CPU oracle: every row of the batched configuration and of the benchmark workload, and rows built
to sit on the edge of the candidate kernel's FP32 decision band. Bit-exact tokens and thresholds."""
import os

import numpy as np
import pytest
import torch

import bench
import lithos_metal_b200 as lm
import oracle
from tests import inputs
from tests.test_gpu_sampling import bf16_tensor

pytestmark = pytest.mark.gpu
THREADS = max(1, len(os.sched_getaffinity(0)))


def gpu_and_oracle(cfg, **extra):
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(np.ascontiguousarray(cfg[k])).cuda() for k in ("temperature", "top_k", "top_p")}
    hist = torch.from_numpy(cfg["history"]).cuda() if cfg.get("history") is not None else None
    pen = dict(repetition_penalty=1.1, presence_penalty=0.5) if hist is not None else {}
    r = lm.sample(x, lm.SamplingParams(draw="inverse_cdf", **pen, **knobs, **extra), history=hist, uniforms=torch.from_numpy(cfg["uniforms"]).cuda(),
                  return_tau=True, return_status=True)
    tok, tau, _ = oracle.sample_batch(cfg["logits"], temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], history=cfg.get("history"),
                                      draw="inverse_cdf", uniforms=cfg["uniforms"], n_threads=THREADS, **pen, **extra)
    return r, tok, tau


def test_every_row_of_the_batched_configuration():
    """Benchmark configuration 3: 256 penalised rows with per-row knobs."""
    r, tok, tau = gpu_and_oracle(inputs.config3())
    status = r.status.cpu().numpy()
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)
    assert not np.any(status & 1) and np.count_nonzero(status & 64) > 100    # nothing on the generic path; most rows with a top_k on the candidate path


def test_every_row_of_the_benchmark_workload():
    """The 4096 rows bench.py times (generated the same way), all of them."""
    inp = bench.make_inputs(torch, bench.TOTAL_ROWS, 0, torch.device("cuda", 0))
    params = lm.SamplingParams(temperature=inp["temperature"], top_k=inp["top_k"], top_p=inp["top_p"], repetition_penalty=bench.RHO,
                               presence_penalty=bench.PI, draw="inverse_cdf")
    r = lm.sample(inp["logits"], params, history=inp["history"], uniforms=inp["uniforms"], return_tau=True, return_status=True)
    hc = bench.host_copy(torch, inp, bench.TOTAL_ROWS)
    tok, tau, _ = oracle.sample_batch(hc["logits"], temperature=hc["temperature"], top_k=hc["top_k"], top_p=hc["top_p"], history=hc["history"],
                                      repetition_penalty=bench.RHO, presence_penalty=bench.PI, draw="inverse_cdf", uniforms=hc["uniforms"], n_threads=THREADS)
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)
    status = r.status.cpu().numpy()
    n_topk = int((hc["top_k"] > 0).sum())
    assert np.count_nonzero(status & 1) <= 2 and np.count_nonzero(status & 64) >= 0.97 * n_topk   # the candidate kernel keeps nearly all of its rows


def test_rows_on_the_edge_of_the_fp32_decision_band():
    """The candidate kernel knows the row's mass only in FP32 and hands a row on when a cumulative-mass boundary lies inside its
    error band around top_p * Z. Here top_p is placed at relative distances 0 .. 1e-4 on both sides of an exact boundary inside the
    top-k set: whichever kernel finishes the row, the threshold must be the oracle's (FP64). Far from the boundary the candidate
    kernel must keep the row (the band is narrow)."""
    base = inputs.config3(rows=8, seed=77)
    deltas = np.array([0.0, 3e-7, -3e-7, 1e-6, -1e-6, 3e-6, -3e-6, 1e-5, -1e-5, 3e-5, -3e-5, 1e-4, -1e-4])
    rows = []
    for r in range(8):
        T = np.float32(0.45 + 0.05 * r)
        z = oracle.bf16_to_f32(base["logits"][r]).astype(np.float64)
        vals, counts = np.unique(z, return_counts=True)
        vals, counts = vals[::-1], counts[::-1]
        cum = np.cumsum(counts * np.exp((vals - vals[0]) / np.float64(T)))
        n_top = np.cumsum(counts)
        i = int(np.searchsorted(n_top, 300))                               # a boundary well inside the top 1000
        for d in deltas:
            rows.append((r, T, np.float32(cum[i] / cum[-1] * (1.0 + d)), d))
    cfg = dict(logits=np.stack([base["logits"][r] for r, _, _, _ in rows]), temperature=np.array([t for _, t, _, _ in rows], np.float32),
               top_k=np.full(len(rows), 1000, np.int32), top_p=np.array([p for _, _, p, _ in rows], np.float32), history=None,
               uniforms=np.linspace(0.05, 0.95, len(rows)).astype(np.float32))
    assert np.all((cfg["top_p"] > 0.3) & (cfg["top_p"] < 1.0))
    r, tok, tau = gpu_and_oracle(cfg)
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)
    on_candidate_path = (r.status.cpu().numpy() & 64) != 0
    far = np.abs(np.array([d for _, _, _, d in rows])) >= 1e-4
    assert on_candidate_path[far].all()                                    # the band does not reach 1e-4
    assert not on_candidate_path[np.array([d for _, _, _, d in rows]) == 0.0].any()   # dead on the boundary: never decided in FP32


@pytest.mark.parametrize("exact_only", [False, True])
def test_draw_over_runs_of_equal_logits_from_both_sources(exact_only):
    """The inverse-CDF draw walks equal logits in index order. With repetition 2.0 and presence 0.5 a penalised logit lands exactly
    on BF16 codes that unpenalised logits of the row carry too (z / 2 - 0.5), so runs of equal values mix penalised and unpenalised
    positions; coarse logits (multiples of 1/4) make the runs long. Uniforms spread over [0, 1) land inside such runs in every
    kernel: rows with a top_k (candidate kernel), without one (histogram kernel), and with exact_only (histogram kernel for all)."""
    rows, vocab = 96, 65536
    rng = np.random.default_rng(123)
    z = np.round(rng.standard_normal((rows, vocab)) * 8.0) / 4.0                                  # values k / 4, |z| up to ~10
    codes = oracle.f32_to_bf16(z.astype(np.float32))
    hist = rng.integers(0, vocab, (rows, 1500)).astype(np.int32)
    top = np.argsort(-z, axis=1)[:, :200]
    hist[:, :200] = top                                                                            # the penalties reach the top of the row
    cfg = dict(logits=codes, temperature=rng.uniform(0.8, 2.5, rows).astype(np.float32),
               top_k=np.where(np.arange(rows) % 3 == 0, 0, np.where(np.arange(rows) % 3 == 1, 40, 700)).astype(np.int32),
               top_p=rng.uniform(0.85, 0.999, rows).astype(np.float32), history=hist, uniforms=np.linspace(0.001, 0.999, rows).astype(np.float32))
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    pen = dict(repetition_penalty=2.0, presence_penalty=0.5)
    r = lm.sample(x, lm.SamplingParams(draw="inverse_cdf", exact_only=exact_only, **pen, **knobs), history=torch.from_numpy(hist).cuda(),
                  uniforms=torch.from_numpy(cfg["uniforms"]).cuda(), return_tau=True, return_status=True)
    tok, tau, _ = oracle.sample_batch(codes, temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], history=hist, draw="inverse_cdf",
                                      uniforms=cfg["uniforms"], n_threads=THREADS, **pen)
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)
    status = r.status.cpu().numpy()
    assert np.count_nonzero(status & 1) <= rows // 8, status                                       # the streaming kernels keep (nearly) all of these rows
    # the drawn tokens do sit in mixed runs: for some rows the token's value is carried by penalised and unpenalised positions alike
    zf = oracle.bf16_to_f32(codes)
    mixed = 0
    for i in range(rows):
        zi = oracle.apply_penalties(zf[i], hist[i], 2.0, 0.5)
        same = np.nonzero(zi == zi[tok[i]])[0]
        pen_ids = np.unique(hist[i])
        mixed += int(np.isin(same, pen_ids).any() and (~np.isin(same, pen_ids)).any())
    assert mixed >= 3, mixed
