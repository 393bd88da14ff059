"""Calls of a few rows: lm_sample cuts every row into slices over the whole GPU (one block per slice, one merge per row).

The reference's sampler dispatches run on the T <= 8 rows of one decode step (monolith/kernels.py:720-775); its own CPU-runnable
configuration is a single FP32 row. The results must be the ones of the row-per-block kernels and of the oracle, bit for bit.
"""
import numpy as np
import pytest
import torch

import oracle
import lithos_metal_b200 as lm
from lithos_metal_b200 import _lib

pytestmark = pytest.mark.gpu
SLICED, GENERIC = _lib.STATUS_SLICED_PATH, 1


def _rows(rows, vocab, seed, dtype, spikes=8):
    rng = np.random.default_rng(seed)
    z = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
    for r in range(rows):
        z[r, rng.choice(vocab, spikes, replace=False)] = 12.0
    if dtype == "bf16":
        codes = oracle.f32_to_bf16(z)
        return torch.from_numpy(codes.view(np.int16)).cuda().view(torch.bfloat16), codes
    return torch.from_numpy(z).cuda(), z


def _check(x, host, *, draw, temperature, top_k, top_p=0.0, min_p=0.0, history=None, rho=1.0, pi=0.0, expect_sliced=True, seed=5, step=2, row_offset=0,
           topp_in_topk=False, exact_only=False):
    rows = x.shape[0]
    u = np.random.default_rng(seed + 100).random(rows).astype(np.float32)
    p = lm.SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, seed=seed, draw=draw, repetition_penalty=rho, presence_penalty=pi,
                          topp_in_topk=topp_in_topk, exact_only=exact_only)
    r = lm.sample(x, p, history=None if history is None else torch.from_numpy(history).cuda(), uniforms=torch.from_numpy(u).cuda(), step=step,
                  row_offset=row_offset, return_tau=True, return_status=True)
    tok, tau, _ = oracle.sample_batch(host, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, topp_in_topk=topp_in_topk, history=history,
                                      repetition_penalty=rho, presence_penalty=pi, draw=draw, uniforms=u, seed=seed, step=step, row_offset=row_offset, n_threads=8)
    st = r.status.cpu().numpy()
    assert bool(np.all(st & SLICED)) == expect_sliced or (not expect_sliced and not np.any(st & SLICED)), st
    assert r.tokens.cpu().tolist() == tok.tolist()
    assert r.tau.cpu().numpy().tobytes() == tau.tobytes()
    return r, st


@pytest.mark.parametrize("draw", ["inverse_cdf", "gumbel"])
@pytest.mark.parametrize("rows", [1, 3, 16, 32])
def test_fp32_rows_with_spikes(rows, draw):
    x, host = _rows(rows, 151936, 1, "f32")
    _check(x, host, draw=draw, temperature=0.7, top_k=20, top_p=0.95)


@pytest.mark.parametrize("top_k,top_p,min_p", [(1, 0.0, 0.0), (16, 0.9, 0.0), (17, 0.0, 0.05), (32, 0.5, 0.0), (50, 0.95, 0.01), (64, 0.99, 0.0)])
def test_bf16_rows_with_penalties(top_k, top_p, min_p):
    rows, vocab = 5, 151936
    x, host = _rows(rows, vocab, 2, "bf16")
    rng = np.random.default_rng(3)
    hist = rng.integers(0, vocab, (rows, 700)).astype(np.int32)
    hist[:, :40] = np.argsort(-oracle.bf16_to_f32(host), axis=1)[:, :40]       # the penalties must reach the top of every row
    hist[0, 50:60] = hist[0, 0]                                               # a repeated id is penalised once
    for draw in ("inverse_cdf", "gumbel"):
        _check(x, host, draw=draw, temperature=0.9, top_k=top_k, top_p=top_p, min_p=min_p, history=hist, rho=1.3, pi=0.4, row_offset=40)


@pytest.mark.parametrize("vocab,top_k,sliced", [(16400, 10, True), (262144, 50, True), (1000000, 8, True), (1000000, 50, True), (8192, 10, False)])
def test_vocabulary_sizes_and_the_limits_of_the_path(vocab, top_k, sliced):
    x, host = _rows(2, vocab, 4, "bf16" if vocab % 8 == 0 else "f32")
    _check(x, host, draw="inverse_cdf", temperature=1.1, top_k=top_k, top_p=0.9, expect_sliced=sliced)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_a_masked_vocabulary_stays_on_the_sliced_path(dtype):
    """-inf logits (constrained decoding): slices with fewer than top_k logits above -inf hand over what they have and one -inf logit."""
    rng = np.random.default_rng(31)
    rows, vocab = 4, 151936
    z = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
    z[0, rng.random(vocab) < 0.9] = -np.inf                                   # nine in ten masked, everywhere
    keep = np.zeros(vocab, bool); keep[1000:1040] = True
    z[1, ~keep] = -np.inf                                                     # 40 logits left: fewer than a top_k of 50
    z[2, :50000] = -np.inf; z[2, 60000:] = -np.inf                            # whole slices masked
    z[3, 5] = -np.inf                                                         # one masked logit
    if dtype == "bf16":
        host = oracle.f32_to_bf16(z)
        x = torch.from_numpy(host.view(np.int16)).cuda().view(torch.bfloat16)
    else:
        host, x = z, torch.from_numpy(z).cuda()
    for draw in ("inverse_cdf", "gumbel"):
        for top_k, top_p in ((20, 0.9), (50, 0.9), (50, 0.0), (1, 0.0)):
            _check(x, host, draw=draw, temperature=0.8, top_k=top_k, top_p=top_p)


def test_rows_with_a_nan_or_an_infinite_maximum_go_to_the_generic_kernel():
    x, host = _rows(3, 151936, 8, "f32")
    x[0, 77] = float("nan"); x[1, 123456] = float("inf")
    u = torch.rand(3, device="cuda")
    for kw in (dict(top_k=20, top_p=0.9), dict(top_k=8)):
        p = lm.SamplingParams(temperature=0.9, draw="inverse_cdf", **kw)
        pe = lm.SamplingParams(temperature=0.9, draw="inverse_cdf", exact_only=True, **kw)
        r = lm.sample(x, p, uniforms=u, return_tau=True, return_status=True)
        e = lm.sample(x, pe, uniforms=u, return_tau=True, return_status=True)
        st = r.status.cpu().numpy()
        assert st[0] & GENERIC and st[1] & GENERIC and st[2] & SLICED, st
        assert r.tokens.cpu().tolist() == e.tokens.cpu().tolist()
        assert r.tau.cpu().numpy().tobytes() == e.tau.cpu().numpy().tobytes()
        assert (st[:2] & ~(GENERIC | SLICED)).tolist() == (e.status.cpu().numpy()[:2] & ~(GENERIC | SLICED)).tolist()


def test_a_top_p_boundary_too_close_for_the_fp32_softmass_goes_to_the_generic_kernel():
    """The slices sum the softmass in FP32; a cumulative mass that meets top_p * total to within that sum's error band is decided by the
    exact kernel instead. Row 0: weights 1 and 1/3 (and nothing else that counts), top_p = 3/4."""
    vocab = 151936
    z = np.full((2, vocab), -40.0, np.float32)
    z[0, 1234] = 10.0; z[0, 99999] = np.float32(10.0 - np.log(3.0))
    z[1] = (np.random.default_rng(12).standard_normal(vocab) * 2).astype(np.float32)
    x = torch.from_numpy(z).cuda()
    r, st = _check(x, z, draw="inverse_cdf", temperature=1.0, top_k=20, top_p=0.75, expect_sliced=False)
    assert st[0] & GENERIC and st[1] & SLICED, st


def test_more_equal_logits_at_the_top_k_boundary_than_the_merge_sorts():
    x, host = _rows(2, 151936, 9, "f32", spikes=0)
    x[0, ::50] = 9.0; host[0, ::50] = 9.0                                     # 3039 equal maxima, about 47 per slice: no record overflows (cap 128), the merge does
    r, st = _check(x, host, draw="inverse_cdf", temperature=1.0, top_k=64, expect_sliced=False)
    assert st[0] & GENERIC and st[1] & SLICED, st


def test_more_ties_than_a_record_holds_go_to_the_generic_kernel():
    x, host = _rows(2, 151936, 6, "f32", spikes=0)
    x[0, 100:300] = 9.0; host[0, 100:300] = 9.0                               # 200 equal maxima inside one slice, top_k 20
    r, st = _check(x, host, draw="inverse_cdf", temperature=1.0, top_k=20, expect_sliced=False)
    assert st[0] & GENERIC and st[1] & SLICED, st


def test_other_knobs_keep_the_row_per_block_kernels():
    x33, host33 = _rows(33, 32768, 7, "bf16")
    _check(x33, host33, draw="inverse_cdf", temperature=0.8, top_k=20, top_p=0.9, expect_sliced=False)      # more rows than the path takes
    x, host = _rows(4, 151936, 7, "bf16")
    _check(x, host, draw="gumbel", temperature=0.8, top_k=40, top_p=0.9, exact_only=True, expect_sliced=False)
    _check(x, host, draw="gumbel", temperature=0.8, top_k=0, top_p=0.9, expect_sliced=False)
    _check(x, host, draw="gumbel", temperature=0.8, top_k=40, top_p=0.9, topp_in_topk=True)
    _check(x, host, draw="inverse_cdf", temperature=0.8, top_k=12, top_p=0.9, topp_in_topk=True)
    _check(x, host, draw="inverse_cdf", temperature=0.8, top_k=64, top_p=0.9, min_p=0.02, topp_in_topk=True)
    k = torch.full((4,), 40, dtype=torch.int32)
    p = lm.SamplingParams(temperature=0.8, top_k=k, seed=1)
    assert not np.any(lm.sample(x, p, return_status=True).status.cpu().numpy() & SLICED)


def test_rows_that_do_not_start_on_a_16_byte_boundary():
    base, host = _rows(3, 40001, 8, "f32")                                    # odd row length: rows 1 and 2 start unaligned
    _check(base, host, draw="inverse_cdf", temperature=0.7, top_k=20, top_p=0.95)
    wide = torch.zeros(3, 40009, device="cuda")
    wide[:, 3:40004] = base                                                   # a view with a stride and an offset
    _check(wide[:, 3:40004], host, draw="inverse_cdf", temperature=0.7, top_k=20, top_p=0.95)


def test_random_configurations_equal_the_exact_kernels():
    """A sweep of seeded random calls (rows, vocabulary, dtype, knobs, draw, penalties, -inf masks, planted ties): the few-row path
    against the same library with LM_FLAG_EXACT_ONLY (the generic kernel, which the other tests hold to the oracle), bit for bit;
    a sample of the calls against the oracle itself."""
    rng = np.random.default_rng(2024)
    checked_with_oracle = 0
    for trial in range(60):
        rows = int(rng.integers(1, 33))
        vocab = int(rng.choice([16384, 20000, 50257, 151936, 131073]))
        dtype = "bf16" if (vocab % 8 == 0 and rng.random() < 0.6) else "f32"
        z = (rng.standard_normal((rows, vocab)) * float(rng.uniform(0.5, 4.0))).astype(np.float32)
        if rng.random() < 0.3:
            z[rng.random((rows, vocab)) < float(rng.uniform(0.3, 0.97))] = -np.inf                # masked vocabulary
            z[np.arange(rows), rng.integers(0, vocab, rows)] = 1.0                                # (never a row of nothing but -inf)
        if rng.random() < 0.3:
            r, n = int(rng.integers(0, rows)), int(rng.integers(2, 40))
            z[r, rng.choice(vocab, n, replace=False)] = np.float32(z[r][np.isfinite(z[r])].max())  # ties at the top
        if dtype == "bf16":
            host = oracle.f32_to_bf16(z)
            x = torch.from_numpy(host.view(np.int16)).cuda().view(torch.bfloat16)
        else:
            host, x = z, torch.from_numpy(z).cuda()
        kw = dict(temperature=float(rng.uniform(0.2, 1.6)), top_k=int(rng.integers(1, 65)), top_p=float(rng.choice([0.0, 0.5, 0.9, 0.99])),
                  min_p=float(rng.choice([0.0, 0.0, 0.02])), draw=str(rng.choice(["inverse_cdf", "gumbel"])), seed=int(rng.integers(0, 1 << 30)),
                  topp_in_topk=bool(rng.random() < 0.2))
        hist = None
        if rng.random() < 0.4:
            hist = rng.integers(0, vocab, (rows, int(rng.integers(1, 600)))).astype(np.int32)
            kw.update(repetition_penalty=float(rng.uniform(1.0, 1.5)), presence_penalty=float(rng.uniform(0.0, 1.0)))
        u = rng.random(rows).astype(np.float32)
        step, off = int(rng.integers(0, 100)), int(rng.integers(0, 1000))
        args = dict(history=None if hist is None else torch.from_numpy(hist).cuda(), uniforms=torch.from_numpy(u).cuda(), step=step, row_offset=off,
                    return_tau=True, return_status=True)
        fast = lm.sample(x, lm.SamplingParams(**kw), **args)
        exact = lm.sample(x, lm.SamplingParams(exact_only=True, **kw), **args)
        st = fast.status.cpu().numpy()
        assert np.all(st & (SLICED | GENERIC)), (trial, st)                                        # every row took the path (or was handed on by it)
        tie = ((st | exact.status.cpu().numpy()) & 4) != 0                                         # Gumbel keys within 4e-6 of one another: flagged, not compared
        assert fast.tau.cpu().numpy().tobytes() == exact.tau.cpu().numpy().tobytes(), (trial, kw, rows, vocab, dtype)
        assert np.all((fast.tokens.cpu().numpy() == exact.tokens.cpu().numpy()) | tie), (trial, kw, rows, vocab, dtype)
        if trial % 10 == 0 and vocab <= 60000:
            tok, tau, _ = oracle.sample_batch(host, temperature=kw["temperature"], top_k=kw["top_k"], top_p=kw["top_p"], min_p=kw["min_p"],
                                              topp_in_topk=kw["topp_in_topk"], history=hist, repetition_penalty=kw.get("repetition_penalty", 1.0),
                                              presence_penalty=kw.get("presence_penalty", 0.0), draw=kw["draw"], uniforms=u, seed=kw["seed"], step=step,
                                              row_offset=off, n_threads=8)
            assert fast.tau.cpu().numpy().tobytes() == tau.tobytes() and np.all((fast.tokens.cpu().numpy() == tok) | tie), trial
            checked_with_oracle += 1
    assert checked_with_oracle >= 2
