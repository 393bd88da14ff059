"""The CUDA sampler against the reference's golden outputs and against the CPU oracle (bit-exact token ids,
thresholds and kept sets; probabilities within 1e-5 relative). All calls go through the C ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import lithos_metal_b200 as lm
from tests import inputs

pytestmark = pytest.mark.gpu


def bf16_tensor(codes: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(codes.view(np.int16)).cuda().view(torch.bfloat16)


@pytest.mark.parametrize("vocab", [248320, 1000, 300])
def test_argmax_edge_cases(golden, vocab):
    lb = inputs.argmax_test_logits(vocab)
    out = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    lm.argmax(bf16_tensor(lb)[:3], out=out[:3])
    got = out.cpu().tolist()
    assert got[:3] == golden["argmax"][str(vocab)][:3] and got[0] == vocab - 1 and got[1] == 5
    assert got[3] == -1                                                   # rows beyond the active ones stay untouched
    assert lm.GreedySampler().forward(bf16_tensor(lb)).cpu().tolist() == golden["argmax"][str(vocab)]
    # the same rows as FP32, and through the sampler entry point with temperature 0
    lf = torch.from_numpy(oracle.bf16_to_f32(lb)).cuda()
    assert lm.argmax(lf).cpu().tolist() == golden["argmax"][str(vocab)]
    assert lm.sample(bf16_tensor(lb), temperature=0.0).tokens.cpu().tolist() == golden["argmax"][str(vocab)]


@pytest.mark.parametrize("rows,vocab", [(1, 151936), (8, 151936), (300, 4096), (2, 7), (5, 8193)])
def test_argmax_shapes_and_strides(rows, vocab):
    rng = np.random.default_rng(rows * 1000 + vocab)
    lb = oracle.f32_to_bf16((rng.standard_normal((rows, vocab + 3)) * 3).astype(np.float32))
    t = bf16_tensor(lb)[:, 1:vocab + 1]                                   # a strided, misaligned view
    exp = oracle.bf16_to_f32(lb)[:, 1:vocab + 1].argmax(-1)
    assert lm.argmax(t).cpu().tolist() == exp.tolist()


@pytest.mark.parametrize("vocab", [1000, 248320])
@pytest.mark.parametrize("name", list(inputs.OPTION_SETS))
def test_draws_equal_the_reference(golden, vocab, name):
    """tests/kernels/test_sampling.py:51-67 of the reference, with the reference's outputs as goldens."""
    opts = inputs.OPTION_SETS[name]
    g = golden["draws"][f"{vocab}/{name}"]
    lb = inputs.sampling_test_logits(vocab, opts)
    x = bf16_tensor(lb)
    s = lm.StochasticSampler(seed=12345, **opts)
    for step in (0, 1, 7):
        r = lm.sample(x, s.params(), step=step, return_tau=True, return_status=True)
        assert r.tau.cpu().tolist() == [np.float32(t) for t in g["tau"]]
        tok, status = r.tokens.cpu().tolist(), r.status.cpu().tolist()
        for i in range(3):
            assert tok[i] == g["tokens"][str(step)][i] or (status[i] & 4), (step, i)   # equal, or flagged as a float32-log near-tie
        assert s.forward(x, step=step).cpu().tolist() == tok
    assert sum(1 for st in status if st & 4) == 0


def test_kept_sets_equal_the_hf_warpers(golden):
    rng = np.random.default_rng(3)
    lb = oracle.f32_to_bf16((rng.standard_normal((2, 4096)) * 3.0).astype(np.float32))
    lf = oracle.bf16_to_f32(lb)
    for name, g in golden["hf_warpers"].items():
        o = dict(g["opts"])
        r = lm.sample(bf16_tensor(lb), return_tau=True, return_probs=True, **o)
        tau = r.tau.cpu().numpy()
        probs = r.probs.cpu().numpy()
        for i in range(2):
            assert np.nonzero(lf[i] >= tau[i])[0].tolist() == g["kept"][i], name
            assert np.nonzero(probs[i])[0].tolist() == g["kept"][i], name


@pytest.mark.parametrize("name", ["plain", "topk", "topp", "minp", "all"])
def test_kept_probabilities_equal_the_reference(golden, name):
    opts = inputs.OPTION_SETS[name]
    lb = inputs.sampling_test_logits(1000, opts)
    g = golden["warped_probabilities"][name]
    p = lm.warped_probabilities(bf16_tensor(lb)[0], **opts)
    assert np.nonzero(p)[0].tolist() == g["idx"]
    np.testing.assert_allclose(p[g["idx"]], g["p"], rtol=1e-5)           # the tolerance the task states for probabilities


def test_known_answer_vector(golden):
    g = golden["known_answer_5"]
    lg = np.array(g["logits"], dtype=np.float32)
    assert lm.thresholds(lg, top_k=3, top_p=0.85) == g["topp"]
    assert lm.thresholds(lg, top_k=3, top_p=0.85, topp_in_topk=True) == g["topp_in_topk"]


def test_config1_single_fp32_row(golden):
    g = golden["config1"]
    z, u = inputs.config1()
    x = torch.from_numpy(z).cuda()
    assert lm.GreedySampler().forward(x).cpu().tolist() == [g["greedy"]]
    opts = dict(temperature=0.7, top_k=20, top_p=0.95)
    r = lm.sample(x, seed=1, return_tau=True, return_probs=True, return_stats=True, **opts)
    assert float(r.tau[0]) == g["tau"] and int(r.tokens[0]) == g["gumbel_token_seed1_step0"]
    p = r.probs[0].cpu().numpy()
    assert np.nonzero(p)[0].tolist() == g["kept_idx"]
    np.testing.assert_allclose(p[g["kept_idx"]], g["kept_p"], rtol=1e-5)
    assert r.stats.cpu().tolist() == [[12.0, 8.0]]
    r = lm.sample(x, draw="inverse_cdf", uniforms=torch.tensor([u]), **opts)
    assert int(r.tokens[0]) == oracle.sample_invcdf(z[0], u, **opts) == g["spikes"][int(np.floor(8 * float(u)))]


def run_both(cfg, draw, rows, seed=77, step=3, row_offset=0, **extra):
    """The same batch through the CUDA library and through the CPU oracle."""
    x = bf16_tensor(cfg["logits"][:rows]) if cfg["logits"].dtype == np.uint16 else torch.from_numpy(cfg["logits"][:rows]).cuda()
    knobs = {k: torch.from_numpy(cfg[k][:rows]).cuda() for k in ("temperature", "top_k", "top_p") if k in cfg}
    hist = cfg.get("history")
    r = lm.sample(x, lm.SamplingParams(seed=seed, draw=draw, repetition_penalty=cfg.get("repetition_penalty", 1.0),
                                       presence_penalty=cfg.get("presence_penalty", 0.0), **knobs, **extra),
                  history=None if hist is None else torch.from_numpy(hist[:rows]).cuda(),
                  uniforms=torch.from_numpy(cfg["uniforms"][:rows]).cuda(), step=step, row_offset=row_offset,
                  return_tau=True, return_stats=True, return_status=True)
    tok, tau, stats = oracle.sample_batch(cfg["logits"][:rows], temperature=cfg["temperature"][:rows], top_k=cfg["top_k"][:rows],
                                          top_p=cfg["top_p"][:rows], history=None if hist is None else hist[:rows],
                                          repetition_penalty=cfg.get("repetition_penalty", 1.0), presence_penalty=cfg.get("presence_penalty", 0.0),
                                          draw=draw, uniforms=cfg["uniforms"][:rows], seed=seed, step=step, row_offset=row_offset, n_threads=8,
                                          **{k: v for k, v in extra.items() if k in ("min_p", "topp_in_topk")})
    return r, tok, tau, stats


@pytest.mark.parametrize("draw", ["inverse_cdf", "gumbel"])
def test_penalised_batch_equals_the_oracle(draw):
    """Benchmark configuration 3 (per-row knobs, 2048-id histories, both penalties) on its first rows."""
    rows = 24
    cfg = inputs.config3(rows=rows)
    r, tok, tau, stats = run_both(cfg, draw, rows, row_offset=1000)
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    status = r.status.cpu().numpy()
    got = r.tokens.cpu().numpy()
    if draw == "gumbel":
        assert np.all((got == tok) | ((status & 4) != 0))
    else:
        np.testing.assert_array_equal(got, tok)
    np.testing.assert_allclose(r.stats.cpu().numpy(), stats, rtol=1e-5)


@pytest.mark.parametrize("vocab,rows", [(300, 5), (1000, 7), (8191, 3), (32768, 4)])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_small_and_ragged_vocabularies(vocab, rows, dtype):
    rng = np.random.default_rng(vocab)
    z = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    cfg = dict(logits=oracle.f32_to_bf16(z) if dtype == "bf16" else z, temperature=rng.uniform(0.3, 1.5, rows).astype(np.float32),
               top_k=rng.choice(np.array([0, 1, 5, 50, vocab + 10], dtype=np.int32), rows), top_p=rng.uniform(0.5, 1.0, rows).astype(np.float32),
               history=rng.integers(-2, vocab + 2, (rows, 64)).astype(np.int32), uniforms=rng.random(rows).astype(np.float32),
               repetition_penalty=1.3, presence_penalty=0.25)
    for draw in ("inverse_cdf", "gumbel"):
        r, tok, tau, stats = run_both(cfg, draw, rows, min_p=0.01)
        np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
        status = r.status.cpu().numpy()
        assert np.all((r.tokens.cpu().numpy() == tok) | ((status & 4) != 0))
        np.testing.assert_allclose(r.stats.cpu().numpy(), stats, rtol=1e-5)


def test_ties_duplicates_and_degenerate_rows():
    V = 4096
    z = np.zeros((4, V), dtype=np.float32)                                 # row 0: every logit equal
    z[1, :] = -np.inf; z[1, 17] = 0.5; z[1, 99] = 0.5                      # row 1: a masked row with two survivors
    z[2, :] = np.repeat(np.arange(V // 8, dtype=np.float32), 8) * 0.01    # row 2: ties of eight everywhere
    z[3, :] = np.linspace(-5, 5, V, dtype=np.float32)
    cfg = dict(logits=oracle.f32_to_bf16(z), temperature=np.array([1.0, 0.5, 0.8, 1.2], np.float32), top_k=np.array([10, 0, 12, 3], np.int32),
               top_p=np.array([0.9, 0.95, 0.5, 0.0], np.float32), uniforms=np.array([0.999999, 0.5, 0.0, 0.3], np.float32))
    r, tok, tau, stats = run_both(cfg, "inverse_cdf", 4)
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)
    np.testing.assert_allclose(r.stats.cpu().numpy(), stats, rtol=1e-5)
    zb = oracle.bf16_to_f32(cfg["logits"])
    assert tau[0] == 0.0 and tok[0] == V - 1 and tau[2] == zb[2, -16]      # ties kept: all of row 0; 16 elements for top_k 12


def test_mixed_greedy_rows_and_repeatability():
    cfg = inputs.config3(rows=8, vocab=32000, hist_len=128)
    cfg["temperature"][::2] = 0.0                                          # every other row greedy
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    hist = torch.from_numpy(cfg["history"]).cuda()
    u = torch.from_numpy(cfg["uniforms"]).cuda()
    p = lm.SamplingParams(draw="inverse_cdf", repetition_penalty=1.1, presence_penalty=0.5, **knobs)
    a = lm.sample(x, p, history=hist, uniforms=u, return_tau=True)
    b = lm.sample(x, p, history=hist, uniforms=u, return_tau=True)
    assert torch.equal(a.tokens, b.tokens) and torch.equal(a.tau, b.tau)   # run twice: identical bits
    for i in range(0, 8, 2):
        z = oracle.apply_penalties(oracle.bf16_to_f32(cfg["logits"][i]), cfg["history"][i], 1.1, 0.5)
        assert int(a.tokens[i]) == oracle.argmax(z)
    # results do not depend on how the batch is split (row-sharded batches): rows 4..7 alone, with their global offset
    s = lm.SamplingParams(seed=9, draw="gumbel", **{k: v[4:] for k, v in knobs.items()})
    full = lm.sample(x, lm.SamplingParams(seed=9, draw="gumbel", **knobs), step=2)
    part = lm.sample(x[4:], s, step=2, row_offset=4)
    assert torch.equal(full.tokens[4:], part.tokens)


def test_invalid_arguments_raise_before_launch():
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        lm.StochasticSampler(temperature=0.0)
    with pytest.raises(ValueError):
        lm.sample(x, temperature=-1.0)
    with pytest.raises(ValueError):
        lm.sample(x, temperature=1.0, draw="inverse_cdf")                  # no uniforms
    with pytest.raises(TypeError):
        lm.sample(x.to(torch.float16), temperature=1.0)
    with pytest.raises(RuntimeError):
        lm.sample(x.cpu(), temperature=1.0)
    bad_t = torch.tensor([float("nan"), 1.0], device="cuda")               # a per-row knob cannot be checked on the host: the row reports -1
    r = lm.sample(x, temperature=bad_t, return_status=True)
    assert int(r.tokens[0]) == -1 and int(r.status[0]) & 16 and int(r.tokens[1]) >= 0


def test_streaming_and_generic_paths_agree():
    """BF16 rows that only ask for tokens take the one-pass streaming kernel; asking for statistics routes the same rows
    through the generic kernel. Same tokens, same thresholds; rows the streaming kernel cannot take fall back by themselves."""
    rows = 40
    cfg = inputs.config3(rows=rows, seed=31)
    cfg["logits"][5, :70000] = 0xFF80                                      # a masked row: 70000 x -inf (counted apart from the codes: stays)
    cfg["logits"][6, :] = oracle.f32_to_bf16(np.float32([1.5]))[0]         # every logit equal: overflows a 16-bit counter -> falls back
    cfg["history"][7, :] = 11                                              # one distinct history id
    cfg["top_k"][8] = 1
    cfg["top_p"][9] = 1.0                                                  # top-p off
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    hist, u = torch.from_numpy(cfg["history"]).cuda(), torch.from_numpy(cfg["uniforms"]).cuda()
    for draw in ("inverse_cdf", "gumbel"):
        for extra in (dict(), dict(min_p=0.02), dict(topp_in_topk=True)):
            p = lm.SamplingParams(seed=5, draw=draw, repetition_penalty=1.1, presence_penalty=0.5, **knobs, **extra)
            fast = lm.sample(x, p, history=hist, uniforms=u, step=1, return_tau=True, return_status=True)
            slow = lm.sample(x, p, history=hist, uniforms=u, step=1, return_tau=True, return_status=True, return_stats=True)
            fs, ss = fast.status.cpu().numpy(), slow.status.cpu().numpy()
            assert np.all(ss & 1) and not (fs[5] & 1) and (fs[6] & 1) and np.count_nonzero(fs & 1) <= 3, fs   # the degenerate row, at most a stray dense one
            assert torch.equal(fast.tau, slow.tau), (draw, extra)
            assert torch.equal(fast.tokens, slow.tokens), (draw, extra)
    tok, tau, _ = oracle.sample_batch(cfg["logits"], temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], history=cfg["history"],
                                      repetition_penalty=1.1, presence_penalty=0.5, draw="inverse_cdf", uniforms=cfg["uniforms"], n_threads=8)
    r = lm.sample(x, lm.SamplingParams(draw="inverse_cdf", repetition_penalty=1.1, presence_penalty=0.5, **knobs), history=hist, uniforms=u, return_tau=True)
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)


def test_streaming_path_with_dense_side_values():
    """Penalised logits that crowd one BF16 bin (equal history targets, thresholds landing on penalised values)."""
    V, rows = 8192, 6
    rng = np.random.default_rng(8)
    z = (rng.standard_normal((rows, V)) * 2).astype(np.float32)
    z[:, :40] = 6.0                                                        # forty equal top logits, all penalised below: 40 side values in one bin
    hist = np.tile(np.arange(40, dtype=np.int32), (rows, 1))
    hist[3:, 20:] = 5000                                                   # rows 3..: only twenty of them penalised
    cfg = dict(logits=oracle.f32_to_bf16(z), temperature=np.full(rows, 0.9, np.float32), top_k=np.array([5, 30, 45, 5, 30, 0], np.int32),
               top_p=np.array([0.0, 0.5, 0.99, 0.3, 0.0, 0.7], np.float32), history=hist, uniforms=rng.random(rows).astype(np.float32),
               repetition_penalty=1.07, presence_penalty=0.013)
    r, tok, tau, _ = run_both(cfg, "inverse_cdf", rows)
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)


@pytest.mark.parametrize("draw", ["inverse_cdf", "gumbel"])
def test_candidate_path_equals_the_oracle(draw):
    """Rows with 1 <= top_k <= 1024 take the one-pass candidate kernel (several rows per block here: grid_limit); check them
    against the CPU oracle like any other, and against the histogram path alone (exact_only)."""
    rows = 36
    cfg = inputs.config3(rows=rows, seed=91)
    cfg["top_k"][:] = np.array([20, 50, 1000, 1, 7, 333], np.int32)[np.arange(rows) % 6]
    cfg["temperature"][3] = 0.05                                            # nearly greedy: the top-p boundary falls inside the top-k set
    cfg["temperature"][10] = 0.11
    z30 = oracle.bf16_to_f32(cfg["logits"][30]) - np.float32(20.0)          # no positive logit: the kernel hands the row back
    cfg["logits"][30] = oracle.f32_to_bf16(z30)
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    hist, u = torch.from_numpy(cfg["history"]).cuda(), torch.from_numpy(cfg["uniforms"]).cuda()
    with_nan = x.clone()
    with_nan[4, 77777] = float("nan")                                       # a NaN row is reported by the exact path, not decided here
    st = lm.sample(with_nan, lm.SamplingParams(seed=5, draw=draw, **knobs), uniforms=u, return_status=True).status.cpu().numpy()
    assert (st[4] & 2) and not (st[4] & 64) and not np.any(np.delete(st, 4) & 2)
    for extra in (dict(), dict(min_p=0.05), dict(topp_in_topk=True)):
        p = lm.SamplingParams(seed=5, draw=draw, repetition_penalty=1.1, presence_penalty=0.5, grid_limit=3, **knobs, **extra)
        r = lm.sample(x, p, history=hist, uniforms=u, step=2, return_tau=True, return_status=True)
        status = r.status.cpu().numpy()
        assert np.count_nonzero(status & 64) >= rows - 5 and not (status[30] & 64), status   # all but row 30 and the odd hand-back
        tok, tau, _ = oracle.sample_batch(cfg["logits"], temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], history=cfg["history"],
                                          repetition_penalty=1.1, presence_penalty=0.5, draw=draw, uniforms=cfg["uniforms"], seed=5, step=2, n_threads=8,
                                          **{k: v for k, v in extra.items()})
        np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
        got = r.tokens.cpu().numpy()
        assert np.all((got == tok) | ((status & 4) != 0)), (extra, np.nonzero(got != tok))
        # and the same rows through the histogram path alone: identical
        q = lm.SamplingParams(seed=5, draw=draw, repetition_penalty=1.1, presence_penalty=0.5, exact_only=True, **knobs, **extra)
        h = lm.sample(x, q, history=hist, uniforms=u, step=2, return_tau=True, return_status=True)
        assert not np.any(h.status.cpu().numpy() & 64)
        assert torch.equal(h.tau, r.tau) and torch.equal(h.tokens, r.tokens)


def test_streaming_draw_over_wide_kept_sets():
    """Rows without a top_k draw through the histogram kernel: kept sets that stay in the
    positive codes, reach into the negative ones (no filter at all, a loose min_p, a row shifted below zero) or
    lie many binades apart must all give the oracle's token. Row 5 holds magnitudes below the kernel's code window
    (2^-39): it is handed to the generic kernel, with the same result."""
    rows, V = 12, 151936
    rng = np.random.default_rng(23)
    z = (rng.standard_normal((rows, V)) * 2).astype(np.float32)
    z[3] -= 30.0                                                            # every logit negative
    z[4] *= 1e-3                                                            # tiny magnitudes: many binades below the maximum
    z[5, ::7] *= 1e-30                                                      # values far outside both windows
    z[6] = np.abs(z[6])                                                     # no negative code at all
    cfg = dict(logits=oracle.f32_to_bf16(z), temperature=np.float32([1.0, 1.5, 0.7, 1.2, 1.0, 0.9, 1.0, 0.3, 1.0, 1.4, 0.6, 1.1]),
               top_k=np.zeros(rows, np.int32), top_p=np.float32([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.9, 0.999, 0.97, 0.5, 1.0]),
               history=rng.integers(0, V, (rows, 64)).astype(np.int32), uniforms=rng.random(rows).astype(np.float32),
               repetition_penalty=1.2, presence_penalty=0.3)
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    for extra in (dict(), dict(min_p=1e-6), dict(min_p=0.01)):
        r = lm.sample(x, lm.SamplingParams(draw="inverse_cdf", repetition_penalty=1.2, presence_penalty=0.3, **knobs, **extra),
                      history=torch.from_numpy(cfg["history"]).cuda(), uniforms=torch.from_numpy(cfg["uniforms"]).cuda(), return_tau=True, return_status=True)
        tok, tau, _ = oracle.sample_batch(cfg["logits"], temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], history=cfg["history"],
                                          repetition_penalty=1.2, presence_penalty=0.3, draw="inverse_cdf", uniforms=cfg["uniforms"], n_threads=8, **extra)
        generic = (r.status.cpu().numpy() & 1) != 0
        assert generic.tolist() == [row == 5 for row in range(rows)], r.status   # all but row 5 through the histogram kernel
        np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
        np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)


def test_large_batch_launch_order():
    """More than sixteen rows per SM: the top-k kernel runs first and the histogram kernel takes its list (smaller batches run the
    two side by side). Same tokens and thresholds as the oracle either way."""
    rows, V = 2600, 32768
    cfg = inputs.config3(rows=rows, vocab=V, hist_len=256, seed=61)
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    hist, u = torch.from_numpy(cfg["history"]).cuda(), torch.from_numpy(cfg["uniforms"]).cuda()
    p = lm.SamplingParams(draw="inverse_cdf", repetition_penalty=1.1, presence_penalty=0.5, **knobs)
    r = lm.sample(x, p, history=hist, uniforms=u, return_tau=True, return_status=True)
    tok, tau, _ = oracle.sample_batch(cfg["logits"], temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], history=cfg["history"],
                                      repetition_penalty=1.1, presence_penalty=0.5, draw="inverse_cdf", uniforms=cfg["uniforms"], n_threads=8)
    status = r.status.cpu().numpy()
    assert np.count_nonzero(status & 64) >= 0.7 * np.count_nonzero(cfg["top_k"] > 0)        # the rows with a top_k went through the top-k kernel
    np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
    np.testing.assert_array_equal(r.tokens.cpu().numpy(), tok)
    small = lm.sample(x[:700], lm.SamplingParams(draw="inverse_cdf", repetition_penalty=1.1, presence_penalty=0.5, **{k: v[:700] for k, v in knobs.items()}),
                      history=hist[:700], uniforms=u[:700], return_tau=True)
    assert torch.equal(small.tokens, r.tokens[:700]) and torch.equal(small.tau, r.tau[:700])


@pytest.mark.parametrize("rows,vocab,calls", [(600, 32768, 300), (2600, 32768, 60)])
def test_back_to_back_calls_are_repeatable(rows, vocab, calls):
    """Many calls in a row on one stream without a host synchronisation in between (each reuses the workspace's counters and
    row lists, in both launch orders): every call returns what the first one did."""
    cfg = inputs.config3(rows=rows, vocab=vocab, hist_len=128, seed=5)
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    hist, u = torch.from_numpy(cfg["history"]).cuda(), torch.from_numpy(cfg["uniforms"]).cuda()
    p = lm.SamplingParams(draw="inverse_cdf", repetition_penalty=1.1, presence_penalty=0.5, **knobs)
    first = lm.sample(x, p, history=hist, uniforms=u, return_tau=True)
    outs = [torch.empty(rows, dtype=torch.int32, device="cuda") for _ in range(calls)]
    for o in outs:
        lm.sample(x, p, history=hist, uniforms=u, out=o)
    torch.cuda.synchronize()
    stacked = torch.stack(outs)
    assert bool((stacked == first.tokens.unsqueeze(0)).all())
    tok, _, _ = oracle.sample_batch(cfg["logits"][:64], temperature=cfg["temperature"][:64], top_k=cfg["top_k"][:64], top_p=cfg["top_p"][:64],
                                    history=cfg["history"][:64], repetition_penalty=1.1, presence_penalty=0.5, draw="inverse_cdf",
                                    uniforms=cfg["uniforms"][:64], n_threads=8)
    np.testing.assert_array_equal(first.tokens[:64].cpu().numpy(), tok)


@pytest.mark.parametrize("rows", [96, 2600])
def test_sampling_call_in_a_cuda_graph(rows):
    """A sampling call captured into a CUDA graph (both launch orders; the small one uses programmatic stream serialization)
    replays to the same tokens as the eager call, several times over."""
    V = 32768
    cfg = inputs.config3(rows=rows, vocab=V, hist_len=64, seed=17)
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    hist, u = torch.from_numpy(cfg["history"]).cuda(), torch.from_numpy(cfg["uniforms"]).cuda()
    p = lm.SamplingParams(draw="inverse_cdf", repetition_penalty=1.1, presence_penalty=0.5, **knobs)
    eager = lm.sample(x, p, history=hist, uniforms=u).tokens.clone()
    out = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            lm.sample(x, p, history=hist, uniforms=u, out=out)
    torch.cuda.synchronize()
    for _ in range(5):
        out.fill_(-7)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)


@pytest.mark.parametrize("draw", ["inverse_cdf", "gumbel"])
def test_top_k_kernel_edge_rows(draw):
    """Rows built to stress the one-pass top-k kernel at a vocabulary it accepts (32768): ties through the k-th rank, more
    ties than it can hold, every logit equal, a -inf mask over most of the row, a +inf logit, a tiny temperature, one
    repeated history id, penalised values crowding the top. Whatever kernel ends up finishing a row, tokens and thresholds
    are the oracle's."""
    V, rows = 32768, 12
    rng = np.random.default_rng(123)
    z = (rng.standard_normal((rows, V)) * 2).astype(np.float32)
    z[0, 100:140] = 7.5                                                     # forty equal logits across the 20th rank
    z[1, :3000] = 8.0                                                       # 3000 equal top logits: more than the kernel's candidate list
    z[2, :] = 1.25                                                          # every logit equal
    z[3, 5000:] = -np.inf                                                   # masked vocabulary
    z[4, 77] = np.inf
    z[6, 9] = 30.0                                                          # far above anything sampled for the cutoff
    z[8, :64] = 6.0                                                         # the top of the row is all penalised (history below)
    z[10] *= 0.01                                                           # tiny logits: few positive codes above the cutoff
    codes = oracle.f32_to_bf16(z)
    hist = rng.integers(0, V, (rows, 512)).astype(np.int32)
    hist[7, :] = 31                                                         # one repeated id
    hist[8, :64] = np.arange(64)
    cfg = dict(logits=codes, temperature=np.float32([0.7, 1.0, 0.9, 1.1, 1.0, 0.02, 0.8, 1.0, 0.9, 1.3, 1.0, 0.6]),
               top_k=np.int32([20, 1000, 5, 50, 20, 50, 20, 7, 50, 1024, 20, 1]), top_p=np.float32([0.9, 0.95, 0.5, 0.9, 0.9, 0.99, 0.8, 0.0, 0.97, 0.9, 0.9, 0.3]),
               history=hist, uniforms=rng.random(rows).astype(np.float32))
    x = bf16_tensor(codes)
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    for extra in (dict(), dict(min_p=0.01), dict(topp_in_topk=True)):
        r = lm.sample(x, lm.SamplingParams(seed=9, draw=draw, repetition_penalty=1.3, presence_penalty=0.4, **knobs, **extra),
                      history=torch.from_numpy(hist).cuda(), uniforms=torch.from_numpy(cfg["uniforms"]).cuda(), step=4, return_tau=True, return_status=True)
        tok, tau, _ = oracle.sample_batch(codes, temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], history=hist,
                                          repetition_penalty=1.3, presence_penalty=0.4, draw=draw, uniforms=cfg["uniforms"], seed=9, step=4, n_threads=8, **extra)
        status = r.status.cpu().numpy()
        keep = np.arange(rows) != 4                                         # the +inf row: weights are NaN by definition, only the threshold is compared
        np.testing.assert_array_equal(r.tau.cpu().numpy(), tau)
        got = r.tokens.cpu().numpy()
        assert np.all((got == tok)[keep] | ((status & 4) != 0)[keep]), (extra, got, tok, status)
        assert np.count_nonzero(status & 64) >= 5                           # the ordinary rows did go through the top-k kernel


def test_penalised_rows_equal_the_reference(golden):
    """16 penalised rows of the batched configuration: the thresholds and Gumbel tokens the reference's own sampling_ref gives on
    the penalised rows (tests/golden), through the candidate kernel and through the histogram kernel alone."""
    g = golden["penalised"]
    cfg = inputs.config3(rows=g["rows"], seed=3)
    x = bf16_tensor(cfg["logits"])
    knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
    for exact_only in (False, True):
        p = lm.SamplingParams(seed=12345, draw="gumbel", repetition_penalty=1.1, presence_penalty=0.5, exact_only=exact_only, **knobs)
        r = lm.sample(x, p, history=torch.from_numpy(cfg["history"]).cuda(), step=1, return_tau=True, return_status=True)
        status = r.status.cpu().numpy()
        assert not np.any(status & 1)
        np.testing.assert_array_equal(r.tau.cpu().numpy(), np.array(g["tau"], dtype=np.float32))
        got = r.tokens.cpu().numpy()
        assert np.all((got == np.array(g["tokens_seed12345_step1"])) | ((status & 4) != 0))


def test_two_streams_sample_at_once_with_their_own_workspaces():
    """Calls that can overlap on the GPU must not share scratch: the host layer keeps one workspace per stream. Two streams run
    different batches again and again, side by side; each gets what it gets alone."""
    cfgs = [inputs.config3(rows=48, vocab=32768, hist_len=256, seed=s) for s in (71, 72)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    work = []
    for cfg in cfgs:
        knobs = {k: torch.from_numpy(cfg[k]).cuda() for k in ("temperature", "top_k", "top_p")}
        work.append((bf16_tensor(cfg["logits"]), lm.SamplingParams(draw="inverse_cdf", repetition_penalty=1.1, presence_penalty=0.5, **knobs),
                     torch.from_numpy(cfg["history"]).cuda(), torch.from_numpy(cfg["uniforms"]).cuda()))
    alone = [lm.sample(x, p, history=h, uniforms=u).tokens.clone() for x, p, h, u in work]
    torch.cuda.synchronize()
    got = [[], []]
    for _ in range(20):
        for i, (x, p, h, u) in enumerate(work):
            with torch.cuda.stream(streams[i]):
                got[i].append(lm.sample(x, p, history=h, uniforms=u).tokens)
    torch.cuda.synchronize()
    for i in range(2):
        assert all(torch.equal(t, alone[i]) for t in got[i])


def test_row_maxima_come_out_of_every_kernel_and_feed_the_verify_step():
    """The reference's sampler leaves each row's maximum for its verify kernels (KEPT_STATS). out_vmax is that: the maximum of the
    (penalised) row, whichever kernel took the row."""
    rows, vocab = 40, 151936
    rng = np.random.default_rng(17)
    codes = oracle.f32_to_bf16((rng.standard_normal((rows, vocab)) * 2).astype(np.float32))
    hist = rng.integers(0, vocab, (rows, 512)).astype(np.int32)
    hist[:, 0] = oracle.bf16_to_f32(codes).argmax(-1)                                 # the raw maximum is penalised in every row
    want = np.stack([oracle.apply_penalties(oracle.bf16_to_f32(codes[r]), hist[r], 1.2, 0.3).max() for r in range(rows)])
    x = bf16_tensor(codes)
    t = torch.from_numpy(np.where(np.arange(rows) % 5 == 0, 0.0, 0.9).astype(np.float32))   # greedy rows among them
    k = torch.from_numpy(np.where(np.arange(rows) % 2 == 0, 0, 30).astype(np.int32))        # histogram-kernel and candidate-kernel rows
    p = lm.SamplingParams(temperature=t, top_k=k, top_p=0.9, repetition_penalty=1.2, presence_penalty=0.3, seed=3)
    for extra in ({}, {"return_stats": True}):                                             # the streaming kernels; the generic kernel
        r = lm.sample(x, p, history=torch.from_numpy(hist).cuda(), return_vmax=True, **extra)
        np.testing.assert_array_equal(r.vmax.cpu().numpy(), want.astype(np.float32))
    few = lm.sample(x[:3], lm.SamplingParams(temperature=0.9, top_k=30, top_p=0.9, seed=3), return_vmax=True, return_status=True)   # the sliced path
    assert np.all(few.status.cpu().numpy() & 256)                                         # (the sliced path took them)
    np.testing.assert_array_equal(few.vmax.cpu().numpy(), oracle.bf16_to_f32(codes[:3]).max(-1))
    # and on to the verify step: thresholds and maxima of the 8 rows from one sampler call
    target, drafts, q, ua, uf = inputs.config2(vocab=vocab, seed=23)
    xt = bf16_tensor(target)
    s = lm.sample(xt, lm.SamplingParams(temperature=0.8, top_k=torch.full((8,), 50, dtype=torch.int32), top_p=0.95, seed=1), return_tau=True, return_vmax=True)
    args = (xt, torch.from_numpy(drafts).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(ua).cuda(), torch.tensor([uf]), "stochastic")
    a = lm.verify(*args, temperature=0.8, tau=s.tau)
    b = lm.verify(*args, temperature=0.8, tau=s.tau, target_vmax=s.vmax)
    assert [v.cpu().tolist() for v in a] == [v.cpu().tolist() for v in b]
    # ... and the kept sets' masses, for every way a step can end (mixed, every draft accepted, first draft rejected) and both residual draws
    for u in (ua, np.zeros(7, np.float32), np.full(7, 0.999, np.float32)):
        for draw in ("inverse_cdf", "gumbel"):
            args = (xt, torch.from_numpy(drafts).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(u).cuda(), torch.tensor([uf]), "stochastic")
            kw = dict(temperature=0.8, tau=s.tau, residual_draw=draw, seed=5, step=2, return_p_draft=True)
            a = lm.verify(*args, **kw)
            b = lm.verify(*args, target_vmax=s.vmax, target_mass=s.mass, **kw)
            assert [v.cpu().tolist() for v in a] == [v.cpu().tolist() for v in b], (draw, u[0])
    # the masses themselves, from every kernel and both of the sampler's draws: the integer sum the oracle forms
    z = oracle.bf16_to_f32(target)
    for draw in ("inverse_cdf", "gumbel"):
        for knobs in (dict(top_k=torch.full((8,), 50, dtype=torch.int32)), dict(top_k=torch.zeros(8, dtype=torch.int32)), dict(top_k=50)):
            r = lm.sample(xt, lm.SamplingParams(temperature=0.8, top_p=0.95, seed=1, draw=draw, **knobs), uniforms=torch.full((8,), 0.3), return_tau=True, return_vmax=True)
            for i in range(8):
                total = C.c_uint64()
                oracle.lib().lmo_sample_invcdf(z[i].ctypes.data_as(C.POINTER(C.c_float)), z.shape[1], float(r.tau[i]), np.float32(0.8), np.float32(0.3), C.byref(total))
                assert int(r.mass[i]) == total.value, (draw, knobs, i)
