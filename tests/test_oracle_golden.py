"""The CPU oracle against the outputs of the reference's own Python code (tests/golden/reference_outputs.json):
thresholds, Gumbel-max tokens, kept-token probabilities, argmax edge cases, the accept-scan state machine, and
the second, independent kept-set oracle (the Hugging Face warpers' masks). No GPU."""
import numpy as np
import pytest

import oracle
from oracle import ref_numpy, spec_models
from tests import inputs


@pytest.mark.parametrize("vocab", [1000, 248320])
@pytest.mark.parametrize("name", list(inputs.OPTION_SETS))
def test_thresholds_and_gumbel_tokens_equal_the_reference(golden, vocab, name):
    opts = inputs.OPTION_SETS[name]
    g = golden["draws"][f"{vocab}/{name}"]
    lb = inputs.sampling_test_logits(vocab, opts)
    assert int(lb.astype(np.uint64).sum()) == g["logits_crc"]          # the regenerated inputs are the reference's inputs
    lf = oracle.bf16_to_f32(lb)
    near_ties = 0
    for i in range(3):
        tau = oracle.thresholds(lf[i], **opts)
        assert np.float32(tau) == np.float32(g["tau"][i])
        for step in (0, 1, 7):
            tok, gap = oracle.sample_gumbel(lf[i], seed=12345, step=step, t=i, **opts)
            if tok != g["tokens"][str(step)][i]:
                assert gap < 4e-6                                      # float32 log differs between libraries only at a near-tie
                near_ties += 1
    assert near_ties == 0


@pytest.mark.parametrize("name", ["plain", "topk", "topp", "minp", "all"])
def test_numpy_restatement_equals_the_reference(golden, name):
    opts = inputs.OPTION_SETS[name]
    lf = oracle.bf16_to_f32(inputs.sampling_test_logits(1000, opts))
    g = golden["draws"][f"1000/{name}"]
    for i in range(3):
        assert ref_numpy.thresholds(lf[i], **opts) == g["tau"][i]
        assert ref_numpy.sample(lf[i], seed=12345, step=7, t=i, **opts) == g["tokens"]["7"][i]


@pytest.mark.parametrize("name", ["plain", "topk", "topp", "minp", "all"])
def test_kept_probabilities_equal_the_reference(golden, name):
    opts = inputs.OPTION_SETS[name]
    lf = oracle.bf16_to_f32(inputs.sampling_test_logits(1000, opts))
    p = oracle.warped_probabilities(lf[0], **opts)
    g = golden["warped_probabilities"][name]
    assert np.nonzero(p)[0].tolist() == g["idx"]                       # the kept index set, exactly
    np.testing.assert_allclose(p[g["idx"]], g["p"], rtol=1e-12)


def test_known_answer_vector(golden):
    g = golden["known_answer_5"]
    lg = np.array(g["logits"], dtype=np.float32)
    assert oracle.thresholds(lg, top_k=3, top_p=0.85) == g["topp"] == lg[2]
    assert oracle.thresholds(lg, top_k=3, top_p=0.85, topp_in_topk=True) == g["topp_in_topk"] == lg[1]


@pytest.mark.parametrize("vocab", [248320, 1000, 300])
def test_argmax_edge_cases(golden, vocab):
    lf = oracle.bf16_to_f32(inputs.argmax_test_logits(vocab))
    got = [oracle.argmax(lf[t]) for t in range(4)]
    assert got == golden["argmax"][str(vocab)]
    assert got[0] == vocab - 1 and got[1] == 5                          # last index of a ragged tail; a tie -> lowest index


def test_kept_sets_equal_the_hf_warpers(golden):
    rng = np.random.default_rng(3)
    lf = oracle.bf16_to_f32(oracle.f32_to_bf16((rng.standard_normal((2, 4096)) * 3.0).astype(np.float32)))
    for name, g in golden["hf_warpers"].items():
        for i in range(2):
            tau = oracle.thresholds(lf[i], **g["opts"])
            assert np.nonzero(lf[i] >= np.float32(tau))[0].tolist() == g["kept"][i], name


def test_config1_outputs(golden):
    g = golden["config1"]
    z, u = inputs.config1()
    assert oracle.argmax(z[0]) == g["greedy"] == min(g["spikes"])      # eight tied spikes: the lowest index wins
    opts = dict(temperature=0.7, top_k=20, top_p=0.95)
    assert oracle.thresholds(z[0], **opts) == g["tau"] == 12.0
    p = oracle.warped_probabilities(z[0], **opts)
    assert np.nonzero(p)[0].tolist() == g["kept_idx"] == g["spikes"]
    np.testing.assert_allclose(p[g["kept_idx"]], g["kept_p"], rtol=1e-12)
    tok, _ = oracle.sample_gumbel(z[0], seed=1, step=0, t=0, **opts)
    assert tok == g["gumbel_token_seed1_step0"]
    # the injected-uniform draw: eight equal weights, so the token is the floor(8u)-th spike
    assert oracle.sample_invcdf(z[0], u, **opts) == g["spikes"][int(np.floor(8 * float(u)))]


def test_accept_scan_model_equals_the_reference_model(golden):
    for case, g in golden["accept_scan"].items():
        got, writes, _ = spec_models.accept_scan(g["state"], g["tokens"], g["ring_cap"], g["eos"], g["ctx_cap"])
        assert got == g["expect"], case
        assert [[a, b] for a, b in writes] == g["writes"], case
        got, writes, _ = spec_models.accept_scan(g["prefill_state"], g["tokens"], g["ring_cap"], g["eos"], g["ctx_cap"])
        assert got == g["prefill_expect"] and not writes, case


def test_spec_exp2_accuracy_and_cdf_target():
    xs = np.linspace(-60, 0, 20001).astype(np.float32)
    got = np.array([oracle.lib().lmo_spec_exp2(float(x)) for x in xs], dtype=np.float64)
    np.testing.assert_allclose(got, np.exp2(xs.astype(np.float64)), rtol=3e-7)
    assert oracle.lib().lmo_spec_exp2(0.0) == 1.0 and oracle.lib().lmo_spec_exp2(-101.0) == 0.0
    assert oracle.lib().lmo_cdf_target(0.0, 1000) == 0 and oracle.lib().lmo_cdf_target(0.99999994, 1 << 60) < (1 << 60)
    assert oracle.lib().lmo_cdf_target(0.5, 1001) == 500


def test_invcdf_draw_follows_the_kept_distribution():
    rng = np.random.default_rng(11)
    lf = np.full(512, -60.0, dtype=np.float32)
    lf[:16] = rng.standard_normal(16) * 1.5
    lf = oracle.bf16_to_f32(oracle.f32_to_bf16(lf))
    p = oracle.warped_probabilities(lf, temperature=0.9)
    n = 4000
    us = np.random.default_rng(5).random(n).astype(np.float32)
    counts = np.bincount([oracle.sample_invcdf(lf, u, temperature=0.9) for u in us], minlength=512)
    sigma = np.sqrt(p * (1 - p) / n)
    assert np.all(np.abs(counts / n - p)[:16] <= 4 * sigma[:16] + 1e-9) and counts[16:].sum() == 0


def test_penalties_apply_once_per_distinct_id():
    z = np.array([2.0, -1.0, 0.5, 3.0], dtype=np.float32)
    out = oracle.apply_penalties(z, [0, 0, 1, -1, 9], 2.0, 0.25)
    np.testing.assert_array_equal(out, np.array([0.75, -2.25, 0.5, 3.0], dtype=np.float32))


def test_verify_models_on_a_small_step():
    target, drafts, q, ua, uf = inputs.config2(vocab=2000, seed=7)
    z = oracle.bf16_to_f32(target)
    drafts = drafts.copy()
    drafts[0] = int(z[0].argmax()); drafts[1] = int(z[1].argmax())        # two drafts the target agrees with
    acc, fin, toks = oracle.verify_greedy(target, drafts)
    assert acc == 2 and fin == int(z[2].argmax()) and toks.tolist() == z.argmax(-1).tolist()
    # all-accept (u = 0) ends on the bonus row; certain reject (q = 1 at the draft, u near 1) at row 0 resamples row 0
    acc, fin, _ = oracle.verify_stochastic(target, drafts, q, np.zeros(7, np.float32), uf)
    assert acc == 7 and fin == oracle.sample_invcdf_index_order(z[7], uf)       # the verify step draws in index order
    acc, fin, _ = oracle.verify_stochastic(target, drafts, q, np.full(7, 0.999, np.float32), uf)
    assert 0 <= acc < 7 and 0 <= fin < 2000


@pytest.mark.parametrize("vocab", [1000, 151936])
@pytest.mark.parametrize("temperature", [0.3, 1.0])
def test_draft_q_equals_the_reference(golden, vocab, temperature):
    """The drafter's draw: the reference's sampling_ref.sample on stream 2000 + k; lse against the float64 log-sum-exp;
    the probabilities rebuilt from (vmax, integer mass) sum to one and reproduce exp(z/T - lse)."""
    g = golden["draft_q"][f"{vocab}/{temperature}"]
    rng = np.random.default_rng(7000 + vocab)
    lb = oracle.f32_to_bf16((rng.standard_normal((7, vocab)) * 2.0).astype(np.float32))
    assert int(lb.astype(np.uint64).sum()) == g["logits_crc"]
    for k in range(7):
        tok, vmax, mass, lse, gap = oracle.draft_q(lb[k], temperature=temperature, seed=12345, step=3, position=k)
        assert tok == g["tokens"][k] or gap < 4e-6
        assert abs(lse - g["lse"][k]) <= 2e-6 * abs(g["lse"][k])
        assert vmax == float(oracle.bf16_to_f32(lb[k]).max())
    q = oracle.draft_probs(lb[0], temperature=temperature, vmax=vmax_of(lb[0]), mass=oracle.draft_q(lb[0], temperature=temperature, seed=1, step=0, position=0)[2])
    z = oracle.bf16_to_f32(lb[0]).astype(np.float64)
    np.testing.assert_allclose(q, np.exp(z / temperature - g["lse"][0]), rtol=2e-5, atol=1e-12)
    assert abs(float(q.astype(np.float64).sum()) - 1.0) < 1e-5


def vmax_of(codes):
    return float(oracle.bf16_to_f32(codes).max())


def confidence_inputs():
    """tests/kernels/test_draft_ops.py:229-235: default_rng(4), gamma 7, hidden 256, rank 64, BF16-rounded weights and bias."""
    rbf = lambda x: oracle.bf16_to_f32(oracle.f32_to_bf16(np.asarray(x, dtype=np.float32)))
    rng = np.random.default_rng(4)
    hidden = oracle.f32_to_bf16(rng.standard_normal((7, 256)).astype(np.float32))
    emb = oracle.f32_to_bf16(rng.standard_normal((7, 64)).astype(np.float32))
    w = rbf(rng.standard_normal(320) * 0.05)
    b = rbf(rng.standard_normal(1) * 0.5)
    return hidden, emb, w, b


def test_confidence_head_equals_the_reference_test_values(golden):
    g = golden["confidence"]
    hidden, emb, w, b = confidence_inputs()
    assert int(hidden.astype(np.uint64).sum() + emb.astype(np.uint64).sum()) == g["inputs_crc"]
    # the reference's bar for its kernel is 2e-3; FP32 accumulation in the kernel's order stays within 1e-6 of the float64 statement
    # unless a BF16 rounding of the dot product flips (one BF16 ulp of the logit moves the sigmoid by < 2e-3)
    for got, want in ((oracle.confidence(hidden, emb, w, float(b[0])), g["with_emb"]),
                      (oracle.confidence(hidden, None, w[:256], float(b[0])), g["hidden_only"]),
                      (oracle.confidence(hidden, None, w[:256], float(b[0]), sts=g["sts"]), g["hidden_only_sts"])):
        assert np.abs(got - np.array(want)).max() <= 2e-3
        assert np.count_nonzero(np.abs(got - np.array(want)) > 1e-6) <= 1


def test_penalised_rows_equal_the_reference(golden):
    """Thresholds and Gumbel tokens of the reference's own sampling_ref on 16 PENALISED rows of the batched benchmark
    configuration (the penalties themselves are this repository's definition; what the reference then computes on the penalised
    FP32 rows is the pin)."""
    g = golden["penalised"]
    cfg = inputs.config3(rows=g["rows"], seed=3)
    assert int(cfg["logits"].astype(np.uint64).sum()) == g["logits_crc"] and int(cfg["history"].astype(np.uint64).sum()) == g["history_crc"]
    tok, tau, _ = oracle.sample_batch(cfg["logits"], temperature=cfg["temperature"], top_k=cfg["top_k"], top_p=cfg["top_p"], history=cfg["history"],
                                      repetition_penalty=1.1, presence_penalty=0.5, draw="gumbel", seed=12345, step=1, n_threads=8)
    np.testing.assert_array_equal(tau, np.array(g["tau"], dtype=np.float32))
    assert tok.tolist() == g["tokens_seed12345_step1"]
