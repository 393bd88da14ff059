"""Draft-side sampling (draft_q) and verification against the drafter's logits, on the GPU through the C ABI."""
import numpy as np
import pytest
import torch

import lithos_metal_b200 as lm
import oracle

pytestmark = pytest.mark.gpu


def bf16_tensor(codes: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(codes.view(np.int16).copy()).cuda().view(torch.bfloat16)


def drafter_rows(vocab: int) -> np.ndarray:
    """The rows of tests/golden/make_golden.py::draft_q_section: 7 draft positions, BF16 N(0, 2^2)."""
    rng = np.random.default_rng(7000 + vocab)
    return oracle.f32_to_bf16((rng.standard_normal((7, vocab)) * 2.0).astype(np.float32))


@pytest.mark.parametrize("vocab", [1000, 151936])
@pytest.mark.parametrize("temperature", [0.3, 1.0])
def test_drafts_equal_the_reference(golden, vocab, temperature):
    """Tokens: what the reference's sampling_ref.sample draws on stream 2000 + k (bit-exact, or flagged as a near-tie of the
    float32 log); lse: the float64 log-sum-exp within 2e-6 relative (the statement is FP32 in the reference); vmax and the
    integer mass: the CPU oracle's, exactly. All seven positions in one call and one position per call give the same."""
    g = golden["draft_q"][f"{vocab}/{temperature}"]
    lb = drafter_rows(vocab)
    assert int(lb.astype(np.uint64).sum()) == g["logits_crc"]
    x = bf16_tensor(lb)
    r = lm.draft_q(x, temperature=temperature, seed=12345, step=3, copy_logits=True)
    tok, status = r.tokens.cpu().numpy(), r.status.cpu().numpy()
    assert np.all((tok == np.array(g["tokens"])) | ((status & 4) != 0)), (tok, g["tokens"], status)
    np.testing.assert_allclose(r.lse.cpu().numpy(), np.array(g["lse"]), rtol=2e-6)
    assert torch.equal(r.q_logits, x)
    for k in range(7):
        t, vmax, mass, lse, _ = oracle.draft_q(lb[k], temperature=temperature, seed=12345, step=3, position=k)
        assert int(r.mass[k]) == mass and float(r.vmax[k]) == vmax and float(r.lse[k]) == np.float32(lse)
        assert t == g["tokens"][k]
        one = lm.draft_q(x[k:k + 1], temperature=temperature, seed=12345, step=3, first_position=k)
        assert int(one.tokens[0]) == int(tok[k]) and int(one.mass[0]) == mass
    f32 = lm.draft_q(x.float(), temperature=temperature, seed=12345, step=3)            # FP32 rows: same values, same draws
    assert torch.equal(f32.tokens, r.tokens) and torch.equal(f32.mass, r.mass)


def test_draft_q_is_the_unfiltered_sampler_draw():
    """The same token as the row sampler draws for an unfiltered row on stream 2000 + k."""
    lb = drafter_rows(151936)
    x = bf16_tensor(lb)
    r = lm.draft_q(x, temperature=0.8, seed=99, step=11)
    s = lm.sample(x, lm.SamplingParams(temperature=0.8, seed=99, draw="gumbel"), step=11, row_offset=2000)
    assert torch.equal(r.tokens, s.tokens)


@pytest.mark.parametrize("temperature", [0.6, 1.0])
def test_verify_from_drafter_logits(temperature):
    """Stochastic verification with q given as the drafter's BF16 logits + draft_q's statistics: the same outcome as the CPU
    oracle fed the probabilities those define, and as the GPU fed the same probabilities as a float32 tensor."""
    V, n = 151936, 7
    rng = np.random.default_rng(404)
    target = oracle.f32_to_bf16((rng.standard_normal((n + 1, V)) * 2.0).astype(np.float32))
    drafter = oracle.f32_to_bf16(oracle.bf16_to_f32(target[:n]) + (rng.standard_normal((n, V)) * 0.5).astype(np.float32))
    tx, dx = bf16_tensor(target), bf16_tensor(drafter)
    for trial in range(6):
        st = lm.draft_q(dx, temperature=temperature, seed=7, step=trial)
        ids = st.tokens
        ua, uf = rng.random(n).astype(np.float32), np.float32(rng.random())
        if trial == 0:
            ua[:] = 0.0                                                     # everything accepted: the bonus row decides
        got = lm.verify(tx, ids, None, torch.from_numpy(ua), torch.tensor([uf]), "stochastic", temperature=temperature, draft_logits=dx,
                        draft_stats=st, return_p_draft=True)
        q = np.stack([oracle.draft_probs(drafter[k], temperature=temperature, vmax=float(st.vmax[k]), mass=int(st.mass[k])) for k in range(n)])
        acc, fin, pd = oracle.verify_stochastic(target, ids.cpu().numpy(), q, ua, uf, temperature=temperature)
        assert (int(got[0]), int(got[1])) == (acc, fin), trial
        np.testing.assert_array_equal(got[3].cpu().numpy(), pd)
        same = lm.verify(tx, ids, torch.from_numpy(q).cuda(), torch.from_numpy(ua), torch.tensor([uf]), "stochastic", temperature=temperature)
        assert (int(same[0]), int(same[1])) == (acc, fin)
        # the whole hand-over of a round: q from the drafter's logits and statistics, the target rows' maxima and masses from the sampler
        kept = lm.sample(tx, lm.SamplingParams(temperature=temperature, top_k=torch.zeros(n + 1, dtype=torch.int32), draw="inverse_cdf"),
                         uniforms=torch.full((n + 1,), 0.5), return_vmax=True)
        both = lm.verify(tx, ids, None, torch.from_numpy(ua), torch.tensor([uf]), "stochastic", temperature=temperature, draft_logits=dx,
                         draft_stats=st, target_vmax=kept.vmax, target_mass=kept.mass)
        assert (int(both[0]), int(both[1])) == (acc, fin), trial
    np.testing.assert_allclose(q.sum(axis=1), 1.0, rtol=1e-5)


def test_draft_q_argument_checks():
    x = torch.zeros(2, 1024, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        lm.draft_q(x, temperature=0.0)
    with pytest.raises(ValueError):
        lm.draft_q(torch.zeros(17, 1024, dtype=torch.bfloat16, device="cuda"), temperature=1.0)
    with pytest.raises(ValueError):
        lm.verify(torch.zeros(3, 1024, dtype=torch.bfloat16, device="cuda"), torch.zeros(2, dtype=torch.int32), None, torch.zeros(2), torch.zeros(1),
                  "stochastic")
    nan = x.clone(); nan[1, 5] = float("nan")
    st = lm.draft_q(nan, temperature=1.0).status.cpu().numpy()
    assert not (st[0] & 2) and (st[1] & 2)
