"""DSpark verification on the GPU against the CPU oracle: accept length and final token bit-exact."""
import numpy as np
import pytest
import torch

import oracle
import lithos_metal_b200 as lm
from tests import inputs
from tests.test_gpu_sampling import bf16_tensor

pytestmark = pytest.mark.gpu


def gpu_verify(target, drafts, q, ua, uf, mode, **kw):
    out = lm.verify(bf16_tensor(target) if target.dtype == np.uint16 else torch.from_numpy(target).cuda(), torch.from_numpy(drafts).cuda(),
                    None if q is None else torch.from_numpy(q).cuda(), None if ua is None else torch.from_numpy(ua).cuda(),
                    None if uf is None else torch.tensor([uf], dtype=torch.float32), mode, **kw)
    return int(out[0]), int(out[1]), out[2].cpu().tolist(), (out[3].cpu().numpy() if len(out) > 3 else None)


@pytest.mark.parametrize("vocab", [151936, 2000, 37])
def test_greedy_verify(vocab):
    target, drafts, _, _, _ = inputs.config2(vocab=vocab, seed=vocab)
    z = oracle.bf16_to_f32(target)
    for n_match in (0, 3, 7):
        d = drafts.copy()
        d[:n_match] = z[:n_match].argmax(-1)
        if n_match < 7 and d[n_match] == z[n_match].argmax():
            d[n_match] = (d[n_match] + 1) % vocab
        acc, fin, toks = oracle.verify_greedy(target, d)
        g_acc, g_fin, g_toks, _ = gpu_verify(target, d, None, None, None, "greedy")
        assert (g_acc, g_fin) == (acc, fin) == (n_match, int(z[n_match].argmax()))
        assert g_toks == d[:acc].tolist() + [fin] + [-1] * (7 - acc)


@pytest.mark.parametrize("vocab,seed", [(151936, 2), (151936, 5), (2000, 7), (300, 9)])
def test_stochastic_verify_equals_the_oracle(vocab, seed):
    """Benchmark configuration 2 (and small vocabularies): random drafts, q = softmax(target + noise), seeded uniforms."""
    target, drafts, q, ua, uf = inputs.config2(vocab=vocab, seed=seed)
    z = oracle.bf16_to_f32(target)
    cases = [(drafts, ua)]
    d2 = drafts.copy(); d2[:4] = z[:4].argmax(-1)                          # likely accepts first
    cases.append((d2, ua))
    cases.append((z[:7].argmax(-1).astype(np.int32), np.zeros(7, np.float32)))          # u = 0: everything accepted, bonus row drawn
    cases.append((drafts, np.full(7, 0.99999, np.float32)))
    for d, u in cases:
        acc, fin, pd = oracle.verify_stochastic(target, d, q, u, uf)
        g_acc, g_fin, g_toks, g_pd = gpu_verify(target, d, q, u, uf, "stochastic", return_p_draft=True)
        assert (g_acc, g_fin) == (acc, fin)
        assert g_toks == d[:acc].tolist() + [fin] + [-1] * (7 - acc)
        np.testing.assert_array_equal(g_pd, pd)


def test_stochastic_verify_with_kept_sets_and_temperature():
    """The general form: every row restricted to its kept set (tau from the sampler), temperature != 1, FP32 logits."""
    target, drafts, q, ua, uf = inputs.config2(vocab=32000, seed=11)
    z = oracle.bf16_to_f32(target)
    T = 0.8
    x = torch.from_numpy(z).cuda()
    tau = lm.sample(x, temperature=T, top_k=50, top_p=0.9, topp_in_topk=True, return_tau=True).tau
    tau_np = tau.cpu().numpy()
    for i in range(8):
        assert tau_np[i] == np.float32(oracle.thresholds(z[i], temperature=float(np.float32(T)), top_k=50, top_p=float(np.float32(0.9)), topp_in_topk=True))
    d = drafts.copy(); d[:3] = z[:3].argmax(-1)
    acc, fin, pd = oracle.verify_stochastic(z, d, q, ua, uf, temperature=T, tau=tau_np)
    out = lm.verify(x, torch.from_numpy(d).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(ua).cuda(), torch.tensor([uf]), "stochastic",
                    temperature=T, tau=tau, return_p_draft=True)
    assert (int(out[0]), int(out[1])) == (acc, fin)
    np.testing.assert_array_equal(out[3].cpu().numpy(), pd)


def test_verify_distribution_matches_the_target():
    """The committed first token is distributed as the target's own softmax whatever the drafter proposes
    (the property the reference checks with a chi-square over seeds, tests/kernels/test_spec_sampling.py:79-118)."""
    rng = np.random.default_rng(21)
    V, n = 64, 3
    z = (rng.standard_normal((n + 1, V)) * 1.5).astype(np.float32)
    qz = z[:n] + rng.standard_normal((n, V)).astype(np.float32)
    q = np.exp(qz - qz.max(-1, keepdims=True)); q = (q / q.sum(-1, keepdims=True)).astype(np.float32)
    p = oracle.warped_probabilities(z[0])
    x, qd = torch.from_numpy(z).cuda(), torch.from_numpy(q).cuda()
    N = 3000
    counts = np.zeros(V)
    u_all = rng.random((N, n + 1)).astype(np.float32)
    draws = np.array([rng.choice(V, p=q[r] / q[r].sum(), size=N) for r in range(n)]).T.astype(np.int32)
    for t in range(N):
        out = lm.verify(x, torch.from_numpy(draws[t]).cuda(), qd, torch.from_numpy(u_all[t, :n]).cuda(), torch.from_numpy(u_all[t, n:]).cuda(), "stochastic")
        counts[int(out[2][0])] += 1
    sigma = np.sqrt(p * (1 - p) / N)
    assert np.all(np.abs(counts / N - p) <= 4.5 * sigma + 1e-9)


def test_repeated_calls_leave_the_workspace_clean():
    target, drafts, q, ua, uf = inputs.config2(vocab=5000, seed=4)
    first = gpu_verify(target, drafts, q, ua, uf, "stochastic")
    for _ in range(5):
        assert gpu_verify(target, drafts, q, ua, uf, "stochastic")[:3] == first[:3]
        gpu_verify(target, drafts, None, None, None, "greedy")
