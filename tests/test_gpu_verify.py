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


@pytest.mark.parametrize("mode", ["greedy", "stochastic"])
def test_verify_commits_the_round_like_accept_scan(mode):
    """verify(..., commit=...) = verify followed by accept_scan on the same StepState: state bytes, token ring and accept log
    equal; a stop token among the accepted drafts truncates the commit; a state that does not describe the round is refused
    (error 4), a finished one is left alone."""
    import lithos_metal_b200 as lm
    V, n = 8192, 7
    rng = np.random.default_rng(77)
    target = oracle.f32_to_bf16((rng.standard_normal((n + 1, V)) * 2.0).astype(np.float32))
    tx = torch.from_numpy(target.view(np.int16).copy()).cuda().view(torch.bfloat16)
    greedy_pick = oracle.bf16_to_f32(target).argmax(axis=1).astype(np.int32)
    layout = lm.StepStateLayout(8, 7)
    for trial in range(4):
        drafts = greedy_pick[:n].copy()
        if trial:
            drafts[rng.integers(1, n)] = 5                                  # a mismatch somewhere: accepted prefix + correction
        q = torch.softmax(tx[:n].float() + 0.3 * torch.randn(n, V, device="cuda", generator=torch.Generator("cuda").manual_seed(trial)), -1)
        ua, uf = torch.from_numpy(rng.random(n).astype(np.float32)), torch.tensor([float(rng.random())])
        eos = int(drafts[1]) if trial == 2 else -1                          # a stop token inside the accepted prefix
        base = {"step": 11, "position": 40, "t_this_step": n + 1, "verify_len": n, "anchor": 3, "pending_tokens": [3] + drafts.tolist(),
                "ring_head": 6, "ring_tail": 2, "gamma": n}
        args = (tx, torch.from_numpy(drafts)) + ((q, ua, uf, "stochastic") if mode == "stochastic" else (None, None, None, "greedy"))
        # separate launches
        st_a, ring_a, log_a = layout.to_device(base), torch.zeros(16, dtype=torch.int64, device="cuda"), torch.zeros(4, dtype=torch.int32, device="cuda")
        out_a = lm.verify(*args)
        lm.accept_scan(layout, st_a, out_a[2], ring_a, eos=eos, log=log_a, ctx_cap=64)
        # one launch
        st_b, ring_b, log_b = layout.to_device(base), torch.zeros(16, dtype=torch.int64, device="cuda"), torch.zeros(4, dtype=torch.int32, device="cuda")
        out_b = lm.verify(*args, commit=dict(layout=layout, state=st_b, ring=ring_b, eos=eos, log=log_b, ctx_cap=64))
        assert all(torch.equal(x, y) for x, y in zip(out_a, out_b))
        assert torch.equal(st_a, st_b) and torch.equal(ring_a, ring_b) and torch.equal(log_a, log_b)
        got = layout.from_device(st_b)
        assert got["accepted"] == int(out_b[0]) and got["step"] == 12 and got["ring_head"] > 6
        if trial == 2:
            assert got["done"] == 1 and got["ring_head"] == 6 + 2           # drafts 0 and 1 (the stop token), nothing after it
    # a state that is not this round's
    st = layout.to_device({"t_this_step": 4, "verify_len": 3, "pending_tokens": [1, 2, 3, 4]})
    ring = torch.zeros(16, dtype=torch.int64, device="cuda")
    lm.verify(*args, commit=dict(layout=layout, state=st, ring=ring))
    got = layout.from_device(st)
    assert got["error"] == 4 and got["done"] == 1 and int(ring.abs().sum()) == 0
    st = layout.to_device({"done": 1, "t_this_step": n + 1, "verify_len": n})
    before = st.clone()
    lm.verify(*args, commit=dict(layout=layout, state=st, ring=ring))
    assert torch.equal(st, before)
    # a prefill chunk: the scan's prefill branch, no token read
    pre = {"prefill_left": 5, "t_this_step": 4, "position": 8, "step": 2}
    st_a, st_b = layout.to_device(pre), layout.to_device(pre)
    lm.accept_scan(layout, st_a, out_a[2], ring)
    lm.verify(*args, commit=dict(layout=layout, state=st_b, ring=ring))
    assert torch.equal(st_a, st_b)


def test_row_maxima_from_the_sampler_spare_an_exchange_and_change_nothing():
    """The reference's verify kernels take each row's maximum from the sampler (KEPT_STATS, sample.metal:273-303). Given them, the
    launch skips its first exchange; accept length, final token and p(draft) must be the ones it finds by itself."""
    target, drafts, q, ua, uf = inputs.config2(vocab=151936, seed=5)
    x = torch.from_numpy(target.view(np.int16)).cuda().view(torch.bfloat16)
    vmax = x.float().amax(dim=1)
    for d, u in ((drafts, ua), (drafts, np.zeros(7, np.float32)), (drafts, np.full(7, 0.999, np.float32))):
        args = (x, torch.from_numpy(d).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(u).cuda(), torch.tensor([uf]), "stochastic")
        a = lm.verify(*args, return_p_draft=True)
        b = lm.verify(*args, return_p_draft=True, target_vmax=vmax)
        assert [t.cpu().tolist() for t in a] == [t.cpu().tolist() for t in b]
    z = oracle.bf16_to_f32(target)
    acc, fin, _ = oracle.verify_stochastic(z, drafts, q, ua, uf)
    out = lm.verify(x, torch.from_numpy(drafts).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(ua).cuda(), torch.tensor([uf]), "stochastic", target_vmax=vmax)
    assert (int(out[0]), int(out[1])) == (acc, fin)
