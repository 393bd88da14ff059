"""GPU-resident control: the sampler, the draft-side draw and the verification step take their round from the device-side
StepState, as the reference's kernels do (kernels/common/sample.metal:172-181, 283-296; argmax.metal:44-46), so that one
captured CUDA graph replays round after round without a host read; the verification step's own randomness (accept stream
3000 + r, Gumbel residual on stream 4000, sample.metal:291-296, 322-346); and the bounded waits of the verification kernel."""
import numpy as np
import pytest
import torch

import lithos_metal_b200 as lm
import oracle
from lithos_metal_b200 import _lib
from tests import inputs
from tests.test_gpu_sampling import bf16_tensor

pytestmark = pytest.mark.gpu
LAYOUT = lm.StepStateLayout(8, 7)
SEED = 0x1234_5678_9ABC_DEF0


def state_for(**fields):
    base = {"rng_lo": SEED & 0xFFFFFFFF, "rng_hi": SEED >> 32}
    base.update(fields)
    return LAYOUT.to_device(base)


def test_sampler_takes_seed_step_and_rows_from_the_state():
    V = 32768
    rng = np.random.default_rng(5)
    x = bf16_tensor(oracle.f32_to_bf16((rng.standard_normal((8, V)) * 2.0).astype(np.float32)))
    p = lm.SamplingParams(temperature=0.9, top_k=40, top_p=0.95, seed=1)   # the seed argument is overridden by the state's
    st = state_for(step=5, t_this_step=3)
    out = torch.full((8,), -7, dtype=torch.int32, device="cuda")
    lm.sample(x, p, out=out, step_state=(LAYOUT, st))
    want = lm.sample(x[:3], lm.SamplingParams(temperature=0.9, top_k=40, top_p=0.95, seed=SEED), step=5).tokens
    assert out[:3].tolist() == want.tolist() and out[3:].tolist() == [-7] * 5            # rows beyond t_this_step untouched
    # rows without a top_k take the histogram kernel, FP32 rows the generic one: same rule
    for logits, q in ((x, lm.SamplingParams(temperature=1.1, top_p=0.9)), (x.float(), lm.SamplingParams(temperature=0.7, top_k=10))):
        out.fill_(-7)
        lm.sample(logits, q, out=out, step_state=(LAYOUT, st))
        q.seed = SEED
        assert out[:3].tolist() == lm.sample(logits[:3], q, step=5).tokens.tolist() and out[3:].tolist() == [-7] * 5
    # a finished generation: nothing is written
    out.fill_(-7)
    lm.sample(x, p, out=out, step_state=(LAYOUT, state_for(step=5, t_this_step=3, done=1)))
    assert out.tolist() == [-7] * 8
    # the drafter's draw reads the same two fields
    d = lm.draft_q(x[:2], temperature=0.8, step_state=(LAYOUT, st))
    e = lm.draft_q(x[:2], temperature=0.8, seed=SEED, step=5)
    assert d.tokens.tolist() == e.tokens.tolist() and d.mass.tolist() == e.mass.tolist()


@pytest.mark.parametrize("residual_draw", ["inverse_cdf", "gumbel"])
def test_verify_with_device_side_randomness_equals_the_oracle(residual_draw):
    """u_accept / u_final from the counter-based noise of (seed, step); the Gumbel form of the final draw."""
    target, drafts, q, _, _ = inputs.config2(vocab=32000, seed=21)
    z = oracle.bf16_to_f32(target)
    for step, d in ((0, drafts), (3, z[:7].argmax(-1).astype(np.int32)), (9, np.concatenate([z[:3].argmax(-1), drafts[3:]]).astype(np.int32))):
        ua = np.array([_lib.lib().lm_uniform01(SEED, step, 3000 + r, 0) for r in range(7)], dtype=np.float32)
        out = lm.verify(bf16_tensor(target), torch.from_numpy(d).cuda(), torch.from_numpy(q).cuda(), None, None, "stochastic", seed=SEED, step=step,
                        residual_draw=residual_draw)
        if residual_draw == "inverse_cdf":
            uf = np.float32(_lib.lib().lm_uniform01(SEED, step, 4000, 0))
            acc, fin, _ = oracle.verify_stochastic(target, d, q, ua, uf)
            assert (int(out[0]), int(out[1])) == (acc, fin)
        else:
            acc, fin, gap = oracle.verify_gumbel(target, d, q, seed=SEED, step=step)
            assert int(out[0]) == acc
            assert int(out[1]) == fin or gap < 4e-6                       # float32 log is library-specific: equal away from near-ties
        assert out[2].tolist() == d[:acc].tolist() + [int(out[1])] + [-1] * (7 - acc)


def run_round(x, q, drafts, conf, st, ring, log, out, threshold, residual_draw, *, host_driven):
    """One speculative round: sampler thresholds -> verification with commit -> staging of the next round."""
    if host_driven:                                                       # the host reads the state and passes the round as arguments
        s = LAYOUT.from_device(st)
        if s["done"]:
            return
        L, step = s["verify_len"], s["step"]
        seed = (s["rng_hi"] << 32) | s["rng_lo"]
        tau = lm.sample(x[:L + 1], lm.SamplingParams(temperature=0.9, top_k=50, seed=seed), step=step, return_tau=True).tau
        d = torch.tensor(s["pending_tokens"][1:L + 1], dtype=torch.int32, device="cuda")
        lm.verify(x[:L + 1], d, q[:L], None, None, "stochastic", temperature=0.9, tau=tau, seed=seed, step=step, residual_draw=residual_draw,
                  out=out[:L + 3], commit=dict(layout=LAYOUT, state=st, ring=ring, log=log))
    else:                                                                 # nothing but launches: every kernel reads the state on the device
        r = lm.sample(x, lm.SamplingParams(temperature=0.9, top_k=50), step_state=(LAYOUT, st), return_tau=True, return_vmax=True)
        # ... and hands the verification the rows' maxima and masses along with the thresholds, as the reference's sampler does
        lm.verify(x, None, q, None, None, "stochastic", temperature=0.9, tau=r.tau, target_vmax=r.vmax, target_mass=r.mass, residual_draw=residual_draw,
                  step_state=(LAYOUT, st), out=out, commit=dict(layout=LAYOUT, state=st, ring=ring, log=log))
    lm.verify_select(LAYOUT, st, drafts, conf, gamma=7, threshold=threshold)


@pytest.mark.parametrize("residual_draw,threshold", [("gumbel", 0.0), ("inverse_cdf", 0.5)])
def test_one_captured_graph_replays_the_rounds_without_a_host_read(residual_draw, threshold):
    """sample -> verify (commit) -> verify_select captured ONCE and replayed eight times equals the eager loop in which the host
    reads the state before every round; the noise moves with the state's step, so the rounds differ."""
    V, rounds = 32768, 8
    rng = np.random.default_rng(31)
    target = oracle.f32_to_bf16((rng.standard_normal((8, V)) * 2.0).astype(np.float32))
    z = oracle.bf16_to_f32(target)
    x = bf16_tensor(target)
    q = torch.softmax(x[:7].float() + 0.5 * torch.randn(7, V, device="cuda", generator=torch.Generator("cuda").manual_seed(3)), -1)
    drafts = torch.from_numpy(z[:7].argmax(-1).astype(np.int32)).cuda()      # likely-accepted drafts: rounds commit several tokens
    conf = torch.tensor([0.9, 0.8, 0.3, 0.7, 0.6, 0.2, 0.9], device="cuda")
    first = {"step": 0, "position": 10, "t_this_step": 8, "verify_len": 7, "anchor": 3, "pending_tokens": [3] + drafts.tolist(), "gamma": 7}
    results = []
    for host_driven in (True, False):
        st = state_for(**first)
        ring, log = torch.zeros(128, dtype=torch.int64, device="cuda"), torch.zeros(16, dtype=torch.int32, device="cuda")
        out = torch.full((10,), -9, dtype=torch.int32, device="cuda")
        args = (x, q, drafts, conf, st, ring, log, out, threshold, residual_draw)
        if host_driven:
            for _ in range(rounds):
                run_round(*args, host_driven=True)
        else:
            run_round(*args, host_driven=False)                            # warm-up outside the capture (first-call set-up), on a scratch state
            st.copy_(state_for(**first)); ring.zero_(); log.zero_()
            torch.cuda.synchronize()
            graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
            with torch.cuda.stream(stream):
                run_round(*args, host_driven=False)                        # the stream's own workspaces, before the capture
                st.copy_(state_for(**first)); ring.zero_(); log.zero_()
                stream.synchronize()
                with torch.cuda.graph(graph, stream=stream):
                    run_round(*args, host_driven=False)
            for _ in range(rounds):
                graph.replay()
        torch.cuda.synchronize()
        results.append((LAYOUT.from_device(st), ring.cpu().numpy().copy(), log.cpu().numpy().copy()))
    (s_host, ring_host, log_host), (s_dev, ring_dev, log_dev) = results
    assert s_dev == s_host and np.array_equal(ring_dev, ring_host) and np.array_equal(log_dev, log_host)
    assert s_dev["step"] == rounds and s_dev["ring_head"] >= rounds and not s_dev["error"]
    accepted = [int(e) & 0xFF for e in log_dev.view(np.uint32)[:rounds]]
    assert len(set(accepted)) > 1 or len(set(ring_dev[:s_dev["ring_head"]] & 0xFFFFFFFF)) > 2     # the rounds are not copies of each other


def test_a_finished_state_leaves_the_verification_outputs_untouched():
    target, drafts, q, ua, uf = inputs.config2(vocab=2000, seed=4)
    st = state_for(done=1, t_this_step=8, verify_len=7)
    before = st.clone()
    out = torch.full((10,), -9, dtype=torch.int32, device="cuda")
    ring = torch.zeros(16, dtype=torch.int64, device="cuda")
    for mode in ("greedy", "stochastic"):
        lm.verify(bf16_tensor(target), None, torch.from_numpy(q).cuda(), None, None, mode, step_state=(LAYOUT, st), out=out,
                  commit=dict(layout=LAYOUT, state=st, ring=ring))
        assert out.tolist() == [-9] * 10 and torch.equal(st, before) and int(ring.abs().sum()) == 0
    # the workspace is clean afterwards: an ordinary call gives the oracle's answer
    acc, fin, _ = oracle.verify_stochastic(target, drafts, q, ua, uf)
    got = lm.verify(bf16_tensor(target), torch.from_numpy(drafts).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(ua).cuda(), torch.tensor([uf]), "stochastic")
    assert (int(got[0]), int(got[1])) == (acc, fin)


@pytest.mark.parametrize("mode", ["greedy", "stochastic"])
def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_clean(mode):
    """The self-test switch makes block 0 withhold its partial results, so the bounded waits between the thread blocks run out
    (a few hundred polls here): the launch ends by itself, reports -1 and error 3 in the state, and leaves the workspace usable."""
    target, drafts, q, ua, uf = inputs.config2(vocab=151936, seed=6)
    x, d, qd = bf16_tensor(target), torch.from_numpy(drafts).cuda(), torch.from_numpy(q).cuda()
    extra = (qd, torch.from_numpy(ua).cuda(), torch.tensor([uf])) if mode == "stochastic" else (None, None, None)
    st = state_for(step=2, position=30, t_this_step=8, verify_len=7, anchor=1, pending_tokens=[1] + drafts.tolist())
    ring = torch.zeros(16, dtype=torch.int64, device="cuda")
    out = lm.verify(x, d, *extra, mode, commit=dict(layout=LAYOUT, state=st, ring=ring), wait_limit=300, selftest=_lib.VERIFY_SELFTEST_WITHHOLD)
    assert int(out[0]) == -1 and int(out[1]) == -1 and out[2].tolist() == [-1] * 8
    got = LAYOUT.from_device(st)
    assert got["error"] == 3 and got["done"] == 1 and int(ring.abs().sum()) == 0
    # the same workspace, an ordinary call: the oracle's answer
    out = lm.verify(x, d, *extra, mode)
    if mode == "stochastic":
        acc, fin, _ = oracle.verify_stochastic(target, drafts, q, ua, uf)
    else:
        acc, fin, _ = oracle.verify_greedy(target, drafts)
    assert (int(out[0]), int(out[1])) == (acc, fin)
