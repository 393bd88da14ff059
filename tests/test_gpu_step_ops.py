"""accept_scan / verify_select / advance on the GPU against the reference's outputs (its own Python model of accept_scan run
on its ten test cases: tests/golden/reference_outputs.json), the expected values its verify_select test states
(tests/kernels/test_draft_ops.py:280-316), and the CPU models."""
import numpy as np
import pytest
import torch

import lithos_metal_b200 as lm
import oracle
from lithos_metal_b200 import step_state as ss
from oracle import spec_models

pytestmark = pytest.mark.gpu
LAYOUT = ss.StepStateLayout(t_max=8, gamma_max=7)


def run_accept(state, tokens, ring_cap=16, eos=-1, ctx_cap=0, lm=False):
    st = LAYOUT.to_device(state)
    ring = torch.zeros(ring_cap, dtype=torch.int64, device="cuda")
    log = torch.zeros(64, dtype=torch.int32, device="cuda")
    ss.accept_scan(LAYOUT, st, torch.tensor(tokens, dtype=torch.int32, device="cuda"), ring, eos=eos, log=log, ctx_cap=ctx_cap, lm=lm)
    got = LAYOUT.from_device(st)
    slots = {i: int(v) for i, v in enumerate(ring.cpu().numpy().view(np.uint64)) if v}
    return got, slots, int(log.cpu().numpy().view(np.uint32)[state["step"] % 64])


def test_accept_scan_equals_the_reference_model(golden):
    for case, g in golden["accept_scan"].items():
        got, ring, entry = run_accept(g["state"], g["tokens"], g["ring_cap"], g["eos"], g["ctx_cap"])
        assert got == g["expect"], case
        assert ring == {slot: val for slot, val in g["writes"]}, case
        if not got["error"]:
            committed = got["position"] - g["state"]["position"] - (g["state"]["t_this_step"] - 1 - g["state"]["verify_len"])
            assert entry == (committed << 16) | (g["state"]["verify_len"] << 8) | got["accepted"], case
        # a prefill chunk only advances and marks its rows for injection
        got, ring, entry = run_accept(g["prefill_state"], g["tokens"], g["ring_cap"], g["eos"], g["ctx_cap"])
        assert got == g["prefill_expect"] and not ring and entry == (4 << 16) | 0xFFFF, case
    # the facts the reference's test asserts on top of the model
    all_ = golden["accept_scan"]["all"]["expect"]
    assert all_["accepted"] == 3 and all_["position"] == 44 and all_["anchor"] == 24 and all_["n_inject"] == 4 and all_["ring_head"] == 7


def test_accept_scan_stop_sets_lm_and_done():
    g = {"position": 40, "step": 5, "ring_head": 3, "ring_tail": 1, "anchor": 9, "t_this_step": 4, "verify_len": 3,
         "pending_tokens": [9, 21, 22, 23, 0, 0, 0, 0], "drafter_ctx_len": 38}
    st = LAYOUT.unpack(LAYOUT.pack(g))
    for kw in (dict(eos=[7, 22]), dict(eos=[]), dict(lm=True), dict(eos=23, ctx_cap=43)):
        got, ring, _ = run_accept(st, [21, 22, 23, 24], **kw)
        eos = kw.get("eos", -1)
        if isinstance(eos, list):                                          # the model takes one id: a list with one hit is that id
            eos = 22 if 22 in eos else -1
        exp, writes, _ = spec_models.accept_scan(st, [21, 22, 23, 24], 16, eos, kw.get("ctx_cap", 0), kw.get("lm", False))
        assert got == exp and ring == dict(writes), kw
    done = dict(st, done=1)
    got, ring, _ = run_accept(done, [21, 22, 23, 24])
    assert got == done and not ring                                        # a finished program returns at its first instruction


def run_select(state, drafts, conf, gamma, threshold, t_max=8, **kw):
    base = LAYOUT.unpack(LAYOUT.pack(state))
    st = LAYOUT.to_device(base)
    ss.verify_select(LAYOUT, st, torch.tensor(drafts, dtype=torch.int32, device="cuda"), torch.tensor(conf, dtype=torch.float32, device="cuda"),
                     gamma=gamma, threshold=threshold, t_max=t_max, **kw)
    got = LAYOUT.from_device(st)
    exp = spec_models.verify_select(base, drafts, conf, gamma=gamma, threshold=threshold, t_max=t_max, **kw)
    assert got == exp, (kw, got, exp)
    return got


def test_verify_select_expected_values_of_the_reference_test():
    drafts, conf = [11, 12, 13, 14, 15], [0.9, 0.6, 0.4, 0.8, 0.1]
    base = {"anchor": 7, "drafter_ctx_len": 10, "n_inject": 3, "t_this_step": 1}
    s = run_select(base, drafts, conf, 5, 0.0)
    assert s["drafter_ctx_len"] == 13 and s["n_inject"] == 0 and s["gamma"] == 5 and s["verify_len"] == 5 and s["t_this_step"] == 6
    assert s["pending_tokens"] == [7, 11, 12, 13, 14, 15, 0, 0] and s["draft_tokens"][:5] == drafts and s["confidence"][:5] == pytest.approx(conf)
    s = run_select(base, drafts, conf, 5, 0.5)
    assert s["verify_len"] == 2 and s["t_this_step"] == 3 and s["pending_tokens"][:4] == [7, 11, 12, 0]
    s = run_select(base, drafts, conf, 5, 0.0, t_max=3)                    # clamped to t_max - 1
    assert s["verify_len"] == 2 and s["t_this_step"] == 3
    s = run_select(dict(base, prefill_left=2, t_this_step=8, pending_tokens=[1, 2, 3, 4, 5, 6, 7, 8]), drafts, conf, 5, 0.0)
    assert s["drafter_ctx_len"] == 13 and s["n_inject"] == 0 and s["t_this_step"] == 8 and s["pending_tokens"] == [1, 2, 3, 4, 5, 6, 7, 8]
    s = run_select(dict(base, done=1), drafts, conf, 5, 0.0)
    assert s["drafter_ctx_len"] == 10 and s["n_inject"] == 3
    cost = [1.0, 1.28, 1.535, 1.79, 2.67, 3.55, 4.4, 5.3]                  # the cost-aware rule: argmax_l (1 + sum a_i) / cost[l]
    s = run_select(base, drafts, conf, 5, 0.0, mode=1, cost=cost)
    a, best, exp_L, e = 1.0, 1.0, 0, 1.0
    for l in range(1, 6):
        a *= conf[l - 1]; e += a
        if e / cost[l] > best:
            best, exp_L = e / cost[l], l
    assert s["verify_len"] == exp_L == 2 and s["t_this_step"] == 3
    assert run_select(base, drafts, conf, 5, 9.0, mode=2)["verify_len"] == 5 and run_select(base, drafts, conf, 5, 9.0, t_max=4, mode=2)["verify_len"] == 3
    assert run_select(base, drafts, conf, 5, 3.0, mode=2)["verify_len"] == 3
    # the context capacity: position 10, so L is clamped to ctx_cap - 11
    pos = dict(base, position=10)
    assert run_select(pos, drafts, conf, 5, 0.0, ctx_cap=13)["verify_len"] == 2
    s = run_select(pos, drafts, conf, 5, 0.0, ctx_cap=11)
    assert s["verify_len"] == 0 and s["t_this_step"] == 1 and s["error"] == 0
    s = run_select(pos, drafts, conf, 5, 0.0, ctx_cap=10)                  # no room for the anchor's row: stop
    assert s["error"] == 2 and s["done"] == 1 and s["t_this_step"] == 1
    assert run_select(pos, drafts, conf, 5, 0.0, ctx_cap=64)["verify_len"] == 5
    assert run_select(pos, drafts, conf, 5, 0.0, lm=True)["drafter_ctx_len"] == 15
    with pytest.raises(ValueError):
        run_select(base, drafts, conf, 5, 0.0, mode=1, cost=[2.0, 3.0])


def test_advance_equals_the_model():
    base = LAYOUT.unpack(LAYOUT.pack({"position": 12, "step": 3, "t_this_step": 2, "ring_head": 5, "ring_tail": 4, "pending_tokens": [4, 5]}))
    for st, kw in ((base, {}), (base, dict(eos=61)), (base, dict(eos=[60, 61])), (base, dict(ctx_cap=14)), (dict(base, prefill_left=1), {}),
                   (dict(base, ring_head=20, ring_tail=4), {}), (dict(base, stop_at=6), {}), (dict(base, done=1), {})):
        dev = LAYOUT.to_device(st)
        ring = torch.zeros(16, dtype=torch.int64, device="cuda")
        ss.advance(LAYOUT, dev, torch.tensor([60, 61], dtype=torch.int32, device="cuda"), ring, **kw)
        eos = kw.get("eos", -1)
        eos = 61 if isinstance(eos, list) else eos
        exp, writes = spec_models.advance(st, [60, 61], 16, eos, kw.get("ctx_cap", 0))
        assert LAYOUT.from_device(dev) == exp, (st, kw)
        assert {i: int(v) for i, v in enumerate(ring.cpu().numpy().view(np.uint64)) if v} == dict(writes)


def test_confidence_head(golden):
    """lm_confidence: bit-exact with the CPU oracle (same FMA order, same BF16 roundings, same fixed exp2) and within the
    reference test's bar of its float64 statement; positions >= gamma untouched; feeds verify_select; silent once done."""
    from tests.test_oracle_golden import confidence_inputs
    g = golden["confidence"]
    hidden, emb, w, b = confidence_inputs()
    as_bf16 = lambda codes: torch.from_numpy(codes.view(np.int16).copy()).cuda().view(torch.bfloat16)
    th, te, tw, tb = as_bf16(hidden), as_bf16(emb), torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
    got = lm.confidence(th, te, tw, tb, gamma=6).cpu().numpy()
    np.testing.assert_array_equal(got[:6], oracle.confidence(hidden, emb, w, float(b[0]))[:6])
    assert got[6] == 0.0 and np.abs(got[:6] - np.array(g["with_emb"])[:6]).max() <= 2e-3
    got = lm.confidence(th, None, tw[:256], tb).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.confidence(hidden, None, w[:256], float(b[0])))
    assert np.abs(got - np.array(g["hidden_only"])).max() <= 2e-3
    got = lm.confidence(th, None, tw[:256], tb, sts=g["sts"]).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.confidence(hidden, None, w[:256], float(b[0]), sts=g["sts"]))
    assert np.abs(got - np.array(g["hidden_only_sts"])).max() <= 2e-3
    # odd widths (not multiples of 32) and the state's done flag
    rng = np.random.default_rng(9)
    h2 = oracle.f32_to_bf16(rng.standard_normal((3, 77)).astype(np.float32)); e2 = oracle.f32_to_bf16(rng.standard_normal((3, 5)).astype(np.float32))
    w2 = (rng.standard_normal(82) * 0.1).astype(np.float32); b2 = np.float32([0.25])
    got = lm.confidence(as_bf16(h2), as_bf16(e2), torch.from_numpy(w2).cuda(), torch.from_numpy(b2).cuda()).cpu().numpy()
    np.testing.assert_array_equal(got, oracle.confidence(h2, e2, w2, 0.25))
    layout = lm.StepStateLayout(8, 7)
    done = layout.to_device({"done": 1})
    out = torch.full((3,), -1.0, device="cuda")
    lm.confidence(as_bf16(h2), as_bf16(e2), torch.from_numpy(w2).cuda(), torch.from_numpy(b2).cuda(), out=out, layout=layout, state=done)
    assert out.cpu().tolist() == [-1.0, -1.0, -1.0]
    with pytest.raises(ValueError):
        lm.confidence(th, None, tw[:256], tb, sts=[0.0])
