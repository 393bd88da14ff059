"""The tile-consumer entry points (lm_tile_begin / lm_tile_consume / lm_tile_finish) against lm_sample on the same logits.

A vocabulary projection that produces its logits in column tiles hands them to the sampler tile by tile
(lm_head_forward writes the whole [T, V] tensor instead, monolith/nn/lm_head.py:50-60). Here the tiles are cut from a
materialised tensor, so the expected tokens are simply what lm_sample (itself checked against the oracle elsewhere in this
suite) and the oracle return for that tensor.
"""
import numpy as np
import pytest
import torch

import oracle
import lithos_metal_b200 as lm
from lithos_metal_b200 import _lib

pytestmark = pytest.mark.gpu


def _logits(rows, vocab, seed, scale=2.0):
    rng = np.random.default_rng(seed)
    codes = oracle.f32_to_bf16((rng.standard_normal((rows, vocab)) * scale).astype(np.float32))
    return torch.from_numpy(codes.view(np.int16)).cuda().view(torch.bfloat16), oracle.bf16_to_f32(codes)


def _feed(ts, x, width, order=None):
    starts = list(range(0, x.shape[1], width))
    if order is not None:
        starts = [starts[i] for i in order(len(starts))]
    for c0 in starts:
        ts.consume(x[:, c0:c0 + width], c0)


@pytest.mark.parametrize("width", [128, 256, 2048])
@pytest.mark.parametrize("draw", ["inverse_cdf", "gumbel"])
def test_tiles_give_the_tokens_of_the_materialised_tensor(width, draw):
    rows, vocab = 48, 151936
    x, _ = _logits(rows, vocab, 5)
    g = np.random.default_rng(6)
    p = lm.SamplingParams(temperature=torch.from_numpy(g.uniform(0.6, 1.2, rows).astype(np.float32)), top_k=torch.from_numpy(g.integers(1, 65, rows).astype(np.int32)),
                          top_p=torch.from_numpy(np.where(g.random(rows) < 0.5, g.uniform(0.7, 0.99, rows), 0.0).astype(np.float32)),
                          min_p=torch.from_numpy(np.where(g.random(rows) < 0.3, 0.02, 0.0).astype(np.float32)), seed=77, draw=draw)
    u = torch.from_numpy(g.random(rows).astype(np.float32)).cuda()
    want = lm.sample(x, p, uniforms=u, step=3, return_tau=True, return_status=True)
    ts = lm.TileSampler(rows, vocab, p)
    _feed(ts, x, width)
    got = ts.finish(uniforms=u, step=3, return_tau=True)
    st = got.status.cpu().numpy()
    assert not np.any(st & _lib.STATUS_TILE_DECLINED), st
    assert np.all(st & _lib.STATUS_CANDIDATE_PATH)
    assert torch.equal(got.tokens, want.tokens)
    assert torch.equal(got.tau, want.tau)
    # and the oracle itself (the same check lm_sample's own tests make)
    codes = x.view(torch.int16).cpu().numpy().view(np.uint16)
    tok, tau, _ = oracle.sample_batch(codes, temperature=p.temperature.numpy(), top_k=p.top_k.numpy(), top_p=p.top_p.numpy(), min_p=p.min_p.numpy(),
                                      draw=draw, uniforms=u.cpu().numpy(), seed=77, step=3, n_threads=8)
    assert got.tokens.cpu().tolist() == tok.tolist()
    assert got.tau.cpu().numpy().tobytes() == tau.tobytes()


def test_tile_order_and_a_second_step_do_not_matter():
    rows, vocab = 16, 65536
    x, _ = _logits(rows, vocab, 9)
    p = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=3, draw="gumbel")
    want = lm.sample(x, p, step=1)
    ts = lm.TileSampler(rows, vocab, p)
    _feed(ts, x, 256, order=lambda n: np.random.default_rng(1).permutation(n))
    assert torch.equal(ts.finish(step=1).tokens, want.tokens)
    x2, _ = _logits(rows, vocab, 10)
    ts.begin()
    _feed(ts, x2, 512, order=lambda n: list(range(n))[::-1])
    assert torch.equal(ts.finish(step=2).tokens, lm.sample(x2, p, step=2).tokens)


def test_float32_tiles_are_rounded_as_the_projection_would_store_them():
    rows, vocab = 8, 32768
    g = torch.Generator(device="cuda").manual_seed(4)
    xf = torch.randn(rows, vocab, device="cuda", generator=g) * 2
    p = lm.SamplingParams(temperature=1.0, top_k=20, seed=8)
    want = lm.sample(xf.to(torch.bfloat16), p)
    ts = lm.TileSampler(rows, vocab, p)
    _feed(ts, xf, 1024)
    assert torch.equal(ts.finish().tokens, want.tokens)


def test_large_top_k_compacts_its_list_on_the_way():
    """top_k 1024 with narrow tiles: the candidate list fills and is cut down to the running top several times."""
    rows, vocab = 6, 151936
    x, _ = _logits(rows, vocab, 21)
    p = lm.SamplingParams(temperature=1.0, top_k=1024, top_p=0.95, seed=5, draw="inverse_cdf")
    u = torch.full((rows,), 0.37, device="cuda")
    want = lm.sample(x, p, uniforms=u, return_tau=True)
    ts = lm.TileSampler(rows, vocab, p)
    _feed(ts, x, 128)
    got = ts.finish(uniforms=u, return_tau=True)
    assert not np.any(got.status.cpu().numpy() & _lib.STATUS_TILE_DECLINED)
    assert torch.equal(got.tokens, want.tokens) and torch.equal(got.tau, want.tau)


@pytest.mark.parametrize("draw", ["inverse_cdf", "gumbel"])
def test_penalised_and_greedy_rows_arrive_in_tiles_too(draw):
    rows, vocab = 24, 151936
    x, host = _logits(rows, vocab, 40)
    g = np.random.default_rng(41)
    hist = g.integers(0, vocab, (rows, 2048)).astype(np.int32)
    hist[:, :64] = np.argsort(-oracle.bf16_to_f32(host), axis=1)[:, :64]            # the penalties reach the top of every row
    t = g.uniform(0.5, 1.3, rows).astype(np.float32); t[::6] = 0.0                   # every sixth row greedy
    k = g.choice([1, 20, 50, 1000], rows).astype(np.int32)
    p = lm.SamplingParams(temperature=torch.from_numpy(t), top_k=torch.from_numpy(k), top_p=torch.from_numpy(g.uniform(0.8, 1.0, rows).astype(np.float32)),
                          repetition_penalty=1.1, presence_penalty=0.5, seed=9, draw=draw)
    u = torch.from_numpy(g.random(rows).astype(np.float32)).cuda()
    h = torch.from_numpy(hist).cuda()
    want = lm.sample(x, p, history=h, uniforms=u, step=2, return_tau=True)
    ts = lm.TileSampler(rows, vocab, p, history=h)
    for rep in range(2):                                                            # the second step reuses the state
        _feed(ts, x, 256 if rep == 0 else 1024)
        got = ts.finish(uniforms=u, step=2, return_tau=True)
        st = got.status.cpu().numpy()
        assert not np.any(st & _lib.STATUS_TILE_DECLINED), st
        assert torch.equal(got.tokens, want.tokens) and torch.equal(got.tau, want.tau)
        ts.begin(h)
    tok, tau, _ = oracle.sample_batch(x.view(torch.int16).cpu().numpy().view(np.uint16), temperature=t, top_k=k, top_p=p.top_p.numpy(), history=hist,
                                      repetition_penalty=1.1, presence_penalty=0.5, draw=draw, uniforms=u.cpu().numpy(), seed=9, step=2, n_threads=8)
    assert want.tokens.cpu().tolist() == tok.tolist()


def test_rows_the_tile_path_does_not_take_are_declined_not_guessed():
    rows, vocab = 5, 32768
    x, _ = _logits(rows, vocab, 30)
    x[1, 100] = float("nan")
    x[2] = -x[2].abs()                                          # no positive logit: the top-k boundary is not above zero
    k = torch.tensor([10, 10, 10, 0, 10], dtype=torch.int32)    # row 3: no top_k
    t = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.0])                 # row 4: greedy (taken: the running argmax)
    p = lm.SamplingParams(temperature=t, top_k=k, seed=1)
    ts = lm.TileSampler(rows, vocab, p)
    _feed(ts, x, 256)
    got = ts.finish()
    st, tok = got.status.cpu().numpy(), got.tokens.cpu().numpy()
    assert not (st[0] & _lib.STATUS_TILE_DECLINED) and tok[0] == int(lm.sample(x[:1], lm.SamplingParams(temperature=1.0, top_k=10, seed=1)).tokens[0])
    assert all(st[r] & _lib.STATUS_TILE_DECLINED and tok[r] == -1 for r in (1, 2, 3)), (st, tok)
    assert st[4] == 0 and tok[4] == int(x[4].float().argmax())


def test_tile_arguments_are_checked():
    L = _lib.lib()
    assert L.lm_tile_state_bytes(0, 4096, 0) == 0 and L.lm_tile_state_bytes(4, 4096, 0) >= 4 * 8192 * 8
    assert L.lm_tile_state_bytes(4, 4096, 1) == L.lm_tile_state_bytes(4, 4096, 0) + 4 * 4096 // 8
    p = lm.SamplingParams(temperature=1.0, top_k=5)
    ts = lm.TileSampler(2, 4096, p)
    x = torch.zeros(2, 4096, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.LithosError):
        ts.consume(x[:, :4096], 0)                              # wider than a tile may be
    with pytest.raises(_lib.LithosError):
        ts.consume(x[:, :256], 4000)                            # runs past the vocabulary
    ts.begin(torch.zeros(2, 8, dtype=torch.int32))                  # no penalties in the knobs: a history changes nothing
    bare = lm.TileSampler(2, 4096, lm.SamplingParams(temperature=1.0, top_k=5, repetition_penalty=1.2))
    with pytest.raises(ValueError):
        bare.begin(torch.zeros(2, 8, dtype=torch.int32))            # built without a history: its state has no room for the ids
