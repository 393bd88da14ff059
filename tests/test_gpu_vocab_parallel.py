"""Vocab-parallel sampling on the GPU: the local and merge kernels with the shards of 2, 4 and 8 ranks emulated on one
device (every shard's records computed one after the other, concatenated as the all-gather would leave them). The
result must equal the single-GPU sampler's on the whole rows, bit for bit, and the CPU model's."""
import numpy as np
import pytest
import torch

import oracle
from oracle import vocab_parallel as vp
import lithos_metal_b200 as lm
from lithos_metal_b200 import parallel
from tests.test_gpu_sampling import bf16_tensor

pytestmark = pytest.mark.gpu


def run_sharded(x, shards, p, uniforms, step=0, row_offset=0):
    backend = parallel.CudaVocabBackend()
    vocab = x.shape[1]
    k = int(p.top_k.max()) if isinstance(p.top_k, torch.Tensor) else int(p.top_k)
    cap = backend.candidate_cap(k)
    recs = []
    for s in range(shards):
        lo, width = parallel.shard_vocab(vocab, s, shards)
        recs.append(backend.local(x[:, lo:lo + width], lo, p, cap, shards))     # [pieces * rows, record bytes]
    gathered = torch.stack(recs).view(-1, x.shape[0], recs[0].shape[1])        # [shards * pieces, rows, record bytes]
    return backend.merge(gathered, p, cap, uniforms, step, row_offset), gathered, cap


@pytest.mark.parametrize("shards", [2, 4, 8])
@pytest.mark.parametrize("draw", ["inverse_cdf", "gumbel"])
def test_config5_equals_the_single_gpu_result(shards, draw):
    """Benchmark configuration 5: 64 rows x 262144 BF16 logits N(0, 2^2), top_k 50, top_p 0.9, temperature 0.8."""
    rng = np.random.default_rng(55)
    rows, vocab = 64, 262144
    codes = oracle.f32_to_bf16(rng.standard_normal((rows, vocab), dtype=np.float32) * np.float32(2.0))
    x = bf16_tensor(codes)
    u = torch.from_numpy(rng.random(rows).astype(np.float32)).cuda()
    p = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=21, draw=draw)
    (tok, tau, status), _, _ = run_sharded(x, shards, p, u, step=4, row_offset=100)
    one = lm.sample(x, p, uniforms=u, step=4, row_offset=100, return_tau=True, return_status=True)
    assert int(status.max()) & ~4 == 0
    assert torch.equal(tau, one.tau)
    assert torch.equal(tok, one.tokens)
    if shards == 8:                                                        # and the CPU definition, on a few rows
        t_o, tau_o, _ = oracle.sample_batch(codes[:6], temperature=0.8, top_k=50, top_p=0.9, draw=draw, uniforms=u[:6].cpu().numpy(), seed=21, step=4,
                                            row_offset=100, n_threads=6)
        np.testing.assert_array_equal(tau[:6].cpu().numpy(), tau_o)
        np.testing.assert_array_equal(tok[:6].cpu().numpy(), t_o)


def test_a_large_top_k_over_eight_shards():
    """top_k 300 over 8 shards: 8 x 368 candidate slots per row, of which the merge puts only those at or above the row's own
    top-k bound in order."""
    rng = np.random.default_rng(56)
    rows, vocab = 16, 151936
    codes = oracle.f32_to_bf16(rng.standard_normal((rows, vocab), dtype=np.float32) * np.float32(2.0))
    x = bf16_tensor(codes)
    u = torch.from_numpy(rng.random(rows).astype(np.float32)).cuda()
    for kw in (dict(top_k=300, top_p=0.9), dict(top_k=128)):
        p = lm.SamplingParams(temperature=0.8, seed=5, draw="inverse_cdf", **kw)
        (tok, tau, status), _, _ = run_sharded(x, 8, p, u, step=2)
        one = lm.sample(x, p, uniforms=u, step=2, return_tau=True)
        assert int(status.max()) & 32 == 0
        assert torch.equal(tau, one.tau)
        assert torch.equal(tok, one.tokens)


def test_a_masked_vocabulary_over_four_shards():
    """-inf logits: a shard with fewer than top_k logits above -inf hands over those and one -inf logit; the result is the oracle's."""
    rng = np.random.default_rng(57)
    rows, vocab = 3, 65536
    z = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
    keep = np.zeros(vocab, bool); keep[20000:20030] = True
    z[0, ~keep] = -np.inf                                                  # 30 logits left, all in one shard
    z[1, rng.random(vocab) < 0.95] = -np.inf
    z[2, :40000] = -np.inf                                                 # two shards masked out, a third partly
    x = torch.from_numpy(z).cuda()
    u = rng.random(rows).astype(np.float32)
    for kw in (dict(top_k=50, top_p=0.9), dict(top_k=20)):
        p = lm.SamplingParams(temperature=0.8, seed=5, draw="inverse_cdf", **kw)
        (tok, tau, status), gathered, cap = run_sharded(x, 4, p, torch.from_numpy(u).cuda())
        t_o, tau_o, _ = oracle.sample_batch(z, temperature=0.8, top_k=kw["top_k"], top_p=kw.get("top_p", 0.0), draw="inverse_cdf", uniforms=u, seed=5, n_threads=3)
        assert int(status.max()) & 32 == 0
        np.testing.assert_array_equal(tau.cpu().numpy(), tau_o)
        np.testing.assert_array_equal(tok.cpu().numpy(), t_o)
    # the records of unsplit shards (a small vocabulary) are the CPU model's
    small = z[:, 18000:22096].copy()
    p = lm.SamplingParams(temperature=0.8, seed=5, draw="inverse_cdf", top_k=50)
    _, gathered, cap = run_sharded(torch.from_numpy(small).cuda(), 4, p, torch.from_numpy(u).cuda())
    g = gathered.cpu().numpy()
    assert g.shape[0] == 4
    for s in range(4):
        lo, width = parallel.shard_vocab(small.shape[1], s, 4)
        a = vp.unpack_record(g[s, 0].tobytes(), cap)
        b = vp.unpack_record(vp.local_record(small[0, lo:lo + width], lo, temperature=0.8, top_k=50, cap=cap), cap)
        assert a[2] == b[2] and sorted(a[5].tolist()) == sorted(b[5].tolist())


def test_records_ties_and_knob_variants():
    rng = np.random.default_rng(3)
    rows, vocab, shards = 9, 8192, 4
    z = (rng.standard_normal((rows, vocab)) * 2).astype(np.float32)
    z[0, 100:140] = 7.5                                                    # 40 tied maxima inside one shard: all of them candidates
    z[1, ::1024] = 8.0                                                     # tied maxima spread over every shard
    z[2, :200] = 9.0                                                       # more ties than a record holds: reported
    x = torch.from_numpy(z).cuda()                                         # FP32 shards
    u = torch.from_numpy(rng.random(rows).astype(np.float32)).cuda()
    for kw in (dict(top_k=20, top_p=0.0), dict(top_k=50, top_p=0.95, min_p=0.01), dict(top_k=30, top_p=0.7, topp_in_topk=True), dict(top_k=1)):
        p = lm.SamplingParams(temperature=0.9, draw="inverse_cdf", **kw)
        (tok, tau, status), gathered, cap = run_sharded(x, shards, p, u)
        status = status.cpu().numpy()
        assert status[2] & 32 and int(tok[2]) == -1 and not np.any(np.delete(status, 2) & 32)
        one = lm.sample(x, p, uniforms=u, return_tau=True)
        keep = np.arange(rows) != 2
        np.testing.assert_array_equal(tau.cpu().numpy()[keep], one.tau.cpu().numpy()[keep])
        np.testing.assert_array_equal(tok.cpu().numpy()[keep], one.tokens.cpu().numpy()[keep])
        # the records against the CPU model: same maximum, same candidate set, same mass
        g = gathered.cpu().numpy()
        for s in range(shards):
            lo, width = parallel.shard_vocab(vocab, s, shards)
            for r in (0, 1, 5):
                a = vp.unpack_record(g[s, r].tobytes(), cap)
                b = vp.unpack_record(vp.local_record(z[r, lo:lo + width], lo, temperature=0.9, top_k=kw["top_k"], cap=cap), cap)
                assert a[0] == b[0] and a[2] == b[2] and sorted(a[5].tolist()) == sorted(b[5].tolist())
                assert abs(a[1] - b[1]) <= 1e-12 * b[1]
                tok_m, tau_m, _ = vp.merge_records([g[t, r].tobytes() for t in range(shards)], cap, temperature=0.9, top_k=kw["top_k"],
                                                   top_p=kw.get("top_p", 0.0), min_p=kw.get("min_p", 0.0), topp_in_topk=kw.get("topp_in_topk", False),
                                                   u=float(u[r]))
                assert tok_m == int(tok[r]) and np.float32(tau_m) == np.float32(float(tau[r]))


def test_invalid_vocab_parallel_requests():
    with pytest.raises(ValueError):
        parallel.VocabParallelSampler(lm.SamplingParams(temperature=0.8, top_k=0, top_p=0.9), 1024, rank=0, world=2)
    with pytest.raises(ValueError):
        parallel.VocabParallelSampler(lm.SamplingParams(temperature=0.8, top_k=1000), 1024, rank=0, world=8)     # 8 x 1064 candidates
    with pytest.raises(ValueError):
        parallel.VocabParallelSampler(lm.SamplingParams(temperature=0.8, top_k=5, repetition_penalty=1.2), 1024, rank=0, world=2)
    s = parallel.VocabParallelSampler(lm.SamplingParams(temperature=0.8, top_k=5, draw="inverse_cdf"), 1024, rank=0, world=1)
    x = torch.randn(3, 1024, device="cuda")
    u = torch.rand(3)
    assert torch.equal(s.sample(x, uniforms=u).tokens, lm.sample(x, s.params, uniforms=u).tokens)      # one shard: the plain sampler


def test_the_sampler_object_with_pieces_and_small_records():
    """VocabParallelSampler on one rank (its records all-gathered with nobody): the shard is cut into pieces, whose records hold twice
    the top_k instead of top_k + 64; the result is the plain sampler's."""
    rng = np.random.default_rng(58)
    x = bf16_tensor(oracle.f32_to_bf16((rng.standard_normal((12, 151936)) * 2).astype(np.float32)))
    u = torch.from_numpy(rng.random(12).astype(np.float32)).cuda()
    for k in (8, 20, 50, 64):
        p = lm.SamplingParams(temperature=0.8, top_k=k, top_p=0.9, draw="inverse_cdf")
        s = parallel.VocabParallelSampler(p, 151936, rank=0, world=1)
        assert s.cap == max(16, (2 * k + 7) // 8 * 8) and s.backend.pieces(1, s.cap, 151936, 12) == 64
        r = s.sample(x, uniforms=u)
        one = lm.sample(x, lm.SamplingParams(exact_only=True, temperature=0.8, top_k=k, top_p=0.9, draw="inverse_cdf"), uniforms=u, return_tau=True)
        assert torch.equal(r.tokens, one.tokens) and torch.equal(r.tau, one.tau) and int(r.status.max()) & 32 == 0
        kept = parallel.VocabParallelSampler(p, 151936, rank=0, world=1, reuse_buffers=True)       # the same with its buffers kept between calls
        for _ in range(2):
            r2 = kept.sample(x, uniforms=u)
            assert torch.equal(r2.tokens, one.tokens) and torch.equal(r2.tau, one.tau)


def test_random_configurations_equal_the_exact_kernel():
    """Seeded random calls (shards, vocabulary, dtype, knobs, draw, -inf masks): local step (in pieces or not) + merge against the
    single-GPU generic kernel on the whole rows, bit for bit."""
    rng = np.random.default_rng(77)
    for trial in range(30):
        shards = int(rng.choice([2, 3, 4, 8]))
        rows = int(rng.integers(1, 40))
        vocab = int(rng.choice([32768, 50257, 151936, 262144]))
        z = (rng.standard_normal((rows, vocab)) * float(rng.uniform(0.5, 3.0))).astype(np.float32)
        if rng.random() < 0.3:
            z[rng.random((rows, vocab)) < 0.9] = -np.inf
            z[np.arange(rows), rng.integers(0, vocab, rows)] = 1.0
        if vocab % 8 == 0 and rng.random() < 0.6:
            x = bf16_tensor(oracle.f32_to_bf16(z))
        else:
            x = torch.from_numpy(z).cuda()
        kw = dict(temperature=float(rng.uniform(0.3, 1.5)), top_k=int(rng.choice([1, 8, 20, 50, 64, 100, 300])), top_p=float(rng.choice([0.0, 0.7, 0.95])),
                  min_p=float(rng.choice([0.0, 0.02])), draw=str(rng.choice(["inverse_cdf", "gumbel"])), seed=int(rng.integers(0, 1 << 30)),
                  topp_in_topk=bool(rng.random() < 0.2))
        u = torch.from_numpy(rng.random(rows).astype(np.float32)).cuda()
        step, off = int(rng.integers(0, 50)), int(rng.integers(0, 500))
        (tok, tau, status), gathered, _ = run_sharded(x, shards, lm.SamplingParams(**kw), u, step=step, row_offset=off)
        exact = lm.sample(x, lm.SamplingParams(exact_only=True, **kw), uniforms=u, step=step, row_offset=off, return_tau=True, return_status=True)
        st = status.cpu().numpy()
        assert not np.any(st & (32 | 2)), (trial, st)
        tie = ((st | exact.status.cpu().numpy()) & 4) != 0
        edge = ((st | exact.status.cpu().numpy()) & 8) != 0                   # a top-p boundary within 1e-12: may fall on the other side (flagged)
        same_tau = tau.cpu().numpy().view(np.uint32) == exact.tau.cpu().numpy().view(np.uint32)
        assert np.all(same_tau | edge), (trial, kw, shards, rows, vocab)
        assert np.all((tok.cpu().numpy() == exact.tokens.cpu().numpy()) | tie | edge), (trial, kw, shards, rows, vocab)
