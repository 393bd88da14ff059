"""The vocabulary projection on the GPU (lm_head) against the CPU restatement and the reference's own outputs, and the decode tail it
starts: projection, then the sampler on its logits. Floating point: a logit may differ from the oracle's by one BF16 unit in the last
place (the FP32 sums are formed in another order); the sampler's result on the kernel's logits is exact again."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from oracle import head
import lithos_metal_b200 as lm
from tests.golden.make_golden import lm_head_inputs

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def bf16(codes):
    return torch.from_numpy(np.ascontiguousarray(codes).view(np.int16)).cuda().view(torch.bfloat16)


def codes_of(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def close_enough(got, want):
    return head.close(got, want)


def test_reference_outputs():
    with open(os.path.join(HERE, "golden", "reference_outputs.json")) as f:
        g = json.load(f)["lm_head"]
    x, w, gamma = lm_head_inputs(g["seed"], g["rows"], g["hidden"], g["vocab"])
    want = lambda key: np.frombuffer(bytes.fromhex(g[key]), dtype=np.uint16).reshape(g["rows"], g["vocab"])
    assert close_enough(codes_of(lm.lm_head(bf16(x), bf16(w))), want("plain"))
    assert close_enough(codes_of(lm.lm_head(bf16(x), bf16(w), bf16(gamma), eps=g["eps"], one_plus=True)), want("norm_one_plus"))
    assert close_enough(codes_of(lm.lm_head(bf16(x), bf16(w), bf16(gamma), eps=g["eps"], one_plus=False)), want("norm_plain_weight"))


@pytest.mark.parametrize("rows,hidden,vocab", [(1, 1024, 32768), (8, 2048, 20011), (3, 4096, 4099), (8, 64, 17)])
def test_shapes_against_the_oracle(rows, hidden, vocab):
    rng = np.random.default_rng(rows * 1000 + vocab)
    x = oracle.f32_to_bf16((rng.standard_normal((rows, hidden)) * 1.2).astype(np.float32))
    w = oracle.f32_to_bf16((rng.standard_normal((vocab, hidden)) * 0.05).astype(np.float32))
    gamma = oracle.f32_to_bf16((rng.standard_normal(hidden) * 0.1).astype(np.float32))
    assert close_enough(codes_of(lm.lm_head(bf16(x), bf16(w))), head.lm_head(x, w))
    assert close_enough(codes_of(lm.lm_head(bf16(x), bf16(w), bf16(gamma), eps=1e-5)), head.lm_head(x, w, gamma, 1e-5))
    # rows of a larger tensor (strides) and an output given by the caller
    wide = torch.zeros(rows, hidden + 64, dtype=torch.bfloat16, device="cuda")
    wide[:, :hidden] = bf16(x)
    out = torch.full((rows, vocab), 7.0, dtype=torch.bfloat16, device="cuda")
    got = lm.lm_head(wide[:, :hidden], bf16(w), out=out)
    assert got.data_ptr() == out.data_ptr() and close_enough(codes_of(out), head.lm_head(x, w))


def test_the_decode_tail_projection_then_sampler():
    """One speculative round's tail on 8 rows: logits from the projection, then thresholds, draw and the verification on them. What
    follows the projection is exact: the same tokens as the CPU oracle gives on the kernel's own logits."""
    rng = np.random.default_rng(5)
    rows, hidden, vocab = 8, 1024, 151936
    x = oracle.f32_to_bf16((rng.standard_normal((rows, hidden))).astype(np.float32))
    w = oracle.f32_to_bf16((rng.standard_normal((vocab, hidden)) * 0.08).astype(np.float32))
    logits = lm.lm_head(bf16(x), bf16(w))
    u = rng.random(rows).astype(np.float32)
    p = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.95, draw="inverse_cdf")
    r = lm.sample(logits, p, uniforms=torch.from_numpy(u).cuda(), return_tau=True, return_status=True)
    host = codes_of(logits)
    tok, tau, _ = oracle.sample_batch(host, temperature=0.8, top_k=50, top_p=0.95, draw="inverse_cdf", uniforms=u, n_threads=8)
    assert r.tokens.cpu().tolist() == tok.tolist() and r.tau.cpu().numpy().tobytes() == tau.tobytes()
    assert close_enough(host, head.lm_head(x, w))
    assert int(lm.argmax(logits[:1])[0]) == int(oracle.bf16_to_f32(host[0]).argmax())


def test_a_vocabulary_shard_of_the_weight_gives_the_bits_of_the_whole():
    """Tensor-parallel heads: every GPU projects onto its own rows of the weight; the logits must not depend on the split."""
    rng = np.random.default_rng(9)
    x = bf16(oracle.f32_to_bf16(rng.standard_normal((8, 512)).astype(np.float32)))
    w = bf16(oracle.f32_to_bf16((rng.standard_normal((40000, 512)) * 0.07).astype(np.float32)))
    whole = lm.lm_head(x, w)
    for shards in (2, 3, 8):
        parts = []
        for s in range(shards):
            lo, width = lm.parallel.shard_vocab(40000, s, shards)
            parts.append(lm.lm_head(x, w[lo:lo + width]))
        assert torch.equal(torch.cat(parts, dim=1).view(torch.int16), whole.view(torch.int16))


def test_argument_checks():
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(100, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        lm.lm_head(torch.zeros(9, 64, dtype=torch.bfloat16, device="cuda"), w)
    with pytest.raises(ValueError):
        lm.lm_head(x.float(), w)
    with pytest.raises(ValueError):
        lm.lm_head(x, torch.zeros(100, 32, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(lm._lib.LithosError):
        lm.lm_head(torch.zeros(2, 48, dtype=torch.bfloat16, device="cuda"), torch.zeros(100, 48, dtype=torch.bfloat16, device="cuda"))   # hidden not a multiple of 64
    assert lm.lm_head(x, w).abs().max().item() == 0.0
