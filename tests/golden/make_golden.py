"""Generates the golden fixtures in this folder by RUNNING THE REFERENCE's own Python code.

Run once, in a container where the reference checkout is available, with its path as the only argument:

    python tests/golden/make_golden.py /path/to/lithos-metal
    python tests/golden/make_golden.py /path/to/lithos-metal --only draft_q      (adds that section, or `confidence` / `penalised` / `lm_head`, to the existing file)

It imports ``monolith.nn.sampling_ref`` / ``monolith.nn.sampler`` / ``monolith.kernels`` / ``monolith.core`` read-only
(numpy and torch are their only dependencies), extracts the ``model_accept`` function from
``tests/kernels/test_draft_ops.py`` by source (the module itself needs the Metal runtime to import), feeds them the
seeded inputs of the reference's own tests plus the benchmark's small configurations, and stores the OUTPUTS
(inputs are regenerated from the recorded seeds by the tests). Nothing here runs at test time.
"""
from __future__ import annotations

import ast
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

OPTION_SETS = {   # tests/kernels/test_sampling.py:52-55
    "plain": dict(temperature=1.0),
    "topk": dict(temperature=0.7, top_k=40),
    "topp": dict(temperature=1.0, top_p=0.9),
    "minp": dict(temperature=1.3, min_p=0.05),
    "all": dict(temperature=0.8, top_k=50, top_p=0.95, min_p=0.02),
    "topp-in-topk": dict(temperature=0.8, top_k=50, top_p=0.9, topp_in_topk=True),
}


def draft_q_section(ref, f32_to_bf16, bf16_to_f32) -> dict:
    """The drafter's draws (kernels/common/sample.metal:212-269): draft position k of a round draws from its own logits row,
    unfiltered, on noise stream 2000 + k; the reference's CPU statement of that draw is ``sampling_ref.sample`` with
    ``t = 2000 + k``. q_lse is stored as the float64 log-sum-exp of z / T (the Metal kernel accumulates it in FP32)."""
    out = {}
    for vocab in (1000, 151936):
        for temperature in (0.3, 1.0):
            rng = np.random.default_rng(7000 + vocab)
            lb = f32_to_bf16((rng.standard_normal((7, vocab)) * 2.0).astype(np.float32))
            lf = bf16_to_f32(lb)
            toks = [int(ref.sample(lf[k], seed=12345, step=3, t=2000 + k, temperature=temperature)) for k in range(7)]
            lse = [float(np.log(np.sum(np.exp(lf[k].astype(np.float64) / temperature)))) for k in range(7)]
            out[f"{vocab}/{temperature}"] = {"tokens": toks, "lse": lse, "logits_crc": int(lb.astype(np.uint64).sum())}
            print("draft_q", vocab, temperature, toks, flush=True)
    return out


def confidence_section(f32_to_bf16, bf16_to_f32) -> dict:
    """The expected values of the reference's confidence-head test (tests/kernels/test_draft_ops.py:228-263), formed by its own
    float64 statement with the reference's BF16 conversions: inputs from default_rng(4), gamma 7, hidden 256, rank 64; the three
    cases of the test (Markov part on, off, per-position STS temperatures). The test's bar for the kernel is 2e-3."""
    rbf = lambda x: bf16_to_f32(f32_to_bf16(np.asarray(x, dtype=np.float32)))
    rng = np.random.default_rng(4)
    gamma, hid, rank = 7, 256, 64
    hidden = f32_to_bf16(rng.standard_normal((gamma, hid)).astype(np.float32))
    emb = f32_to_bf16(rng.standard_normal((gamma, rank)).astype(np.float32))
    w = rbf(rng.standard_normal(hid + rank) * 0.05)
    b = rbf(rng.standard_normal(1) * 0.5)
    feats = np.concatenate([bf16_to_f32(hidden), bf16_to_f32(emb)], axis=1).astype(np.float64)
    z = rbf(rbf(feats @ w.astype(np.float64)) + b[0])
    with_emb = 1.0 / (1.0 + np.exp(-z.astype(np.float64)))
    z2 = rbf(rbf(bf16_to_f32(hidden).astype(np.float64) @ w[:hid].astype(np.float64)) + b[0])
    sts = [0.5, 1.0, 2.0, 1.5, 0.8, 1.2, 3.0]
    return {"with_emb": with_emb.tolist(), "hidden_only": (1.0 / (1.0 + np.exp(-z2.astype(np.float64)))).tolist(),
            "sts": sts, "hidden_only_sts": (1.0 / (1.0 + np.exp(-z2.astype(np.float64) / np.array(sts)))).tolist(),
            "inputs_crc": int(hidden.astype(np.uint64).sum() + emb.astype(np.uint64).sum())}


def penalised_section(ref, f32_to_bf16, bf16_to_f32) -> dict:
    """Thresholds and Gumbel draws of the reference's own ``sampling_ref`` on PENALISED rows of the batched benchmark
    configuration: 16 rows of 151936 BF16 logits N(0, 2^2), per-row temperature / top_k / top_p, a 2048-id history per row. The
    reference has no penalties; they are applied here in binary32 the way this repository defines them (for every distinct
    history id: z = z / rho if z > 0 else z * rho, then z = z - pi), and the reference then sees arbitrary FP32 rows
    (``thresholds`` walks ~3800 distinct values per row: about half a second each)."""
    rows, vocab, hist_len, rho, pi = 16, 151936, 2048, np.float32(1.1), np.float32(0.5)
    rng = np.random.default_rng(3)                                          # the recipe of tests/inputs.config3(rows=16)
    lb = f32_to_bf16((rng.standard_normal((rows, vocab), dtype=np.float32) * np.float32(2.0)))
    temperature = rng.uniform(0.3, 1.5, rows).astype(np.float32)
    top_k = rng.choice(np.array([0, 20, 50, 1000], dtype=np.int32), rows)
    top_p = rng.uniform(0.8, 1.0, rows).astype(np.float32)
    history = rng.integers(0, vocab, (rows, hist_len)).astype(np.int32)
    taus, toks = [], []
    for r in range(rows):
        z = bf16_to_f32(lb[r]).astype(np.float32).copy()
        ids = np.unique(history[r])
        v = z[ids]
        z[ids] = (np.where(v > 0, v / rho, v * rho).astype(np.float32) - pi).astype(np.float32)
        opts = dict(temperature=float(temperature[r]), top_k=int(top_k[r]), top_p=float(top_p[r]))
        taus.append(float(ref.thresholds(z, **opts)))
        toks.append(int(ref.sample(z, seed=12345, step=1, t=r, **opts)))
        print("penalised", r, opts, taus[-1], toks[-1], flush=True)
    return {"rows": rows, "tau": taus, "tokens_seed12345_step1": toks, "logits_crc": int(lb.astype(np.uint64).sum()),
            "history_crc": int(history.astype(np.uint64).sum())}


def lm_head_inputs(seed: int = 77, rows: int = 5, hidden: int = 256, vocab: int = 600):
    """The seeded inputs of the lm_head section, as BF16 codes (uint16): hidden states, weight [vocab, hidden], norm weight."""
    rng = np.random.default_rng(seed)

    def codes(a):
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return (codes(rng.standard_normal((rows, hidden)) * 1.5), codes(rng.standard_normal((vocab, hidden)) * 0.06), codes(rng.standard_normal(hidden) * 0.2))


def lm_head_section() -> dict:
    """The reference's own definitions of the lm_head op (monolith/nn/oracle.py: linear, rms_norm) on seeded BF16 inputs: the logits
    as BF16 codes, hex, row-major [rows, vocab]; without the norm, with it (1 + weight), and with a plain weight."""
    import torch
    from monolith.nn import oracle as nn_oracle
    x, w, g = lm_head_inputs()

    def t(c):
        return torch.from_numpy((c.astype(np.uint32) << 16).view(np.float32).copy()).to(torch.bfloat16)

    def hexed(y):
        return y.view(torch.int16).numpy().view(np.uint16).tobytes().hex()
    xt, wt, gt = t(x), t(w), t(g)
    return {"seed": 77, "rows": 5, "hidden": 256, "vocab": 600, "eps": 1e-6,
            "plain": hexed(nn_oracle.linear(xt, wt)),
            "norm_one_plus": hexed(nn_oracle.linear(nn_oracle.rms_norm(xt, gt, 1e-6, one_plus=True), wt)),
            "norm_plain_weight": hexed(nn_oracle.linear(nn_oracle.rms_norm(xt, gt, 1e-6, one_plus=False), wt))}


def main(ref_root: str, only: str = "") -> None:
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    if only in ("draft_q", "confidence", "penalised", "lm_head"):                                  # add this section to the existing file without redoing the rest
        from monolith.formats.fp import bf16_to_f32, f32_to_bf16
        from monolith.nn import sampling_ref as ref
        path = os.path.join(HERE, "reference_outputs.json")
        with open(path) as f:
            out = json.load(f)
        if only == "draft_q":
            out["draft_q"] = draft_q_section(ref, f32_to_bf16, bf16_to_f32)
        elif only == "lm_head":
            out["lm_head"] = lm_head_section()
        elif only == "penalised":
            out["penalised"] = penalised_section(ref, f32_to_bf16, bf16_to_f32)
        else:
            out["confidence"] = confidence_section(f32_to_bf16, bf16_to_f32)
        with open(path, "w") as f:
            json.dump(out, f, indent=1, sort_keys=True)
        print("updated", path)
        return
    import torch
    from monolith import kernels
    from monolith.core import StepStateLayout
    from monolith.formats.fp import bf16_to_f32, f32_to_bf16
    from monolith.nn import sampling_ref as ref
    from monolith.nn.sampler import GreedySampler, StochasticSampler

    out = {}

    # ---- tests/kernels/test_sampling.py:51-67: draws and thresholds, BF16 logits N(0, 4^2), seed 12345, steps 0/1/7
    draws = {}
    for vocab in (1000, 248320):
        for name, opts in OPTION_SETS.items():
            rng = np.random.default_rng(vocab + len(opts))
            lb = f32_to_bf16((rng.standard_normal((3, vocab)) * 4.0).astype(np.float32))
            lf = bf16_to_f32(lb)
            taus = [ref.thresholds(lf[i], **opts) for i in range(3)]
            toks = {str(step): [ref.sample(lf[i], seed=12345, step=step, t=i, **opts) for i in range(3)] for step in (0, 1, 7)}
            draws[f"{vocab}/{name}"] = {"tau": [float(t) for t in taus], "tokens": toks, "logits_crc": int(lb.astype(np.uint64).sum())}
            print("draws", vocab, name, taus, toks, flush=True)
    out["draws"] = draws

    # ---- kept-token probability vectors (sampling_ref.warped_probabilities) for V = 1000, stored sparsely
    probs = {}
    for name, opts in OPTION_SETS.items():
        if name == "topp-in-topk":
            continue                                   # warped_probabilities has no topp_in_topk argument
        rng = np.random.default_rng(1000 + len(opts))
        lf = bf16_to_f32(f32_to_bf16((rng.standard_normal((3, 1000)) * 4.0).astype(np.float32)))
        p = ref.warped_probabilities(lf[0], **opts)
        nz = np.nonzero(p)[0]
        probs[name] = {"idx": nz.tolist(), "p": [float(x) for x in p[nz]]}
    out["warped_probabilities"] = probs

    # ---- tests/contract/test_nn_lowering.py:321-323: the five-logit known answer for the two top-p orders
    lg = np.log(np.array([0.5, 0.3, 0.1, 0.06, 0.04], dtype=np.float32))
    out["known_answer_5"] = {"topp": float(ref.thresholds(lg, top_k=3, top_p=0.85)),
                             "topp_in_topk": float(ref.thresholds(lg, top_k=3, top_p=0.85, topp_in_topk=True)),
                             "logits": [float(x) for x in lg]}

    # ---- tests/kernels/test_embed_stat_argmax.py:99-111: argmax edge cases through GreedySampler.forward
    arg = {}
    for vocab in (248320, 1000, 300):
        rng = np.random.default_rng(vocab)
        logits = rng.standard_normal((4, vocab)).astype(np.float32) * 4
        logits[0, vocab - 1] = 100.0
        logits[1, 5] = logits[1, 7] = 50.0
        logits[1, 5] = logits[1, 7]
        logits[2] = -np.abs(logits[2]) - 1
        lf = bf16_to_f32(f32_to_bf16(logits))
        arg[str(vocab)] = GreedySampler().forward(torch.from_numpy(lf)).tolist()
    out["argmax"] = arg

    # ---- HF warpers as an independent kept-set oracle (tests/kernels/test_sampling.py:70-88)
    try:
        from transformers import MinPLogitsWarper, TopKLogitsWarper, TopPLogitsWarper
        rng = np.random.default_rng(3)
        lf = bf16_to_f32(f32_to_bf16((rng.standard_normal((2, 4096)) * 3.0).astype(np.float32)))
        hf = {}
        for name, opts, warper in [("topk", dict(temperature=1.0, top_k=25), TopKLogitsWarper(25)),
                                   ("topp", dict(temperature=1.0, top_p=0.8), TopPLogitsWarper(0.8)),
                                   ("minp", dict(temperature=1.0, min_p=0.1), MinPLogitsWarper(0.1)),
                                   ("topk-topp", dict(temperature=1.0, top_k=25, top_p=0.8, topp_in_topk=True),
                                    lambda ids, s: TopPLogitsWarper(0.8)(ids, TopKLogitsWarper(25)(ids, s)))]:
            kept = [np.nonzero(np.isfinite(warper(None, torch.from_numpy(lf[i:i + 1]).clone())[0].numpy()))[0].tolist() for i in range(2)]
            hf[name] = {"opts": opts, "kept": kept}
        out["hf_warpers"] = hf
    except Exception as e:                              # pragma: no cover
        print("HF warpers skipped:", e)

    # ---- benchmark configuration 1: one FP32 row, V = 151936, N(0, 2^2), 8 spikes at +12, seed 0
    rng = np.random.default_rng(0)
    V = 151936
    z = (rng.standard_normal(V) * 2.0).astype(np.float32)
    spikes = rng.choice(V, size=8, replace=False)
    z[spikes] = 12.0
    greedy = int(GreedySampler().forward(torch.from_numpy(z[None]))[0])
    opts = dict(temperature=0.7, top_k=20, top_p=0.95)
    tau = ref.thresholds(z, **opts)
    p = ref.warped_probabilities(z, **opts)
    nz = np.nonzero(p)[0]
    tok = int(StochasticSampler(0.7, 20, 0.95, seed=1).forward(torch.from_numpy(z[None]))[0])
    out["config1"] = {"spikes": sorted(int(s) for s in spikes), "greedy": greedy, "tau": float(tau), "kept_idx": nz.tolist(),
                      "kept_p": [float(x) for x in p[nz]], "gumbel_token_seed1_step0": tok}
    print("config1", out["config1"], flush=True)

    # ---- accept_scan: the reference's own Python model, taken from its test file by source
    src = open(os.path.join(ref_root, "tests/kernels/test_draft_ops.py")).read()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "model_accept")
    ns = {}
    exec(compile(ast.Module([fn], []), "model_accept", "exec"), ns)
    model_accept = ns["model_accept"]
    layout = StepStateLayout(t_max=8, gamma_max=7)
    cases = {}
    for case in ["all", "partial", "none", "eos_draft", "eos_bonus", "first_token", "overflow", "wrap", "context_full", "context_room"]:
        st = layout.unpack(layout.pack({}))
        st.update(position=40, step=5, ring_head=3, ring_tail=1, anchor=9, t_this_step=4, verify_len=3, pending_tokens=[9, 21, 22, 23, 0, 0, 0, 0])
        tokens, eos, cap, ctx_cap = [21, 22, 23, 24], -1, 16, 0
        if case == "context_full":
            ctx_cap = 44
        elif case == "context_room":
            ctx_cap = 45
        if case == "partial":
            tokens = [21, 50, 23, 24]
        elif case == "none":
            tokens = [51, 22, 23, 24]
        elif case == "eos_draft":
            tokens, eos = [21, 22, 23, 24], 22
        elif case == "eos_bonus":
            tokens, eos = [21, 50, 23, 24], 50
        elif case == "first_token":
            st.update(t_this_step=3, verify_len=0, pending_tokens=[101, 102, 103, 0, 0, 0, 0, 0], ring_head=0, ring_tail=0)
            tokens = [31, 32, 33]
        elif case == "overflow":
            st.update(ring_head=17, ring_tail=0)
        elif case == "wrap":
            st.update(ring_head=15, ring_tail=13)
        exp, writes = model_accept(st, tokens, cap, eos, ctx_cap)
        pre = dict(st, prefill_left=2, t_this_step=4)
        exp_pre, _ = model_accept(pre, tokens, cap, eos, ctx_cap)
        cases[case] = {"state": st, "tokens": tokens, "eos": eos, "ring_cap": cap, "ctx_cap": ctx_cap, "expect": exp,
                       "writes": [[int(a), int(b)] for a, b in writes], "prefill_state": pre, "prefill_expect": exp_pre}
    out["accept_scan"] = cases

    # ---- binary contracts: StepState layout and the parameter records
    out["step_state"] = {"offsets_8_7": layout.offsets, "size_8_7": layout.size}
    out["sample_params_hex"] = kernels.sample_params(vocab=151936, t_active=8, n_sg=40, top_k=20, temperature=0.7, top_p=0.95, min_p=0.0,
                                                     seed=(7 << 32) | 5, step=3, topp_in_topk=True).hex()
    out["select_params_hex"] = kernels.select_params(7, 0.5, 8, mode=1, cost=[1.0, 1.28, 1.5], log_cap=4, ctx_cap=64).hex()
    out["accept_params_hex"] = kernels.accept_params(16, 2, 64, ctx_cap=44).hex()

    out["draft_q"] = draft_q_section(ref, f32_to_bf16, bf16_to_f32)
    out["confidence"] = confidence_section(f32_to_bf16, bf16_to_f32)
    out["penalised"] = penalised_section(ref, f32_to_bf16, bf16_to_f32)
    out["lm_head"] = lm_head_section()

    with open(os.path.join(HERE, "reference_outputs.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", os.path.join(HERE, "reference_outputs.json"))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[3] if len(sys.argv) > 3 and sys.argv[2] == "--only" else "")
