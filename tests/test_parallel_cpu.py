"""Multi-GPU host logic on CPU ranks (gloo, world size 2): the vocab-parallel record exchange, the row-sharded split with
global row offsets, and a rank that never joins. The kernels are replaced by the CPU oracle; no GPU is involved."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import oracle
from lithos_metal_b200 import parallel

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(case, world, tmp_path, timeout=240):
    port = str(free_port())
    outs = [str(tmp_path / f"{case}_{r}.npz") for r in range(world)]
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "gloo_worker.py"), case, str(r), str(world), port, outs[r]],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    logs = []
    for p in procs:
        try:
            logs.append(p.communicate(timeout=timeout)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            logs.append("timeout")
    assert all(p.returncode == 0 for p in procs), logs
    return [np.load(o) for o in outs]


def test_shard_arithmetic():
    for total, world in ((4096, 8), (11, 2), (3, 4), (262144, 8)):
        blocks = [parallel.shard_rows(total, r, world) for r in range(world)]
        assert blocks[0][0] == 0 and sum(c for _, c in blocks) == total
        assert all(blocks[i][0] + blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
        assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1
    with pytest.raises(ValueError):
        parallel.shard_rows(8, 2, 2)


def test_vocab_parallel_exchange_equals_one_device(tmp_path):
    res = run_ranks("vocab", 2, tmp_path)
    rng = np.random.default_rng(17)
    rows, vocab = 6, 4096
    z = oracle.bf16_to_f32(oracle.f32_to_bf16((rng.standard_normal((rows, vocab)) * 2).astype(np.float32)))
    z[1, :300] = 9.5
    u = rng.random(rows).astype(np.float32)
    for draw in ("inverse_cdf", "gumbel"):
        tok, tau, _ = oracle.sample_batch(z, temperature=0.8, top_k=50, top_p=0.9, draw=draw, uniforms=u, seed=5, step=3, row_offset=10)
        for r in res:                                              # every rank holds the single-device result
            if draw == "inverse_cdf":
                keep = r[draw + "_status"] == 0
                assert keep.sum() == rows - 1 and not keep[1]      # the 300-way tie overflows a record and is reported, not hidden
                np.testing.assert_array_equal(r[draw + "_tokens"][keep], tok[keep])
                np.testing.assert_array_equal(r[draw + "_tau"][keep], tau[keep])
                assert r[draw + "_tokens"][1] == -1
            else:
                keep = r[draw + "_status"] == 0
                np.testing.assert_array_equal(r[draw + "_tokens"][keep], tok[keep])
        np.testing.assert_array_equal(res[0][draw + "_tokens"], res[1][draw + "_tokens"])


def test_row_sharded_split_equals_the_whole_batch(tmp_path):
    res = run_ranks("rows", 2, tmp_path)
    rng = np.random.default_rng(17)
    total, vocab = 11, 2048
    z = oracle.f32_to_bf16((rng.standard_normal((total, vocab)) * 2).astype(np.float32))
    T = rng.uniform(0.5, 1.2, total).astype(np.float32)
    tok, _, _ = oracle.sample_batch(z, temperature=T, top_k=20, top_p=0.9, draw="gumbel", seed=9, step=2)
    for r in res:
        np.testing.assert_array_equal(r["tokens"], tok)
    assert (int(res[0]["first"]), int(res[0]["count"]), int(res[1]["first"]), int(res[1]["count"])) == (0, 6, 6, 5)


def test_a_rank_that_never_joins_ends_the_collective_with_an_error(tmp_path):
    res = run_ranks("absent", 2, tmp_path)
    assert int(res[0]["joined"]) == 1 and int(res[0]["error"]) == 1 and int(res[1]["joined"]) == 0
