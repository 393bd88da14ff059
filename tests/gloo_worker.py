"""One CPU rank of the multi-GPU host-logic tests (gloo). Launched by tests/test_parallel_cpu.py as
``python tests/gloo_worker.py <case> <rank> <world> <port> <out.npz>``. The compute steps are the CPU oracle standing in for
the CUDA kernels (test infrastructure); what is under test is the host layer: sharding arithmetic, record exchange,
global row offsets, identical results on every rank."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle                                                    # noqa: E402
from oracle import vocab_parallel as vp                          # noqa: E402
from lithos_metal_b200 import parallel                           # noqa: E402
from lithos_metal_b200.sampler import SamplingParams             # noqa: E402


class NumpyVocabBackend:
    """The vocab-parallel backend interface on numpy (records in the CUDA library's byte layout)."""

    def candidate_cap(self, top_k):
        return vp.candidate_cap(top_k)

    def record_bytes(self, cap):
        return vp.record_bytes(cap)

    def local(self, logits, shard_start, p, cap, shards=1):
        z = logits.numpy()
        half = z.shape[1] // 2                                              # two pieces per shard, piece-major like the CUDA backend's records
        recs = [np.frombuffer(vp.local_record(z[r, lo:hi], shard_start + lo, temperature=float(p.temperature), top_k=int(p.top_k), cap=cap), np.uint8)
                for lo, hi in ((0, half), (half, z.shape[1])) for r in range(z.shape[0])]
        return torch.from_numpy(np.stack(recs).copy())

    def merge(self, gathered, p, cap, uniforms, step, row_offset):
        g = gathered.numpy()
        out = [vp.merge_records([g[s, r].tobytes() for s in range(g.shape[0])], cap, temperature=float(p.temperature), top_k=int(p.top_k),
                                top_p=float(p.top_p), min_p=float(p.min_p), topp_in_topk=p.topp_in_topk, draw=p.draw,
                                u=0.0 if uniforms is None else float(uniforms[r]), seed=p.seed, step=step, t=row_offset + r) for r in range(g.shape[1])]
        return (torch.tensor([o[0] for o in out], dtype=torch.int32), torch.tensor([o[1] for o in out], dtype=torch.float32),
                torch.tensor([o[2] for o in out], dtype=torch.int32))


def main():
    case, rank, world, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(17)
    if case == "vocab":
        rows, vocab = 6, 4096
        z = oracle.bf16_to_f32(oracle.f32_to_bf16((rng.standard_normal((rows, vocab)) * 2).astype(np.float32)))
        z[1, :300] = 9.5                                          # a plateau of 300 tied maxima in shard 0: more ties than a record holds
        u = rng.random(rows).astype(np.float32)
        res = {}
        for draw in ("inverse_cdf", "gumbel"):
            p = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=5, draw=draw)
            s = parallel.VocabParallelSampler(p, vocab, backend=NumpyVocabBackend())
            lo, width = parallel.shard_vocab(vocab, rank, world)
            r = s.sample(torch.from_numpy(z[:, lo:lo + width].copy()), uniforms=torch.from_numpy(u), step=3, row_offset=10)
            res[draw + "_tokens"], res[draw + "_tau"], res[draw + "_status"] = r.tokens.numpy(), r.tau.numpy(), r.status.numpy()
        np.savez(out, **res)
    elif case == "rows":
        total, vocab = 11, 2048                                   # 11 rows over 2 ranks: an uneven split
        z = oracle.f32_to_bf16((rng.standard_normal((total, vocab)) * 2).astype(np.float32))
        T = rng.uniform(0.5, 1.2, total).astype(np.float32)
        first, count = parallel.shard_rows(total, rank, world)
        tok, _, _ = oracle.sample_batch(z[first:first + count], temperature=T[first:first + count], top_k=20, top_p=0.9, draw="gumbel", seed=9, step=2,
                                        row_offset=first)
        mine = torch.full((total,), -9, dtype=torch.int32)
        mine[first:first + count] = torch.from_numpy(tok)
        dist.all_reduce(mine, op=dist.ReduceOp.MAX)               # test-only exchange to compare against the unsharded batch
        np.savez(out, tokens=mine.numpy(), first=first, count=count)
    elif case == "absent":
        # a rank that never joins the exchange: the others' collective ends with an error after a short timeout (no GPU involved)
        import datetime
        dist.destroy_process_group()
        os.environ["MASTER_PORT"] = str(int(port) + 1)
        if rank == 1:
            np.savez(out, joined=0)
            return
        try:
            dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
            t = torch.zeros(4)
            dist.all_reduce(t)
            np.savez(out, joined=1, error=0)
        except Exception as e:                                    # the expected path
            np.savez(out, joined=1, error=1, text=str(type(e).__name__))
        return
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
