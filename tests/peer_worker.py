"""Worker of tests/test_gpu_peer_exchange.py: one process per GPU (torchrun), the vocab-parallel sampler with the records read in place
from the peers' memory, several steps in a row (the two record buffers take turns), against the single-GPU sampler on the whole rows."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import lithos_metal_b200 as lm                                               # noqa: E402
from lithos_metal_b200 import parallel                                       # noqa: E402


def main() -> None:
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    rows, vocab = 12, 151936
    p = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.9, draw="inverse_cdf")
    sampler = parallel.VocabParallelSampler(p, vocab, exchange="peer")
    lo, width = parallel.shard_vocab(vocab, rank, world)
    ok = True
    for step in range(5):
        full = (torch.randn(rows, vocab, generator=g, device=dev) * 2.0).to(torch.bfloat16)      # the same rows on every rank
        u = torch.rand(rows, generator=g, device=dev)
        r = sampler.sample(full[:, lo:lo + width].contiguous(), uniforms=u, step=step)
        one = lm.sample(full, lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.9, draw="inverse_cdf", exact_only=True), uniforms=u, step=step, return_tau=True)
        ok = ok and torch.equal(r.tokens, one.tokens) and torch.equal(r.tau, one.tau)
    in_place = any(v is not None for v in sampler._peer.values())
    flag = torch.tensor([int(ok), int(in_place)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PEER_EXCHANGE", "ok" if int(flag[0]) else "MISMATCH", "in_place" if int(flag[1]) else "all_gather_fallback", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
