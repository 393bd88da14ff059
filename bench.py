#!/usr/bin/env python
"""Benchmark of the generation-control hot path on B200.

A "step" is one pass of the fused sampler over one batch of synthetic logits: the row-sharded large-batch
configuration (4096 rows x 151936 BF16 logits from N(0, 2^2); per-row temperature U[0.3, 1.5], top_k from
{0, 20, 50, 1000}, top_p U[0.8, 1.0]; repetition penalty 1.1 and presence penalty 0.5 over a 2048-id history per row;
injected uniforms), rows split evenly over the ranks, no collective. Prints ONE JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

``value`` is rows/s with the inputs resident in HBM (CUDA events, max over ranks); ``e2e`` is the same metric through
the public API with HOST (pinned) inputs, copies inside the timed region; ``roofline`` relates the sampler kernel's
algorithmic bytes per launch to the measured HBM copy peak; ``cpu_baseline`` is the CPU oracle (a C restatement
of the reference's numpy sampler) timed on this host's cores on a bounded sample of the same workload.
``--impl reference`` times that CPU path alone, as the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

VOCAB = 151936
TOTAL_ROWS = 4096
HIST_LEN = 2048
RHO, PI = 1.1, 0.5
SEED = 1234
ROW_BYTES = VOCAB * 2 + HIST_LEN * 4 + 4 * 4 + 4          # logits + history + (T, k, p, u) + token: algorithmic bytes per row
METRIC, UNIT = "sampled_rows_per_s", "rows/s"
WORKLOAD = ("row-sharded penalised sampling: 4096 rows x 151936 bf16 logits N(0,2^2), per-row T~U[0.3,1.5], top_k in {0,20,50,1000}, "
            "top_p~U[0.8,1.0], repetition 1.1 + presence 0.5 over 2048-id histories, inverse-CDF draw from injected uniforms")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier measurement on this pool)"


def ncu_traffic():
    """DRAM bytes per row of one sampling call: dram__bytes_read.sum + dram__bytes_write.sum of the top-k kernel and of the
    histogram kernel, from one ncu capture of the 4096-row workload itself (a call's traffic is this times its rows). The
    figures are typed in from that capture; `captured_at` names the commit whose kernels were captured."""
    return TRAFFIC


# (top-k kernel read + write) + (histogram kernel read + write) over the 4096 rows of one call
TRAFFIC = {"dram_bytes_per_row": (1038539000 + 5840384 + 397207000 + 37092864) / 4096, "captured_at": "89b19b4"}


def launches_per_call(lm, rows: int) -> int:
    """Kernels one lm_sample call launches on this workload (per rank): top-k kernel, histogram kernel, generic kernel; with at
    most 5 rows per SM the two sampler kernels run side by side and a row-listing kernel plus a second (usually empty) launch
    of the histogram kernel join them (the rule is lm_sample's, lithos_metal_b200/csrc/lithos_b200.cu)."""
    from lithos_metal_b200 import _lib
    sms = _lib.lib().lm_device_sm_count()
    return 3 if rows > 5 * max(sms, 1) else 5


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown," \
        "clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index), "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def make_inputs(torch, rows: int, row_offset: int, device):
    """Seeded synthetic inputs of the workload's shapes and distributions, generated on the device."""
    g = torch.Generator(device=device)
    g.manual_seed(SEED + row_offset)
    logits = torch.empty(rows, VOCAB, dtype=torch.bfloat16, device=device)
    for r0 in range(0, rows, 256):                                         # bounded temporaries
        n = min(256, rows - r0)
        logits[r0:r0 + n] = (torch.randn(n, VOCAB, generator=g, device=device) * 2.0).to(torch.bfloat16)
    temperature = torch.rand(rows, generator=g, device=device) * 1.2 + 0.3
    top_k = torch.tensor([0, 20, 50, 1000], dtype=torch.int32, device=device)[torch.randint(0, 4, (rows,), generator=g, device=device)]
    top_p = torch.rand(rows, generator=g, device=device) * 0.2 + 0.8
    history = torch.randint(0, VOCAB, (rows, HIST_LEN), generator=g, device=device, dtype=torch.int32)
    uniforms = torch.rand(rows, generator=g, device=device)
    return dict(logits=logits, temperature=temperature, top_k=top_k.contiguous(), top_p=top_p, history=history, uniforms=uniforms)


def cpu_rows_per_s(inp_host, n_rows: int, n_threads: int, repeats: int = 1):
    """The C oracle over the first n_rows of a host copy of the workload, all host threads; rows/s (best of repeats)."""
    import numpy as np
    import oracle
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        tok, _, _ = oracle.sample_batch(inp_host["logits"][:n_rows], temperature=inp_host["temperature"][:n_rows], top_k=inp_host["top_k"][:n_rows],
                                        top_p=inp_host["top_p"][:n_rows], history=inp_host["history"][:n_rows], repetition_penalty=RHO,
                                        presence_penalty=PI, draw="inverse_cdf", uniforms=inp_host["uniforms"][:n_rows], n_threads=n_threads)
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
    return n_rows / best, tok


def penalised_rows(hc, rows):
    """FP32 rows `rows` of a host copy with the penalties applied in binary32 (this repository's definition; the reference has none)."""
    import numpy as np
    import oracle
    out = []
    for r in rows:
        z = oracle.bf16_to_f32(hc["logits"][r]).astype(np.float32).copy()
        ids = np.unique(hc["history"][r])
        v = z[ids]
        z[ids] = (np.where(v > 0, v / np.float32(RHO), v * np.float32(RHO)).astype(np.float32) - np.float32(PI)).astype(np.float32)
        out.append(z)
    return out


_AS_SHIPPED = {}


def _as_shipped_row(i):
    ref, zs, hc = _AS_SHIPPED["ref"], _AS_SHIPPED["rows"], _AS_SHIPPED["hc"]
    return int(ref.sample(zs[i], seed=SEED, step=0, t=i, temperature=float(hc["temperature"][i]), top_k=int(hc["top_k"][i]), top_p=float(hc["top_p"][i])))


def as_shipped_baseline(hc, cores: int):
    """The reference's numpy sampler AS SHIPPED (monolith/nn/sampling_ref.py `sample`: thresholds + Gumbel-max draw), placed
    under oracle/_ref by oracle/make_ref.py: rows/s of a single process and of a multiprocessing.Pool over the host's cores, on
    a bounded subset of the workload's rows (a row with top-p costs ~0.3 s). The penalties, which the reference does not have,
    are applied beforehand and are not timed."""
    from oracle import make_ref
    ref = make_ref.load()
    if ref is None:
        return {"unavailable": "oracle/_ref/sampling_ref.py is not there (python oracle/make_ref.py <reference checkout> places it)"}
    import multiprocessing as mp
    n_single, n_pool = 8, max(8, min(len(hc["temperature"]), 2 * cores))
    _AS_SHIPPED.update(ref=ref, hc=hc, rows=penalised_rows(hc, range(n_pool)))
    _as_shipped_row(0)
    t0 = time.perf_counter()
    single = [_as_shipped_row(i) for i in range(n_single)]
    t_single = time.perf_counter() - t0
    try:
        with mp.get_context("fork").Pool(cores) as pool:
            pool.map(_as_shipped_row, range(min(cores, n_pool)))             # workers started and warm
            t0 = time.perf_counter()
            pooled = pool.map(_as_shipped_row, range(n_pool), chunksize=1)
            t_pool = time.perf_counter() - t0
        pool_v, same = n_pool / t_pool, pooled[:n_single] == single
    except OSError as e:
        pool_v, same = None, f"pool unavailable: {e}"
    return {"single_process_rows_per_s": n_single / t_single, "pool_rows_per_s": pool_v, "unit": UNIT, "cores": cores, "kind": "reference",
            "sample": f"{n_single} rows single process, {n_pool} rows over a Pool of {cores}; the reference's own Gumbel-max draw (it has no "
                      "inverse-CDF draw), penalties applied beforehand and not timed", "pool_equals_single": same}


def host_copy(torch, inp, n_rows: int):
    import numpy as np
    return dict(logits=inp["logits"][:n_rows].view(torch.int16).cpu().numpy().view(np.uint16), temperature=inp["temperature"][:n_rows].cpu().numpy(),
                top_k=inp["top_k"][:n_rows].cpu().numpy(), top_p=inp["top_p"][:n_rows].cpu().numpy(), history=inp["history"][:n_rows].cpu().numpy(),
                uniforms=inp["uniforms"][:n_rows].cpu().numpy())


def reference_arm(args, rank: int, world: int) -> None:
    """The reference's CPU path (its numpy sampler restated in C, every host thread), timed on a bounded sample."""
    if rank != 0:
        return
    import numpy as np
    import oracle
    cores = len(os.sched_getaffinity(0))
    n_rows = max(64, min(512, 2 * cores))
    rng = np.random.default_rng(SEED)
    inp = dict(logits=oracle.f32_to_bf16(rng.standard_normal((n_rows, VOCAB), dtype=np.float32) * np.float32(2.0)),
               temperature=rng.uniform(0.3, 1.5, n_rows).astype(np.float32), top_k=rng.choice(np.array([0, 20, 50, 1000], np.int32), n_rows),
               top_p=rng.uniform(0.8, 1.0, n_rows).astype(np.float32), history=rng.integers(0, VOCAB, (n_rows, HIST_LEN)).astype(np.int32),
               uniforms=rng.random(n_rows).astype(np.float32))
    for _ in range(args.warmup):
        cpu_rows_per_s(inp, n_rows, cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_rows_per_s(inp, n_rows, cores)
    dt = time.perf_counter() - t0
    value = n_rows * args.steps / dt
    sample = f"{n_rows} rows of the workload per step, C restatement of monolith/nn/sampling_ref.py (oracle/lm_oracle.c), {cores} threads"
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
                      "data": "synthetic", "config": {"workload": WORKLOAD, "vocab": VOCAB, "rows_per_step": n_rows},
                      "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
                      "cpu_baseline_as_shipped": as_shipped_baseline(inp, cores),
                      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=TOTAL_ROWS, help="total rows over all ranks (default: the workload's 4096)")
    ap.add_argument("--skip-extras", action="store_true", help="skip the e2e, CPU-baseline, small-batch and verify legs")
    ap.add_argument("--verify-only", action="store_true", help="run only the DSpark verify / draft legs (plain launches first, then the timed graphs)")
    ap.add_argument("--head-only", action="store_true", help="run only the lm_head legs (the projection alone, and the decode tail behind it)")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        reference_arm(args, rank, world)
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    import lithos_metal_b200 as lm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.verify_only:
        if rank == 0:
            print(json.dumps({"verify": bench_verify(torch, lm, dev)}))
        return
    if args.head_only:
        if rank == 0:
            print(json.dumps({"lm_head": bench_lm_head(torch, lm, dev)}))
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    total_rows = args.rows
    rows = total_rows // world
    row_offset = rank * rows
    inp = make_inputs(torch, rows, row_offset, dev)
    # inputs larger than L2 (126 MB) between timed iterations: rotate over as many copies as it takes to pass 512 MB
    n_buf = max(1, -(-512 * 2**20 // (rows * VOCAB * 2)))
    logit_bufs = [inp["logits"]] + [inp["logits"].clone() for _ in range(n_buf - 1)]
    params = lm.SamplingParams(temperature=inp["temperature"], top_k=inp["top_k"], top_p=inp["top_p"], repetition_penalty=RHO, presence_penalty=PI,
                               draw="inverse_cdf")
    tokens = torch.empty(rows, dtype=torch.int32, device=dev)

    def step(i: int):
        lm.sample(logit_bufs[i % n_buf], params, history=inp["history"], uniforms=inp["uniforms"], row_offset=row_offset, out=tokens)

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    for i in range(args.warmup):
        step(i)
    sync_all()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        sync_all()
        ev0.record()
        for i in range(args.steps):
            step(i)
        ev1.record()
        sync_all()
        elapsed_ms = ev0.elapsed_time(ev1)
        if elapsed_ms < 300:                                               # give nvidia-smi time for a few samples under the same load
            t_end = time.perf_counter() + 0.5
            i = 0
            while time.perf_counter() < t_end:
                step(i); i += 1
                if i % 8 == 0:
                    torch.cuda.synchronize(dev)
            torch.cuda.synchronize(dev)
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = total_rows / (ms_per_step * 1e-3)
    peak, peak_src = peaks()
    achieved = rows * ROW_BYTES / (ms_per_step * 1e-3) / 1e9              # per GPU: one launch covers this rank's rows
    traffic = ncu_traffic()
    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
           "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 logits; f64/u64 selection arithmetic", "data": "synthetic",
           "config": {"workload": WORKLOAD, "vocab": VOCAB, "total_rows": total_rows, "rows_per_gpu": rows, "parallelism": f"rows/{world}, no collective",
                      "l2": f"inputs larger than L2: {n_buf} logits buffer(s) of {rows * VOCAB * 2 / 2**20:.0f} MiB rotated"},
           "logits_gbs_per_gpu": rows * VOCAB * 2 / (ms_per_step * 1e-3) / 1e9,
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                        "frac_of_nominal_8TBs": achieved / 8000.0, "algorithmic_bytes_per_row": ROW_BYTES,
                        "traffic": (traffic["dram_bytes_per_row"] * rows if traffic else None)},
           "gpu_launches": launches_per_call(lm, rows) * args.steps, "clocks": clocks.summary()}
    out["roofline"]["launch"] = ("one sampling call = sample_topk_kernel (rows with a top_k) + sample_hist_kernel (the other rows) + "
                                 "sample_generic_kernel (rows handed on: none here)" + (" + the row-listing kernel and a second sample_hist_kernel launch "
                                 "(side-by-side order up to 5 rows per SM)" if launches_per_call(lm, rows) == 5 else "") + "; duration = CUDA events around the call")

    if not args.skip_extras:
        # ---- e2e: host (pinned) inputs -> public API -> tokens on the host, copies inside the timed region
        e2e_steps = max(3, min(args.steps, 5))
        host = {k: torch.empty(v.shape, dtype=v.dtype, pin_memory=True).copy_(v) for k, v in inp.items()}
        host_tok = torch.empty(rows, dtype=torch.int32, pin_memory=True)
        h2d = sum(v.numel() * v.element_size() for v in host.values())

        def e2e_step():
            d = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
            p = lm.SamplingParams(temperature=d["temperature"], top_k=d["top_k"], top_p=d["top_p"], repetition_penalty=RHO, presence_penalty=PI,
                                  draw="inverse_cdf")
            r = lm.sample(d["logits"], p, history=d["history"], uniforms=d["uniforms"], row_offset=row_offset)
            host_tok.copy_(r.tokens, non_blocking=True)

        e2e_step()
        sync_all()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        sync_all()
        e2e_s = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        out["e2e"] = {"value": total_rows * e2e_steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": rows * 4,
                      "steps": e2e_steps, "note": "pinned host logits/history/knobs copied in every step; PCIe-bound"}
        del host

        if rank == 0 and world == 1:
            # ---- the small-batch configuration (256 rows) and the DSpark verify step, reported beside the headline
            small = {k: v[:256] for k, v in inp.items()}
            sp = lm.SamplingParams(temperature=small["temperature"], top_k=small["top_k"], top_p=small["top_p"], repetition_penalty=RHO,
                                   presence_penalty=PI, draw="inverse_cdf")
            # 256-row calls on the 16 different 256-row slices of this rank's logits (1.2 GB: far larger than L2), captured in one
            # CUDA graph so that the time is the GPU's, not the host's launch path
            slices = []
            for j in range(rows // 256):
                sl = slice(256 * j, 256 * (j + 1))
                slices.append((inp["logits"][sl], lm.SamplingParams(temperature=inp["temperature"][sl], top_k=inp["top_k"][sl], top_p=inp["top_p"][sl],
                                                                    repetition_penalty=RHO, presence_penalty=PI, draw="inverse_cdf"),
                               inp["history"][sl], inp["uniforms"][sl]))
            t256 = _graph_us(torch, dev, [(lambda z=z, p=p, h=h, u=u: lm.sample(z, p, history=h, uniforms=u, out=tokens[:256])) for z, p, h, u in slices]) * 1e-3
            out["batch256"] = {"us_per_launch": 1e3 * t256, "rows_per_s": 256 / (t256 * 1e-3), "algorithmic_gbs": 256 * ROW_BYTES / (t256 * 1e-3) / 1e9,
                               "frac_of_peak": 256 * ROW_BYTES / (t256 * 1e-3) / 1e9 / peak, "l2": f"{len(slices)} different 256-row inputs in turn ({len(slices) * 256 * VOCAB * 2 >> 20} MiB)",
                               "timing": f"CUDA graph of {len(slices)} calls, min of 8 replays"}
            out["verify"] = bench_verify(torch, lm, dev)
            # ---- CPU baseline on this host's cores: a bounded sample of the same workload
            cores = len(os.sched_getaffinity(0))
            n_cpu = max(64, min(512, 2 * cores))
            hc = host_copy(torch, inp, n_cpu)
            cpu_rows_per_s(hc, min(n_cpu, cores), cores)
            cpu_v, cpu_tok = cpu_rows_per_s(hc, n_cpu, cores)
            out["cpu_baseline"] = {"value": cpu_v, "unit": UNIT, "cores": cores, "kind": "port",
                                   "sample": f"first {n_cpu} rows of the workload, C restatement of monolith/nn/sampling_ref.py (oracle/lm_oracle.c), {cores} threads"}
            out["cpu_baseline_as_shipped"] = as_shipped_baseline(hc, cores)
            # outside every timed region: EVERY row of the workload against the oracle
            step(0)
            torch.cuda.synchronize(dev)
            _, all_tok = cpu_rows_per_s(host_copy(torch, inp, rows), rows, cores)
            gpu_tok = tokens.cpu().numpy()
            out["cpu_baseline"]["tokens_equal_gpu"] = bool((gpu_tok == all_tok).all())
            out["cpu_baseline"]["rows_compared"] = int(rows)
            out["config1"] = bench_config1(torch, lm, dev)
            out["config5_single_gpu"] = bench_config5_single(torch, lm, dev)
            out["lm_head"] = bench_lm_head(torch, lm, dev)
    if world > 1 and not args.skip_extras:
        out["vocab_parallel"] = bench_vocab_parallel(torch, dist, lm, dev, rank, world, args.warmup)
        out["tensor_parallel_decode_tail"] = bench_tp_tail(torch, dist, lm, dev, rank, world, args.warmup)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def _min_us(torch, dev, call, flush=None, n=20, warm=3):
    ts = []
    for i in range(warm + n):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); call(); b.record()
        torch.cuda.synchronize(dev)
        if i >= warm:
            ts.append(a.elapsed_time(b) * 1e3)
    return min(ts)


def _graph_us(torch, dev, calls, replays=8):
    """Microseconds per call of `calls` (closures that enqueue work on the current stream), captured once in a CUDA graph and
    replayed: the minimum over the replays of (graph time / number of calls)."""
    for c in calls[:3]:
        c()
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for c in calls:
            c()
    best = float("inf")
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(replays):
        a.record(); graph.replay(); b.record()
        torch.cuda.synchronize(dev)
        best = min(best, a.elapsed_time(b) * 1e3 / len(calls))
    return best


def bench_config1(torch, lm, dev):
    """Configuration 1: one FP32 row of 151936 logits N(0, 2^2) with 8 spikes at +12; greedy, then temperature 0.7 / top_k 20 /
    top_p 0.95 with an injected uniform. Microseconds per call over 256 different such rows in turn (155 MB: larger than L2),
    the calls captured in one CUDA graph (a single-row call is shorter than the host's launch path)."""
    g = torch.Generator(device=dev); g.manual_seed(0)
    n = 256
    z = torch.randn(n, VOCAB, generator=g, device=dev) * 2.0
    z.scatter_(1, torch.rand(n, VOCAB, generator=g, device=dev).topk(8, dim=1).indices, 12.0)
    u = torch.rand(n, generator=torch.Generator(device=dev).manual_seed(1), device=dev)
    p = lm.SamplingParams(temperature=0.7, top_k=20, top_p=0.95, draw="inverse_cdf")
    out = torch.empty(1, dtype=torch.int32, device=dev)
    greedy = _graph_us(torch, dev, [(lambda i=i: lm.argmax(z[i:i + 1], out=out)) for i in range(n)])
    stochastic = _graph_us(torch, dev, [(lambda i=i: lm.sample(z[i:i + 1], p, uniforms=u[i:i + 1], out=out)) for i in range(n)])
    return {"workload": "1 row x 151936 fp32, 8 spikes at +12", "greedy_us": greedy, "stochastic_us": stochastic,
            "timing": f"CUDA graph of {n} calls on {n} different rows ({n * VOCAB * 4 >> 20} MiB), min of 8 replays"}


def bench_lm_head(torch, lm, dev):
    """The vocabulary projection in front of the sampler (the reference's lm_head op: 8 rows of a speculative round, hidden 4096,
    151936 x 4096 BF16 weights = 1.24 GB, larger than L2, read once per call; final norm fused), alone and as the head of the
    decode tail: projection, sampler on its 8 rows of logits (thresholds and row statistics), stochastic verification."""
    g = torch.Generator(device=dev); g.manual_seed(SEED)
    rows, hidden = 8, 4096
    x = torch.randn(rows, hidden, generator=g, device=dev).to(torch.bfloat16)
    w = (torch.randn(VOCAB, hidden, generator=g, device=dev) * 0.03).to(torch.bfloat16)
    gamma = (torch.randn(hidden, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    logits = torch.empty(rows, VOCAB, dtype=torch.bfloat16, device=dev)
    head_us = _graph_us(torch, dev, [lambda: lm.lm_head(x, w, gamma, out=logits)] * 8)
    drafts = torch.randint(0, VOCAB, (7,), generator=g, device=dev, dtype=torch.int32)
    q = torch.softmax(torch.randn(7, VOCAB, generator=g, device=dev) * 2.0, dim=-1)
    ua, uf, u8 = torch.rand(7, generator=g, device=dev), torch.rand(1, generator=g, device=dev), torch.full((8,), 0.5, device=dev)
    p = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.95, draw="inverse_cdf")

    def tail():
        lm.lm_head(x, w, gamma, out=logits)
        r = lm.sample(logits, p, uniforms=u8, return_tau=True, return_vmax=True)
        lm.verify(logits, drafts, q, ua, uf, "stochastic", temperature=0.8, tau=r.tau, target_vmax=r.vmax, target_mass=r.mass)
    tail_us = _graph_us(torch, dev, [tail] * 8)
    weight_bytes = VOCAB * hidden * 2
    return {"workload": f"{rows} rows x hidden {hidden} -> {VOCAB} logits, BF16 weights ({weight_bytes >> 20} MiB, read once per call), RMSNorm fused",
            "us_per_call": head_us, "weight_gbs": weight_bytes / (head_us * 1e-6) / 1e9, "frac_of_peak": weight_bytes / (head_us * 1e-6) / 1e9 / peaks()[0],
            "decode_tail_us": tail_us, "decode_tail": "lm_head -> lm_sample (8 rows, top_k 50, top_p 0.95, row statistics out) -> lm_verify (stochastic, statistics in)",
            "timing": "CUDA graph of 8 calls, min of 8 replays"}


def bench_config5_single(torch, lm, dev):
    """Configuration 5 on ONE GPU through lm_sample (the result the vocab-parallel mode must reproduce): 64 rows x 262144 BF16."""
    g = torch.Generator(device=dev); g.manual_seed(SEED)
    full = (torch.randn(64, 262144, generator=g, device=dev) * 2.0).to(torch.bfloat16)
    u = torch.rand(64, generator=g, device=dev)
    p = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.9, draw="inverse_cdf")
    flush = torch.empty(256 * 2**20, dtype=torch.uint8, device=dev)
    us = _min_us(torch, dev, lambda: lm.sample(full, p, uniforms=u), flush)
    return {"workload": "64 rows x 262144 bf16, top_k 50, top_p 0.9, T 0.8, whole rows on one GPU", "us_per_step": us,
            "frac_of_peak": 64 * 262144 * 2 / (us * 1e-6) / 1e9 / peaks()[0], "timing": "L2 flushed, min of 20"}


def _peer_exchange_us(torch, dist, dev, make_sampler, step_of, expect, warmup, n=20):
    """The same step with the records read in place from the peers' memory (symmetric memory over NVLink, a barrier over the ranks on
    the stream, no collective): microseconds per step (max over ranks) and whether every rank's tokens are the expected ones; or why
    not. Never raises: the all-gather figures stand on their own."""
    try:
        sampler = make_sampler()
        r = None
        for _ in range(max(3, warmup)):
            r = step_of(sampler)
        torch.cuda.synchronize(dev)
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            r = step_of(sampler)
        b.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([a.elapsed_time(b) / n], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        used = torch.tensor([int(any(v is not None for v in sampler._peer.values()))], device=dev)
        same = torch.tensor([int(torch.equal(expect, r.tokens))], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        dist.all_reduce(used, op=dist.ReduceOp.MIN)
        res = {"us_per_step": 1e3 * float(t.item()), "tokens_equal_single_gpu_on_every_rank": bool(same.item()),
               "records_read_in_place_from_peers": bool(used.item())}
    except Exception as e:                                                  # (the ranks fail together or not at all: the setup is collective)
        return {"unavailable": repr(e)[:200]}
    try:
        # the same steps as one CUDA graph per rank (two steps: both record buffers), replayed: without the host's launch path
        side = torch.cuda.Stream(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(2):
                    r = step_of(sampler)
        torch.cuda.synchronize(dev)
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize(dev)
        same = torch.tensor([int(torch.equal(expect, r.tokens))], device=dev)
        dist.barrier()
        a.record()
        for _ in range(n // 2):
            graph.replay()
        b.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([a.elapsed_time(b) / (2 * (n // 2))], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        res["us_per_step_graph"] = 1e3 * float(t.item())
        res["graph_tokens_equal"] = bool(same.item())
    except Exception as e:
        res["graph"] = "unavailable: " + repr(e)[:160]
    return res


def bench_vocab_parallel(torch, dist, lm, dev, rank, world, warmup):
    """The vocab-parallel configuration (64 rows x 262144 BF16 logits N(0, 2^2), top_k 50, top_p 0.9, temperature 0.8), the
    vocabulary split over the ranks: per-step time of local kernel + NCCL all-gather + merge kernel (CUDA events, max over
    ranks), and whether every rank's tokens equal rank 0's single-GPU result on the whole rows."""
    from lithos_metal_b200 import parallel
    rows, vocab = 64, 262144
    g = torch.Generator(device=dev)
    g.manual_seed(SEED)                                                    # every rank generates the same full rows, keeps its shard
    full = (torch.randn(rows, vocab, generator=g, device=dev) * 2.0).to(torch.bfloat16)
    u = torch.rand(rows, generator=g, device=dev)
    p = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.9, draw="inverse_cdf")
    sampler = parallel.VocabParallelSampler(p, vocab)
    lo, width = parallel.shard_vocab(vocab, rank, world)
    shard = full[:, lo:lo + width].contiguous()
    for _ in range(max(3, warmup)):
        r = sampler.sample(shard, uniforms=u)
    torch.cuda.synchronize(dev)
    dist.barrier()
    n = 20
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        r = sampler.sample(shard, uniforms=u)
    b.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([a.elapsed_time(b) / n], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # the three parts of a step, each timed on its own (CUDA events, max over ranks): local kernel, NCCL all-gather, merge kernel
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    parts = torch.zeros(3, dtype=torch.float64, device=dev)
    for _ in range(n):
        ev[0].record()
        rec = sampler.backend.local(shard, sampler.shard_start, p, sampler.cap, world)
        ev[1].record()
        flat = torch.empty(world * rec.shape[0], rec.shape[1], dtype=rec.dtype, device=dev)
        dist.all_gather_into_tensor(flat, rec)
        ev[2].record()
        sampler.backend.merge(flat.view(-1, rows, rec.shape[1]), p, sampler.cap, u, 0, 0)
        ev[3].record()
        torch.cuda.synchronize(dev)
        parts += torch.tensor([ev[i].elapsed_time(ev[i + 1]) for i in range(3)], dtype=torch.float64, device=dev)
    parts /= n
    dist.all_reduce(parts, op=dist.ReduceOp.MAX)
    one = lm.sample(full, p, uniforms=u).tokens
    same = torch.tensor([int(torch.equal(one, r.tokens))], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    ms = float(t.item())
    return {"workload": "64 rows x 262144 bf16, vocab split over the ranks, top_k 50, top_p 0.9, T 0.8", "us_per_step": 1e3 * ms,
            "rows_per_s": rows / (ms * 1e-3), "local_kernel_us": 1e3 * float(parts[0]), "allgather_us": 1e3 * float(parts[1]),
            "merge_kernel_us": 1e3 * float(parts[2]), "parts_timing": "each part between its own CUDA events with a synchronize per step (launch gaps included), max over ranks",
            "allgather_bytes_per_rank": int(rec.numel()), "records_per_row_and_rank": int(rec.shape[0] // rows),
            "tokens_equal_single_gpu_on_every_rank": bool(same.item()),
            "peer_records": _peer_exchange_us(torch, dist, dev, lambda: parallel.VocabParallelSampler(p, vocab, exchange="peer"),
                                              lambda sm: sm.sample(shard, uniforms=u), one, warmup)}


def bench_tp_tail(torch, dist, lm, dev, rank, world, warmup):
    """The decode tail with the vocabulary projection split over the ranks (a tensor-parallel head): every rank projects the 8 rows onto
    its own vocab/world rows of the 151936 x 4096 BF16 weight (lm_head on a shard gives the bits of the whole), then the vocab-parallel
    sampler on the local logits (records, one all-gather, merge). Microseconds per step (CUDA events, max over ranks), and whether every
    rank's tokens equal the single-GPU tail's (projection onto the whole weight, then lm_sample) computed on rank 0's GPU."""
    from lithos_metal_b200 import parallel
    rows, hidden = 8, 4096
    g = torch.Generator(device=dev); g.manual_seed(SEED)                   # the same tensors on every rank; a rank keeps its shard of the weight
    x = torch.randn(rows, hidden, generator=g, device=dev).to(torch.bfloat16)
    gamma = (torch.randn(hidden, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    u = torch.rand(rows, generator=g, device=dev)
    w = (torch.randn(VOCAB, hidden, generator=g, device=dev) * 0.03).to(torch.bfloat16)
    p = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.95, draw="inverse_cdf")
    one = lm.sample(lm.lm_head(x, w, gamma), p, uniforms=u).tokens
    lo, width = parallel.shard_vocab(VOCAB, rank, world)
    w_local = w[lo:lo + width].clone()
    del w
    sampler = parallel.VocabParallelSampler(p, VOCAB, reuse_buffers=True)
    local = torch.empty(rows, width, dtype=torch.bfloat16, device=dev)

    def step():
        lm.lm_head(x, w_local, gamma, out=local)
        return sampler.sample(local, uniforms=u)
    for _ in range(max(3, warmup)):
        r = step()
    torch.cuda.synchronize(dev)
    dist.barrier()
    n = 20
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        r = step()
    b.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([a.elapsed_time(b) / n], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    same = torch.tensor([int(torch.equal(one, r.tokens))], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    return {"workload": f"8 rows x hidden 4096 -> {VOCAB} logits over {world} ranks ({width} vocabulary rows each), then top_k 50 / top_p 0.95 sampling over the ranks",
            "us_per_step": 1e3 * float(t.item()), "weight_bytes_per_rank": int(width * hidden * 2),
            "timing": "20 steps between CUDA events (host launches included), max over ranks",
            "tokens_equal_single_gpu_on_every_rank": bool(same.item()),
            "peer_records": _peer_exchange_us(torch, dist, dev, lambda: parallel.VocabParallelSampler(p, VOCAB, exchange="peer"),
                                              lambda sm: (lm.lm_head(x, w_local, gamma, out=local), sm.sample(local, uniforms=u))[1], one, warmup)}


def bench_verify(torch, lm, dev):
    """One DSpark step (7 drafts + bonus row, V = 151936, BF16 target, FP32 draft probabilities): GPU microseconds per
    step, measured over a CUDA graph of 20 back-to-back steps so that host launch overhead is not in the number."""
    g = torch.Generator(device=dev)
    g.manual_seed(SEED)
    target = (torch.randn(8, VOCAB, generator=g, device=dev) * 2.0).to(torch.bfloat16)
    drafts = torch.randint(0, VOCAB, (7,), generator=g, device=dev, dtype=torch.int32)
    drafts[:3] = target[:3].float().argmax(-1).to(torch.int32)
    q = torch.softmax(target[:7].float() + torch.randn(7, VOCAB, generator=g, device=dev) * 0.5, dim=-1)
    ua, uf = torch.rand(7, generator=g, device=dev), torch.rand(1, generator=g, device=dev)
    # the drafter's side of the same round: seven BF16 logits rows, sampled one position per call as a Markov drafter does
    drafter = (target[:7].float() + torch.randn(7, VOCAB, generator=g, device=dev) * 0.5).to(torch.bfloat16)
    stats = lm.draft_q(drafter, temperature=1.0, seed=SEED, step=0)
    # the two ends of the stochastic step: every draft accepted (no residual: two exchanges between the blocks), and the first
    # draft rejected (the residual of row 0 is summed and drawn from: three exchanges)
    u_zero, u_one = torch.zeros(7, device=dev), torch.full((7,), 0.999, device=dev)
    kept = lm.sample(target, lm.SamplingParams(temperature=1.0, top_k=torch.zeros(8, dtype=torch.int32), draw="inverse_cdf"), uniforms=torch.full((8,), 0.5), return_vmax=True)
    vmax, mass = kept.vmax, kept.mass                                  # what the sampler leaves for the verify step (no thresholds here)
    worst = drafts.clone()
    worst[0] = (q[0] / torch.softmax(target[0].float(), dim=-1)).argmax().to(torch.int32)       # the token the drafter overrates most
    round_params = lm.SamplingParams(temperature=0.8, top_k=50, top_p=0.95, draw="inverse_cdf")
    u8 = torch.full((8,), 0.5, device=dev)

    def round_tail(with_stats: bool):
        r = lm.sample(target, round_params, uniforms=u8, return_tau=True, return_vmax=with_stats)
        return lm.verify(target, drafts, q, ua, uf, "stochastic", temperature=0.8, tau=r.tau, target_vmax=r.vmax, target_mass=r.mass)

    calls = {"stochastic": lambda: lm.verify(target, drafts, q, ua, uf, "stochastic"),
             "stochastic_all_accepted": lambda: lm.verify(target, drafts, q, u_zero, uf, "stochastic"),
             "stochastic_first_rejected": lambda: lm.verify(target, worst, q, u_one, uf, "stochastic"),
             # the row maxima handed over by the sampler, as the reference's verify kernels get them (KEPT_STATS): one exchange fewer
             "stochastic_given_row_max": lambda: lm.verify(target, drafts, q, ua, uf, "stochastic", target_vmax=vmax),
             # ... and the rows' masses too (both halves of KEPT_STATS: what lm_sample leaves in out_vmax / out_mass): one exchange in all
             "stochastic_given_row_stats": lambda: lm.verify(target, drafts, q, ua, uf, "stochastic", target_vmax=vmax, target_mass=mass),
             "stochastic_given_row_stats_first_rejected": lambda: lm.verify(target, worst, q, u_one, uf, "stochastic", target_vmax=vmax, target_mass=mass),
             # the tail of a speculative step as the reference runs it: the sampler on the 8 rows (thresholds top_k 50 / top_p 0.95,
             # temperature 0.8; it leaves tau and, in the second form, the rows' maxima and masses), then the verification
             "round_sample_then_verify": lambda: round_tail(False),
             "round_sample_then_verify_given_row_stats": lambda: round_tail(True),
             "stochastic_q_logits": lambda: lm.verify(target, stats.tokens, None, ua, uf, "stochastic", draft_logits=drafter, draft_stats=stats),
             # both hand-overs of a round at once: q from the drafter's logits and statistics, the target rows' maxima and masses from the sampler
             "stochastic_q_logits_given_row_stats": lambda: lm.verify(target, stats.tokens, None, ua, uf, "stochastic", draft_logits=drafter, draft_stats=stats,
                                                                      target_vmax=vmax, target_mass=mass),
             "greedy": lambda: lm.verify(target, drafts, mode="greedy"),
             "draft_q_one_position": lambda: lm.draft_q(drafter[3:4], temperature=1.0, seed=SEED, step=0, first_position=3)}
    res = {"accept_len": {"stochastic": int(calls["stochastic"]()[0]), "stochastic_all_accepted": int(calls["stochastic_all_accepted"]()[0]),
                          "stochastic_first_rejected": int(calls["stochastic_first_rejected"]()[0])}}
    for mode, call in calls.items():
        for _ in range(3):
            call()
        torch.cuda.synchronize(dev)
        side = torch.cuda.Stream(dev)
        graph = torch.cuda.CUDAGraph()
        n = 20
        try:
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(n):
                        call()
            torch.cuda.synchronize(dev)
            graph.replay()
            torch.cuda.synchronize(dev)
            best = None
            for _ in range(10):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); graph.replay(); b.record()
                torch.cuda.synchronize(dev)
                t = a.elapsed_time(b) * 1e3 / n
                best = t if best is None or t < best else best
            res[mode + "_us_per_step"] = best
            res["timing"] = "CUDA graph of 20 steps, min of 10 replays"
        except Exception as e:                                             # graph capture unavailable: time single launches
            torch.cuda.synchronize(dev)
            ts = []
            for _ in range(20):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); call(); b.record()
                torch.cuda.synchronize(dev)
                ts.append(a.elapsed_time(b) * 1e3)
            res[mode + "_us_per_step"] = min(ts)
            res["timing"] = f"single launches, min of 20 (graph capture failed: {type(e).__name__})"
    res["bytes_algorithmic_min"] = 8 * VOCAB * 2 + VOCAB * 4
    res["bytes_one_pass"] = 8 * VOCAB * 2 + 7 * VOCAB * 4
    res["bytes_one_pass_q_logits"] = 8 * VOCAB * 2 + 7 * VOCAB * 2
    return res


if __name__ == "__main__":
    main()
