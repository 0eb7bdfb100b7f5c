#!/usr/bin/env python
"""Benchmark of the hot path: the chained per-pass op mix of one forward pass, token-sharded over N GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference|reference-cuda]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

One step = one pass over ONE batch of 65,536 tokens whose rows are split over the N GPUs (strong scaling: rank
k owns rows [k*65536/N, (k+1)*65536/N), generated from per-row-block seeds so the batch is the same for every
N): 1 embedding gather, 42 fused residual-add + RMSNorm, 21 gated RMSNorm, 17 relu^2 = 81 launches, 2,693,380
algorithmic HBM bytes per token, no collective on the path.  The pass is captured once in a CUDA graph and
replayed inside the timed loop (--eager host-launches it instead).
Rank 0 prints ONE JSON line.  `value` is device-timed whole-job tokens/s over exactly K steps with every
input resident in HBM (65,536 x K / max-over-ranks time); `weak` is the same measurement with 65,536 tokens
PER GPU; `e2e` is the pass through the host-buffer call (ids copied in from pinned memory, result row copied
back) timed by the wall clock; `roofline` describes the dominant kernel (add + RMSNorm) and `kernels` all four,
from a second run of the same K steps in which a CUDA event is recorded after every launch
(`traced_ms_per_step` is that run's step time); `parity_check` compares sampled rows of the timed pass's output
with the CPU oracle after the timed region; `allgather` (N > 1) is an NCCL all-gather of the output rows, timed
separately and never part of `value`.

--impl reference        the torch golden formulation on the host cores (all threads), a bounded token sample
--impl reference-cuda   the reference's OWN CUDA kernels (recompiled for sm_100a into oracle/_ref) on the GPU,
                        unfused as the reference runs them (add kernel, then rmsnorm kernel)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "achieved HBM GB/s (% of B200 peak) and tokens/s per fused op at 1/2/4/8 GPUs"
GLOBAL_TOKENS = 65536
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0

# algorithmic HBM bytes per token and per launch kind (each activation byte crosses HBM once)
BYTES_PER_TOKEN = {"embedding": 2 * 3136 * 2 + 4, "add_rmsnorm": 4 * 3136 * 2, "gated_rmsnorm": 3 * 6144 * 2,
                   "relu2": 2 * 12544 * 2}


# ------------------------------------------------------------------------------------------------
# rank plumbing (works with gloo on CPU and nccl on GPU)
# ------------------------------------------------------------------------------------------------
def _reduce(value: float, op) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=op)
    return float(t.item())


def max_over_ranks(value: float) -> float:
    return _reduce(value, dist.ReduceOp.MAX)


def sum_over_ranks(value: float) -> float:
    return _reduce(value, dist.ReduceOp.SUM)


def barrier() -> None:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def measured_peak() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (6650 GB/s, earlier measurement on this pool)"


# ------------------------------------------------------------------------------------------------
# clock sampling during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.samples: list[list[str]] = []
        self.proc = None
        self.thread = None
        sel = []
        try:
            sel = ["-i", str(torch.cuda.get_device_properties(device_index).uuid)]
            if not sel[1].startswith("GPU-"):
                sel[1] = "GPU-" + sel[1]
        except Exception:
            sel = []
        self.cmd = ["nvidia-smi", *sel, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"]

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self) -> None:
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append([time.perf_counter()] + parts)

    def summary(self, t0: float, t1: float, strict: bool = False) -> dict:
        """Median SM clock, maximum power and the slowdown reasons seen in the samples taken inside [t0, t1]."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        samples = list(self.samples)
        inside = [s[1:] for s in samples if t0 <= s[0] <= t1 + (0.0 if strict else 0.15)]
        for s in inside or ([] if strict else [s[1:] for s in samples[-3:]]):
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
                power.append(float(s[2]))
            except ValueError:
                continue
            for name, flag in zip(names, s[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}

    def stop(self) -> None:
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)
        self.proc = None


# ------------------------------------------------------------------------------------------------
# the B200 arm
# ------------------------------------------------------------------------------------------------
class TracedChain:
    """ChainPass whose ops record a CUDA event after every launch, so each launch's device time is known."""

    def __init__(self, cp):
        self.cp = cp
        self.kinds: list[str] = []
        self.events: list[torch.cuda.Event] = []

    def run(self) -> None:
        from nemotron_infer_b200 import chain, ops
        cp, b = self.cp, self.cp.buf

        def mark(kind):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.kinds.append(kind)
            self.events.append(ev)

        mark("start")
        cur, other = b.hidden
        ops.embedding(b.table, b.ids, out=cur, err_flag=b.err_flag)
        mark("embedding")
        n_m = 0
        for i, kind in enumerate(cp.schedule):
            if kind == "M":
                ops.rmsnorm_gated(b.y, b.z, b.gated_w[n_m], chain.D_INNER // chain.N_GROUPS, out=b.gated_out)
                n_m += 1
                mark("gated_rmsnorm")
            elif kind == "-":
                ops.relu2(b.u, out=b.act)
                mark("relu2")
            ops.add_rmsnorm(cur, b.mixer_out[i % len(b.mixer_out)], b.norm_w[i], out_res=other, out=b.normed)
            mark("add_rmsnorm")
            cur, other = other, cur

    def per_kind_ms(self) -> dict[str, list[float]]:
        out: dict[str, list[float]] = {}
        for i in range(1, len(self.events)):
            if self.kinds[i] == "start":
                continue
            out.setdefault(self.kinds[i], []).append(self.events[i - 1].elapsed_time(self.events[i]))
        return out


def cpu_chain_tokens_per_s(tokens: int, reps: int, threads: int) -> tuple[float, float]:
    """Times the torch golden formulation of the same 81-op chain on the host cores."""
    from oracle import torch_golden as og
    from nemotron_infer_b200 import chain
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16
    vocab = 131072
    table = torch.empty(vocab, chain.HIDDEN, dtype=bf)
    for lo in range(0, vocab, 16384):
        table[lo:lo + 16384] = (0.02 * torch.randn(16384, chain.HIDDEN, generator=g)).to(bf)
    ids = torch.randint(0, vocab, (tokens,), generator=g)
    mix = [torch.randn(tokens, chain.HIDDEN, generator=g).to(bf) for _ in range(2)]
    y, z = (torch.randn(tokens, chain.D_INNER, generator=g).to(bf) for _ in range(2))
    u = (2 * torch.randn(tokens, chain.INTER, generator=g)).to(bf)
    nw = 1 + 0.1 * torch.randn(chain.N_LAYERS, chain.HIDDEN, generator=g)
    gw = 1 + 0.1 * torch.randn(21, chain.D_INNER, generator=g)
    sched = chain.layer_schedule()

    def one_pass():
        h = og.embedding(ids, table)
        n_m = 0
        for i, kind in enumerate(sched):
            if kind == "M":
                og.gated_rmsnorm_bf16(y, z, gw[n_m], chain.D_INNER // chain.N_GROUPS)
                n_m += 1
            elif kind == "-":
                og.relu2_bf16(u)
            h, n = og.add_rmsnorm_bf16(h, mix[i % 2], nw[i])
        return n

    one_pass()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return tokens / med, med * 1e3


def timed_passes(step, steps: int) -> float:
    """Device time in ms of exactly `steps` calls of `step` on the current stream: barrier + synchronize on both
    sides, two CUDA events on the launching stream, max over ranks."""
    barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    barrier()
    return max_over_ranks(ev0.elapsed_time(ev1))


def parity_sample(cp, n_rows: int, seed: int) -> dict:
    """Checks rows of the pass that was just timed against the CPU oracle (outside every timed region).

    `n_rows` rows of this rank's shard (first, last, the rest drawn at random) are recomputed with
    oracle/torch_golden.py from the same inputs: the whole 42-layer residual chain for final_hidden and normed,
    the last gated RMSNorm and relu^2.  The ops are independent per row, so a row subset is a complete check of
    those rows."""
    from oracle import torch_golden as og
    from nemotron_infer_b200 import chain
    b, T = cp.buf, cp.tokens
    g = torch.Generator().manual_seed(seed)
    pick = torch.unique(torch.cat([torch.tensor([0, T - 1]), torch.randint(0, T, (max(n_rows - 2, 0),), generator=g)]))
    sel = pick.to(b.ids.device)
    cpu = lambda t: t.index_select(0, sel).cpu()  # noqa: E731
    ids = cpu(b.ids).long()
    h = og.embedding(torch.arange(ids.numel()), b.table.index_select(0, ids.to(b.table.device)).cpu())
    mix = [cpu(m) for m in b.mixer_out]
    norm_w, gated_w = b.norm_w.cpu(), b.gated_w.cpu()
    for i in range(chain.N_LAYERS):
        h, normed = og.add_rmsnorm_bf16(h, mix[i % len(mix)], norm_w[i])
    gated = og.gated_rmsnorm_bf16(cpu(b.y), cpu(b.z), gated_w[20], chain.D_INNER // chain.N_GROUPS)
    act = og.relu2_bf16(cpu(b.u))
    bits = lambda t: t.contiguous().view(torch.int16)  # noqa: E731
    rep_n = og.ulp_report(cpu(b.normed), normed)
    rep_g = og.ulp_report(cpu(b.gated_out), gated)
    exact = {"final_hidden": bool(torch.equal(bits(cpu(cp.final_hidden)), bits(h))),
             "act": bool(torch.equal(bits(cpu(b.act)), bits(act)))}
    return {"rows": int(pick.numel()), "max_ulp": int(max(rep_n["max_ulp"], rep_g["max_ulp"])),
            "mismatch_frac": {"normed": rep_n["mismatch_frac"], "gated_out": rep_g["mismatch_frac"]},
            "bit_exact": [k for k, v in exact.items() if v], "not_bit_exact": [k for k, v in exact.items() if not v],
            "err_flag": int(b.err_flag.item())}


def run_b200(args, rank: int, world: int, local_rank: int) -> dict | None:
    from nemotron_infer_b200 import _lib, chain, ops
    lib = _lib.load()                       # raises if the CUDA library is missing: there is no fallback
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (B200); no CPU path exists for the product arm")
    torch.cuda.set_device(local_rank)
    _lib.check(lib.nmt_set_device(local_rank), "nmt_set_device")
    dev = f"cuda:{local_rank}"
    G = args.tokens                          # ONE batch of G tokens; rank k of n owns rows shard_range(G, k, n)
    lo, hi = chain.shard_range(G, rank, world)
    T = hi - lo
    cp = chain.ChainPass(T, dev, init=chain.batch_shard(G, lo, hi, dev, seed=1234))
    for _ in range(max(args.warmup, 3)):
        cp.run()
    torch.cuda.synchronize()
    if args.eager:
        step, launches_per_step, mode = cp.run, cp.launches_per_pass, "81 host-side launches per pass"
    else:
        cp.capture()
        step, launches_per_step = cp.replay, cp.graph_launches
        mode = f"one CUDA-graph replay per pass ({cp.graph_launches} kernel nodes, programmatic dependent launch edges)"

    # the sampler starts ahead of the timed region (nvidia-smi takes a moment to come up) and keeps the GPU
    # busy meanwhile; only samples inside the timed window are reported
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(5):
        step()
    launches0 = ops.launch_count()
    t_start = time.perf_counter()
    ms_total = timed_passes(step, args.steps)
    t_end = time.perf_counter()
    launches = (ops.launch_count() - launches0) if args.eager else launches_per_step * args.steps

    # The same K steps once more with a CUDA event after every launch: per-kernel durations for the roofline.
    # (Kept out of the region `value` is taken from: 82 event records per step cost ~1 % and keep consecutive
    # kernels from overlapping their launch with the previous kernel's tail.)
    traced = TracedChain(cp)
    tv0, tv1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tv0.record()
    for _ in range(args.steps):
        traced.run()
    tv1.record()
    torch.cuda.synchronize()
    traced_ms = tv0.elapsed_time(tv1) / args.steps
    t_end = time.perf_counter()
    barrier()
    clocks = sampler.summary(t_start, t_end) if sampler else None

    # the timed pass's own output against the CPU oracle, on sampled rows of every rank's shard
    step()
    torch.cuda.synchronize()
    par = parity_sample(cp, args.parity_rows, seed=99 + rank)
    par_bad = sum_over_ranks(float(par["max_ulp"] > 1 or bool(par["not_bit_exact"]) or par["err_flag"] != 0))
    par_rows = sum_over_ranks(par["rows"])
    par_ulp = max_over_ranks(par["max_ulp"])

    # Optional: gather every rank's output rows (NCCL over NVLink).  Not part of the metric: the path itself has no
    # exchange step; this only says what assembling the full [G, 3136] tensor on every GPU would add.
    allgather = None
    if args.allgather and world > 1 and G % world == 0:
        full = torch.empty(G, 3136, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            dist.all_gather_into_tensor(full, cp.buf.normed)
        ag_ms = timed_passes(lambda: dist.all_gather_into_tensor(full, cp.buf.normed), args.steps) / args.steps
        recv = (world - 1) * T * 3136 * 2
        allgather = {"ms": round(ag_ms, 4), "bytes_received_per_gpu": recv, "gbs_per_gpu": round(recv / ag_ms / 1e6, 1),
                     "backend": "nccl all_gather_into_tensor", "note": "timed separately; not included in value or e2e"}
        del full

    # end to end through the host-buffer call: ids from pinned host memory, the last row (and, second figure,
    # every row) of the result back to pinned host memory, wall clock
    ids_host = cp.buf.ids.cpu().pin_memory()
    cp.run_from_host(ids_host)
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cp.run_from_host(ids_host)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    rows_host = torch.empty(T, 3136, dtype=torch.bfloat16).pin_memory()
    cp.run_from_host(ids_host, full_output=rows_host)
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cp.run_from_host(ids_host, full_output=rows_host)
    e2e_all_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    del rows_host

    per_kind = traced.per_kind_ms()
    local = {k: (statistics.mean(v), len(v)) for k, v in per_kind.items()}

    # weak scaling beside it (N > 1): G tokens PER GPU, i.e. a batch of N*G tokens sharded the same way
    weak = None
    if world > 1 and not args.no_weak:
        del cp, traced
        torch.cuda.empty_cache()
        wp = chain.ChainPass(G, dev, init=chain.batch_shard(G * world, rank * G, (rank + 1) * G, dev, seed=4321))
        if args.eager:
            wstep = wp.run
        else:
            wp.capture()
            wstep = wp.replay
        for _ in range(max(args.warmup, 3)):
            wstep()
        w_ms = timed_passes(wstep, args.steps)
        weak = {"value": round(G * world * args.steps / (w_ms * 1e-3), 1), "unit": "tokens/s", "scaling": "weak",
                "tokens_per_gpu": G, "global_tokens": G * world, "ms_per_step": round(w_ms / args.steps, 4)}
        del wp
        torch.cuda.empty_cache()
    if rank != 0:
        return None
    peak, peak_src = measured_peak()
    traffic = {}
    tp = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if os.path.exists(tp):
        traffic = json.load(open(tp))
    kernels = {}
    for kind, (mean_ms, n) in local.items():
        bytes_launch = BYTES_PER_TOKEN[kind] * T
        ach = bytes_launch / (mean_ms * 1e-3) / 1e9
        t_tok = traffic.get(kind, {}).get("dram_bytes_per_token")
        kernels[kind] = {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(ach / peak, 4), "frac_of_nominal_8000": round(ach / NOMINAL_HBM_GBS, 4),
                         "traffic": (t_tok * T if t_tok else None), "algorithmic_bytes": bytes_launch,
                         "avg_launch_ms": round(mean_ms, 4), "launches": n, "tokens_per_launch": T,
                         "tokens_per_s": round(T / (mean_ms * 1e-3), 1)}
    value = G * args.steps / (ms_total * 1e-3)
    gbs = value * chain.bytes_per_token(4) / 1e9
    out = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "BASELINE.json configs[4]: chained per-pass op mix (1 embedding gather, 42 add+RMSNorm "
                               "@3136, 21 gated RMSNorm @6144/8 groups, 17 relu^2 @12544) over ONE batch of "
                               f"{G} tokens, rows split over the GPUs (rank k of n owns rows [k*G/n, (k+1)*G/n)), no collective",
                   "global_tokens": G, "tokens_per_gpu": T, "ids": "int32", "bytes_per_token": chain.bytes_per_token(4),
                   "launch": mode,
                   "l2": ("every activation tensor of a shard and the 822 MB table exceed the 126 MB L2; no flush"
                          if T * 3136 * 2 > 126 * 2**20 else
                          "a shard's 3136-wide tensors are smaller than the 126 MB L2, but consecutive launches of the pass "
                          "touch different tensors and the pass moves > 20 GB between two uses of the same bytes; no flush")},
        "traced_ms_per_step": round(traced_ms, 4),
        "hbm_gbs": round(gbs, 1), "hbm_gbs_per_gpu": round(gbs / world, 1),
        "hbm_frac_of_measured_peak": round(gbs / world / peak, 4),
        "hbm_frac_of_nominal_8000": round(gbs / world / NOMINAL_HBM_GBS, 4),
        "roofline": dict(kernels["add_rmsnorm"], kernel="rmsnorm_ctarow_kernel<3,1,true> (fused residual add + RMSNorm, 3136 wide)",
                         peak_source=peak_src),
        "kernels": kernels,
        "e2e": {"value": round(G * args.steps / e2e_s, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": G * 4, "d2h_bytes_per_step": 3136 * 2 * world,
                "ms_per_step": round(e2e_s / args.steps * 1e3, 4),
                "call": "ChainPass.run_from_host(ids in pinned host memory) -> last token's normed hidden state on the host",
                "all_rows": {"value": round(G * args.steps / e2e_all_s, 1), "unit": "tokens/s",
                             "h2d_bytes_per_step": G * 4, "d2h_bytes_per_step": G * 3136 * 2,
                             "ms_per_step": round(e2e_all_s / args.steps * 1e3, 4),
                             "call": "the same call returning every normed row [T, 3136] to pinned host memory; from 32,768 tokens per GPU up the pass runs as 4 row ranges and each range's copy overlaps the next range's kernels"}},
        "gpu_launches": int(launches),
        "parity_check": {"rows": int(par_rows), "max_ulp": int(par_ulp), "mismatch_frac": par["mismatch_frac"],
                         "bit_exact": par["bit_exact"], "ok": par_bad == 0,
                         "against": "oracle/torch_golden.py on the same rows of the timed batch (first, last, random), "
                                    "after the timed region; mismatch_frac is rank 0's"},
        "clocks": clocks,
    }
    if weak:
        out["weak"] = weak
    elif world == 1:
        out["weak"] = {"value": out["value"], "unit": "tokens/s", "scaling": "weak", "tokens_per_gpu": G,
                       "global_tokens": G, "ms_per_step": out["ms_per_step"], "note": "identical to the strong figure at 1 GPU"}
    if allgather:
        out["allgather"] = allgather
    if world == 1 and not args.no_per_op:
        out["ops_at_config_sizes"] = per_op_at_config_sizes(dev, peak, sampler)
    if sampler:
        sampler.stop()
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        v, ms = cpu_chain_tokens_per_s(args.cpu_tokens, 3, threads)
        out["cpu_baseline"] = {"value": round(v, 1), "unit": "tokens/s", "cores": threads, "kind": "port",
                               "sample": f"the same 81-op chain in the torch golden formulation (oracle/torch_golden.py) on "
                                         f"{args.cpu_tokens} tokens, median of 3 passes after 1 warm-up, {ms:.0f} ms per pass, "
                                         f"torch {torch.__version__} with {threads} threads"}
    return out


def per_op_at_config_sizes(dev: str, peak: float, sampler) -> dict:
    """BASELINE.json configs[1..3] (and the gather) at their own sizes, each op alone.

    Bandwidth-sized cases: batches of back-to-back launches over rotating buffer sets larger than L2, CUDA events,
    median over ~0.4 s of launches, with the median SM clock seen during that window (us x MHz = SM cycles per
    launch, which separates a power-capped clock from a fixed per-launch cost).  T = 1 and 64 are latency cases:
    microseconds per launch inside a CUDA-graph replay, no GB/s."""
    from nemotron_infer_b200 import microbench as mb
    per_op = {}
    for name, op, tok in (("add_rmsnorm", "add_rmsnorm", 8192), ("gated", "gated", 16384), ("relu2", "relu2", 8192),
                          ("embedding", "embedding", 65536), ("add_rmsnorm_65536", "add_rmsnorm", 65536)):
        probe = mb.run_op(op, tok, 5, 3, dev, 10, False)
        reps = max(10, min(4000, int(0.4e6 / max(probe["median_us"] * 10, 1.0))))
        t0 = time.perf_counter()
        r = mb.run_op(op, tok, reps, 3, dev, 10, False)
        t1 = time.perf_counter()
        mhz = sampler.summary(t0, t1, strict=True)["sm_mhz"] if sampler else None
        per_op[name] = {"tokens": tok, "us_per_launch": r["median_us"], "achieved_gbs": r["gbs"],
                        "frac_of_measured_peak": round(r["gbs"] / peak, 4),
                        "frac_of_nominal_8000": round(r["gbs"] / NOMINAL_HBM_GBS, 4), "tokens_per_s": r["tokens_per_s"],
                        "sm_mhz_median": mhz,
                        "kcycles_per_launch": round(r["median_us"] * mhz / 1e3, 2) if mhz else None}
        torch.cuda.empty_cache()
    for tok in (1, 64):
        r = mb.run_op("add_rmsnorm", tok, 50, 3, dev, 20, True)
        per_op[f"add_rmsnorm_T{tok}"] = {"tokens": tok, "us_per_launch": r["median_us"],
                                         "mode": "CUDA-graph replay of 20 launches; latency-bound, no GB/s figure"}
    return per_op


# ------------------------------------------------------------------------------------------------
# reference arms
# ------------------------------------------------------------------------------------------------
def run_reference_cpu(args, world: int) -> dict:
    threads = os.cpu_count() or 1
    reps = max(args.steps, 1)
    v, ms = cpu_chain_tokens_per_s(args.cpu_tokens, reps, threads)
    sample = (f"reference formulation (tools/dump_*.py golden functions restated in oracle/torch_golden.py) of the "
              f"81-op chain on {args.cpu_tokens} tokens per step, {threads} host threads, torch {torch.__version__}; "
              f"the reference has no CPU implementation of these ops other than this torch formulation")
    out = {"impl": "reference", "metric": METRIC, "value": round(v, 1), "unit": "tokens/s", "n_gpus": world,
           "steps": reps, "warmup": 1, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": "BASELINE.json configs[4] chained per-pass op mix, bounded sample",
                      "tokens_per_step": args.cpu_tokens},
           "cpu_baseline": {"value": round(v, 1), "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
           "e2e": {"value": round(v, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if torch.cuda.is_available() and os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libnemotron_ref.so")):
        try:
            out["reference_cuda"] = run_reference_cuda(args, 0, quiet=True)
        except Exception as e:  # the CPU figure stands on its own
            out["reference_cuda"] = {"unavailable": f"{type(e).__name__}: {e}"}
    return out


def run_reference_cuda(args, local_rank: int, quiet: bool = False) -> dict:
    """The reference's own kernels (oracle/_ref, compiled from its headers for sm_100a), same chain, unfused."""
    import ctypes
    from nemotron_infer_b200 import chain
    path = os.path.join(ROOT, "oracle", "_ref", "libnemotron_ref.so")
    if not os.path.exists(path):
        return {"impl": "reference-cuda", "unavailable": "oracle/_ref/libnemotron_ref.so was not built (reference checkout absent at build time)"}
    R = ctypes.CDLL(path)
    torch.cuda.set_device(local_rank)
    R.ref_set_device(local_rank)
    T = args.tokens
    cp = chain.ChainPass(T, f"cuda:{local_rank}", ids_dtype=torch.int64, seed=1234)
    b = cp.buf
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    sz, fl = ctypes.c_size_t, ctypes.c_float
    gs = chain.D_INNER // chain.N_GROUPS

    def one_pass():
        cur, other = b.hidden
        R.ref_embedding_i64(p(b.table), p(b.ids), p(cur), sz(T), 3136, None)
        n_m = 0
        for i, kind in enumerate(cp.schedule):
            if kind == "M":
                R.ref_rmsnorm_gated_bf16(p(b.y), p(b.z), p(b.gated_w[n_m]), p(b.gated_out), sz(T), sz(chain.D_INNER), sz(gs), fl(1e-5), None)
                n_m += 1
            elif kind == "-":
                R.ref_relu2_bf16(p(b.u), p(b.act), sz(T * chain.INTER), None)
            R.ref_add_bf16(p(cur), p(b.mixer_out[i % 2]), p(other), sz(T * chain.HIDDEN), None)
            R.ref_rmsnorm_bf16(p(other), p(b.normed), p(b.norm_w[i]), sz(T), sz(chain.HIDDEN), fl(1e-5), None)
            cur, other = other, cur

    for _ in range(3):
        one_pass()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = max(args.steps, 1)
    ev0.record()
    for _ in range(steps):
        one_pass()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / steps
    v = T / (ms * 1e-3)
    return {"impl": "reference-cuda", "value": round(v, 1), "unit": "tokens/s", "ms_per_step": round(ms, 4),
            "launches_per_step": 1 + 42 * 2 + 21 + 17, "tokens": T, "steps": steps,
            "hbm_gbs_on_fused_byte_model": round(v * chain.bytes_per_token(8) / 1e9, 1),
            "what": "nemotron_infer's ops/reduce.cuh, ops/elementwise.cuh, ops/embedding.cuh kernels, unmodified, "
                    "recompiled for sm_100a, legacy default stream, int64 ids, add and rmsnorm as separate launches"}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-cuda"])
    ap.add_argument("--tokens", type=int, default=GLOBAL_TOKENS, help="tokens of the ONE batch that is split over the GPUs")
    ap.add_argument("--eager", action="store_true", help="host-launch every kernel instead of replaying the captured pass")
    ap.add_argument("--no-weak", action="store_true", help="skip the extra weak-scaling figure (N > 1)")
    ap.add_argument("--no-per-op", action="store_true", help="skip the per-op figures at the config sizes (N = 1)")
    ap.add_argument("--parity-rows", type=int, default=256, help="rows per rank checked against the oracle after timing")
    ap.add_argument("--cpu-tokens", type=int, default=2048, help="token sample of the CPU legs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allgather", action=argparse.BooleanOptionalAction, default=True,
                    help="also time an NCCL all-gather of the output rows (N > 1), reported separately, never in value")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    # Libraries (NCCL's version banner, for one) write to stdout; keep stdout for the ONE JSON line.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj: dict) -> None:
        os.write(json_fd, (json.dumps(obj) + "\n").encode())

    if args.impl == "reference":
        if rank == 0:
            emit(run_reference_cpu(args, world))
        return
    if args.impl == "reference-cuda":
        if rank == 0:
            emit(run_reference_cuda(args, local_rank))
        return

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    try:
        out = run_b200(args, rank, world, local_rank)
        if rank == 0 and out is not None:
            emit(out)
    finally:
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
