"""Per-op timing of the hot-path kernels at the benchmark shapes (the counterpart of the reference's
in-test perf fixtures, tests/ops/test_reduce.cu:362-463, test_elementwise.cu:534-701, test_embedding.cu:196-221).

    python -m nemotron_infer_b200.microbench [--op all|add_rmsnorm|rmsnorm|gated|gated_model|relu2|add|embedding|chain]
                                             [--tokens T] [--reps R] [--warmup W] [--tune key=value ...]
                                             [--graph] [--fixed-cost]

Each op runs on buffer sets that are rotated so that consecutive launches never touch the same bytes and
the sets together exceed twice the 126 MB L2.  Timing is by CUDA events on the launching stream around
BATCHES of back-to-back launches (--batch, default 10), so a figure includes the launch gaps a real
sequence of kernels has but not the cost of an event record between every two launches.  One JSON line
per op: median / min microseconds per launch, algorithmic GB/s, tokens/s, and the fraction of the nominal
8000 GB/s and of the measured copy peak.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from . import _lib, ops

BF = torch.bfloat16
NOMINAL_GBS = 8000.0
L2_BYTES = 126 * 1024 * 1024

# op -> (default tokens of the benchmark configuration, algorithmic bytes per token)
SHAPES = {
    "add_rmsnorm": (8192, 4 * 3136 * 2),
    "rmsnorm": (8192, 2 * 3136 * 2),
    "gated": (16384, 3 * 6144 * 2),          # 8 groups of 768
    "gated_model": (16384, 3 * 7680 * 2),    # the model's own shape: 8 groups of 960
    "relu2": (8192, 2 * 12544 * 2),
    "add": (8192, 3 * 3136 * 2),
    "embedding": (65536, 2 * 3136 * 2 + 4),
    # rows too wide for one CTA's registers (not a model shape): bulk-staged row shares + cluster reduction
    "add_rmsnorm_wide": (2048, 4 * 65536 * 2),
    "rmsnorm_wide": (2048, 2 * 65536 * 2),
    "conv1d_split": (16384, 9728 * (2 + 2)),                     # xBC in, x | B | C out (Mamba-2 conv1d + SiLU)
    # single-token decode projections (weight streaming): "tokens" is the number of output rows N here
    "gemv_up": (12544, 3136),        # up_proj   N = 12544, K = 3136: 3136 weight bytes per output row
    "gemv_down": (3136, 12544),      # down_proj N = 3136,  K = 12544
    "gemv_out": (3136, 7680),        # Mamba-2 out_proj N = 3136, K = 7680 (in_proj: --op gemv_up --tokens 17504)
    "gemv_o": (3136, 5120),          # attention o_proj N = 3136, K = 5120 (q / k / v: --op gemv_up --tokens 5120 / 1024)
    "ssm_step": (1, 2 * 96 * 80 * 128 * 4),   # per sequence: the fp32 state [96, 80, 128] read and written once
    "sdpa_decode": (512, 2 * 8 * 128 * 2),    # per cached token: one K and one V row of each of the 8 KV heads
    # e4m3 activation quantisation (the step after the norm / activation in the FP8 blocks)
    "quantize_fp8": (8192, 3136 * (2 + 2 + 1)),                  # amax pass + quantising pass over [T, 3136]
    "add_rmsnorm_quant_fp8": (8192, 3136 * (2 + 2 + 2 + 2 + 1)),  # x, r -> out_res ; out_res -> e4m3
    "relu2_quant_fp8": (8192, 12544 * (2 + 2 + 1)),              # u twice in, e4m3 out
    "gated_quant_fp8": (16384, 6144 * (2 + 2 + 2 + 2 + 1)),      # y, z -> bf16 out (+max) ; bf16 out -> e4m3
}


def measured_peak() -> float | None:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"])
    except Exception:
        return None


def make_case(op: str, T: int, dev):
    rn = lambda *s: torch.randn(*s, device=dev)  # noqa: E731
    if op in ("add_rmsnorm", "rmsnorm", "add", "add_rmsnorm_wide", "rmsnorm_wide"):
        cols = 65536 if op.endswith("_wide") else 3136
        x, r = rn(T, cols).to(BF), rn(T, cols).to(BF)
        w = 1 + 0.1 * rn(cols)
        o1, o2 = torch.empty_like(x), torch.empty_like(x)
        if op.startswith("add_rmsnorm"):
            return lambda: ops.add_rmsnorm(x, r, w, out_res=o1, out=o2)
        if op.startswith("rmsnorm"):
            return lambda: ops.rmsnorm(x, w, out=o1)
        return lambda: ops.add(x, r, out=o1)
    if op in ("gated", "gated_model"):
        cols, gs = (6144, 768) if op == "gated" else (7680, 960)
        y, z = rn(T, cols).to(BF), rn(T, cols).to(BF)
        w = 1 + 0.1 * rn(cols)
        o = torch.empty_like(y)
        return lambda: ops.rmsnorm_gated(y, z, w, gs, out=o)
    if op == "relu2":
        u = (2 * rn(T, 12544)).to(BF)
        o = torch.empty_like(u)
        return lambda: ops.relu2(u, out=o)
    if op.startswith("gemv"):
        K = SHAPES[op][1]
        W = (rn(T, K) * 20).clamp(-448, 448).to(torch.float8_e4m3fn)
        x = rn(K).to(BF)
        sc = torch.rand(T, device=dev) * 0.01
        y = torch.empty(T, dtype=BF, device=dev)
        return lambda: ops.gemv_w8a16(x, W, sc, out=y)
    if op == "sdpa_decode":
        H_Q, H_KV = 40, 8
        q, kn, vn = rn(H_Q, 128).to(BF), rn(H_KV, 128).to(BF), rn(H_KV, 128).to(BF)
        k, v = rn(H_KV, T + 1, 128).to(BF), rn(H_KV, T + 1, 128).to(BF)
        o = torch.empty(H_Q, 128, dtype=BF, device=dev)
        ws = torch.empty(max(16, _lib.load().nmt_sdpa_decode_workspace_bytes(T, H_Q)), dtype=torch.uint8, device=dev)
        return lambda: ops.sdpa_decode(q, k, v, kn, vn, T, out=o, workspace=ws)
    if op == "ssm_step":
        H, P, N, G = 96, 80, 128, 8
        x, dt = rn(T, H * P).to(BF), (rn(T, H) - 1).to(BF)
        A_log, D, bias = torch.log(1 + 15 * torch.rand(H, device=dev)), 1 + 0.1 * rn(H), 0.5 * rn(H)
        Bm, Cm = rn(T, G, N).to(BF), rn(T, G, N).to(BF)
        state = 0.3 * rn(T, H, P, N)
        y = torch.empty(T, H * P, dtype=BF, device=dev)
        return lambda: ops.ssm_decode_step(x, dt, A_log, Bm, Cm, D, state, dt_bias=bias, out=y)
    if op == "conv1d_split":
        xbc = rn(1, T, 9728).to(BF)
        w, b = 0.2 * rn(9728, 4), 0.1 * rn(9728)
        return lambda: ops.causal_conv1d_silu(xbc, w, b, split=(7680, 1024, 1024))
    if op == "quantize_fp8":
        x = rn(T, 3136).to(BF)
        q = torch.empty(T, 3136, dtype=torch.float8_e4m3fn, device=dev)
        return lambda: ops.quantize_fp8(x, out=q)
    if op == "relu2_quant_fp8":
        u = (2 * rn(T, 12544)).to(BF)
        q = torch.empty(T, 12544, dtype=torch.float8_e4m3fn, device=dev)
        return lambda: ops.quantize_fp8(u, out=q, relu2_first=True)
    if op == "gated_quant_fp8":
        y, z = rn(T, 6144).to(BF), rn(T, 6144).to(BF)
        w = 1 + 0.1 * rn(6144)
        o = torch.empty_like(y)
        q = torch.empty(T, 6144, dtype=torch.float8_e4m3fn, device=dev)
        return lambda: ops.rmsnorm_gated_quant_fp8(y, z, w, 768, out_bf16=o, out=q)
    if op == "add_rmsnorm_quant_fp8":
        x, r = rn(T, 3136).to(BF), rn(T, 3136).to(BF)
        w = 1 + 0.1 * rn(3136)
        o1 = torch.empty_like(x)
        q = torch.empty(T, 3136, dtype=torch.float8_e4m3fn, device=dev)
        ws = ops.fp8_workspace(T, dev)
        return lambda: ops.rmsnorm_quant_fp8(x, w, r=r, out_res=o1, out=q, workspace=ws)
    if op == "embedding":
        table = make_case.table if getattr(make_case, "table", None) is not None else (0.02 * rn(131072, 3136)).to(BF)
        make_case.table = table
        ids = torch.randint(0, 131072, (T,), device=dev, dtype=torch.int32)
        o = torch.empty(T, 3136, dtype=BF, device=dev)
        return lambda: ops.embedding(table, ids, out=o)
    raise ValueError(op)


def run_op(op: str, T: int, reps: int, warmup: int, dev, batch: int = 10, graph: bool = False) -> dict:
    _, bpt = SHAPES[op]
    nbytes = bpt * T
    # enough buffer sets that a launch never finds its tensors in L2 (at most 8; the small per-sequence state of the SSM
    # step, which in a decode step is evicted by 3 GB of weights between two uses, gets as many as that takes)
    nsets = max(2, min(48 if op in ("ssm_step", "sdpa_decode") else 8, -(-2 * L2_BYTES // max(nbytes, 1)) + 1))
    if op in ("ssm_step", "sdpa_decode"):
        batch = max(batch, nsets)                 # one timed interval walks every set once
    fns = [make_case(op, T, dev) for _ in range(nsets)]
    for i in range(max(warmup, 3)):
        fns[i % nsets]()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    if graph:
        # Kernels of a few microseconds are bound by the host's launch rate when driven from Python; a CUDA graph
        # of one batch (rotating over the buffer sets) shows the device-side rate a captured decode loop gets.
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for k in range(batch):
                fns[k % nsets]()
        g.replay()
        torch.cuda.synchronize()
        evs[0].record()
        for i in range(reps):
            g.replay()
            evs[i + 1].record()
    else:
        evs[0].record()
        n = 0
        for i in range(reps):
            for _ in range(batch):
                fns[n % nsets]()
                n += 1
            evs[i + 1].record()
    torch.cuda.synchronize()
    us = sorted(evs[i].elapsed_time(evs[i + 1]) * 1e3 / batch for i in range(reps))
    med, mn = statistics.median(us), us[0]
    peak = measured_peak()
    gbs = nbytes / med / 1e3
    return {"op": op, "tokens": T, "bytes_per_token": bpt, "buffer_sets": nsets, "reps": reps, "batch": batch, "graph": graph,
            "median_us": round(med, 2), "min_us": round(mn, 2), "gbs": round(gbs, 1),
            "gbs_best": round(nbytes / mn / 1e3, 1), "tokens_per_s": round(T / med * 1e6, 0),
            "frac_of_nominal_8000": round(gbs / NOMINAL_GBS, 4),
            "frac_of_measured_peak": round(gbs / peak, 4) if peak else None}


def run_fixed_cost(op: str, T: int, reps: int, dev) -> dict:
    """Separates a launch's steady cost from what does not grow with the number of launches: CUDA graphs of
    n = 1 ... 32 back-to-back launches (rotating buffer sets), median replay time, least-squares line
    time(n) = fixed + n * per_launch."""
    pts = {}
    for n in (1, 2, 4, 8, 16, 32):
        r = run_op(op, T, reps, 3, dev, n, True)
        pts[n] = r["median_us"] * n
    xs, ys = list(pts), [pts[n] for n in pts]
    mx, my = sum(xs) / len(xs), sum(ys) / len(ys)
    slope = sum((a - mx) * (b - my) for a, b in zip(xs, ys)) / sum((a - mx) ** 2 for a in xs)
    nbytes = SHAPES[op][1] * T
    return {"op": op, "tokens": T, "us_by_launches": {str(k): round(v, 1) for k, v in pts.items()},
            "per_launch_us": round(slope, 2), "fixed_us": round(my - slope * mx, 2),
            "steady_gbs": round(nbytes / slope / 1e3, 1), "steady_frac_of_nominal_8000": round(nbytes / slope / 1e3 / NOMINAL_GBS, 4)}


def run_chain(T: int, reps: int, dev) -> dict:
    """Latency of the whole 81-launch pass at a (small) token count: host-launched vs one CUDA-graph replay."""
    from . import chain
    cp = chain.ChainPass(T, dev, vocab=chain.VOCAB if T >= 4096 else 8192)
    out = {"op": "chain", "tokens": T, "launches_per_pass": cp.launches_per_pass}
    cp.capture()
    for name, fn in (("eager", cp.run), ("graph", cp.replay)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        out[f"{name}_us_per_pass"] = round(us, 1)
        out[f"{name}_tokens_per_s"] = round(T / us * 1e6, 0)
        out[f"{name}_gbs"] = round(chain.bytes_per_token(4) * T / us / 1e3, 1)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="all")
    ap.add_argument("--tokens", type=int, default=0, help="0 = the benchmark configuration's token count")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=10, help="back-to-back launches per timed interval")
    ap.add_argument("--graph", action="store_true", help="capture each batch in a CUDA graph (default for the gemv ops)")
    ap.add_argument("--fixed-cost", action="store_true", help="graphs of 1 ... 32 launches: per-launch cost and fixed cost of each op")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--tune", action="append", default=[], metavar="key=value")
    a = ap.parse_args()
    torch.cuda.set_device(a.device)
    _lib.check(_lib.load().nmt_set_device(a.device), "nmt_set_device")
    for kv in a.tune:
        k, v = kv.split("=")
        ops.tune(k, int(v))
    names = list(SHAPES) if a.op == "all" else a.op.split(",")
    for op in names:
        if op == "chain":
            print(json.dumps(run_chain(a.tokens or 64, a.reps, f"cuda:{a.device}")), flush=True)
            continue
        T = a.tokens or SHAPES[op][0]
        if a.fixed_cost:
            print(json.dumps(run_fixed_cost(op, T, a.reps, f"cuda:{a.device}")), flush=True)
            torch.cuda.empty_cache()
            continue
        print(json.dumps(run_op(op, T, a.reps, a.warmup, f"cuda:{a.device}", a.batch, a.graph or op.startswith("gemv") or op in ("ssm_step", "sdpa_decode"))), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
