"""Per-op timing of the hot-path kernels at the benchmark shapes (the counterpart of the reference's
in-test perf fixtures, tests/ops/test_reduce.cu:362-463, test_elementwise.cu:534-701, test_embedding.cu:196-221).

    python -m nemotron_infer_b200.microbench [--op all|add_rmsnorm|rmsnorm|gated|gated_model|relu2|add|embedding]
                                             [--tokens T] [--reps R] [--warmup W] [--tune key=value ...]

Each op runs on buffer sets that are rotated so that consecutive launches never touch the same bytes and
the sets together exceed twice the 126 MB L2; every launch is bracketed by CUDA events on the launching
stream.  One JSON line per op: median / min microseconds, algorithmic GB/s, tokens/s, and the fraction of
the nominal 8000 GB/s and of the measured copy peak.
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
}


def measured_peak() -> float | None:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"])
    except Exception:
        return None


def make_case(op: str, T: int, dev):
    rn = lambda *s: torch.randn(*s, device=dev)  # noqa: E731
    if op in ("add_rmsnorm", "rmsnorm", "add"):
        x, r = rn(T, 3136).to(BF), rn(T, 3136).to(BF)
        w = 1 + 0.1 * rn(3136)
        o1, o2 = torch.empty_like(x), torch.empty_like(x)
        if op == "add_rmsnorm":
            return lambda: ops.add_rmsnorm(x, r, w, out_res=o1, out=o2)
        if op == "rmsnorm":
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
    if op == "embedding":
        table = make_case.table if getattr(make_case, "table", None) is not None else (0.02 * rn(131072, 3136)).to(BF)
        make_case.table = table
        ids = torch.randint(0, 131072, (T,), device=dev, dtype=torch.int32)
        o = torch.empty(T, 3136, dtype=BF, device=dev)
        return lambda: ops.embedding(table, ids, out=o)
    raise ValueError(op)


def run_op(op: str, T: int, reps: int, warmup: int, dev) -> dict:
    _, bpt = SHAPES[op]
    nbytes = bpt * T
    nsets = max(2, min(8, -(-2 * L2_BYTES // max(nbytes, 1)) + 1))
    fns = [make_case(op, T, dev) for _ in range(nsets)]
    for i in range(max(warmup, 3)):
        fns[i % nsets]()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    evs[0].record()
    for i in range(reps):
        fns[i % nsets]()
        evs[i + 1].record()
    torch.cuda.synchronize()
    us = sorted(evs[i].elapsed_time(evs[i + 1]) * 1e3 for i in range(reps))
    med, mn = statistics.median(us), us[0]
    peak = measured_peak()
    gbs = nbytes / med / 1e3
    return {"op": op, "tokens": T, "bytes_per_token": bpt, "buffer_sets": nsets, "reps": reps,
            "median_us": round(med, 2), "min_us": round(mn, 2), "gbs": round(gbs, 1),
            "gbs_best": round(nbytes / mn / 1e3, 1), "tokens_per_s": round(T / med * 1e6, 0),
            "frac_of_nominal_8000": round(gbs / NOMINAL_GBS, 4),
            "frac_of_measured_peak": round(gbs / peak, 4) if peak else None}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="all")
    ap.add_argument("--tokens", type=int, default=0, help="0 = the benchmark configuration's token count")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
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
        T = a.tokens or SHAPES[op][0]
        print(json.dumps(run_op(op, T, a.reps, a.warmup, f"cuda:{a.device}")), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
