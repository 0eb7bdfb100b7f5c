"""Generates the golden fixtures in this directory FROM THE REFERENCE'S OWN CODE.

Run where the reference checkout is available (its location comes from --reference or the REFERENCE_ROOT
environment variable):

    python tests/golden/make_golden.py --reference <path to nemotron_infer>

Two sources, neither of which copies reference text into this repository:

1. The reference's golden emitters tools/dump_mlp_block.py and
   tools/dump_mamba_block.py are executed UNMODIFIED from a scratch copy (they
   write next to themselves and the mounted reference is read-only).  From their
   raw float32 dumps we keep the stage tensors that pin the hot-path ops:
     mlp:   input, block_norm_w -> normed (RMSNorm);  up -> act (relu^2);
            input + down -> expected (residual add); up_proj_w / down_proj_w for the whole-block check
     mamba: input, block_norm_w -> normed;  scan_y, gate, gnorm_w -> gnormed (gated RMSNorm);
            xbc, conv1d_w, conv1d_b -> xbc_conv (causal conv1d + SiLU)
2. The functions `plain_rmsnorm` and `gated_rmsnorm` are lifted out of
   tools/dump_mamba_block.py with `ast` at run time and evaluated on the seeded
   inputs of the benchmark configurations (small row counts, full widths), with
   the bf16 conventions of the hot path (bf16 storage, fp32 math, residual sum
   rounded before the norm).  relu^2 / residual add / embedding use the same
   torch expressions the emitters use (F.relu(u).pow(2), a + b, F.embedding).

Outputs: dump_mlp_block.npz, dump_mamba_block.npz, dump_attention_block.npz (tools/dump_attention_block.py, run
unmodified the same way: input, the five weights, normed, expected), cfg_bf16.npz, cfg0_fp32.npz.
bf16 tensors are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import argparse
import ast
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import torch_golden as og  # noqa: E402  (only for the seeded input generators)


def run_dump(reference: str, script: str, sub: str) -> dict[str, np.ndarray]:
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, "tools"))
        shutil.copy(os.path.join(reference, "tools", script), os.path.join(tmp, "tools", script))
        subprocess.run([sys.executable, os.path.join(tmp, "tools", script)], check=True,
                       stdout=subprocess.DEVNULL)
        d = os.path.join(tmp, "tests", "data", sub)
        out = {f[:-4]: np.fromfile(os.path.join(d, f), dtype="<f4") for f in os.listdir(d) if f.endswith(".bin")}
        out["meta"] = np.array(open(os.path.join(d, "meta.txt")).read())
        return out


def lift_functions(path: str, names: list[str]) -> dict:
    tree = ast.parse(open(path).read())
    ns = {"torch": torch, "F": F}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    missing = [n for n in names if n not in ns]
    if missing:
        raise RuntimeError(f"{path} no longer defines {missing}")
    return ns


def bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.bfloat16
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"),
                    help="the reference checkout (default: $REFERENCE_ROOT, else a directory named 'reference' beside this repository)")
    a = ap.parse_args()
    torch.set_num_threads(1)          # fixed summation order for the fixtures

    mlp = run_dump(a.reference, "dump_mlp_block.py", "mlp_block")
    keep = ["input", "block_norm_w", "up_proj_w", "down_proj_w", "normed", "up", "act", "down", "expected", "meta"]
    np.savez_compressed(os.path.join(HERE, "dump_mlp_block.npz"), **{k: mlp[k] for k in keep})

    mam = run_dump(a.reference, "dump_mamba_block.py", "mamba_block")
    keep = ["input", "block_norm_w", "in_proj_w", "conv1d_w", "conv1d_b", "A_log", "D", "dt_bias", "gnorm_w", "out_proj_w",
            "normed", "xbc", "xbc_conv", "scan_y", "gate", "gnormed", "mixer_out", "expected", "meta"]
    np.savez_compressed(os.path.join(HERE, "dump_mamba_block.npz"), **{k: mam[k] for k in keep})

    att = run_dump(a.reference, "dump_attention_block.py", "attention_block")
    keep = ["input", "block_norm_w", "q_proj_w", "k_proj_w", "v_proj_w", "o_proj_w", "normed", "expected", "meta"]
    np.savez_compressed(os.path.join(HERE, "dump_attention_block.npz"), **{k: att[k] for k in keep})

    ref = lift_functions(os.path.join(a.reference, "tools", "dump_mamba_block.py"), ["plain_rmsnorm", "gated_rmsnorm"])
    plain_rmsnorm, gated_rmsnorm = ref["plain_rmsnorm"], ref["gated_rmsnorm"]
    bf = torch.bfloat16
    fx: dict[str, np.ndarray] = {}

    # cfg1: residual add + RMSNorm, width 3136, first 6 rows of the seeded stream.
    x, r, w = og.cfg1_inputs(6)
    res = (x.float() + r.float()).to(bf)                       # residual + mixer_out, stored as bf16
    fx.update(cfg1_x=bits(x), cfg1_r=bits(r), cfg1_w=w.numpy(), cfg1_out_res=bits(res),
              cfg1_out=bits(plain_rmsnorm(res, w, 1e-5).to(bf)),
              cfg1_plain_out=bits(plain_rmsnorm(x, w, 1e-5).to(bf)))
    # cfg2: gated RMSNorm at 6144 / 768 and at the model's 7680 / 960.
    for tag, cols, gs in (("cfg2", 6144, 768), ("cfg2m", 7680, 960)):
        y, z, w = og.cfg2_inputs(4, cols)
        fx.update({f"{tag}_y": bits(y), f"{tag}_z": bits(z), f"{tag}_w": w.numpy(),
                   f"{tag}_out": bits(gated_rmsnorm(y, w, z, gs, 1e-5).to(bf))})
    # cfg3: relu^2 at width 12544.
    u = og.cfg3_inputs(3)
    fx.update(cfg3_u=bits(u), cfg3_out=bits(F.relu(u.float()).pow(2).to(bf)))
    # cfg4: embedding gather, width 3136, a 64-row table (ids include both ends and repeats).
    table, ids = og.cfg4_inputs(40, vocab=64)
    ids[:4] = torch.tensor([0, 63, 63, 0], dtype=ids.dtype)
    fx.update(cfg4_table=bits(table), cfg4_ids=ids.numpy().astype(np.int64),
              cfg4_out=bits(F.embedding(ids.long(), table)))
    np.savez_compressed(os.path.join(HERE, "cfg_bf16.npz"), **fx)

    # cfg0: fp32 RMSNorm on the CPU golden formulation; first 8 rows of x[512, 3136].
    x, w = og.cfg0_inputs()
    np.savez_compressed(os.path.join(HERE, "cfg0_fp32.npz"), x=x[:8].numpy(), w=w.numpy(),
                        out=plain_rmsnorm(x[:8], w, 1e-5).numpy())
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
