"""Helpers shared by the block-level GPU tests: the three builds of oracle/ref_blocks_wrapper.cu (the reference's
own blocks on its kernels, on the drop-in headers, and in their fused forms), fixtures from the reference's dump
scripts, and per-row e4m3 weights."""
import ctypes
import os

import pytest
import torch

from conftest import ROOT, golden
from oracle import torch_golden as og

BF = torch.bfloat16
_LIBS = {}


def load_blocks(kind):
    """kind: 'stock' | 'shim' | 'fused'."""
    if kind in _LIBS:
        return _LIBS[kind]
    path = os.path.join(ROOT, "oracle", "_ref", f"libref_blocks_{kind}.so")
    if not os.path.exists(path):
        pytest.skip(f"{os.path.basename(path)} not built (needs the reference checkout at build time: make -C oracle blocks)")
    lib = ctypes.CDLL(path)
    lib.blk_set_device(torch.cuda.current_device())
    _LIBS[kind] = lib
    return lib


def p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def fusion_counters(nmt):
    a, b = ctypes.c_int64(0), ctypes.c_int64(0)
    assert nmt.nmt_fusion_counters(ctypes.byref(a), ctypes.byref(b)) == 0
    return a.value, b.value


def rel_l2(got, want):
    got, want = got.float(), want.float()
    return ((got - want).norm() / want.norm().clamp_min(1e-12)).item()


def fp8_rows(w):
    """Per-output-row e4m3 weights and scales, as the reference tests quantise them (tests/ops/test_gemm.cu:521-531)."""
    q, s = og.quant_weight_perrow(w.float().cpu())
    return q.cuda(), s.cuda()


def mlp_fixture():
    d = golden("dump_mlp_block.npz")
    f = lambda k, *shape: torch.from_numpy(d[k].copy()).reshape(*shape).cuda()  # noqa: E731
    return dict(x=f("input", 8, 64), nw=f("block_norm_w", 64), up=f("up_proj_w", 256, 64),
                down=f("down_proj_w", 64, 256), want=f("expected", 8, 64))


MAMBA_KEYS = ["input", "block_norm_w", "in_proj_w", "conv1d_w", "conv1d_b", "A_log", "D", "dt_bias", "gnorm_w", "out_proj_w"]
# tools/dump_mamba_block.py: HIDDEN 64, H 4, P 16, N 16, G 2, K 4, S 24
MAMBA = dict(HIDDEN=64, H=4, P=16, N=16, G=2, K=4, S=24, INTER=64, CONV_DIM=128, PROJ=196)


def mamba_fixture():
    d = golden("dump_mamba_block.npz")
    g = {k: torch.from_numpy(d[k].copy()).cuda() for k in MAMBA_KEYS}
    g["want"] = torch.from_numpy(d["expected"].copy()).reshape(24, 64).cuda()
    return g


def attn_fixture():
    d = golden("dump_attention_block.npz")
    f = lambda k, *shape: torch.from_numpy(d[k].copy()).reshape(*shape).cuda()  # noqa: E731
    # tools/dump_attention_block.py: HIDDEN 256, 4 query heads, 2 KV heads, head 128, S 40
    return dict(x=f("input", 40, 256), nw=f("block_norm_w", 256), q=f("q_proj_w", 512, 256), k=f("k_proj_w", 256, 256),
                v=f("v_proj_w", 256, 256), o=f("o_proj_w", 256, 512), want=f("expected", 40, 256))


def run_mlp_bf16(lib, x, nw, up, down):
    out = torch.empty_like(x)
    assert lib.blk_mlp_forward_bf16(p(x), p(nw), p(up), p(down), p(out), x.shape[0], x.shape[1], up.shape[0]) == 0
    return out


def run_mamba_bf16(lib, g, x=None, S=None, conv_state=None, ssm_state=None):
    x = g["input"].to(BF) if x is None else x
    S = x.numel() // 64 if S is None else S
    out = torch.empty(S, 64, dtype=BF, device="cuda")
    in_proj, out_proj = g["in_proj_w"].to(BF), g["out_proj_w"].to(BF)      # named: p() keeps an address, not the tensor
    rc = lib.blk_mamba_forward_bf16(p(x), p(g["block_norm_w"]), p(in_proj), p(g["conv1d_w"]), p(g["conv1d_b"]),
                                    p(g["A_log"]), p(g["D"]), p(g["dt_bias"]), p(g["gnorm_w"]), p(out_proj),
                                    p(out), 1, S, p(conv_state), p(ssm_state))
    torch.cuda.synchronize()
    assert rc == 0
    return out
