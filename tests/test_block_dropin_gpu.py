"""Block-level drop-in check: the reference's OWN MLP block (model/mlp_block.cuh, unmodified) compiled twice by
oracle/Makefile -- once on its own kernels, once on include/nemotron_b200_shim + libnemotron_b200.so -- must give
the golden block output of the reference's dump script within the reference's block-test tolerances
(tests/model/test_mlp_block.cu:124,150: fp32 1e-3, bf16 1.5e-1)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import ROOT, golden

pytestmark = pytest.mark.gpu


def _load(name):
    path = os.path.join(ROOT, "oracle", "_ref", name)
    if not os.path.exists(path):
        pytest.skip(f"{name} not built (needs the reference checkout at build time: make -C oracle blocks)")
    lib = ctypes.CDLL(path)
    lib.blk_set_device(torch.cuda.current_device())
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.fixture(scope="module")
def mlp_golden():
    d = golden("dump_mlp_block.npz")
    f = lambda k, *shape: torch.from_numpy(d[k].copy()).reshape(*shape).cuda()  # noqa: E731
    return dict(x=f("input", 8, 64), nw=f("block_norm_w", 64), up=f("up_proj_w", 256, 64),
                down=f("down_proj_w", 64, 256), want=f("expected", 8, 64))


@pytest.mark.parametrize("which", ["libref_mlp_stock.so", "libref_mlp_shim.so"])
def test_reference_mlp_block_matches_its_golden(built_lib, mlp_golden, which):
    lib, g = _load(which), mlp_golden
    before = built_lib.nmt_launch_count()
    out = torch.empty_like(g["x"])
    assert lib.blk_mlp_forward_fp32(_p(g["x"]), _p(g["nw"]), _p(g["up"]), _p(g["down"]), _p(out), 8, 64, 256) == 0
    torch.cuda.synchronize()
    lib.blk_reset_allocator()
    assert (out - g["want"]).abs().max().item() < 1e-3
    bf = torch.bfloat16
    outb = torch.empty(8, 64, dtype=bf, device="cuda")
    xb, upb, downb = g["x"].to(bf), g["up"].to(bf), g["down"].to(bf)
    assert lib.blk_mlp_forward_bf16(_p(xb), _p(g["nw"]), _p(upb), _p(downb), _p(outb), 8, 64, 256) == 0
    torch.cuda.synchronize()
    lib.blk_reset_allocator()
    assert (outb.float() - g["want"]).abs().max().item() < 1.5e-1
    launched = built_lib.nmt_launch_count() - before
    # the shim build runs rmsnorm, relu^2 and the residual add of both passes on this library: 6 launches
    assert launched == (6 if "shim" in which else 0)
    lib.blk_free_allocator()


def test_mlp_block_at_model_width_shim_equals_stock(built_lib):
    stock, shim = _load("libref_mlp_stock.so"), _load("libref_mlp_shim.so")
    M, H, I = 96, 3136, 12544
    g = torch.Generator(device="cuda").manual_seed(3)
    bf = torch.bfloat16
    x = torch.randn(M, H, generator=g, device="cuda").to(bf)
    nw = (1 + 0.1 * torch.randn(H, generator=g, device="cuda")).contiguous()
    up = (0.02 * torch.randn(I, H, generator=g, device="cuda")).to(bf)
    down = (0.02 * torch.randn(H, I, generator=g, device="cuda")).to(bf)
    outs = []
    for lib in (stock, shim):
        out = torch.empty(M, H, dtype=bf, device="cuda")
        assert lib.blk_mlp_forward_bf16(_p(x), _p(nw), _p(up), _p(down), _p(out), M, H, I) == 0
        torch.cuda.synchronize()
        lib.blk_free_allocator()
        outs.append(out.float())
    # Same GEMMs, same inputs; the norm may differ by one bf16 ulp per element (association order), which the
    # 3136-long dot products average out: the block outputs agree to bf16 resolution.
    rel = ((outs[0] - outs[1]).norm() / outs[0].norm()).item()
    assert rel < 5e-3, rel
    assert (outs[0] - outs[1]).abs().max().item() < 0.15


@pytest.fixture(scope="module")
def mamba_golden():
    d = golden("dump_mamba_block.npz")
    f = lambda k: torch.from_numpy(d[k].copy()).cuda()  # noqa: E731
    names = ["input", "block_norm_w", "in_proj_w", "conv1d_w", "conv1d_b", "A_log", "D", "dt_bias", "gnorm_w", "out_proj_w"]
    g = {k: f(k) for k in names}
    g["want"] = f("expected").reshape(24, 64)
    return g


def _run_mamba(lib, g, bf16):
    bf = torch.bfloat16
    cast = (lambda t: t.to(bf)) if bf16 else (lambda t: t)
    x, in_proj, out_proj = cast(g["input"]), cast(g["in_proj_w"]), cast(g["out_proj_w"])
    out = torch.empty(24, 64, dtype=x.dtype, device="cuda")
    fn = lib.blk_mamba_forward_bf16 if bf16 else lib.blk_mamba_forward_fp32
    rc = fn(_p(x), _p(g["block_norm_w"]), _p(in_proj), _p(g["conv1d_w"]), _p(g["conv1d_b"]), _p(g["A_log"]), _p(g["D"]),
            _p(g["dt_bias"]), _p(g["gnorm_w"]), _p(out_proj), _p(out), 1, 24)
    torch.cuda.synchronize()
    lib.blk_free_allocator()
    assert rc == 0
    return out.float()


def test_reference_mamba_block_on_the_drop_in_matches_its_golden(built_lib, mamba_golden):
    """The reference's Mamba-2 block, unchanged, with its RMSNorm, gated RMSNorm and residual add served by this
    library, reproduces the golden of tools/dump_mamba_block.py within the reference's own block-test
    tolerances (tests/model/test_mamba_block.cu: fp32 1e-3, bf16 1.5e-1)."""
    shim = _load("libref_mamba_shim.so")
    before = built_lib.nmt_launch_count()
    out32 = _run_mamba(shim, mamba_golden, bf16=False)
    assert (out32 - mamba_golden["want"]).abs().max().item() < 1e-3
    out16 = _run_mamba(shim, mamba_golden, bf16=True)
    assert (out16 - mamba_golden["want"]).abs().max().item() < 1.5e-1
    assert built_lib.nmt_launch_count() - before == 6        # norm, gated norm, add: once per precision


def test_reference_mamba_block_on_its_own_kernels_is_reported(mamba_golden):
    """Same block on the reference's own kernels.  Its gated RMSNorm reduces through a shared-memory word that all
    32 lanes of a warp store to (ops/reduce.cuh:280-287); where that race resolves wrongly the block misses its
    own golden.  Recorded, not asserted: the outcome belongs to the reference, not to this library."""
    stock = _load("libref_mamba_stock.so")
    for bf16, tol in ((False, 1e-3), (True, 1.5e-1)):
        err = (_run_mamba(stock, mamba_golden, bf16) - mamba_golden["want"]).abs().max().item()
        print(f"reference mamba block on its own kernels, {'bf16' if bf16 else 'fp32'}: max abs err {err:.3e} "
              f"(reference tolerance {tol:g}) -> {'within' if err < tol else 'OUTSIDE'}")
