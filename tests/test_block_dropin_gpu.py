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
