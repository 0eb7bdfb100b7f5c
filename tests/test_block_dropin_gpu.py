"""Block-level drop-in check: the reference's OWN blocks (model/{mlp,mamba,attention}_block.cuh, unmodified), compiled
by oracle/Makefile on their own kernels ("stock"), on include/nemotron_b200_shim + libnemotron_b200.so ("shim") and
with model/blocks_b200.cuh pre-included ("fused"), must give the golden block output of the reference's dump scripts
within the reference's block-test tolerances (tests/model/test_mlp_block.cu:124,150, test_mamba_block.cu,
test_attention_block.cu:129,156: fp32 1e-3 / 2e-3, bf16 1.5e-1 / 2e-1)."""
import pytest
import torch

from blocks_common import BF, attn_fixture, load_blocks, mamba_fixture, mlp_fixture, p, rel_l2, run_mamba_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mlp_golden():
    return mlp_fixture()


@pytest.fixture(scope="module")
def mamba_golden():
    return mamba_fixture()


@pytest.fixture(scope="module")
def attn_golden():
    return attn_fixture()


@pytest.mark.parametrize("which", ["stock", "shim", "fused"])
def test_reference_mlp_block_matches_its_golden(built_lib, mlp_golden, which):
    lib, g = load_blocks(which), mlp_golden
    before = built_lib.nmt_launch_count()
    out = torch.empty_like(g["x"])
    assert lib.blk_mlp_forward_fp32(p(g["x"]), p(g["nw"]), p(g["up"]), p(g["down"]), p(out), 8, 64, 256) == 0
    torch.cuda.synchronize()
    lib.blk_reset_allocator()
    assert (out - g["want"]).abs().max().item() < 1e-3
    outb = torch.empty(8, 64, dtype=BF, device="cuda")
    xb, upb, downb = g["x"].to(BF), g["up"].to(BF), g["down"].to(BF)
    assert lib.blk_mlp_forward_bf16(p(xb), p(g["nw"]), p(upb), p(downb), p(outb), 8, 64, 256) == 0
    torch.cuda.synchronize()
    lib.blk_reset_allocator()
    assert (outb.float() - g["want"]).abs().max().item() < 1.5e-1
    launched = built_lib.nmt_launch_count() - before
    # on the drop-in, rmsnorm, relu^2 and the residual add of both passes run on this library: 6 launches
    assert launched == (0 if which == "stock" else 6)
    lib.blk_free_allocator()


def test_mlp_block_at_model_width_shim_equals_stock(built_lib):
    stock, shim = load_blocks("stock"), load_blocks("shim")
    M, H, I = 96, 3136, 12544
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(M, H, generator=g, device="cuda").to(BF)
    nw = (1 + 0.1 * torch.randn(H, generator=g, device="cuda")).contiguous()
    up = (0.02 * torch.randn(I, H, generator=g, device="cuda")).to(BF)
    down = (0.02 * torch.randn(H, I, generator=g, device="cuda")).to(BF)
    outs = []
    for lib in (stock, shim):
        out = torch.empty(M, H, dtype=BF, device="cuda")
        assert lib.blk_mlp_forward_bf16(p(x), p(nw), p(up), p(down), p(out), M, H, I) == 0
        torch.cuda.synchronize()
        lib.blk_free_allocator()
        outs.append(out.float())
    # Same GEMMs, same inputs; the norm may differ by one bf16 ulp per element (association order), which the
    # 3136-long dot products average out: the block outputs agree to bf16 resolution.
    assert rel_l2(outs[1], outs[0]) < 5e-3
    assert (outs[0] - outs[1]).abs().max().item() < 0.15


def _run_mamba_fp32(lib, g):
    out = torch.empty(24, 64, device="cuda")
    rc = lib.blk_mamba_forward_fp32(p(g["input"]), p(g["block_norm_w"]), p(g["in_proj_w"]), p(g["conv1d_w"]), p(g["conv1d_b"]),
                                    p(g["A_log"]), p(g["D"]), p(g["dt_bias"]), p(g["gnorm_w"]), p(g["out_proj_w"]), p(out), 1, 24)
    torch.cuda.synchronize()
    lib.blk_free_allocator()
    assert rc == 0
    return out


@pytest.mark.parametrize("which", ["shim", "fused"])
def test_reference_mamba_block_on_the_drop_in_matches_its_golden(built_lib, mamba_golden, which):
    """The reference's Mamba-2 block with its RMSNorm, gated RMSNorm and residual add served by this library (and, in
    the fused form, its conv1d + SiLU writing x | B | C directly) reproduces the golden of tools/dump_mamba_block.py
    within the reference's own block-test tolerances (tests/model/test_mamba_block.cu: fp32 1e-3, bf16 1.5e-1)."""
    lib = load_blocks(which)
    before = built_lib.nmt_launch_count()
    out32 = _run_mamba_fp32(lib, mamba_golden)
    assert (out32 - mamba_golden["want"]).abs().max().item() < 1e-3
    out16 = run_mamba_bf16(lib, mamba_golden)
    torch.cuda.synchronize()
    lib.blk_free_allocator()
    assert (out16.float() - mamba_golden["want"]).abs().max().item() < 1.5e-1
    # norm, gated norm, add once per precision; the fused bf16 form adds the split-fused conv1d
    assert built_lib.nmt_launch_count() - before == (6 if which == "shim" else 7)


def test_fused_mamba_prefill_equals_the_unfused_block_bit_for_bit(mamba_golden):
    """conv1d + SiLU with the x | B | C split fused must not change a byte of the block output or of the conv state."""
    outs = []
    for which in ("shim", "fused"):
        lib = load_blocks(which)
        conv_state = torch.zeros(1, 128, 3, device="cuda")
        ssm_state = torch.zeros(1, 4, 16, 16, device="cuda")
        out = run_mamba_bf16(lib, mamba_golden, conv_state=conv_state, ssm_state=ssm_state)
        torch.cuda.synchronize()
        lib.blk_free_allocator()
        outs.append((out, conv_state, ssm_state))
    # the reference's conv kernel and this library's agree to 1 bf16 ulp, not always to the bit: compare at block tolerance,
    # and the raw-input conv state exactly
    assert (outs[0][0].float() - outs[1][0].float()).abs().max().item() < 2e-2
    assert torch.equal(outs[0][1], outs[1][1])
    assert rel_l2(outs[1][2], outs[0][2]) < 2e-2


def test_reference_mamba_block_on_its_own_kernels_is_reported(mamba_golden):
    """Same block on the reference's own kernels.  Its gated RMSNorm reduces through a shared-memory word that all
    32 lanes of a warp store to (ops/reduce.cuh:280-287); where that race resolves wrongly the block misses its
    own golden.  Recorded, not asserted: the outcome belongs to the reference, not to this library."""
    stock = load_blocks("stock")
    want = mamba_golden["want"]
    for bf16, tol in ((False, 1e-3), (True, 1.5e-1)):
        got = run_mamba_bf16(stock, mamba_golden).float() if bf16 else _run_mamba_fp32(stock, mamba_golden)
        torch.cuda.synchronize()
        stock.blk_free_allocator()
        err = (got - want).abs().max().item()
        print(f"reference mamba block on its own kernels, {'bf16' if bf16 else 'fp32'}: max abs err {err:.3e} "
              f"(reference tolerance {tol:g}) -> {'within' if err < tol else 'OUTSIDE'}")


@pytest.mark.parametrize("which", ["stock", "shim"])
def test_reference_attention_block_matches_its_golden(built_lib, attn_golden, which):
    """model/attention_block.cuh:107-226 with its pre-norm and residual add on this library, against the golden of
    tools/dump_attention_block.py at the reference's tolerances (tests/model/test_attention_block.cu:129,156)."""
    lib, g = load_blocks(which), attn_golden
    before = built_lib.nmt_launch_count()
    out = torch.empty_like(g["x"])
    assert lib.blk_attn_forward_fp32(p(g["x"]), p(g["nw"]), p(g["q"]), p(g["k"]), p(g["v"]), p(g["o"]), p(out), 40) == 0
    torch.cuda.synchronize()
    lib.blk_reset_allocator()
    assert (out - g["want"]).abs().max().item() < 2e-3
    b = {k: g[k].to(BF) for k in ("x", "q", "k", "v", "o")}
    outb = torch.empty(40, 256, dtype=BF, device="cuda")
    assert lib.blk_attn_forward_bf16(p(b["x"]), p(g["nw"]), p(b["q"]), p(b["k"]), p(b["v"]), p(b["o"]), p(outb), 40,
                                     None, None, 0) == 0
    torch.cuda.synchronize()
    lib.blk_free_allocator()
    assert (outb.float() - g["want"]).abs().max().item() < 2e-1
    assert built_lib.nmt_launch_count() - before == (0 if which == "stock" else 4)      # norm + add, twice


@pytest.mark.parametrize("which", ["shim", "fused"])
def test_attention_prefill_then_decode_on_the_drop_in(attn_golden, which):
    """The reference's hand-off check (tests/model/test_attention_block.cu:196-243): prefill S-1 tokens into the KV cache,
    decode token S, compare with row S-1 of the full-sequence golden (rel L2 < 0.1).  "shim": the reference's decode
    attention kernels; "fused": the integration header, where sdpa_decode_bf16 is this library's."""
    lib, g = load_blocks(which), attn_golden
    S = 40
    b = {k: g[k].to(BF) for k in ("x", "q", "k", "v", "o")}
    kc = torch.zeros(2, S, 128, dtype=BF, device="cuda")
    vc = torch.zeros(2, S, 128, dtype=BF, device="cuda")
    pre = torch.empty(S - 1, 256, dtype=BF, device="cuda")
    assert lib.blk_attn_forward_bf16(p(b["x"]), p(g["nw"]), p(b["q"]), p(b["k"]), p(b["v"]), p(b["o"]), p(pre), S - 1,
                                     p(kc), p(vc), S) == 0
    lib.blk_reset_allocator()
    tok = b["x"][S - 1].contiguous()
    dec = torch.empty(256, dtype=BF, device="cuda")
    assert lib.blk_attn_decode_bf16(p(tok), p(g["nw"]), p(b["q"]), p(b["k"]), p(b["v"]), p(b["o"]), p(kc), p(vc), S - 1, S,
                                    p(dec)) == 0
    torch.cuda.synchronize()
    lib.blk_free_allocator()
    assert rel_l2(dec, g["want"][S - 1]) < 0.1
    assert (pre.float() - g["want"][:S - 1]).abs().max().item() < 2e-1
