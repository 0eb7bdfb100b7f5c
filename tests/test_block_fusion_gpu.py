"""The fused forms inside REAL blocks.

1. Cross-block fusion: with the next block's norm weight announced (nmt_fuse_next_norm), the closing residual add of
   the reference's block i and the pre-norm of block i+1 run as ONE launch of the fused add + RMSNorm kernel, with the
   block code, its signatures and its allocator untouched.  Checked on stacks of two of the reference's own blocks
   (MLP -> MLP, Mamba-2 -> MLP, attention -> MLP) against the goldens of its dump scripts and the dump scripts'
   formulation of the MLP block, at the reference's block tolerances (tests/model/test_mlp_block.cu:124,150), and at
   model width against the unfused stack.
2. The FP8 and single-token block forms of include/nemotron_b200_shim/model/blocks_b200.cuh against the same blocks on
   this library's single ops (byte-identical), against the reference's own kernels, and against the goldens with the
   reference's FP8 tolerances (tests/model/test_mlp_block.cu:184, test_mamba_block.cu:241,368)."""
import pytest
import torch

from blocks_common import (BF, MAMBA, attn_fixture, fp8_rows, fusion_counters, load_blocks, mamba_fixture, mlp_fixture, p,
                           rel_l2, run_mamba_bf16, run_mlp_bf16)
from oracle import torch_golden as og

pytestmark = pytest.mark.gpu
EPS = 1e-5


def _mlp_weights(hidden, inter, seed):
    g = torch.Generator().manual_seed(seed)
    nw = 1 + 0.1 * torch.randn(hidden, generator=g)
    up = torch.randn(inter, hidden, generator=g) / hidden ** 0.5
    down = torch.randn(hidden, inter, generator=g) / inter ** 0.5
    return nw.cuda(), up.cuda(), down.cuda()


def _second_mlp(lib, nmt, first_block, x, nw2, up2, down2, announce):
    """Runs `first_block(out1)` then the reference's MLP block on its output, the way engine.py drives layers: rewind the
    allocator before each block; optionally announce the second block's norm weight before the first."""
    nmt.nmt_fusion_reset()
    lib.blk_reset_allocator()
    if announce:
        assert nmt.nmt_fuse_next_norm(p(nw2), EPS) == 0
    out1 = first_block()
    lib.blk_reset_allocator()
    out2 = run_mlp_bf16(lib, out1, nw2, up2.to(BF), down2.to(BF))
    torch.cuda.synchronize()
    return out1, out2


def _pair(built_lib, first_block, x, nw2, up2, down2, expect_launches_unfused):
    lib = load_blocks("shim")
    results = {}
    for announce in (False, True):
        f0, e0 = fusion_counters(built_lib)
        before = built_lib.nmt_launch_count()
        out1, out2 = _second_mlp(lib, built_lib, lambda: first_block(lib), x, nw2, up2, down2, announce)
        launched = built_lib.nmt_launch_count() - before
        f1, e1 = fusion_counters(built_lib)
        results[announce] = (out1, out2, launched, f1 - f0, e1 - e0)
    lib.blk_free_allocator()
    u, f = results[False], results[True]
    assert u[2] == expect_launches_unfused and u[3:] == (0, 0)
    assert f[2] == expect_launches_unfused - 1, "one launch fewer per block boundary"
    assert f[3:] == (1, 1), "one fused tail, one skipped head"
    assert torch.equal(u[0].view(torch.int16), f[0].view(torch.int16)), "the residual stream itself must not change"
    return u, f


def test_two_stacked_mlp_blocks_fuse_the_boundary_and_meet_the_golden(built_lib):
    g = mlp_fixture()
    nw2, up2, down2 = _mlp_weights(64, 256, seed=21)
    xb, upb, downb = g["x"].to(BF), g["up"].to(BF), g["down"].to(BF)
    u, f = _pair(built_lib, lambda lib: run_mlp_bf16(lib, xb, g["nw"], upb, downb), xb, nw2, up2, down2,
                 expect_launches_unfused=6)
    want1 = g["want"].cpu()
    want2 = og.mlp_block(want1, nw2.cpu(), up2.cpu(), down2.cpu())
    for out1, out2 in (u[:2], f[:2]):
        assert (out1.float().cpu() - want1).abs().max().item() < 1.5e-1
        assert (out2.float().cpu() - want2).abs().max().item() < 1.5e-1
    assert rel_l2(f[1], u[1]) < 1e-2


def test_mamba_then_mlp_fuses_the_boundary_and_meets_the_golden(built_lib):
    g = mamba_fixture()
    nw2, up2, down2 = _mlp_weights(64, 256, seed=22)
    u, f = _pair(built_lib, lambda lib: run_mamba_bf16(lib, g), None, nw2, up2, down2, expect_launches_unfused=6)
    want1 = g["want"].cpu()
    want2 = og.mlp_block(want1, nw2.cpu(), up2.cpu(), down2.cpu())
    for out1, out2 in (u[:2], f[:2]):
        assert (out1.float().cpu() - want1).abs().max().item() < 1.5e-1
        assert (out2.float().cpu() - want2).abs().max().item() < 1.5e-1
    assert rel_l2(f[1], u[1]) < 1e-2


def test_attention_then_mlp_fuses_the_boundary_and_meets_the_golden(built_lib):
    g = attn_fixture()
    b = {k: g[k].to(BF) for k in ("x", "q", "k", "v", "o")}
    nw2, up2, down2 = _mlp_weights(256, 512, seed=23)

    def attn(lib):
        out = torch.empty(40, 256, dtype=BF, device="cuda")
        assert lib.blk_attn_forward_bf16(p(b["x"]), p(g["nw"]), p(b["q"]), p(b["k"]), p(b["v"]), p(b["o"]), p(out), 40,
                                         None, None, 0) == 0
        return out
    u, f = _pair(built_lib, attn, None, nw2, up2, down2, expect_launches_unfused=5)
    want1 = g["want"].cpu()
    want2 = og.mlp_block(want1, nw2.cpu(), up2.cpu(), down2.cpu())
    for out1, out2 in (u[:2], f[:2]):
        assert (out1.float().cpu() - want1).abs().max().item() < 2e-1
        assert rel_l2(out2.cpu(), want2) < 2e-2
    assert rel_l2(f[1], u[1]) < 1e-2


def test_model_width_pair_fused_equals_unfused_to_bf16_resolution(built_lib):
    M, H, I = 192, 3136, 12544
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(M, H, generator=g, device="cuda").to(BF)
    ws = []
    for _ in range(2):
        ws.append(((1 + 0.1 * torch.randn(H, generator=g, device="cuda")).contiguous(),
                   (0.02 * torch.randn(I, H, generator=g, device="cuda")).to(BF),
                   (0.02 * torch.randn(H, I, generator=g, device="cuda")).to(BF)))
    (nw1, up1, down1), (nw2, up2, down2) = ws
    u, f = _pair(built_lib, lambda lib: run_mlp_bf16(lib, x, nw1, up1, down1), x, nw2, up2.float(), down2.float(),
                 expect_launches_unfused=6)
    assert rel_l2(f[1], u[1]) < 5e-3 and (f[1].float() - u[1].float()).abs().max().item() < 0.15


def test_fusion_falls_back_when_the_pattern_does_not_match(built_lib):
    """Announced, but the next block's pre-norm tensor is somewhere else (allocator not rewound): the fused tail still
    runs, the head finds no match and runs the plain norm - same results, no skipped head.  And an announcement is
    used at most once."""
    lib = load_blocks("shim")
    g = mlp_fixture()
    xb, upb, downb = g["x"].to(BF), g["up"].to(BF), g["down"].to(BF)
    nw2, up2, down2 = _mlp_weights(64, 256, seed=21)
    built_lib.nmt_fusion_reset()
    lib.blk_reset_allocator()
    want1 = run_mlp_bf16(lib, xb, g["nw"], upb, downb)
    lib.blk_reset_allocator()
    want2 = run_mlp_bf16(lib, want1, nw2, up2.to(BF), down2.to(BF))
    torch.cuda.synchronize()
    f0, e0 = fusion_counters(built_lib)
    lib.blk_reset_allocator()
    assert built_lib.nmt_fuse_next_norm(p(nw2), EPS) == 0
    out1 = run_mlp_bf16(lib, xb, g["nw"], upb, downb)
    out2 = run_mlp_bf16(lib, out1, nw2, up2.to(BF), down2.to(BF))          # no rewind: other workspace addresses
    out3 = run_mlp_bf16(lib, out2, nw2, up2.to(BF), down2.to(BF))          # no announcement left: plain add, plain norm
    torch.cuda.synchronize()
    f1, e1 = fusion_counters(built_lib)
    assert (f1 - f0, e1 - e0) == (1, 0)
    assert torch.equal(out1.view(torch.int16), want1.view(torch.int16))
    assert torch.equal(out2.view(torch.int16), want2.view(torch.int16))
    assert torch.isfinite(out3.float()).all()
    # a weight that is not 16-byte aligned is refused, a NULL weight withdraws the announcement
    assert built_lib.nmt_fuse_next_norm(nw2.data_ptr() + 4, EPS) == 2
    assert built_lib.nmt_fuse_next_norm(None, EPS) == 0
    lib.blk_free_allocator()
    built_lib.nmt_fusion_reset()


def test_a_launch_between_the_fused_tail_and_the_head_drops_the_pending_norm(built_lib):
    """The head is skipped only when it is the very next launch of this library on the thread: here relu^2 rewrites the
    rows in between, and the head must run its norm on the new rows."""
    T, H = 64, 3136
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(T, H, generator=g, device="cuda").to(BF)
    m = torch.randn(T, H, generator=g, device="cuda").to(BF)
    w1 = (1 + 0.1 * torch.randn(H, generator=g, device="cuda")).contiguous()
    w2 = (1 + 0.1 * torch.randn(H, generator=g, device="cuda")).contiguous()
    y, out, want = (torch.empty(T, H, dtype=BF, device="cuda") for _ in range(3))
    built_lib.nmt_fusion_reset()
    f0, e0 = fusion_counters(built_lib)
    assert built_lib.nmt_block_head_rmsnorm_bf16(p(x), p(y), p(w1), T, H, EPS, None) == 0
    assert built_lib.nmt_fuse_next_norm(p(w2), EPS) == 0
    assert built_lib.nmt_block_tail_add_bf16(p(x), p(m), p(out), T * H, None) == 0          # fused: y = norm(out) * w2
    assert built_lib.nmt_relu2_bf16(p(out), p(out), T * H, None) == 0                       # rows change under it
    assert built_lib.nmt_block_head_rmsnorm_bf16(p(out), p(y), p(w2), T, H, EPS, None) == 0
    assert built_lib.nmt_rmsnorm_bf16(p(out), p(want), p(w2), T, H, EPS, None) == 0
    torch.cuda.synchronize()
    f1, e1 = fusion_counters(built_lib)
    assert (f1 - f0, e1 - e0) == (1, 0)
    assert torch.equal(y.view(torch.int16), want.view(torch.int16))
    # and with nothing in between the same sequence does skip the head
    assert built_lib.nmt_block_head_rmsnorm_bf16(p(x), p(y), p(w1), T, H, EPS, None) == 0
    assert built_lib.nmt_fuse_next_norm(p(w2), EPS) == 0
    assert built_lib.nmt_block_tail_add_bf16(p(x), p(m), p(out), T * H, None) == 0
    assert built_lib.nmt_block_head_rmsnorm_bf16(p(out), p(y), p(w2), T, H, EPS, None) == 0
    assert built_lib.nmt_rmsnorm_bf16(p(out), p(want), p(w2), T, H, EPS, None) == 0
    torch.cuda.synchronize()
    f2, e2 = fusion_counters(built_lib)
    assert (f2 - f1, e2 - e1) == (1, 1)
    # y now comes from the fused kernel, which spreads a row over another number of threads than the plain norm:
    # the two may differ by one bf16 ulp in a few elements (summation order)
    rep = og.ulp_report(y.cpu(), want.cpu())
    assert rep["max_ulp"] <= 1 and rep["mismatch_frac"] <= 0.005, rep
    built_lib.nmt_fusion_reset()


# ---------------------------------------------------------------------------------------------------------------
# FP8 and single-token block forms
# ---------------------------------------------------------------------------------------------------------------
def _mlp_fp8(lib, x, nw, upq, ups, downq, downs, hidden, inter):
    out = torch.empty_like(x)
    assert lib.blk_mlp_forward_fp8(p(x), p(nw), p(upq), p(ups), p(downq), p(downs), p(out), x.shape[0], hidden, inter) == 0
    torch.cuda.synchronize()
    lib.blk_free_allocator()
    return out


def test_fp8_mlp_block_prefill_fused_equals_unfused_and_meets_the_golden(built_lib):
    g = mlp_fixture()
    xb = g["x"].to(BF)
    upq, ups = fp8_rows(g["up"])
    downq, downs = fp8_rows(g["down"])
    outs, launches = {}, {}
    for which in ("stock", "shim", "fused"):
        before = built_lib.nmt_launch_count()
        outs[which] = _mlp_fp8(load_blocks(which), xb, g["nw"], upq, ups, downq, downs, 64, 256)
        launches[which] = built_lib.nmt_launch_count() - before
    # the reference's tolerance against the fp32 golden (tests/model/test_mlp_block.cu:184)
    for which, out in outs.items():
        assert rel_l2(out, g["want"]) < 0.3, which
    # same FP8 GEMM inputs, same GEMMs: the fused form changes no output byte
    assert torch.equal(outs["fused"].view(torch.int16), outs["shim"].view(torch.int16))
    assert rel_l2(outs["fused"], outs["stock"]) < 2e-2
    # shim: norm, relu^2, add on this library, quantiser the reference's; fused: norm+quant (2 kernels), relu^2+quant (2), add
    assert launches == {"stock": 0, "shim": 3, "fused": 5}


def test_fp8_mlp_block_at_model_width_prefill_and_single_token(built_lib):
    H, I = 3136, 12544
    g = torch.Generator().manual_seed(4)
    nw = (1 + 0.1 * torch.randn(H, generator=g)).cuda()
    upq, ups = fp8_rows(0.02 * torch.randn(I, H, generator=g))
    downq, downs = fp8_rows(0.02 * torch.randn(H, I, generator=g))
    for M in (64, 1):
        x = torch.randn(M, H, generator=g).to(BF).cuda()
        outs, launches = {}, {}
        for which in ("stock", "shim", "fused"):
            before = built_lib.nmt_launch_count()
            outs[which] = _mlp_fp8(load_blocks(which), x, nw, upq, ups, downq, downs, H, I)
            launches[which] = built_lib.nmt_launch_count() - before
        assert torch.equal(outs["fused"].view(torch.int16), outs["shim"].view(torch.int16)), M
        assert rel_l2(outs["fused"], outs["stock"]) < 2e-2, M
        if M == 1:
            # single token: norm, up_proj GEMV, relu^2, down_proj GEMV, add -> two launches
            assert launches == {"stock": 0, "shim": 5, "fused": 2}
        else:
            assert launches == {"stock": 0, "shim": 3, "fused": 5}


def test_single_token_fp8_mlp_block_latency_three_ways(built_lib):
    """The reference's FP8 MLP block for one token at model width, timed on the device: on the reference's own kernels
    (5 launches), on this library's single ops (5 launches) and in fused form (2 launches).  Four weight sets (4 x 79 MB)
    rotate so that no call finds its matrices in L2, as in a 42-layer decode step.  The figures go to the session's
    report; the assertions are only the order and a factor of two over the reference's kernels."""
    from conftest import ULP_LOG
    H, I, SETS, CALLS = 3136, 12544, 4, 48
    g = torch.Generator().manual_seed(6)
    nw = (1 + 0.1 * torch.randn(H, generator=g)).cuda()
    x = torch.randn(1, H, generator=g).to(BF).cuda()
    sets = []
    for _ in range(SETS):
        upq, ups = fp8_rows(0.02 * torch.randn(I, H, generator=g))
        downq, downs = fp8_rows(0.02 * torch.randn(H, I, generator=g))
        sets.append((upq, ups, downq, downs))
    out = torch.empty_like(x)
    us = {}
    for which in ("stock", "shim", "fused"):
        lib = load_blocks(which)

        def call(i):
            upq, ups, downq, downs = sets[i % SETS]
            assert lib.blk_mlp_forward_fp8(p(x), p(nw), p(upq), p(ups), p(downq), p(downs), p(out), 1, H, I) == 0
            lib.blk_reset_allocator()
        for i in range(8):
            call(i)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        for _ in range(3):
            t0.record()
            for i in range(CALLS):
                call(i)
            t1.record()
            torch.cuda.synchronize()
            best = min(best, t0.elapsed_time(t1) * 1e3 / CALLS)
        us[which] = best
        lib.blk_free_allocator()
    ULP_LOG.append(dict(what="latency_us mlp_block_forward_fp8 one token 3136/12544 (reference kernels / this library's ops / fused)",
                        stock=round(us["stock"], 2), shim=round(us["shim"], 2), fused=round(us["fused"], 2)))
    assert us["shim"] < us["stock"] and us["fused"] < us["shim"] * 1.25, us
    assert us["stock"] / us["fused"] > 2.0, us


def test_prefill_fp8_mlp_block_latency_three_ways(built_lib):
    """The same block for 4096 tokens: the two FP8 GEMMs (cuBLASLt, the reference's own calls, identical in the three
    builds) plus what surrounds them - norm, quantise, relu^2, quantise, add: 9 launches of the reference's kernels, or
    norm + add of this library around the reference's quantisers (shim), or norm+quantise, relu^2+quantise and add in 5
    launches of this library (fused).  Figures go to the session's report."""
    from conftest import ULP_LOG
    M, H, I, CALLS = 4096, 3136, 12544, 12
    g = torch.Generator().manual_seed(9)
    nw = (1 + 0.1 * torch.randn(H, generator=g)).cuda()
    x = torch.randn(M, H, generator=g).to(BF).cuda()
    upq, ups = fp8_rows(0.02 * torch.randn(I, H, generator=g))
    downq, downs = fp8_rows(0.02 * torch.randn(H, I, generator=g))
    out = torch.empty_like(x)
    us = {}
    for which in ("stock", "shim", "fused"):
        lib = load_blocks(which)

        def call():
            assert lib.blk_mlp_forward_fp8(p(x), p(nw), p(upq), p(ups), p(downq), p(downs), p(out), M, H, I) == 0
            lib.blk_reset_allocator()
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        for _ in range(3):
            t0.record()
            for _ in range(CALLS):
                call()
            t1.record()
            torch.cuda.synchronize()
            best = min(best, t0.elapsed_time(t1) * 1e3 / CALLS)
        us[which] = best
        lib.blk_free_allocator()
    ULP_LOG.append(dict(what="latency_us mlp_block_forward_fp8 4096 tokens 3136/12544 (reference kernels / this library's ops / fused)",
                        stock=round(us["stock"], 1), shim=round(us["shim"], 1), fused=round(us["fused"], 1)))
    assert us["fused"] < us["stock"], us


def _mamba_fp8_weights(g):
    inq, ins = fp8_rows(g["in_proj_w"].reshape(MAMBA["PROJ"], 64))
    outq, outs = fp8_rows(g["out_proj_w"].reshape(64, 64))
    return inq, ins, outq, outs


def _mamba_prefill_then_decode(lib, g, fp8):
    """The reference's hand-off check (tests/model/test_mamba_block.cu:247-308, 311-370): prefill S-1 tokens, decode
    token S from the states the prefill left, compare with row S-1 of the full-sequence golden."""
    S = MAMBA["S"]
    x = g["input"].reshape(S, 64).to(BF)
    conv_state = torch.zeros(1, MAMBA["CONV_DIM"], 3, device="cuda")
    ssm_state = torch.zeros(1, MAMBA["H"], MAMBA["P"], MAMBA["N"], device="cuda")
    pre = torch.empty(S - 1, 64, dtype=BF, device="cuda")
    dec = torch.empty(64, dtype=BF, device="cuda")
    tok = x[S - 1].contiguous()
    common = (p(g["conv1d_w"]), p(g["conv1d_b"]), p(g["A_log"]), p(g["D"]), p(g["dt_bias"]), p(g["gnorm_w"]))
    if fp8:
        inq, ins, outq, outs = _mamba_fp8_weights(g)
        assert lib.blk_mamba_forward_fp8(p(x), p(g["block_norm_w"]), p(inq), p(ins), *common, p(outq), p(outs), p(pre), 1, S - 1,
                                         p(conv_state), p(ssm_state)) == 0
        lib.blk_reset_allocator()
        assert lib.blk_mamba_decode_fp8(p(tok), p(g["block_norm_w"]), p(inq), p(ins), *common, p(outq), p(outs), p(conv_state),
                                        p(ssm_state), p(dec), 1) == 0
    else:
        inw, outw = g["in_proj_w"].to(BF), g["out_proj_w"].to(BF)
        assert lib.blk_mamba_forward_bf16(p(x), p(g["block_norm_w"]), p(inw), *common, p(outw), p(pre), 1, S - 1, p(conv_state),
                                          p(ssm_state)) == 0
        lib.blk_reset_allocator()
        assert lib.blk_mamba_decode_bf16(p(tok), p(g["block_norm_w"]), p(inw), *common, p(outw), p(conv_state), p(ssm_state),
                                         p(dec), 1) == 0
    torch.cuda.synchronize()
    lib.blk_free_allocator()
    return pre, dec, conv_state, ssm_state


@pytest.mark.parametrize("which", ["shim", "fused"])
def test_mamba_prefill_then_decode_bf16(built_lib, which):
    g = mamba_fixture()
    before = built_lib.nmt_launch_count()
    pre, dec, conv_state, _ = _mamba_prefill_then_decode(load_blocks(which), g, fp8=False)
    launched = built_lib.nmt_launch_count() - before
    want = g["want"]
    assert (dec.float() - want[MAMBA["S"] - 1]).abs().max().item() < 1.5e-1      # test_mamba_block.cu:303
    assert (pre.float() - want[:MAMBA["S"] - 1]).abs().max().item() < 1.5e-1
    # the conv window after the decode step holds the last three raw xBC rows; finite and changed by the step
    assert torch.isfinite(conv_state).all()
    # norm, gated norm, add per block call; the fused forms add the split-fused conv (prefill), the conv step and the
    # state-space step (decode)
    assert launched == (6 if which == "shim" else 9)


@pytest.mark.parametrize("which", ["shim", "fused"])
def test_mamba_prefill_then_decode_fp8(built_lib, which):
    g = mamba_fixture()
    before = built_lib.nmt_launch_count()
    pre, dec, _, _ = _mamba_prefill_then_decode(load_blocks(which), g, fp8=True)
    launched = built_lib.nmt_launch_count() - before
    want = g["want"]
    assert rel_l2(dec, want[MAMBA["S"] - 1]) < 0.35                             # test_mamba_block.cu:368
    assert rel_l2(pre, want[:MAMBA["S"] - 1]) < 0.3                             # test_mamba_block.cu:241
    if which == "shim":
        # prefill: norm, gated norm, add; decode: norm, 3 in_proj GEMVs, gated norm, out_proj GEMV, add
        assert launched == 3 + 7
    else:
        # prefill: norm+quant (2), conv+split, gated norm with maximum + quantiser (2), add; decode: norm+in_proj GEMV,
        # + conv step, state-space step, gated norm + out_proj GEMV + add
        assert launched == 6 + 3


def test_mamba_fp8_decode_fused_equals_unfused_bit_for_bit(built_lib):
    """Same states in, same token: the 5-launch decode block returns the bytes of the 12-launch one."""
    g = mamba_fixture()
    inq, ins, outq, outs = _mamba_fp8_weights(g)
    gen = torch.Generator().manual_seed(77)
    tok = torch.randn(64, generator=gen).to(BF).cuda()
    conv0 = torch.randn(1, MAMBA["CONV_DIM"], 3, generator=gen).cuda()
    ssm0 = (0.1 * torch.randn(1, MAMBA["H"], MAMBA["P"], MAMBA["N"], generator=gen)).cuda()
    common = (p(g["conv1d_w"]), p(g["conv1d_b"]), p(g["A_log"]), p(g["D"]), p(g["dt_bias"]), p(g["gnorm_w"]))
    res = {}
    for which in ("shim", "fused"):
        lib = load_blocks(which)
        conv, ssm = conv0.clone(), ssm0.clone()
        dec = torch.empty(64, dtype=BF, device="cuda")
        assert lib.blk_mamba_decode_fp8(p(tok), p(g["block_norm_w"]), p(inq), p(ins), *common, p(outq), p(outs), p(conv), p(ssm),
                                        p(dec), 1) == 0
        torch.cuda.synchronize()
        lib.blk_free_allocator()
        res[which] = (dec, conv, ssm)
    # the conv step of the reference and of this library agree to 1 bf16 ulp; everything else is this library's in both
    assert (res["shim"][0].float() - res["fused"][0].float()).abs().max().item() < 5e-2
    assert torch.equal(res["shim"][1], res["fused"][1]), "conv window"
    assert rel_l2(res["fused"][2], res["shim"][2]) < 2e-2


def _attn_fp8_weights(g):
    out = []
    for k in ("q", "k", "v", "o"):
        out.extend(p(t) for t in _keep(fp8_rows(g[k])))
    return out


_KEPT = []


def _keep(ts):
    _KEPT.append(ts)          # the pointers handed to the block must outlive the launches
    return ts


def _attention_fp8_prefill_then_decode(built_lib, which):
    """model/attention_block.cuh:286-414 at the tolerances of tests/model/test_attention_block.cu:161-300: the full
    sequence, then prefill of S-1 tokens into the KV cache and a decode step for token S."""
    lib, g = load_blocks(which), attn_fixture()
    S = 40
    x = g["x"].to(BF)
    w = _attn_fp8_weights(g)
    before = built_lib.nmt_launch_count()
    full = torch.empty(S, 256, dtype=BF, device="cuda")
    assert lib.blk_attn_forward_fp8(p(x), p(g["nw"]), *w, p(full), S, None, None, 0) == 0
    lib.blk_reset_allocator()
    kc = torch.zeros(2, S, 128, dtype=BF, device="cuda")
    vc = torch.zeros(2, S, 128, dtype=BF, device="cuda")
    pre = torch.empty(S - 1, 256, dtype=BF, device="cuda")
    assert lib.blk_attn_forward_fp8(p(x), p(g["nw"]), *w, p(pre), S - 1, p(kc), p(vc), S) == 0
    lib.blk_reset_allocator()
    tok = x[S - 1].contiguous()
    dec = torch.empty(256, dtype=BF, device="cuda")
    assert lib.blk_attn_decode_fp8(p(tok), p(g["nw"]), *w, p(kc), p(vc), S - 1, S, p(dec)) == 0
    torch.cuda.synchronize()
    lib.blk_free_allocator()
    launched = built_lib.nmt_launch_count() - before
    assert rel_l2(full, g["want"]) < 0.3
    assert rel_l2(pre, g["want"][:S - 1]) < 0.3
    assert rel_l2(dec, g["want"][S - 1]) < 0.35
    # shim (the reference's own quantiser): per prefill norm and add = 2; decode norm, 4 GEMVs, add = 6
    # fused: per prefill norm+quantise (2), quantiser (2), add = 5; decode 3 GEMVs with the norm inside, the decode
    # attention (2), o_proj GEMV + add = 6
    assert launched == {"stock": 0, "shim": 10, "fused": 16}[which]
    return full, pre, dec


@pytest.mark.parametrize("which", ["stock", "shim", "fused"])
def test_attention_fp8_prefill_then_decode(built_lib, which):
    _attention_fp8_prefill_then_decode(built_lib, which)


def test_attention_fp8_fused_equals_unfused_bit_for_bit(built_lib):
    res = {which: _attention_fp8_prefill_then_decode(built_lib, which) for which in ("shim", "fused")}
    for a, b, name in zip(res["shim"][:2], res["fused"][:2], ("full sequence", "prefill")):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), name
    # the decode step of the fused build also runs this library's decode attention, whose fp32 sums associate differently
    # from the reference kernel's: equal to bf16 resolution, not necessarily bit for bit
    assert rel_l2(res["fused"][2], res["shim"][2]) < 1e-2
