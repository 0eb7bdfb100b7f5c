"""Mamba-2 causal conv1d + SiLU with the x | B | C split, against the golden formulation of the reference's
emitter (tools/dump_mamba_block.py:126-130), its dumped stage tensors, and the reference's own kernel."""
import ctypes

import pytest
import torch

from conftest import golden
from oracle import torch_golden as og

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def ops(built_lib):
    from nemotron_infer_b200 import ops as _ops
    built_lib.nmt_set_device(torch.cuda.current_device())
    return _ops


def make(batch, S, C, seed=0):
    g = torch.Generator().manual_seed(seed + S + C)
    x = torch.randn(batch, S, C, generator=g).to(BF)
    w = 0.2 * torch.randn(C, 4, generator=g)
    b = 0.1 * torch.randn(C, generator=g)
    return x, w, b


def test_fp32_twin_matches_the_dump_stage(ops):
    d = golden("dump_mamba_block.npz")
    x = torch.from_numpy(d["xbc"].copy()).reshape(1, 24, 128)
    w = torch.from_numpy(d["conv1d_w"].copy()).reshape(128, 4)
    b = torch.from_numpy(d["conv1d_b"].copy())
    y, state = ops.causal_conv1d_silu(x.cuda(), w.cuda(), b.cuda(), return_state=True)
    torch.testing.assert_close(y.cpu().reshape(-1), torch.from_numpy(d["xbc_conv"]), rtol=1e-5, atol=1e-5)
    assert torch.equal(state.cpu(), og.conv_state_tail(x))


@pytest.mark.parametrize("batch,S,C,split", [(1, 24, 128, None), (1, 4096, 9728, (7680, 1024, 1024)), (2, 100, 9728, (7680, 1024, 1024)),
                                            (3, 1, 64, (32, 16, 16)), (1, 2, 64, None), (2, 3, 8, None), (1, 33, 128, (8, 120)),
                                            (1, 65, 256, (256,))])
def test_bf16_conv_against_golden(ops, batch, S, C, split):
    x, w, b = make(batch, S, C)
    want = og.causal_conv1d_silu_bf16(x, w, b)
    out, state = ops.causal_conv1d_silu(x.cuda(), w.cuda(), b.cuda(), split=split, return_state=True)
    got = torch.cat([o.cpu() for o in out], dim=-1) if split is not None else out.cpu()
    rep = og.ulp_report(got, want)
    assert rep["max_ulp"] <= 1 and rep["mismatch_frac"] <= 0.02, rep
    assert torch.equal(state.cpu(), og.conv_state_tail(x))
    # the split only changes where a vector is stored, never its value
    whole = ops.causal_conv1d_silu(x.cuda(), w.cuda(), b.cuda()).cpu()
    assert torch.equal(whole.view(torch.int16), got.view(torch.int16))


@pytest.mark.parametrize("batch,C,split", [(1, 9728, (7680, 1024, 1024)), (3, 9728, (7680, 1024, 1024)), (2, 64, None), (1, 8, None),
                                           (5, 256, (8, 248))])
def test_decode_step_continues_the_prefill(ops, batch, C, split):
    """Prefill S tokens, then feed the next tokens one at a time through the decode step: every step must match the
    golden step formula on the carried state AND the prefill over the longer sequence (the same causal window)."""
    S, steps = 37, 6
    x, w, b = make(batch, S + steps, C, seed=11)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    _, state = ops.causal_conv1d_silu(xd[:, :S].contiguous(), wd, bd, return_state=True)
    want_all = og.causal_conv1d_silu_bf16(x, w, b)
    ostate = og.conv_state_tail(x[:, :S])
    for t in range(S, S + steps):
        xt = xd[:, t].contiguous()
        out = ops.causal_conv1d_silu_decode(xt, wd, bd, state, split=split)
        got = torch.cat([o.cpu() for o in out], dim=-1) if split is not None else out.cpu()
        want_step, ostate = og.causal_conv1d_decode_bf16(x[:, t], w, b, ostate)
        for want in (want_step, want_all[:, t]):
            # one bf16 ulp, except where the taps nearly cancel: there the fp32 sum's last bits (fma or not, order)
            # are many ulps of a tiny result, so those elements get an absolute bar instead
            big = want.float().abs() >= 1e-2
            rep = og.ulp_report(got[big], want[big])
            assert rep["max_ulp"] <= 1 and rep["mismatch_frac"] <= 0.02, (t, rep)
            assert float((got.float() - want.float())[~big].abs().max()) <= 1e-4 if bool((~big).any()) else True
        assert torch.equal(state.cpu(), ostate), t                   # the window holds raw inputs: exact
    assert torch.equal(state.cpu(), og.conv_state_tail(x))


def test_decode_step_argument_checks(built_lib):
    L = built_lib
    B = 0x7F0000000000
    f = L.nmt_causal_conv1d_silu_decode_split_bf16
    assert f(B, B, B, B, B, B, 7680, 1024, 1024, B, 0, None) == 0          # empty batch
    assert f(B, B, B, B, B, B, 7684, 1024, 1024, B, 1, None) == 3          # segment not a multiple of 8 channels
    assert f(B, B, B, B, B, B, 7680, 1024, 1024, None, 1, None) == 1       # the state is not optional here
    assert f(B, B, B, B, B, B, 7680, 1024, 1024, B + 4, 1, None) == 2      # state must be 16-byte aligned
    assert f(B, B, B, B, None, B, 7680, 1024, 1024, B, 1, None) == 1       # a non-empty segment needs its tensor


def test_conv_against_reference_kernel(ops, ref_kernels):
    if ref_kernels is None or not hasattr(ref_kernels, "ref_causal_conv1d_bf16"):
        pytest.skip("reference conv1d kernel not built")
    x, w, b = make(2, 300, 9728, seed=5)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    ref = torch.empty_like(xd)
    ref_state = torch.zeros(2, 9728, 3, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    ref_kernels.ref_set_device(torch.cuda.current_device())
    assert ref_kernels.ref_causal_conv1d_bf16(p(xd), p(wd), p(bd), p(ref), p(ref_state), 9728, 300, 2, None) == 0
    torch.cuda.synchronize()
    got, state = ops.causal_conv1d_silu(xd, wd, bd, return_state=True)
    rep = og.ulp_report(got, ref)
    assert rep["max_ulp"] <= 1 and rep["mismatch_frac"] <= 0.02, rep
    assert torch.equal(state, ref_state)


def test_conv_argument_checks(built_lib):
    L = built_lib
    B = 0x7F0000000000
    assert L.nmt_causal_conv1d_silu_split_bf16(B, B, B, B, None, None, 128, 0, 0, None, 0, 1, None) == 0      # S == 0
    assert L.nmt_causal_conv1d_silu_split_bf16(B, B, B, B, None, None, 100, 0, 0, None, 4, 1, None) == 3     # n0 % 8
    assert L.nmt_causal_conv1d_silu_split_bf16(B, B, B, B, None, None, 64, 64, 0, None, 4, 1, None) == 1     # out1 missing
    assert L.nmt_causal_conv1d_silu_split_bf16(B + 2, B, B, B, None, None, 64, 0, 0, None, 4, 1, None) == 2  # alignment
