"""nmt_ssm_decode_step_bf16 (the single-token Mamba-2 recurrence) through the C ABI: against the oracle
(oracle/torch_golden.ssm_decode_step, pinned to the dump script's scan on CPU), against the reference's own kernel
(ops/mamba2/ssm.cuh, bit for bit), over several tokens, at the model's dimensions and at ragged ones."""
import ctypes

import pytest
import torch

from oracle import torch_golden as og

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def ops(built_lib):
    from nemotron_infer_b200 import ops as _ops
    assert torch.cuda.is_available()
    built_lib.nmt_set_device(torch.cuda.current_device())
    return _ops


def p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _case(batch, H, P, N, G, seed, with_bias=True):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    d = dict(x=rn(batch, H * P).to(BF), dt=(rn(batch, H) - 1).to(BF), A_log=torch.log(1 + 15 * torch.rand(H, generator=g)),
             B=rn(batch, G, N).to(BF), C=rn(batch, G, N).to(BF), D=1 + 0.1 * rn(H), dt_bias=(0.5 * rn(H)) if with_bias else None,
             state=0.3 * rn(batch, H, P, N))
    return {k: (v.cuda() if v is not None else None) for k, v in d.items()}


def _oracle(c, batch, H, P):
    ys, states = [], []
    for b in range(batch):
        y, s = og.ssm_decode_step(c["x"][b].cpu().reshape(H, P), c["dt"][b].cpu(), c["A_log"].cpu(), c["B"][b].cpu(), c["C"][b].cpu(),
                                  c["D"].cpu(), c["state"][b].cpu(), c["dt_bias"].cpu() if c["dt_bias"] is not None else None)
        ys.append(y.reshape(H * P))
        states.append(s)
    return torch.stack(ys), torch.stack(states)


@pytest.mark.parametrize("batch,H,P,N,G,bias", [(1, 96, 80, 128, 8, True), (3, 96, 80, 128, 8, True), (1, 4, 16, 16, 2, True),
                                                 (2, 6, 5, 96, 3, False), (1, 2, 3, 200, 1, True), (1, 8, 7, 33, 4, True)])
def test_against_the_oracle(ops, batch, H, P, N, G, bias):
    c = _case(batch, H, P, N, G, seed=H * 1000 + N, with_bias=bias)
    want_y, want_state = _oracle(c, batch, H, P)
    state = c["state"].clone()
    y = ops.ssm_decode_step(c["x"], c["dt"], c["A_log"], c["B"], c["C"], c["D"], state, dt_bias=c["dt_bias"])
    torch.cuda.synchronize()
    # the state is fp32 arithmetic of three multiplies and an add per element: equal to the oracle up to the fused
    # multiply-add's single rounding
    assert (state.cpu() - want_state).abs().max().item() <= 1e-6 * max(1.0, want_state.abs().max().item())
    # y is a sum of up to 256 products of mixed sign: the order of the additions shows in the last bits of a small sum,
    # so the bound is one bf16 ulp of the value or 1e-6 of the sum of magnitudes, whichever is larger
    err = (y.float().cpu() - want_y).abs()
    mags = (want_state.abs() * c["C"].float().cpu().repeat_interleave(H // G, dim=1)[:, :, None, :].abs()).sum(-1).reshape(batch, H * P)
    assert bool((err <= torch.maximum(want_y.abs() * 2.0 ** -7, 2e-6 * mags + 1e-30)).all()), err.max().item()


def test_softplus_branches_and_clamps(ops):
    """dt + bias above 20 passes through, below -20 gives a step of zero (state and y = D x unchanged by B), and the
    clamp arguments bound the step (ops/mamba2/ssm.cuh:72-76)."""
    H, P, N, G = 4, 8, 32, 2
    c = _case(1, H, P, N, G, seed=3)
    c["dt"] = torch.tensor([[25.0, -30.0, 0.5, -0.5]]).to(BF).cuda()
    c["dt_bias"] = torch.zeros(H).cuda()
    want_y, want_state = _oracle(c, 1, H, P)
    state = c["state"].clone()
    y = ops.ssm_decode_step(c["x"], c["dt"], c["A_log"], c["B"], c["C"], c["D"], state, dt_bias=c["dt_bias"])
    assert (state.cpu() - want_state).abs().max().item() <= 1e-6 * max(1.0, want_state.abs().max().item())
    assert torch.equal(state[0, 1], c["state"][0, 1]), "a step of zero leaves the head's state as it was"
    assert og.ulp_report(y.cpu(), want_y.to(BF))["max_ulp"] <= 1
    # clamp: dt_max = 0.1 caps every head's step
    state2 = c["state"].clone()
    ops.ssm_decode_step(c["x"], c["dt"], c["A_log"], c["B"], c["C"], c["D"], state2, dt_bias=c["dt_bias"], dt_max=0.1)
    dA = torch.exp(-torch.exp(c["A_log"][0]) * 0.1)
    new00 = c["state"][0, 0, 0] * dA + 0.1 * c["B"][0, 0].float() * c["x"][0, 0].float()
    assert torch.allclose(state2[0, 0, 0], new00, rtol=1e-5, atol=1e-6)


def test_bit_identical_to_the_reference_kernel_over_several_tokens(ops, ref_kernels):
    if ref_kernels is None or not hasattr(ref_kernels, "ref_ssm_decode_bf16"):
        pytest.skip("oracle/_ref/libnemotron_ref.so not built with the SSM door (needs the reference checkout at build time)")
    ref_kernels.ref_set_device(torch.cuda.current_device())
    for batch, H, P, N, G in ((1, 96, 80, 128, 8), (2, 96, 80, 128, 8), (1, 4, 16, 16, 2)):
        c = _case(batch, H, P, N, G, seed=11 + batch)
        mine, theirs = c["state"].clone(), c["state"].clone()
        y_ref = torch.empty(batch, H * P, dtype=BF, device="cuda")
        gen = torch.Generator().manual_seed(5)
        for _ in range(4):                                         # the state is carried from token to token
            x = torch.randn(batch, H * P, generator=gen).to(BF).cuda()
            dt = (torch.randn(batch, H, generator=gen) - 1).to(BF).cuda()
            y = ops.ssm_decode_step(x, dt, c["A_log"], c["B"], c["C"], c["D"], mine, dt_bias=c["dt_bias"])
            assert ref_kernels.ref_ssm_decode_bf16(p(x), p(dt), p(c["A_log"]), p(c["B"]), p(c["C"]), p(c["D"]), p(c["dt_bias"]),
                                                   p(theirs), p(y_ref), batch, H, P, N, G, None) == 0
            torch.cuda.synchronize()
            assert torch.equal(mine, theirs), (batch, H, "state")
            assert torch.equal(y.view(torch.int16), y_ref.view(torch.int16)), (batch, H, "y")


def test_rejections_and_empty_batch(built_lib):
    H, P, N, G = 4, 8, 32, 2
    c = _case(1, H, P, N, G, seed=1)
    y = torch.empty(1, H * P, dtype=BF, device="cuda")
    args = lambda **kw: [p(kw.get("x", c["x"])), p(c["dt"]), p(c["A_log"]), p(c["B"]), p(c["C"]), p(c["D"]), p(c["dt_bias"]),  # noqa: E731
                         p(kw.get("state", c["state"])), p(y)]
    before = built_lib.nmt_launch_count()
    assert built_lib.nmt_ssm_decode_step_bf16(*args(), 0, H, P, N, G, 0.0, 1e30, None) == 0            # empty batch: nothing to do
    assert built_lib.nmt_ssm_decode_step_bf16(*args(), 1, H, P, N, 3, 0.0, 1e30, None) == 3            # heads % groups != 0
    assert built_lib.nmt_ssm_decode_step_bf16(*args(), 1, H, P, 512, G, 0.0, 1e30, None) == 5          # state size beyond 256
    assert built_lib.nmt_ssm_decode_step_bf16(*args(state=None), 1, H, P, N, G, 0.0, 1e30, None) == 1
    odd = ctypes.c_void_p(c["x"].data_ptr() + 1)
    a = args()
    a[0] = odd
    assert built_lib.nmt_ssm_decode_step_bf16(*a, 1, H, P, N, G, 0.0, 1e30, None) == 2
    assert built_lib.nmt_launch_count() == before
