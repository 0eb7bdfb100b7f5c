"""nmt_sdpa_decode_bf16 (attention of one query token over the KV cache, then the cache append) through the C ABI:
against the oracle (oracle/torch_golden.sdpa_decode), against the reference's own kernels, over several appended tokens,
at the model's head counts (40 query / 8 KV heads) and the dump script's (4 / 2), short and long caches."""
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


def _case(H_Q, H_KV, cap, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    return dict(q=(scale * rn(H_Q, 128)).to(BF).cuda(), k=rn(H_KV, cap, 128).to(BF).cuda(), v=rn(H_KV, cap, 128).to(BF).cuda(),
                kn=rn(H_KV, 128).to(BF).cuda(), vn=rn(H_KV, 128).to(BF).cuda())


def _close(got, want, what):
    """fp32 accumulation in another order than the oracle's, then one bf16 rounding: a few units of the last bf16 place
    of the largest output of the head (the outputs of a head are an average of the same V rows, so they share a scale)."""
    err = (got.float().cpu() - want).abs()
    tol = want.abs().amax(dim=-1, keepdim=True) * 2.0 ** -7 + 1e-6
    assert bool((err <= tol).all()), (what, err.max().item(), tol.min().item())


@pytest.mark.parametrize("H_Q,H_KV,S,cap", [(40, 8, 512, 1024), (40, 8, 1, 64), (40, 8, 63, 64), (40, 8, 65, 128), (40, 8, 1024, 1025), (40, 8, 1025, 1100), (40, 8, 5000, 5001), (40, 8, 40000, 40001),
                                            (4, 2, 39, 40), (8, 8, 200, 256), (16, 2, 130, 256), (8, 2, 4097, 8192)])
def test_against_the_oracle(ops, H_Q, H_KV, S, cap):
    c = _case(H_Q, H_KV, cap, seed=H_Q * 100 + S, scale=3.0)        # larger logits: a peaked softmax
    want = og.sdpa_decode(c["q"].cpu(), c["k"].cpu(), c["v"].cpu(), S)
    k, v = c["k"].clone(), c["v"].clone()
    out = ops.sdpa_decode(c["q"], k, v, c["kn"], c["vn"], S)
    torch.cuda.synchronize()
    _close(out, want, "output")
    # the append: position S holds the new rows, nothing else changed
    assert torch.equal(k[:, S].view(torch.int16), c["kn"].view(torch.int16)) and torch.equal(v[:, S].view(torch.int16), c["vn"].view(torch.int16))
    k[:, S], v[:, S] = c["k"][:, S], c["v"][:, S]
    assert torch.equal(k.view(torch.int16), c["k"].view(torch.int16)) and torch.equal(v.view(torch.int16), c["v"].view(torch.int16))


def test_empty_cache_gives_zero_and_still_appends(ops):
    c = _case(40, 8, 16, seed=2)
    k, v = c["k"].clone(), c["v"].clone()
    out = ops.sdpa_decode(c["q"], k, v, c["kn"], c["vn"], 0)
    assert torch.count_nonzero(out).item() == 0
    assert torch.equal(k[:, 0].view(torch.int16), c["kn"].view(torch.int16))


def test_against_the_reference_kernels_over_appended_tokens(ops, ref_kernels):
    if ref_kernels is None or not hasattr(ref_kernels, "ref_sdpa_decode_bf16"):
        pytest.skip("oracle/_ref/libnemotron_ref.so not built with the attention door (needs the reference checkout at build time)")
    ref_kernels.ref_set_device(torch.cuda.current_device())
    for H_Q, H_KV, S0, cap in ((40, 8, 300, 512), (4, 2, 20, 64)):
        c = _case(H_Q, H_KV, cap, seed=9)
        mine_k, mine_v, ref_k, ref_v = c["k"].clone(), c["v"].clone(), c["k"].clone(), c["v"].clone()
        o_ref = torch.empty(H_Q, 128, dtype=BF, device="cuda")
        gen = torch.Generator().manual_seed(4)
        for step in range(5):                                      # the caches grow by one row per token
            q = torch.randn(H_Q, 128, generator=gen).to(BF).cuda()
            kn, vn = torch.randn(H_KV, 128, generator=gen).to(BF).cuda(), torch.randn(H_KV, 128, generator=gen).to(BF).cuda()
            o = ops.sdpa_decode(q, mine_k, mine_v, kn, vn, S0 + step)
            assert ref_kernels.ref_sdpa_decode_bf16(p(q), p(ref_k), p(ref_v), p(o_ref), p(kn), p(vn), S0 + step, cap, H_Q, H_KV, None) == 0
            torch.cuda.synchronize()
            assert torch.equal(mine_k.view(torch.int16), ref_k.view(torch.int16)) and torch.equal(mine_v.view(torch.int16), ref_v.view(torch.int16))
            _close(o, o_ref.float().cpu(), (H_Q, step))


def test_rejections(built_lib):
    c = _case(40, 8, 64, seed=1)
    out = torch.empty(40, 128, dtype=BF, device="cuda")
    ws = torch.empty(built_lib.nmt_sdpa_decode_workspace_bytes(32, 40), dtype=torch.uint8, device="cuda")
    call = lambda *a: built_lib.nmt_sdpa_decode_bf16(p(c["q"]), p(c["k"]), p(c["v"]), p(out), p(c["kn"]), p(c["vn"]), *a)  # noqa: E731
    before = built_lib.nmt_launch_count()
    assert call(32, 64, 40, 8, 64, p(ws), None) == 5               # head size other than 128
    assert call(32, 64, 40, 7, 128, p(ws), None) == 3              # heads not a multiple of kv heads
    assert call(32, 64, 24, 8, 128, p(ws), None) == 5              # 3 query heads per kv head: no kernel
    assert call(64, 64, 40, 8, 128, p(ws), None) == 3              # no room for the new row
    assert call(32, 64, 40, 8, 128, None, None) == 1
    assert built_lib.nmt_launch_count() == before
    assert built_lib.nmt_sdpa_decode_workspace_bytes(512, 40) == 40 * 16 * 130 * 4
