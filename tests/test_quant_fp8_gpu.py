"""Per-tensor e4m3 activation quantisation, alone and fused with the op that produces its input.  The unfused
quantiser restates ops/gemm.cuh:257-307 operation for operation and must be bit-exact; the fused forms must
equal "this library's op -> bf16 tensor -> quantiser" bit for bit and the golden composition within the norm's
one-ulp tolerance."""
import ctypes
import os

import pytest
import torch

from conftest import ROOT
from oracle import torch_golden as og

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def ops(built_lib):
    from nemotron_infer_b200 import ops as _ops
    built_lib.nmt_set_device(torch.cuda.current_device())
    return _ops


def bytes_of(t):
    return t.contiguous().view(torch.uint8).cpu()


@pytest.mark.parametrize("shape,scale", [((8192, 3136), 1.0), ((64, 12544), 30.0), ((1, 8), 1e-3), ((333, 24), 1e4)])
def test_quantizer_is_bit_exact(ops, shape, scale):
    g = torch.Generator().manual_seed(shape[0] + shape[1])
    x = (scale * torch.randn(*shape, generator=g)).to(BF)
    want_q, want_s = og.quantize_fp8(x)
    q, s = ops.quantize_fp8(x.cuda())
    assert float(s.item()) == float(want_s)
    assert torch.equal(bytes_of(q), bytes_of(want_q))


def test_quantizer_edge_cases(ops):
    z = torch.zeros(16, 64, dtype=BF)
    q, s = ops.quantize_fp8(z.cuda())
    assert float(s.item()) == pytest.approx(1.0 / 448.0, rel=1e-7) and int(bytes_of(q).sum()) == 0
    x = torch.tensor([448.0, -448.0, 1.0, -0.0, 3e38, -3e38, 1e-30, 0.5], dtype=BF)   # huge range: small values flush
    want_q, want_s = og.quantize_fp8(x)
    q, s = ops.quantize_fp8(x.cuda())
    assert float(s.item()) == float(want_s) and torch.equal(bytes_of(q), bytes_of(want_q))
    q, s = ops.quantize_fp8(torch.empty(0, 8, dtype=BF, device="cuda"))
    assert q.numel() == 0


def test_quantizer_matches_reference_kernels(ops):
    path = os.path.join(ROOT, "oracle", "_ref", "libref_blocks_stock.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libref_blocks_stock.so not built")
    R = ctypes.CDLL(path)
    R.blk_set_device(torch.cuda.current_device())
    x = (3 * torch.randn(4096, 3136, generator=torch.Generator().manual_seed(1))).to(BF).cuda()
    ref_q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device="cuda")
    ref_s = torch.zeros(1, device="cuda")
    amax = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    assert R.blk_quantize_activation_fp8(p(x), p(ref_q), p(ref_s), p(amax), ctypes.c_size_t(x.numel())) == 0
    torch.cuda.synchronize()
    q, s = ops.quantize_fp8(x)
    assert float(s.item()) == float(ref_s.item())
    assert torch.equal(bytes_of(q), bytes_of(ref_q))


def test_relu2_quant_equals_relu2_then_quant(ops):
    u = og.cfg3_inputs(2048)
    want_q, want_s = og.quantize_fp8(og.relu2_bf16(u))
    q, s = ops.quantize_fp8(u.cuda(), relu2_first=True)
    assert float(s.item()) == float(want_s)
    assert torch.equal(bytes_of(q), bytes_of(want_q))
    neg = -u.abs()                                     # nothing survives the relu: all-zero tensor, scale 1/448
    q, s = ops.quantize_fp8(neg.cuda(), relu2_first=True)
    assert int(bytes_of(q).sum()) == 0 and float(s.item()) == pytest.approx(1.0 / 448.0, rel=1e-7)


@pytest.mark.parametrize("T,cols", [(8192, 3136), (1, 3136), (77, 1024), (5, 64), (300, 4096), (40, 12544)])
def test_norm_quant_fused_equals_unfused_and_golden(ops, T, cols):
    x, r, w = og.cfg1_inputs(T, cols)
    xd, rd, wd = x.cuda(), r.cuda(), w.cuda()
    # fused: residual add + norm + quantise
    res, q, s = ops.rmsnorm_quant_fp8(xd, wd, r=rd)
    # this library, unfused: the same arithmetic through a bf16 tensor
    res2, normed2 = ops.add_rmsnorm(xd, rd, wd)
    q2, s2 = ops.quantize_fp8(normed2)
    assert torch.equal(res.view(torch.int16), res2.view(torch.int16))
    assert float(s.item()) == float(s2.item())
    assert torch.equal(bytes_of(q), bytes_of(q2)), "fusion must not change a single byte"
    # golden composition: the norm may sit one bf16 ulp away, so the scale may move by one bf16 step of the maximum
    want_res, want_normed = og.add_rmsnorm_bf16(x, r, w)
    want_q, want_s = og.quantize_fp8(want_normed)
    assert torch.equal(res.cpu(), want_res)
    assert abs(float(s.item()) - float(want_s)) <= float(want_s) * 2.0 ** -7
    d = (og.e4m3_ordered(q.cpu()) - og.e4m3_ordered(want_q)).abs()
    assert int(d.max()) <= 1
    if float(s.item()) == float(want_s):
        assert float((d != 0).float().mean()) < 0.02
    # plain norm + quantise
    q3, s3 = ops.rmsnorm_quant_fp8(xd, wd)
    q4, s4 = ops.quantize_fp8(ops.rmsnorm(xd, wd))
    assert float(s3.item()) == float(s4.item()) and torch.equal(bytes_of(q3), bytes_of(q4))


@pytest.mark.parametrize("cols", [20480, 20488, 24576, 32768])
def test_norm_quant_wide_rows_follow_the_unfused_norms_summation_order(ops, cols):
    """Plain norms of 20,488 - 32,768 columns run in a kernel that adds the warps' partial sums as a butterfly, the
    narrower ones (and every fused add + norm) sequentially; the quantiser's statistics pass must add in the same
    order or rstd can differ in its last bit.  Many rows make a last-bit difference show."""
    T = 512
    x, r, w = og.cfg1_inputs(T, cols)
    xd, rd, wd = x.cuda(), r.cuda(), w.cuda()
    q, s = ops.rmsnorm_quant_fp8(xd, wd)
    q2, s2 = ops.quantize_fp8(ops.rmsnorm(xd, wd))
    assert float(s.item()) == float(s2.item()) and torch.equal(bytes_of(q), bytes_of(q2)), "plain norm + quantise"
    res, q, s = ops.rmsnorm_quant_fp8(xd, wd, r=rd)
    res2, normed2 = ops.add_rmsnorm(xd, rd, wd)
    q2, s2 = ops.quantize_fp8(normed2)
    assert torch.equal(res.view(torch.int16), res2.view(torch.int16))
    assert float(s.item()) == float(s2.item()) and torch.equal(bytes_of(q), bytes_of(q2)), "add + norm + quantise"


@pytest.mark.parametrize("qrows", [1, 2, 4])
def test_norm_quant_pass_layouts_agree(ops, qrows):
    """The e4m3 pass handles 1, 2 or 4 rows per CTA: same bytes from all, including from a source that is only
    16-byte aligned."""
    try:
        ops.tune("quant.rows_per_cta", qrows)
        for T, cols in ((1027, 3136), (3, 16), (50, 4096), (9, 8200)):
            x, r, w = og.cfg1_inputs(T, cols)
            xd, rd, wd = x.cuda(), r.cuda(), w.cuda()
            res, q, s = ops.rmsnorm_quant_fp8(xd, wd, r=rd)
            _, normed = ops.add_rmsnorm(xd, rd, wd)
            q2, s2 = ops.quantize_fp8(normed)
            assert float(s.item()) == float(s2.item()) and torch.equal(bytes_of(q), bytes_of(q2)), (T, cols)
            # 16-byte aligned but not 32-byte aligned x (plain norm + quant reads x in pass 2)
            buf = torch.empty(T * cols + 8, dtype=BF, device="cuda")
            xo = buf[8:].view(T, cols)
            xo.copy_(xd)
            assert xo.data_ptr() % 32 == 16
            q3, s3 = ops.rmsnorm_quant_fp8(xo, wd)
            q4, s4 = ops.quantize_fp8(ops.rmsnorm(xd, wd))
            assert float(s3.item()) == float(s4.item()) and torch.equal(bytes_of(q3), bytes_of(q4)), (T, cols)
    finally:
        ops.tune("quant.rows_per_cta", 0)


@pytest.mark.parametrize("T,cols,gs", [(4096, 6144, 768), (300, 7680, 960), (7, 192, 64), (5, 120, 12), (3, 8192, 4096)])
def test_gated_norm_quant_equals_gated_then_quant(ops, T, cols, gs):
    y, z, w = og.cfg2_inputs(T, cols)
    yd, zd, wd = y.cuda(), z.cuda(), w.cuda()
    out, q, s = ops.rmsnorm_gated_quant_fp8(yd, zd, wd, gs)
    out2 = ops.rmsnorm_gated(yd, zd, wd, gs)
    q2, s2 = ops.quantize_fp8(out2)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
    assert float(s.item()) == float(s2.item()) and torch.equal(bytes_of(q), bytes_of(q2))
    want_q, want_s = og.quantize_fp8(og.gated_rmsnorm_bf16(y, z, w, gs))
    assert abs(float(s.item()) - float(want_s)) <= float(want_s) * 2.0 ** -7
    assert int((og.e4m3_ordered(q.cpu()) - og.e4m3_ordered(want_q)).abs().max()) <= 1


def test_norm_quant_in_place_residual_and_reused_workspace(ops):
    x, r, w = og.cfg1_inputs(513)
    ws = ops.fp8_workspace(513, "cuda")
    ws.fill_(0xFF)                                      # the workspace needs no initialisation
    xd = x.cuda()
    res, q, s = ops.rmsnorm_quant_fp8(xd, w.cuda(), r=r.cuda(), out_res=xd, workspace=ws)
    res2, normed2 = ops.add_rmsnorm(x.cuda(), r.cuda(), w.cuda())
    q2, s2 = ops.quantize_fp8(normed2)
    assert torch.equal(xd.view(torch.int16), res2.view(torch.int16))
    assert float(s.item()) == float(s2.item()) and torch.equal(bytes_of(q), bytes_of(q2))
    # second call on the same workspace with smaller values: the running maximum must start from zero again
    xs = (0.01 * x.float()).to(BF).cuda()
    q5, s5 = ops.rmsnorm_quant_fp8(xs, w.cuda(), workspace=ws)
    q6, s6 = ops.quantize_fp8(ops.rmsnorm(xs, w.cuda()))
    assert float(s5.item()) == float(s6.item()) and torch.equal(bytes_of(q5), bytes_of(q6))
