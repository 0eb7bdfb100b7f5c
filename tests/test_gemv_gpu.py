"""W8A16 GEMV (single-token decode projection) against the reference test's CPU formulation
(tests/ops/test_gemm.cu:505-513), its input recipe and tolerance (:539-589), and the reference's own kernel."""
import ctypes

import pytest
import torch

from oracle import torch_golden as og

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def ops(built_lib):
    from nemotron_infer_b200 import ops as _ops
    built_lib.nmt_set_device(torch.cuda.current_device())
    return _ops


def check(got, want):
    """The reference test's bar (max(0.02, 2 %)) and, tighter, the bf16 rounding of the exact sum: fp32 partial
    sums in a different order may move the result by an ulp only when the sum nearly cancels."""
    got, want = got.float().cpu(), want.float()
    tol = torch.maximum(torch.full_like(want, 0.02), 0.02 * want.abs())
    assert bool(((got - want).abs() <= tol).all())
    rep = og.ulp_report(got.to(BF), want.to(BF))
    assert rep["mismatch_frac"] <= 0.05 and rep["max_ulp"] <= 4, rep


def test_reference_test_recipe(ops):
    N, K = 64, 3136                                  # tests/ops/test_gemm.cu:541-546
    x = ((torch.arange(K) * 13 % 17).float() * 0.1 - 0.8).to(BF)
    Wf = ((torch.arange(N * K) * 7 % 23).float() * 0.05 - 0.55).reshape(N, K)
    W, sc = og.quant_weight_perrow(Wf)
    check(ops.gemv_w8a16(x.cuda(), W.cuda(), sc.cuda()), og.gemv_w8a16(x, W, sc))


@pytest.mark.parametrize("N,K", [(12544, 3136), (3136, 12544), (3136, 7680), (17504, 3136), (1, 16), (7, 48), (33, 8192),
                                 (5, 20000), (131, 4096 + 16)])
def test_model_and_odd_shapes(ops, N, K):
    g = torch.Generator().manual_seed(N + K)
    x = torch.randn(K, generator=g).to(BF)
    W, sc = og.quant_weight_perrow(0.05 * torch.randn(N, K, generator=g))
    check(ops.gemv_w8a16(x.cuda(), W.cuda(), sc.cuda()), og.gemv_w8a16(x, W, sc))


def test_every_e4m3_value_and_split_variants(ops):
    # one row per e4m3 bit pattern (NaN patterns excluded) against a one-hot x: the conversion must be exact
    codes = torch.tensor([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=torch.uint8)
    K = 16
    W = torch.zeros(codes.numel(), K, dtype=torch.uint8)
    W[:, 5] = codes
    W = W.view(torch.float8_e4m3fn)
    x = torch.zeros(K, dtype=BF)
    x[5] = 1.0
    sc = torch.ones(codes.numel())
    got = ops.gemv_w8a16(x.cuda(), W.cuda(), sc.cuda()).cpu().float()
    assert torch.equal(got, W.float()[:, 5])
    g = torch.Generator().manual_seed(3)
    xk = torch.randn(6272, generator=g).to(BF)
    Wk, sk = og.quant_weight_perrow(0.05 * torch.randn(100, 6272, generator=g))
    want = og.gemv_w8a16(xk, Wk, sk)
    try:
        for variant, split, per_sm in ((1, 2, 1), (1, 4, 2), (1, 8, 3), (2, 1, 1), (2, 2, 2), (2, 4, 1), (2, 8, 3)):
            ops.tune("gemv.variant", variant)        # 1 = whole-unit loads, 2 = looped loads
            ops.tune("gemv.split", split)
            ops.tune("gemv.ctas_per_sm", per_sm)
            check(ops.gemv_w8a16(xk.cuda(), Wk.cuda(), sk.cuda()), want)
    finally:
        for k in ("gemv.variant", "gemv.split", "gemv.ctas_per_sm"):
            ops.tune(k, 0)


def test_tensor_core_path_positions_and_codes(ops):
    """K a multiple of 64 takes the mma.sync kernel, whose lanes visit k in a permuted order: a diagonal W against
    an x of distinct values proves W and x use the same permutation, and every e4m3 code converts exactly."""
    codes = torch.tensor([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=torch.uint8)
    for K in (64, 128, 448, 3136):
        N = K
        W = torch.zeros(N, K, dtype=torch.uint8)
        W[torch.arange(N), torch.arange(K)] = codes[torch.arange(N) % codes.numel()]
        W = W.view(torch.float8_e4m3fn)
        x = (1 + (torch.arange(K) % 128).float() / 128).to(BF)           # exact in bf16 and f16, distinct within a chunk pair
        x = x * torch.tensor([1.0, -2.0, 0.5, 4.0])[(torch.arange(K) // 128) % 4].to(BF)
        sc = torch.ones(N)
        got = ops.gemv_w8a16(x.cuda(), W.cuda(), sc.cuda()).cpu()
        want = (W.float()[torch.arange(N), torch.arange(K)] * x.float()).to(BF)
        assert torch.equal(got, want), K


def test_tensor_core_path_keeps_small_elements_of_x_exact(ops):
    """x is staged as f16 after scaling max|x| into [2^14, 2^15): every bf16 element within 2^-28 of the largest keeps
    all 8 significant bits.  One-hot weight rows read single elements of x back, over 18 binades below the maximum and
    every 8-bit significand; the fp32-product kernel (variant 1) must agree."""
    K = 64 * 18
    mant = 1 + (torch.arange(K) % 128).float() / 128                      # every 8-bit significand
    expo = -(torch.arange(K) // 64).float()                               # 2^0 ... 2^-17, 64 elements each
    x = (mant * torch.pow(torch.tensor(2.0), expo)).to(BF)
    x[0] = 1.9921875                                                      # the maximum: 1.1111111b
    W = torch.zeros(K, K)
    W[torch.arange(K), torch.arange(K)] = 1.0
    Wq, sc = W.to(torch.float8_e4m3fn), torch.ones(K)
    try:
        for variant in (3, 1):
            ops.tune("gemv.variant", variant)
            got = ops.gemv_w8a16(x.cuda(), Wq.cuda(), sc.cuda()).float().cpu()
            assert torch.equal(got, x.float()), variant
    finally:
        ops.tune("gemv.variant", 0)


def test_tcgen05_path_splits_x_exactly_within_twelve_binades_of_its_maximum(ops):
    """Variant 5 multiplies the e4m3 weights with x split into two e4m3 terms after scaling max|x| into [128, 256): every
    element within 2^-12 of the largest must come back exactly (all 8 significant bits of the bf16), smaller ones with an
    absolute error of at most 2^-17 of the largest."""
    K = 64 * 18
    mant = 1 + (torch.arange(K) % 128).float() / 128
    expo = -(torch.arange(K) // 64).float()
    x = (mant * torch.pow(torch.tensor(2.0), expo)).to(BF)
    x[0] = 1.9921875
    W = torch.zeros(K, K)
    W[torch.arange(K), torch.arange(K)] = 1.0
    Wq, sc = W.to(torch.float8_e4m3fn), torch.ones(K)
    want = x.float()
    try:
        ops.tune("gemv.variant", 5)
        got = ops.gemv_w8a16(x.cuda(), Wq.cuda(), sc.cuda()).float().cpu()
    finally:
        ops.tune("gemv.variant", 0)
    exact = expo >= -12
    assert torch.equal(got[exact], want[exact])
    assert float((got - want).abs().max()) <= 2.0 ** -17 * 1.9921875


@pytest.mark.parametrize("variant", [3, 5])
@pytest.mark.parametrize("scale", [1e30, 1e-30, 3e4, 2.0 ** -20])
def test_tensor_core_path_x_magnitudes(ops, scale, variant):
    """x is staged as f16 times a power of two taken from max|x|: huge and tiny vectors must come out as accurately
    as ordinary ones."""
    g = torch.Generator().manual_seed(17)
    N, K = 96, 3136
    x = (torch.randn(K, generator=g) * scale).to(BF)
    W, sc = og.quant_weight_perrow(0.05 * torch.randn(N, K, generator=g))
    try:
        ops.tune("gemv.variant", variant)
        got = ops.gemv_w8a16(x.cuda(), W.cuda(), sc.cuda()).float().cpu()
    finally:
        ops.tune("gemv.variant", 0)
    want = og.gemv_w8a16(x, W, sc).float()
    rep = og.ulp_report(got.to(BF), want.to(BF))
    assert rep["mismatch_frac"] <= 0.05 and rep["max_ulp"] <= 4, rep


@pytest.mark.parametrize("N,K", [(40, 64), (9, 192), (300, 16384), (50, 16448), (1000, 512), (17, 32704), (5000, 3136),
                                 (1237, 12544), (333, 7680), (148 * 8 + 1, 128)])
def test_tensor_core_path_slicing(ops, built_lib, N, K):
    """Shapes that exercise one chunk per row, uneven slices, the register-held and re-read x staging, many
    k-streams per tile and ragged last tiles; every stream count the knob allows."""
    g = torch.Generator().manual_seed(N * 7 + K)
    x = torch.randn(K, generator=g).to(BF)
    W, sc = og.quant_weight_perrow(0.05 * torch.randn(N, K, generator=g))
    want = og.gemv_w8a16(x, W, sc)
    try:
        for streams in (0, 1, 2, 4, 8):
            for chunks in (0, 2, 4):
                for per_sm in (0, 1):
                    ops.tune("gemv.streams", streams)
                    ops.tune("gemv.unit_chunks", chunks)
                    ops.tune("gemv.ctas_per_sm", per_sm)
                    check(ops.gemv_w8a16(x.cuda(), W.cuda(), sc.cuda()), want)
        for k in ("gemv.streams", "gemv.unit_chunks", "gemv.ctas_per_sm"):
            ops.tune(k, 0)
        ops.tune("gemv.variant", 5)                  # tcgen05 + TMA; shapes it does not take fall through to the default
        for kparts in (0, 1, 2, 4, 8):
            for stages in (0, 1, 2, 7):
                ops.tune("gemv.kparts", kparts)
                ops.tune("gemv.ring_stages", stages)
                check(ops.gemv_w8a16(x.cuda(), W.cuda(), sc.cuda()), want)
    finally:
        for k in ("gemv.streams", "gemv.unit_chunks", "gemv.ctas_per_sm", "gemv.variant", "gemv.kparts", "gemv.ring_stages"):
            ops.tune(k, 0)
    assert built_lib.nmt_device_wait_timeouts() == 0


@pytest.mark.parametrize("variant", [3, 5])
@pytest.mark.parametrize("N,K", [(12544, 3136), (3136, 12544), (17504, 3136), (3136, 7680), (40, 64), (16, 10240)])
def test_fused_decode_forms_are_byte_identical_to_the_separate_ops(ops, N, K, variant):
    """norm -> GEMV -> relu^2 / residual add as one launch: same bytes as this library's separate kernels, and the
    oracle's composition of the same steps within the GEMV tolerance.  Both tensor-core kernels."""
    ops.tune("gemv.variant", variant)
    try:
        _fused_forms(ops, N, K, variant)
    finally:
        ops.tune("gemv.variant", 0)


def _fused_forms(ops, N, K, variant):
    g = torch.Generator().manual_seed(N + 3 * K)
    x = (2 * torch.randn(K, generator=g)).to(BF)
    nw = og.norm_weight(K, g)
    W, sc = og.quant_weight_perrow(0.05 * torch.randn(N, K, generator=g))
    res = torch.randn(N, generator=g).to(BF)
    xd, nwd, Wd, scd, resd = x.cuda(), nw.cuda(), W.cuda(), sc.cuda(), res.cuda()
    normed = ops.rmsnorm(xd.view(1, K), nwd).view(K)
    y_plain = ops.gemv_w8a16(normed, Wd, scd)
    cases = {
        "norm": (dict(norm_w=nwd), y_plain),
        "norm+relu2": (dict(norm_w=nwd, activation="relu2"), ops.relu2(y_plain)),
        "residual": (dict(residual=resd), ops.add(resd, ops.gemv_w8a16(xd, Wd, scd))),
        "relu2": (dict(activation="relu2"), ops.relu2(ops.gemv_w8a16(xd, Wd, scd))),
        "norm+relu2+residual": (dict(norm_w=nwd, activation="relu2", residual=resd), ops.add(resd, ops.relu2(y_plain))),
    }
    # the norm prologue exists up to 10,240 columns (the model norms 3136); the tcgen05 kernel runs it on four warps: 5,120
    with_norm = K <= (10240 if variant == 3 else 5120)
    for name, (kw, want) in cases.items():
        if "norm" in name and not with_norm:
            continue
        n0 = ops.launch_count()
        got = ops.gemv_w8a16_fused(xd, Wd, scd, **kw)
        assert ops.launch_count() == n0 + 1, name
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), name
    buf = resd.clone()                                   # the residual stream updated in place
    ops.gemv_w8a16_fused(xd, Wd, scd, residual=buf, out=buf)
    assert torch.equal(buf.view(torch.int16), cases["residual"][1].view(torch.int16))
    # oracle composition (torch golden formulation of each step)
    # (the norm may sit one bf16 ulp from the golden's in a few elements, which a nearly cancelling row sum
    # magnifies in ulps, so only the reference test's absolute / relative bar applies here)
    if not with_norm:
        return
    want_n = og.rmsnorm_bf16(x.view(1, K), nw).view(K)
    want_y = og.gemv_w8a16(want_n, W, sc).float()
    got_y = ops.gemv_w8a16_fused(xd, Wd, scd, norm_w=nwd).float().cpu()
    assert bool(((got_y - want_y).abs() <= torch.maximum(torch.full_like(want_y, 0.02), 0.02 * want_y.abs())).all())
    want_mlp = og.relu2_bf16(og.gemv_w8a16(want_n, W, sc).to(BF))
    got_mlp = ops.gemv_w8a16_fused(xd, Wd, scd, norm_w=nwd, activation="relu2").float().cpu()
    tol = torch.maximum(torch.full_like(want_mlp.float(), 0.02), 0.04 * want_mlp.float().abs())     # the square doubles the relative error
    assert bool(((got_mlp - want_mlp.float()).abs() <= tol).all())


def test_fused_gemv_argument_checks(built_lib):
    L = built_lib
    B = 0x7F0000000000
    assert L.nmt_gemv_w8a16_fused(B, B, 1e-5, B, B, 0, B, B, 0, 3136, None) == 0          # N == 0: nothing to do
    assert L.nmt_gemv_w8a16_fused(B, B, 1e-5, B, B, 2, B, B, 4, 3136, None) == 3          # unknown activation
    assert L.nmt_gemv_w8a16_fused(B, B, 1e-5, None, B, 0, B, B, 4, 3136, None) == 1
    assert L.nmt_gemv_w8a16_fused(B + 4, B, 1e-5, B, B, 0, None, B, 4, 3136, None) == 2   # norm prologue wants 16-byte x
    assert L.nmt_gemv_w8a16_fused(B, None, 1e-5, B, B, 0, None, B, 4, 3152, None) == 5    # K % 64 != 0: no fused form
    assert L.nmt_gemv_w8a16_fused(B, B, 1e-5, B, B, 0, None, B, 4, 12544, None) == 5      # norm prologue beyond 10240 columns


def test_against_reference_kernel(ops, ref_kernels):
    if ref_kernels is None or not hasattr(ref_kernels, "ref_gemv_fp8"):
        pytest.skip("reference gemv kernel not built")
    g = torch.Generator().manual_seed(9)
    N, K = 12544, 3136
    x = torch.randn(K, generator=g).to(BF).cuda()
    W, sc = og.quant_weight_perrow(0.05 * torch.randn(N, K, generator=g))
    Wd, sd = W.cuda(), sc.cuda()
    ref = torch.empty(N, dtype=BF, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    ref_kernels.ref_set_device(torch.cuda.current_device())
    assert ref_kernels.ref_gemv_fp8(p(x), p(Wd), p(sd), p(ref), N, K, None) == 0
    torch.cuda.synchronize()
    got = ops.gemv_w8a16(x, Wd, sd)
    rep = og.ulp_report(got, ref)
    assert rep["max_ulp"] <= 4 and rep["mismatch_frac"] <= 0.05, rep


def test_gemv_argument_checks(built_lib):
    L = built_lib
    B = 0x7F0000000000
    assert L.nmt_gemv_w8a16(B, B, B, B, 0, 3136, None) == 0
    assert L.nmt_gemv_w8a16(B, B, B, B, 4, 3130, None) == 3
    assert L.nmt_gemv_w8a16(B, None, B, B, 4, 3136, None) == 1
    assert L.nmt_gemv_w8a16(B, B + 8, B, B, 4, 3136, None) == 2
    assert L.nmt_gemv_w8a16(B, B, B, B, 4, 64000, None) == 5


@pytest.mark.parametrize("N,K,gs,with_res", [(3136, 7680, 960, True), (3136, 7680, 960, False), (64, 64, 32, True), (512, 6144, 768, True),
                                            (130, 1024, 8, True), (77, 2048, 2048, False)])
def test_gated_norm_gemv_equals_the_separate_ops(ops, N, K, gs, with_res):
    """nmt_gemv_w8a16_gated = nmt_rmsnorm_gated_bf16 -> nmt_gemv_w8a16_fused(residual), byte for byte (the Mamba-2 decode
    block's model/mamba_block.cuh:504-514)."""
    g = torch.Generator().manual_seed(N + K + gs)
    y = torch.randn(K, generator=g).to(BF).cuda()
    z = (2 * torch.randn(K, generator=g)).to(BF).cuda()
    gw = (1 + 0.1 * torch.randn(K, generator=g)).cuda()
    Wq, sc = og.quant_weight_perrow(0.05 * torch.randn(N, K, generator=g))
    Wq, sc = Wq.cuda(), sc.cuda()
    res = torch.randn(N, generator=g).to(BF).cuda() if with_res else None
    normed = ops.rmsnorm_gated(y.view(1, K), z.view(1, K), gw, gs).view(K)
    want = ops.gemv_w8a16_fused(normed, Wq, sc, residual=res)
    got = ops.gemv_w8a16_gated(y, z, gw, gs, Wq, sc, residual=res)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_gated_norm_gemv_rejections(built_lib):
    K, N = 1024, 64
    y = torch.zeros(K, dtype=BF, device="cuda")
    gw = torch.ones(K, device="cuda")
    W = torch.zeros(N, K, dtype=torch.float8_e4m3fn, device="cuda")
    sc = torch.ones(N, device="cuda")
    out = torch.zeros(N, dtype=BF, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    call = lambda gs, k=K: built_lib.nmt_gemv_w8a16_gated(p(y), p(y), p(gw), 1e-5, gs, p(W), p(sc), None, p(out), N, k, None)  # noqa: E731
    before = built_lib.nmt_launch_count()
    assert call(100) == 3            # group size not a multiple of 8
    assert call(96) == 3             # does not divide K
    assert call(8, 1000) == 3        # K not a multiple of 64
    assert built_lib.nmt_gemv_w8a16_gated(p(y), None, p(gw), 1e-5, 128, p(W), p(sc), None, p(out), N, K, None) == 1
    assert built_lib.nmt_launch_count() == before


@pytest.mark.parametrize("dims", [dict(HID=3136, INTER=7680, GN=1024, H=96), dict(HID=64, INTER=64, GN=32, H=4)])
def test_in_proj_with_conv_step_equals_the_separate_ops(ops, built_lib, dims):
    """nmt_gemv_w8a16_fused_conv_step = nmt_gemv_w8a16_fused (norm folded in) -> nmt_causal_conv1d_silu_decode_split_bf16,
    byte for byte: x | B | C, the conv window, and the gate / dt rows (model/mamba_block.cuh:473-497), over three tokens."""
    HID, INTER, GN, H = dims["HID"], dims["INTER"], dims["GN"], dims["H"]
    CONV = INTER + 2 * GN
    PROJ = INTER + CONV + H
    g = torch.Generator().manual_seed(HID)
    nw = (1 + 0.1 * torch.randn(HID, generator=g)).cuda()
    Wq, sc = og.quant_weight_perrow(0.05 * torch.randn(PROJ, HID, generator=g))
    Wq, sc = Wq.cuda(), sc.cuda()
    cw, cb = (0.3 * torch.randn(CONV, 4, generator=g)).cuda(), (0.1 * torch.randn(CONV, generator=g)).cuda()
    st_a = (0.5 * torch.randn(1, CONV, 3, generator=g)).cuda()
    st_b = st_a.clone()
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    for _ in range(3):
        x = torch.randn(HID, generator=g).to(BF).cuda()
        proj = ops.gemv_w8a16_fused(x, Wq, sc, norm_w=nw)
        want = ops.causal_conv1d_silu_decode(proj[INTER:INTER + CONV].view(1, CONV), cw, cb, st_a, split=(INTER, GN, GN))
        y = torch.full((PROJ,), 7.0, dtype=BF, device="cuda")
        outs = [torch.empty(n, dtype=BF, device="cuda") for n in (INTER, GN, GN)]
        before = built_lib.nmt_launch_count()
        assert built_lib.nmt_gemv_w8a16_fused_conv_step(p(x), p(nw), 1e-5, p(Wq), p(sc), p(y), PROJ, HID, INTER, p(cw), p(cb), p(st_b),
                                                        p(outs[0]), p(outs[1]), p(outs[2]), INTER, GN, GN, None) == 0
        assert built_lib.nmt_launch_count() - before == 1
        torch.cuda.synchronize()
        for got, w in zip(outs, want):
            assert torch.equal(got.view(torch.int16), w.reshape(-1).view(torch.int16))
        assert torch.equal(st_a, st_b), "conv window"
        assert torch.equal(y[:INTER].view(torch.int16), proj[:INTER].view(torch.int16)), "gate rows"
        assert torch.equal(y[INTER + CONV:].view(torch.int16), proj[INTER + CONV:].view(torch.int16)), "dt rows"
        assert bool((y[INTER:INTER + CONV].float() == 7.0).all()), "the xBC rows are not stored"


def test_conv_step_form_without_conv_rows_is_the_plain_fused_gemv(ops, built_lib):
    N, K = 200, 1024
    g = torch.Generator().manual_seed(12)
    x = torch.randn(K, generator=g).to(BF).cuda()
    nw = (1 + 0.1 * torch.randn(K, generator=g)).cuda()
    Wq, sc = og.quant_weight_perrow(0.05 * torch.randn(N, K, generator=g))
    Wq, sc = Wq.cuda(), sc.cuda()
    want = ops.gemv_w8a16_fused(x, Wq, sc, norm_w=nw)
    y = torch.empty(N, dtype=BF, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    assert built_lib.nmt_gemv_w8a16_fused_conv_step(p(x), p(nw), 1e-5, p(Wq), p(sc), p(y), N, K, 0, None, None, None, None, None, None,
                                                    0, 0, 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(y.view(torch.int16), want.view(torch.int16))
    # a conv range that does not fit the rows is refused, and so is a missing window
    assert built_lib.nmt_gemv_w8a16_fused_conv_step(p(x), p(nw), 1e-5, p(Wq), p(sc), p(y), N, K, 150, p(nw), p(nw), p(nw), p(y), None, None,
                                                    64, 0, 0, None) == 3
    assert built_lib.nmt_gemv_w8a16_fused_conv_step(p(x), p(nw), 1e-5, p(Wq), p(sc), p(y), N, K, 0, p(nw), p(nw), None, p(y), None, None,
                                                    64, 0, 0, None) == 1
