"""The allocation-free form of the fused add + RMSNorm + e4m3 quantiser, called through the C ABI.

`nmt_add_rmsnorm_quant_fp8_static` is for hosts that have no way to hand the library a workspace: the reference's
engine refuses to call cudaMalloc / cudaFree between layers, a bare foreign-function binding owns no device
allocator, and a server whose memory is fully committed cannot count on a late allocation.  Its scratch is an
array inside the library, shared by every call, so this test runs it twice in a row (with the larger values
FIRST, so that a running maximum left over from call one would be caught in call two) and requires both results
to be identical, byte for byte, to the workspace form `nmt_add_rmsnorm_quant_fp8`.

This file sorts last on purpose: a run that stops at the first failure has by then run every other test.
"""
import pytest
import torch

from oracle import torch_golden as og

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
MAX_ROWS = 65536            # NMT_STATIC_SCRATCH_MAX_ROWS in include/nemotron_b200.h


def _run_both(lib, x, r, w):
    """Calls the workspace form and the static form on the same inputs; returns their outputs."""
    rows, cols = x.shape
    outs = []
    for static in (False, True):
        res = torch.empty_like(x)
        q = torch.zeros(rows, cols, dtype=torch.float8_e4m3fn, device=x.device)
        scale = torch.zeros(1, device=x.device)
        if static:
            st = lib.nmt_add_rmsnorm_quant_fp8_static(x.data_ptr(), r.data_ptr(), w.data_ptr(), res.data_ptr(),
                                                      q.data_ptr(), scale.data_ptr(), rows, cols, 1e-5, None)
        else:
            ws = torch.empty(int(lib.nmt_fp8_workspace_bytes(rows)), dtype=torch.uint8, device=x.device)
            st = lib.nmt_add_rmsnorm_quant_fp8(x.data_ptr(), r.data_ptr(), w.data_ptr(), res.data_ptr(), q.data_ptr(),
                                               scale.data_ptr(), ws.data_ptr(), rows, cols, 1e-5, None)
        assert st == 0, lib.nmt_status_string(st)
        torch.cuda.synchronize()
        outs.append((res, q.view(torch.uint8), float(scale.item())))
    return outs


def test_static_scratch_form_matches_workspace_form_twice_in_a_row(built_lib):
    lib = built_lib
    assert lib.nmt_set_device(torch.cuda.current_device()) == 0
    x, r, w = (t.cuda() for t in og.cfg1_inputs(1500))
    first = (8.0 * x.float()).to(BF), r, w                        # call 1: large magnitudes
    second = (0.05 * x.float()).to(BF)[:333].contiguous(), (0.05 * r.float()).to(BF)[:333].contiguous(), w   # call 2: smaller, fewer rows
    for args in (first, second):
        (res_ws, q_ws, s_ws), (res_st, q_st, s_st) = _run_both(lib, *args)
        assert torch.equal(res_st.view(torch.int16), res_ws.view(torch.int16))
        assert s_st == s_ws and s_st > 0.0
        assert torch.equal(q_st, q_ws)
    # and the second call really used its own maximum, not the first call's
    assert _run_both(lib, *second)[1][2] < _run_both(lib, *first)[1][2]


def test_static_scratch_form_at_exactly_the_row_limit(built_lib):
    """rows == NMT_STATIC_SCRATCH_MAX_ROWS writes the last float of the built-in array: the only size at which a
    miscounted array length would show.  Narrow rows keep the case at about a megabyte per tensor."""
    lib = built_lib
    assert lib.nmt_set_device(torch.cuda.current_device()) == 0
    g = torch.Generator().manual_seed(65536)
    x = torch.randn(MAX_ROWS, 8, generator=g).to(BF).cuda()
    r = torch.randn(MAX_ROWS, 8, generator=g).to(BF).cuda()
    x[MAX_ROWS - 1] = 3.0 * x[MAX_ROWS - 1]                      # the last row carries a rstd of its own
    w = og.norm_weight(8, g).cuda()
    for _ in range(2):
        (res_ws, q_ws, s_ws), (res_st, q_st, s_st) = _run_both(lib, x, r, w)
        assert torch.equal(res_st.view(torch.int16), res_ws.view(torch.int16))
        assert s_st == s_ws and s_st > 0.0
        assert torch.equal(q_st, q_ws)
    want_res, want = og.add_rmsnorm_bf16(x.cpu(), r.cpu(), w.cpu())
    q_want, s_want = og.quantize_fp8(want)
    assert torch.equal(res_st.cpu().view(torch.int16), want_res.view(torch.int16))
    assert abs(s_st - float(s_want)) <= 1e-6 * float(s_want) + 1e-12


def test_static_scratch_form_rejects_too_many_rows_and_allocates_nothing(built_lib):
    lib = built_lib
    lib.nmt_set_device(torch.cuda.current_device())
    x, r, w = (t.cuda() for t in og.cfg1_inputs(64))
    res = torch.empty_like(x)
    q = torch.empty(64, 3136, dtype=torch.float8_e4m3fn, device="cuda")
    scale = torch.zeros(1, device="cuda")
    launches = lib.nmt_launch_count()
    st = lib.nmt_add_rmsnorm_quant_fp8_static(x.data_ptr(), r.data_ptr(), w.data_ptr(), res.data_ptr(), q.data_ptr(),
                                              scale.data_ptr(), MAX_ROWS + 1, 3136, 1e-5, None)
    assert st == 6 and b"NMT_STATIC_SCRATCH_MAX_ROWS" in lib.nmt_status_string(st)
    assert lib.nmt_launch_count() == launches, "a rejected call launches nothing"
    # (one call first, so that the driver has loaded the kernels' code before free memory is sampled)
    assert lib.nmt_add_rmsnorm_quant_fp8_static(x.data_ptr(), r.data_ptr(), w.data_ptr(), res.data_ptr(), q.data_ptr(),
                                                scale.data_ptr(), 64, 3136, 1e-5, None) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    st = lib.nmt_add_rmsnorm_quant_fp8_static(x.data_ptr(), r.data_ptr(), w.data_ptr(), res.data_ptr(), q.data_ptr(),
                                              scale.data_ptr(), 64, 3136, 1e-5, None)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert st == 0 and free_after == free_before, "the call must not take device memory"
