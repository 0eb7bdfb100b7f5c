"""Randomly drawn shapes (fixed seed) for every op on the path, against the torch golden formulation: the
parametrised tests pin the model's and the benchmark's shapes, this one walks the space in between - odd row
counts, widths that leave ragged last vectors per thread, group sizes that are not powers of two."""
import numpy as np
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


def _ulp_ok(got, want, what):
    rep = og.ulp_report(got, want)
    assert rep["max_ulp"] <= 1 and rep["mismatch_frac"] <= 0.05, (what, rep)


def test_random_norm_shapes(ops):
    rng = np.random.default_rng(20240)
    for _ in range(40):
        rows = int(rng.integers(1, 70))
        cols = 8 * int(rng.integers(1, 2600))                       # up to 20,800 columns
        g = torch.Generator().manual_seed(rows * 7919 + cols)
        x = (float(rng.uniform(0.05, 30)) * torch.randn(rows, cols, generator=g)).to(BF)
        r = torch.randn(rows, cols, generator=g).to(BF)
        w = og.norm_weight(cols, g)
        want_res, want = og.add_rmsnorm_bf16(x, r, w)
        got_res, got = ops.add_rmsnorm(x.cuda(), r.cuda(), w.cuda())
        assert torch.equal(got_res.cpu(), want_res), (rows, cols)
        _ulp_ok(got, want, ("add_rmsnorm", rows, cols))
        _ulp_ok(ops.rmsnorm(x.cuda(), w.cuda()), og.rmsnorm_bf16(x, w), ("rmsnorm", rows, cols))


def test_random_gated_shapes(ops):
    rng = np.random.default_rng(20241)
    for _ in range(40):
        rows = int(rng.integers(1, 40))
        gs = 8 * int(rng.integers(1, 257))                          # group size up to 2048, any multiple of 8
        groups = int(rng.integers(1, 13))
        cols = gs * groups
        g = torch.Generator().manual_seed(rows * 104729 + cols + gs)
        y = torch.randn(rows, cols, generator=g).to(BF)
        z = (float(rng.uniform(0.2, 6)) * torch.randn(rows, cols, generator=g)).to(BF)
        w = og.norm_weight(cols, g)
        _ulp_ok(ops.rmsnorm_gated(y.cuda(), z.cuda(), w.cuda(), gs), og.gated_rmsnorm_bf16(y, z, w, gs), ("gated", rows, cols, gs))


def test_random_elementwise_and_gather_shapes(ops):
    rng = np.random.default_rng(20242)
    for _ in range(40):
        n = 8 * int(rng.integers(1, 300000))
        g = torch.Generator().manual_seed(n)
        a = (3 * torch.randn(n, generator=g)).to(BF)
        b = torch.randn(n, generator=g).to(BF)
        assert torch.equal(ops.relu2(a.cuda()).cpu().view(torch.int16), og.relu2_bf16(a).view(torch.int16)), n
        assert torch.equal(ops.add(a.cuda(), b.cuda()).cpu().view(torch.int16), og.add_bf16(a, b).view(torch.int16)), n
    for _ in range(20):
        vocab = int(rng.integers(1, 5000))
        hidden = 8 * int(rng.integers(1, 700))
        T = int(rng.integers(1, 6000))
        g = torch.Generator().manual_seed(vocab * 31 + hidden + T)
        table = torch.randn(vocab, hidden, generator=g).to(BF)
        dtype = torch.int32 if rng.integers(0, 2) else torch.int64
        ids = torch.randint(0, vocab, (T,), generator=g).to(dtype)
        got = ops.embedding(table.cuda(), ids.cuda()).cpu()
        assert torch.equal(got.view(torch.int16), og.embedding(ids.long(), table).view(torch.int16)), (vocab, hidden, T)
