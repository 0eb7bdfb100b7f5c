"""The reference's whole pybind module (nemotron_infer/csrc/include/binding.cu, unmodified) built by oracle/Makefile
twice: on its own kernels, and with include/nemotron_b200_shim/model/blocks_b200.cuh pre-included, i.e. as the drop-in
a maintainer would ship.  Both must offer the 16 functions and the constants of binding.cu:214-245 and agree on the
block outputs at model width; on the drop-in the hot-path ops must be this library's launches, and a layer loop
driven the way engine.py:254-272 drives it must fuse its block boundaries once the next norm weight is announced."""
import importlib.util
import os

import pytest
import torch

from blocks_common import BF, fp8_rows, fusion_counters, rel_l2
from conftest import ROOT

NAMES = ["reset_allocator", "free_allocator", "sync", "embedding", "rmsnorm", "lm_head", "mamba_forward", "mamba_decode",
         "attn_forward", "attn_decode", "mlp_forward", "mamba_forward_fp8", "mamba_decode_fp8", "attn_forward_fp8",
         "attn_decode_fp8", "mlp_forward_fp8"]
CONSTANTS = dict(HIDDEN=3136, H=96, P=80, N=128, G=8, CONV_K=4, H_Q=40, H_KV=8, HEAD=128, INTER=12544, VOCAB=131072,
                 CONV_DIM=9728, IN_PROJ=17504)
_MODS = {}


def load_binding(kind):
    """kind: 'stock' | 'b200'.  The drop-in is a module called `binding`, like the reference's; the stock build was given
    the module name `binding_stock` at compile time, because pybind11 keeps one module per name in a process."""
    if kind in _MODS:
        return _MODS[kind]
    name = "binding" if kind == "b200" else "binding_stock"
    path = os.path.join(ROOT, "oracle", "_ref", "binding_b200", "binding.so") if kind == "b200" else \
        os.path.join(ROOT, "oracle", "_ref", "binding_stock.so")
    if not os.path.exists(path):
        pytest.skip(f"{path} not built (needs the reference checkout at build time: make -C oracle binding)")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _MODS[kind] = mod
    return mod


@pytest.mark.parametrize("kind", ["stock", "b200"])
def test_module_offers_the_reference_surface(kind):
    m = load_binding(kind)
    for name in NAMES:
        assert callable(getattr(m, name)), name
    for name, value in CONSTANTS.items():
        assert getattr(m, name) == value, name
    assert load_binding("stock") is not load_binding("b200")


def _ptr(t):
    return t.data_ptr()


def _weights(seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")  # noqa: E731
    H, I, QD, KD = 3136, 12544, 40 * 128, 8 * 128
    return dict(nw=(1 + 0.1 * rn(H)).contiguous(), up=(0.02 * rn(I, H)).to(BF), down=(0.02 * rn(H, I)).to(BF),
                anw=(1 + 0.1 * rn(H)).contiguous(), q=(0.02 * rn(QD, H)).to(BF), k=(0.02 * rn(KD, H)).to(BF),
                v=(0.02 * rn(KD, H)).to(BF), o=(0.02 * rn(H, QD)).to(BF), nw3=(1 + 0.1 * rn(H)).contiguous())


@pytest.mark.gpu
def test_mlp_and_attention_forward_agree_between_the_two_builds(built_lib):
    stock, b200 = load_binding("stock"), load_binding("b200")
    w = _weights(5)
    S = 64
    x = torch.randn(S, 3136, generator=torch.Generator(device="cuda").manual_seed(6), device="cuda").to(BF)
    outs = {}
    for name, m in (("stock", stock), ("b200", b200)):
        before = built_lib.nmt_launch_count()
        mlp = torch.empty_like(x)
        att = torch.empty_like(x)
        m.reset_allocator()
        m.mlp_forward(_ptr(x), _ptr(w["nw"]), _ptr(w["up"]), _ptr(w["down"]), _ptr(mlp), S)
        m.reset_allocator()
        m.attn_forward(_ptr(x), _ptr(w["anw"]), _ptr(w["q"]), _ptr(w["k"]), _ptr(w["v"]), _ptr(w["o"]), _ptr(att), S, 0, 0, 0)
        m.sync()
        torch.cuda.synchronize()
        m.free_allocator()
        outs[name] = (mlp, att, built_lib.nmt_launch_count() - before)
    assert outs["stock"][2] == 0 and outs["b200"][2] == 5          # mlp: norm, relu^2, add; attention: norm, add
    for i, what in ((0, "mlp_forward"), (1, "attn_forward")):
        assert torch.isfinite(outs["b200"][i].float()).all(), what
        assert rel_l2(outs["b200"][i], outs["stock"][i]) < 5e-3, what
        assert (outs["b200"][i].float() - outs["stock"][i].float()).abs().max().item() < 0.15, what


@pytest.mark.gpu
def test_embedding_and_final_norm_through_the_module(built_lib):
    b200 = load_binding("b200")
    from oracle import torch_golden as og
    g = torch.Generator().manual_seed(8)
    table = (0.02 * torch.randn(4096, 3136, generator=g)).to(BF)         # the module takes no vocabulary size; ids stay below 4096
    ids = torch.randint(0, 4096, (33,), generator=g)
    nw = og.norm_weight(3136, g)
    td, idd, nwd = table.cuda(), ids.cuda(), nw.cuda()
    hidden = torch.empty(33, 3136, dtype=BF, device="cuda")
    normed = torch.empty_like(hidden)
    before = built_lib.nmt_launch_count()
    b200.embedding(_ptr(td), _ptr(idd), _ptr(hidden), 33)
    b200.rmsnorm(_ptr(hidden), _ptr(normed), _ptr(nwd), 33)
    b200.sync()
    torch.cuda.synchronize()
    assert built_lib.nmt_launch_count() - before == 2
    want = og.embedding(ids, table)
    assert torch.equal(hidden.cpu().view(torch.int16), want.view(torch.int16))
    assert og.ulp_report(normed, og.rmsnorm_bf16(want, nw))["max_ulp"] <= 1


@pytest.mark.gpu
def test_layer_loop_fuses_block_boundaries_when_the_next_norm_is_announced(built_lib):
    """Three layers (MLP, attention, MLP) and the final norm, driven like engine.py:254-272 (reset_allocator before every
    layer, hidden ping-pong).  With the next layer's norm weight announced before each block, both inner boundaries
    run as one fused launch and the next block's norm is skipped; the result equals the unannounced loop's."""
    m = load_binding("b200")
    w = _weights(11)
    S = 48
    x = torch.randn(S, 3136, generator=torch.Generator(device="cuda").manual_seed(12), device="cuda").to(BF)
    layers = [("mlp", w["nw"]), ("attn", w["anw"]), ("mlp", w["nw3"])]

    def run(announce):
        built_lib.nmt_fusion_reset()
        hbuf = [x.clone(), torch.empty_like(x)]
        cur, other = hbuf
        for i, (kind, nw) in enumerate(layers):
            m.reset_allocator()
            if announce and i + 1 < len(layers):
                assert built_lib.nmt_fuse_next_norm(layers[i + 1][1].data_ptr(), 1e-5) == 0
            if kind == "mlp":
                m.mlp_forward(_ptr(cur), _ptr(nw), _ptr(w["up"]), _ptr(w["down"]), _ptr(other), S)
            else:
                m.attn_forward(_ptr(cur), _ptr(nw), _ptr(w["q"]), _ptr(w["k"]), _ptr(w["v"]), _ptr(w["o"]), _ptr(other), S, 0, 0, 0)
            cur, other = other, cur
        m.reset_allocator()
        final = torch.empty_like(x)
        m.rmsnorm(_ptr(cur), _ptr(final), _ptr(w["nw"]), S)
        m.sync()
        torch.cuda.synchronize()
        return cur.clone(), final

    run(False)                                   # first pass creates the allocator's slabs
    f0, e0 = fusion_counters(built_lib)
    l0 = built_lib.nmt_launch_count()
    hid_u, fin_u = run(False)
    l1 = built_lib.nmt_launch_count()
    hid_f, fin_f = run(True)
    l2 = built_lib.nmt_launch_count()
    f1, e1 = fusion_counters(built_lib)
    m.free_allocator()
    assert l1 - l0 == 3 + 2 + 3 + 1 and l2 - l1 == (l1 - l0) - 2
    assert (f1 - f0, e1 - e0) == (2, 2)
    assert rel_l2(hid_f, hid_u) < 5e-3 and rel_l2(fin_f, fin_u) < 5e-3
    assert torch.isfinite(fin_f.float()).all()


@pytest.mark.gpu
def test_fp8_mlp_forward_prefill_and_single_token_agree_between_the_two_builds(built_lib):
    stock, b200 = load_binding("stock"), load_binding("b200")
    g = torch.Generator().manual_seed(4)
    nw = (1 + 0.1 * torch.randn(3136, generator=g)).cuda()
    upq, ups = fp8_rows(0.02 * torch.randn(12544, 3136, generator=g))
    downq, downs = fp8_rows(0.02 * torch.randn(3136, 12544, generator=g))
    for M, want_launches in ((32, 5), (1, 2)):
        x = torch.randn(M, 3136, generator=g).to(BF).cuda()
        outs = {}
        for name, m in (("stock", stock), ("b200", b200)):
            before = built_lib.nmt_launch_count()
            out = torch.empty_like(x)
            m.reset_allocator()
            m.mlp_forward_fp8(_ptr(x), _ptr(nw), _ptr(upq), _ptr(ups), _ptr(downq), _ptr(downs), _ptr(out), M)
            m.sync()
            torch.cuda.synchronize()
            m.free_allocator()
            outs[name] = (out, built_lib.nmt_launch_count() - before)
        assert outs["stock"][1] == 0 and outs["b200"][1] == want_launches
        assert rel_l2(outs["b200"][0], outs["stock"][0]) < 2e-2, M
