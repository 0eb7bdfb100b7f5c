"""Pins the CPU oracle (oracle/torch_golden.py, oracle/ref_loops.c) to fixtures that the reference's own
code produced (tests/golden/make_golden.py): the unmodified dump scripts and the lifted golden functions."""
import numpy as np
import torch

from conftest import bf16_from_bits, fptr, golden
from oracle import torch_golden as og


def _t(a):
    return torch.from_numpy(np.asarray(a).copy())


def test_plain_rmsnorm_matches_mlp_dump_stage():
    d = golden("dump_mlp_block.npz")
    x = _t(d["input"]).reshape(8, 64)
    got = og.plain_rmsnorm(x, _t(d["block_norm_w"]))
    torch.testing.assert_close(got.reshape(-1), _t(d["normed"]), rtol=1e-6, atol=1e-6)


def test_relu2_and_residual_match_mlp_dump_stages():
    d = golden("dump_mlp_block.npz")
    torch.testing.assert_close(og.relu2(_t(d["up"])), _t(d["act"]), rtol=0, atol=0)
    torch.testing.assert_close(og.residual_add(_t(d["input"]), _t(d["down"])), _t(d["expected"]), rtol=0, atol=0)


def test_mlp_block_formula_matches_mlp_dump_output():
    d = golden("dump_mlp_block.npz")
    got = og.mlp_block(_t(d["input"]).reshape(8, 64), _t(d["block_norm_w"]), _t(d["up_proj_w"]).reshape(256, 64),
                       _t(d["down_proj_w"]).reshape(64, 256))
    torch.testing.assert_close(got.reshape(-1), _t(d["expected"]), rtol=1e-5, atol=1e-5)


def test_plain_rmsnorm_matches_attention_dump_stage():
    d = golden("dump_attention_block.npz")
    x = _t(d["input"]).reshape(40, 256)
    torch.testing.assert_close(og.plain_rmsnorm(x, _t(d["block_norm_w"])).reshape(-1), _t(d["normed"]),
                               rtol=1e-6, atol=1e-6)


def test_norms_match_mamba_dump_stages():
    d = golden("dump_mamba_block.npz")
    x = _t(d["input"]).reshape(24, 64)
    torch.testing.assert_close(og.plain_rmsnorm(x, _t(d["block_norm_w"])).reshape(-1), _t(d["normed"]),
                               rtol=1e-6, atol=1e-6)
    y = _t(d["scan_y"]).reshape(24, 64)
    z = _t(d["gate"]).reshape(24, 64)
    got = og.gated_rmsnorm(y, _t(d["gnorm_w"]), z, 32)
    torch.testing.assert_close(got.reshape(-1), _t(d["gnormed"]), rtol=1e-5, atol=1e-6)


def test_conv1d_matches_mamba_dump_stage():
    d = golden("dump_mamba_block.npz")
    x = _t(d["xbc"]).reshape(1, 24, 128)
    got = og.causal_conv1d_silu(x, _t(d["conv1d_w"]).reshape(128, 4), _t(d["conv1d_b"]))
    torch.testing.assert_close(got.reshape(-1), _t(d["xbc_conv"]), rtol=1e-6, atol=1e-6)
    tail = og.conv_state_tail(x)
    assert torch.equal(tail[0, :, 2], x[0, 23]) and torch.equal(tail[0, :, 0], x[0, 21])


def test_cfg0_fp32_rmsnorm_fixture():
    d = golden("cfg0_fp32.npz")
    x, w = og.cfg0_inputs()
    np.testing.assert_array_equal(x[:8].numpy(), d["x"])          # the seeded stream itself is pinned
    np.testing.assert_array_equal(w.numpy(), d["w"])
    torch.testing.assert_close(og.plain_rmsnorm(x[:8], w), _t(d["out"]), rtol=1e-6, atol=1e-6)


def test_bf16_config_fixtures():
    d = golden("cfg_bf16.npz")
    x, r, w = bf16_from_bits(d["cfg1_x"]), bf16_from_bits(d["cfg1_r"]), _t(d["cfg1_w"])
    sx, sr, sw = og.cfg1_inputs(6)
    assert torch.equal(sx, x) and torch.equal(sr, r) and torch.equal(sw, w)
    out_res, out = og.add_rmsnorm_bf16(x, r, w)
    assert torch.equal(out_res, bf16_from_bits(d["cfg1_out_res"]))
    assert og.ulp_report(out, bf16_from_bits(d["cfg1_out"]))["max_ulp"] <= 1
    assert og.ulp_report(og.rmsnorm_bf16(x, w), bf16_from_bits(d["cfg1_plain_out"]))["max_ulp"] <= 1
    for tag, gs in (("cfg2", 768), ("cfg2m", 960)):
        y, z, w = bf16_from_bits(d[f"{tag}_y"]), bf16_from_bits(d[f"{tag}_z"]), _t(d[f"{tag}_w"])
        rep = og.ulp_report(og.gated_rmsnorm_bf16(y, z, w, gs), bf16_from_bits(d[f"{tag}_out"]))
        assert rep["max_ulp"] <= 1 and rep["mismatch_frac"] < 1e-3, rep
    u = bf16_from_bits(d["cfg3_u"])
    assert torch.equal(og.relu2_bf16(u), bf16_from_bits(d["cfg3_out"]))
    table, ids = bf16_from_bits(d["cfg4_table"]), _t(d["cfg4_ids"])
    assert torch.equal(og.embedding(ids, table), bf16_from_bits(d["cfg4_out"]))


def test_bf16_add_is_single_rounding():
    # The fused kernel adds in fp32 and rounds once; torch's bf16 add must agree bit for bit.
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(1 << 16, generator=g) * torch.logspace(-6, 6, 1 << 16)).to(torch.bfloat16)
    b = torch.randn(1 << 16, generator=g).to(torch.bfloat16)
    assert torch.equal(og.add_bf16(a, b), a + b)


def test_ulp_distance_helper():
    bf = torch.bfloat16
    a = torch.tensor([1.0, -1.0, 0.0, -0.0, float("nan"), 1.0], dtype=bf)
    b = torch.tensor([1.0078125, -1.0078125, -0.0, 0.0, float("nan"), float("nan")], dtype=bf)
    assert og.bf16_ulp_distance(a, b).tolist() == [1, 1, 0, 0, 0, 1 << 16]


def test_c_restatement_agrees_with_torch_formulation(oracle_c):
    rng = np.random.default_rng(0)
    rows, cols, gs = 5, 192, 64
    x = rng.uniform(-3, 3, (rows, cols)).astype(np.float32)
    z = rng.uniform(-2, 2, (rows, cols)).astype(np.float32)
    w = rng.uniform(-1.5, 1.5, cols).astype(np.float32)
    y = np.empty_like(x)
    oracle_c.orc_rmsnorm_f32(fptr(x), fptr(y), fptr(w), rows, cols, 1e-5)
    np.testing.assert_allclose(y, og.plain_rmsnorm(_t(x), _t(w)).numpy(), rtol=2e-6, atol=2e-6)
    oracle_c.orc_gated_f32(fptr(x), fptr(y), fptr(w), fptr(z), rows, cols, gs, 1e-5)
    np.testing.assert_allclose(y, og.gated_rmsnorm(_t(x), _t(w), _t(z), gs).numpy(), rtol=3e-6, atol=3e-6)
    oracle_c.orc_relu2_f32(fptr(x), fptr(y), x.size)
    np.testing.assert_array_equal(y, og.relu2(_t(x)).numpy())
    # bf16 rounding helper == torch's round-to-nearest-even
    v = rng.standard_normal(4096).astype(np.float32) * 10.0 ** rng.integers(-20, 20, 4096).astype(np.float32)
    got = np.array([oracle_c.orc_bf16_round(float(t)) for t in v], dtype=np.float32)
    np.testing.assert_array_equal(got, _t(v).to(torch.bfloat16).float().numpy())
    # the bf16 loop (w quantised to bf16, as the reference's test does) stays within its 0.5 tolerance
    # of the torch formulation, and within 2 ulp where |w| is exactly representable
    wq = _t(w).to(torch.bfloat16).float().numpy()
    oracle_c.orc_rmsnorm_bf16(fptr(x), fptr(y), fptr(wq), rows, cols, 1e-5)
    ref = og.rmsnorm_bf16(_t(x).to(torch.bfloat16), _t(wq))
    assert og.ulp_report(_t(y).to(torch.bfloat16), ref)["max_ulp"] <= 1


def test_c_embedding_loop(oracle_c):
    import ctypes
    d = golden("cfg_bf16.npz")
    table, ids = d["cfg4_table"].astype(np.uint16), d["cfg4_ids"].astype(np.int64)
    out = np.zeros((ids.size, table.shape[1]), dtype=np.uint16)
    oracle_c.orc_embedding_u16(table.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)),
                               ids.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                               out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), ids.size, table.shape[1])
    np.testing.assert_array_equal(out, d["cfg4_out"])


def test_ssm_decode_step_iterated_reproduces_the_dump_scripts_scan():
    """The single-token recurrence (oracle of ops/mamba2/ssm.cuh:43-103), stepped over the 24 tokens of
    tools/dump_mamba_block.py from a zero state, must give the chunked scan's output `scan_y` of that script: x, B, C from
    its `xbc_conv`, dt from its `normed` and `in_proj_w` (the last H rows), A_log / D / dt_bias as dumped."""
    d = golden("dump_mamba_block.npz")
    H, P, N, G, S, INTER, CONV, HID = 4, 16, 16, 2, 24, 64, 128, 64
    f = lambda k, *shape: torch.from_numpy(d[k].copy()).reshape(*shape)  # noqa: E731
    conv = f("xbc_conv", S, CONV)
    proj_dt = f("normed", S, HID) @ f("in_proj_w", INTER + CONV + H, HID)[INTER + CONV:].T
    A_log, D, dt_bias = f("A_log", H), f("D", H), f("dt_bias", H)
    state = torch.zeros(H, P, N)
    ys = []
    for t in range(S):
        x, B, C = conv[t, :INTER].reshape(H, P), conv[t, INTER:INTER + G * N].reshape(G, N), conv[t, INTER + G * N:].reshape(G, N)
        y, state = og.ssm_decode_step(x, proj_dt[t], A_log, B, C, D, state, dt_bias)
        ys.append(y.reshape(INTER))
    got = torch.stack(ys)
    want = f("scan_y", S, INTER)
    assert (got - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())
