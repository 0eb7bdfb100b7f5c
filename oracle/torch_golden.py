"""TEST INFRASTRUCTURE — the CPU oracle.  Never imported by the product package.

Restates, in torch on the CPU, the formulation of each hot-path op that the
reference's golden emitters use (paths relative to the reference root):

  plain_rmsnorm   tools/dump_mlp_block.py:28-31 (same text at tools/dump_mamba_block.py:89-92,
                  tools/dump_attention_block.py:38-41, tools/ref_full_model.py:73-75)
  gated_rmsnorm   tools/dump_mamba_block.py:81-86 (tools/ref_full_model.py:76-80)
  relu2           tools/dump_mlp_block.py:49      (tools/ref_full_model.py:137)
  residual_add    tools/dump_mlp_block.py:53
  embedding       tools/ref_full_model.py:140

The bf16 forms evaluate the same formulas in fp32 on the upcast bf16 inputs and
round the result to bf16 (round to nearest even); the fused add+norm rounds the
residual sum to bf16 BEFORE the norm, because the reference writes the sum as a
bf16 tensor (ops/elementwise.cuh:241-245) that the next block's RMSNorm reads
back (ops/reduce.cuh:154-171).

Pinned: tests/test_oracle.py checks every function here against fixtures in
tests/golden/ that were produced by the reference's own functions and by its
unmodified dump scripts (tests/golden/make_golden.py).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

EPS = 1e-5


# --- the five formulas, fp32 ---------------------------------------------------

def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    x = x.float()
    var = x.pow(2).mean(-1, keepdim=True)
    return (x * torch.rsqrt(var + eps)) * weight


def gated_rmsnorm(x: torch.Tensor, weight: torch.Tensor, z: torch.Tensor, group_size: int,
                  eps: float = EPS) -> torch.Tensor:
    x = x.float() * F.silu(z.float())
    xg = x.reshape(*x.shape[:-1], x.shape[-1] // group_size, group_size)
    rstd = torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + eps)
    return (xg * rstd).reshape(x.shape) * weight


def relu2(u: torch.Tensor) -> torch.Tensor:
    return F.relu(u.float()).pow(2)


def residual_add(x: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    return x + r


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return F.embedding(ids.long(), table)


# --- bf16 forms (bf16 storage, fp32 math, one rounding per stored tensor) -------

def rmsnorm_bf16(x: torch.Tensor, w: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    assert x.dtype == torch.bfloat16 and w.dtype == torch.float32
    return plain_rmsnorm(x, w, eps).to(torch.bfloat16)


def add_bf16(x: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    assert x.dtype == torch.bfloat16 and r.dtype == torch.bfloat16
    return (x.float() + r.float()).to(torch.bfloat16)


def add_rmsnorm_bf16(x: torch.Tensor, r: torch.Tensor, w: torch.Tensor, eps: float = EPS):
    out_res = add_bf16(x, r)
    return out_res, rmsnorm_bf16(out_res, w, eps)


def gated_rmsnorm_bf16(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, group_size: int,
                       eps: float = EPS) -> torch.Tensor:
    assert y.dtype == torch.bfloat16 and z.dtype == torch.bfloat16 and w.dtype == torch.float32
    return gated_rmsnorm(y, w, z, group_size, eps).to(torch.bfloat16)


def relu2_bf16(u: torch.Tensor) -> torch.Tensor:
    assert u.dtype == torch.bfloat16
    return relu2(u).to(torch.bfloat16)


# --- the whole MLP block (tools/dump_mlp_block.py:42-53), used as the golden of stacked-block tests ------------

def mlp_block(x: torch.Tensor, norm_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    """out = x + down(relu(up(rmsnorm(x)))^2), fp32, weights in nn.Linear layout [out, in]."""
    x = x.float()
    return residual_add(x, F.linear(relu2(F.linear(plain_rmsnorm(x, norm_w, eps), up_w)), down_w))


# --- Mamba-2 depthwise causal conv1d + SiLU (tools/dump_mamba_block.py:126-130; tools/ref_full_model.py mamba()) ---

def causal_conv1d_silu(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """x [batch, S, C]; w [C, K] (the emitter's [C, 1, K] flattened); b [C]."""
    S, C, K = x.shape[1], x.shape[2], w.shape[1]
    h = x.float().transpose(1, 2)
    h = F.conv1d(h, w.reshape(C, 1, K), bias=b, padding=K - 1, groups=C)[..., :S]
    return F.silu(h.transpose(1, 2))


def causal_conv1d_silu_bf16(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    assert x.dtype == torch.bfloat16
    return causal_conv1d_silu(x, w, b).to(torch.bfloat16)


def conv_state_tail(x: torch.Tensor, K: int = 4) -> torch.Tensor:
    """[batch, C, K-1] fp32: the last K-1 raw inputs per channel, zero-padded on the left when S < K-1
    (what causal_conv1d_prefill leaves for the decode step, ops/mamba2/causal_conv1d.cuh:86-92)."""
    batch, S, C = x.shape
    pad = F.pad(x.float().transpose(1, 2), (K - 1, 0))
    return pad[..., pad.shape[-1] - (K - 1):].contiguous()


# --- W8A16 GEMV (tests/ops/test_gemm.cu:505-531: gemv_fp8_ref and quant_weight_perrow) -------------------------

def causal_conv1d_decode_bf16(x_t: torch.Tensor, w: torch.Tensor, b: torch.Tensor, state: torch.Tensor):
    """One decode step (ops/mamba2/causal_conv1d.cuh:409-429): x_t [batch, C] bf16, state [batch, C, K-1] fp32.
    acc = b + sum_k w[:, k] * state[..., k] + w[:, K-1] * x_t; returns (silu(acc) as bf16, shifted state)."""
    xf = x_t.float()
    acc = b.expand_as(xf).clone()
    for k in range(w.shape[1] - 1):
        acc = acc + w[:, k] * state[..., k]
    acc = acc + w[:, -1] * xf
    new_state = torch.cat([state[..., 1:], xf.unsqueeze(-1)], dim=-1)
    return F.silu(acc).to(torch.bfloat16), new_state


def ssm_decode_step(x: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor, B: torch.Tensor, C: torch.Tensor, D: torch.Tensor,
                    state: torch.Tensor, dt_bias: torch.Tensor | None = None):
    """One token of the Mamba-2 recurrence in the arithmetic of ops/mamba2/ssm.cuh:43-103 (fp32 throughout): x [H, P],
    dt [H], B and C [G, N], state [H, P, N]; consecutive heads share a B / C group (h -> h // (H / G), the convention
    tools/dump_mamba_block.py:140-145 states).  Returns (y [H, P] fp32 before rounding, new state)."""
    H, P, N = state.shape
    G = B.shape[0]
    dtv = dt.float() + (dt_bias.float() if dt_bias is not None else 0.0)
    dtv = torch.where(dtv > 20.0, dtv, torch.where(dtv < -20.0, torch.zeros_like(dtv), torch.log1p(torch.exp(dtv))))
    dA = torch.exp(-torch.exp(A_log.float()) * dtv)
    Bh = B.float().repeat_interleave(H // G, dim=0)
    Ch = C.float().repeat_interleave(H // G, dim=0)
    xf = x.float()
    new = state.float() * dA[:, None, None] + (dtv[:, None] * xf)[:, :, None] * Bh[:, None, :]
    y = (new * Ch[:, None, :]).sum(-1) + D.float()[:, None] * xf
    return y, new


def sdpa_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, s_cache: int) -> torch.Tensor:
    """One query token over the first s_cache cached positions, the formulation of tools/dump_attention_block.py
    (softmax(q K^T / sqrt(d)) V with consecutive query heads sharing a KV head) restricted to what the decode kernel of
    ops/attention/sdpa_decode.cuh:98-115 covers: positions [0, s_cache), the new token not included.  fp32; q [H_Q, D],
    caches [H_KV, cap, D]."""
    H_Q, D = q.shape
    H_KV = k_cache.shape[0]
    if s_cache == 0:
        return torch.zeros(H_Q, D)
    K = k_cache[:, :s_cache].float().repeat_interleave(H_Q // H_KV, dim=0)      # [H_Q, s, D]
    V = v_cache[:, :s_cache].float().repeat_interleave(H_Q // H_KV, dim=0)
    scores = torch.einsum("hd,hsd->hs", q.float(), K) / (D ** 0.5)
    return torch.einsum("hs,hsd->hd", torch.softmax(scores, dim=-1), V)


def quant_weight_perrow(Wf: torch.Tensor):
    """Per-output-row e4m3 quantisation of an fp32 weight matrix: (W_e4m3, w_scale)."""
    amax = Wf.abs().amax(dim=1)
    scale = amax / 448.0
    scale = torch.where(scale < 1e-10, torch.full_like(scale, 1.0 / 448.0), scale)
    q = torch.clamp(Wf * (1.0 / scale)[:, None], -448.0, 448.0).to(torch.float8_e4m3fn)
    return q, scale.float()


def gemv_w8a16(x: torch.Tensor, W: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """y[n] = (sum_k float(W[n,k]) * float(x[k])) * w_scale[n], as fp32 (round to bf16 for the kernel's output).
    Accumulated in float64 here so that the checker itself adds no summation-order noise."""
    assert W.dtype == torch.float8_e4m3fn and x.dtype == torch.bfloat16
    return ((W.float().double() @ x.float().double()) * w_scale.double()).float()


# --- per-tensor e4m3 quantisation of a bf16 activation tensor -----------------------
# Restates fp8_amax_kernel + fp8_quant_kernel (ops/gemm.cuh:257-289): amax = max|x| over the bf16 tensor,
# s = amax / 448 (1/448 when s < 1e-10), q = e4m3(clamp(x * (1/s), -448, 448)), all in fp32.

def quantize_fp8(x: torch.Tensor):
    assert x.dtype == torch.bfloat16
    xf = x.float()
    amax = xf.abs().max() if xf.numel() else torch.zeros(())
    s = (amax / torch.tensor(448.0)).to(torch.float32)
    if float(s) < 1e-10:
        s = torch.tensor(1.0 / 448.0, dtype=torch.float32)
    inv = (torch.tensor(1.0, dtype=torch.float32) / s).to(torch.float32)
    q = torch.clamp(xf * inv, -448.0, 448.0).to(torch.float8_e4m3fn)
    return q, s


def e4m3_ordered(t: torch.Tensor) -> torch.Tensor:
    bits = t.contiguous().view(torch.uint8).to(torch.int32)
    mag = bits & 0x7F
    return torch.where((bits & 0x80) != 0, -mag, mag)


# --- comparison helpers ----------------------------------------------------------

def bf16_ordered(t: torch.Tensor) -> torch.Tensor:
    """Maps bf16 values to integers that are monotone in the value (+0 and -0 both map to 0)."""
    bits = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    mag = bits & 0x7FFF
    return torch.where((bits & 0x8000) != 0, -mag, mag)


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Element-wise distance in bf16 units in the last place; NaN vs NaN counts as 0, NaN vs number as 2^16."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.shape == b.shape
    d = (bf16_ordered(a) - bf16_ordered(b)).abs()
    na, nb = torch.isnan(a), torch.isnan(b)
    d = torch.where(na & nb, torch.zeros_like(d), d)
    d = torch.where(na ^ nb, torch.full_like(d, 1 << 16), d)
    return d


def ulp_report(got: torch.Tensor, want: torch.Tensor) -> dict:
    d = bf16_ulp_distance(got.cpu(), want.cpu())
    n = d.numel()
    return {"max_ulp": int(d.max()) if n else 0,
            "mismatch": int((d != 0).sum()),
            "mismatch_frac": float((d != 0).sum()) / max(n, 1),
            "n": n}


# --- seeded inputs of the benchmark configurations --------------------------------
# Every tensor is drawn in fp32 from torch.Generator().manual_seed(seed) and then cast.

def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def norm_weight(cols: int, g: torch.Generator) -> torch.Tensor:
    return 1.0 + 0.1 * torch.randn(cols, generator=g, dtype=torch.float32)


def cfg0_inputs(rows: int = 512, cols: int = 3136, seed: int = 0):
    """fp32 RMSNorm: x ~ N(0,1), w = 1 + 0.1 N(0,1)."""
    g = _gen(seed)
    x = torch.randn(rows, cols, generator=g, dtype=torch.float32)
    return x, norm_weight(cols, g)


def cfg1_inputs(T: int, cols: int = 3136, seed: int = 0):
    """bf16 residual add + RMSNorm: x, r ~ N(0,1) -> bf16, w fp32."""
    g = _gen(seed)
    x = torch.randn(T, cols, generator=g, dtype=torch.float32).to(torch.bfloat16)
    r = torch.randn(T, cols, generator=g, dtype=torch.float32).to(torch.bfloat16)
    return x, r, norm_weight(cols, g)


def cfg2_inputs(T: int, cols: int = 6144, seed: int = 0):
    """bf16 gated RMSNorm: y, z ~ N(0,1) -> bf16, w fp32."""
    g = _gen(seed)
    y = torch.randn(T, cols, generator=g, dtype=torch.float32).to(torch.bfloat16)
    z = torch.randn(T, cols, generator=g, dtype=torch.float32).to(torch.bfloat16)
    return y, z, norm_weight(cols, g)


def cfg3_inputs(T: int, cols: int = 12544, seed: int = 0):
    """bf16 relu^2: u ~ N(0, 2^2) -> bf16."""
    g = _gen(seed)
    return (2.0 * torch.randn(T, cols, generator=g, dtype=torch.float32)).to(torch.bfloat16)


def cfg4_inputs(T: int, vocab: int = 131072, hidden: int = 3136, seed: int = 0, ids_dtype=torch.int32):
    """Embedding: table ~ N(0, 0.02^2) -> bf16, ids uniform in [0, vocab)."""
    g = _gen(seed)
    table = (0.02 * torch.randn(vocab, hidden, generator=g, dtype=torch.float32)).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (T,), generator=g, dtype=torch.int64).to(ids_dtype)
    return table, ids
