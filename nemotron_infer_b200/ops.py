"""Tensor-level operators over the C-ABI library (torch tensors in, torch tensors out).

torch is used for device memory and streams only; every operator validates its
arguments, takes `data_ptr()` of each tensor (the same hand-off the reference's
engine does, engine.py:40-42) and calls libnemotron_b200.so on torch's current
stream.  There is no eager/PyTorch fallback: a CPU tensor or a missing library
raises.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import NemotronB200Error  # noqa: F401  (re-exported)

EPS = 1e-5


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev(*ts: torch.Tensor) -> None:
    for t in ts:
        if not t.is_cuda:
            raise ValueError("nemotron_infer_b200 operators run on CUDA tensors only (no CPU fallback)")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous (row stride == cols)")
    dev = ts[0].device
    if any(t.device != dev for t in ts):
        raise ValueError("all tensors must live on the same device")


def _rows_cols(t: torch.Tensor) -> tuple[int, int]:
    cols = t.shape[-1] if t.dim() else 1
    return (t.numel() // cols if cols else 0), cols


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = EPS, out: torch.Tensor | None = None) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dim; bf16 or fp32 x, fp32 w."""
    out = torch.empty_like(x) if out is None else out
    _dev(x, w, out)
    if w.dtype != torch.float32 or out.dtype != x.dtype or out.shape != x.shape:
        raise ValueError("w must be fp32 and out must match x")
    rows, cols = _rows_cols(x)
    if w.numel() != cols:
        raise ValueError("w must have one entry per column")
    lib = _lib.load()
    if x.dtype == torch.bfloat16:
        st = lib.nmt_rmsnorm_bf16(x.data_ptr(), out.data_ptr(), w.data_ptr(), rows, cols, eps, _stream())
    elif x.dtype == torch.float32:
        st = lib.nmt_rmsnorm_f32(x.data_ptr(), out.data_ptr(), w.data_ptr(), rows, cols, eps, _stream())
    else:
        raise ValueError("x must be bf16 or fp32")
    _lib.check(st, "rmsnorm")
    return out


def add_rmsnorm(x: torch.Tensor, r: torch.Tensor, w: torch.Tensor, eps: float = EPS,
                out_res: torch.Tensor | None = None, out: torch.Tensor | None = None):
    """(out_res, out) with out_res = bf16(x + r) and out = rmsnorm(out_res) * w, in one pass over HBM."""
    out_res = torch.empty_like(x) if out_res is None else out_res
    out = torch.empty_like(x) if out is None else out
    _dev(x, r, w, out_res, out)
    if x.dtype != torch.bfloat16 or r.dtype != x.dtype or out.dtype != x.dtype or out_res.dtype != x.dtype:
        raise ValueError("x, r, out_res and out must be bf16")
    if w.dtype != torch.float32:
        raise ValueError("w must be fp32")
    if not (x.shape == r.shape == out.shape == out_res.shape):
        raise ValueError("x, r, out_res and out must have the same shape")
    rows, cols = _rows_cols(x)
    if w.numel() != cols:
        raise ValueError("w must have one entry per column")
    st = _lib.load().nmt_add_rmsnorm_bf16(x.data_ptr(), r.data_ptr(), w.data_ptr(), out_res.data_ptr(),
                                          out.data_ptr(), rows, cols, eps, _stream())
    _lib.check(st, "add_rmsnorm")
    return out_res, out


def rmsnorm_gated(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, group_size: int, eps: float = EPS,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """out = (g * rsqrt(mean_group(g^2) + eps)) * w with g = y * silu(z); bf16 or fp32."""
    out = torch.empty_like(y) if out is None else out
    _dev(y, z, w, out)
    if z.dtype != y.dtype or out.dtype != y.dtype or w.dtype != torch.float32:
        raise ValueError("y, z and out must share a dtype and w must be fp32")
    if not (y.shape == z.shape == out.shape):
        raise ValueError("y, z and out must have the same shape")
    rows, cols = _rows_cols(y)
    if w.numel() != cols:
        raise ValueError("w must have one entry per column")
    lib = _lib.load()
    fn = {torch.bfloat16: lib.nmt_rmsnorm_gated_bf16, torch.float32: lib.nmt_rmsnorm_gated_f32}.get(y.dtype)
    if fn is None:
        raise ValueError("y must be bf16 or fp32")
    _lib.check(fn(y.data_ptr(), z.data_ptr(), w.data_ptr(), out.data_ptr(), rows, cols, int(group_size), eps,
                  _stream()), "rmsnorm_gated")
    return out


def relu2(u: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = relu(u)^2; bf16 or fp32."""
    out = torch.empty_like(u) if out is None else out
    _dev(u, out)
    if out.dtype != u.dtype or out.shape != u.shape:
        raise ValueError("out must match u")
    lib = _lib.load()
    fn = {torch.bfloat16: lib.nmt_relu2_bf16, torch.float32: lib.nmt_relu2_f32}.get(u.dtype)
    if fn is None:
        raise ValueError("u must be bf16 or fp32")
    _lib.check(fn(u.data_ptr(), out.data_ptr(), u.numel(), _stream()), "relu2")
    return out


def add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = a + b; bf16 (single rounding) or fp32."""
    out = torch.empty_like(a) if out is None else out
    _dev(a, b, out)
    if b.dtype != a.dtype or out.dtype != a.dtype or not (a.shape == b.shape == out.shape):
        raise ValueError("a, b and out must match")
    lib = _lib.load()
    fn = {torch.bfloat16: lib.nmt_add_bf16, torch.float32: lib.nmt_add_f32}.get(a.dtype)
    if fn is None:
        raise ValueError("a must be bf16 or fp32")
    _lib.check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream()), "add")
    return out


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None,
              err_flag: torch.Tensor | None = None, check_range: bool = True) -> torch.Tensor:
    """out[i, :] = table[ids[i], :]; bf16 table, int32 or int64 ids.  With check_range, an id outside
    [0, vocab) zero-fills its row and sets err_flag (device int32[1]) instead of reading out of bounds."""
    vocab, hidden = table.shape
    out = torch.empty((ids.numel(), hidden), dtype=table.dtype, device=table.device) if out is None else out
    _dev(table, ids, out)
    if table.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise ValueError("table and out must be bf16")
    if out.numel() != ids.numel() * hidden:
        raise ValueError("out must hold ids.numel() rows of table width")
    lib = _lib.load()
    fn = {torch.int64: lib.nmt_embedding_bf16_i64, torch.int32: lib.nmt_embedding_bf16_i32}.get(ids.dtype)
    if fn is None:
        raise ValueError("ids must be int32 or int64")
    if err_flag is not None:
        _dev(err_flag)
        if err_flag.dtype != torch.int32:
            raise ValueError("err_flag must be int32")
    _lib.check(fn(table.data_ptr(), ids.data_ptr(), out.data_ptr(), ids.numel(), hidden,
                  vocab if check_range else 0, err_flag.data_ptr() if err_flag is not None else None, _stream()),
               "embedding")
    return out


def causal_conv1d_silu(xbc: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, split: tuple[int, ...] | None = None,
                       return_state: bool = False):
    """Depthwise causal conv1d (4 taps) + bias + SiLU over xbc [batch, S, conv_dim] (bf16 or fp32), w [conv_dim, 4],
    bias [conv_dim] fp32.  With split=(n0, n1, n2) the bf16 result comes back as three contiguous tensors
    (the x | B | C inputs of the scan) instead of one; return_state adds the [batch, conv_dim, 3] fp32 tail."""
    if xbc.dim() != 3:
        raise ValueError("xbc must be [batch, S, conv_dim]")
    batch, S, C = xbc.shape
    _dev(xbc, w, bias)
    if w.dtype != torch.float32 or bias.dtype != torch.float32 or w.numel() != C * 4 or bias.numel() != C:
        raise ValueError("w must be fp32 [conv_dim, 4] and bias fp32 [conv_dim]")
    state = torch.empty(batch, C, 3, dtype=torch.float32, device=xbc.device) if return_state else None
    sp = state.data_ptr() if state is not None else None
    lib = _lib.load()
    if xbc.dtype == torch.float32:
        if split is not None:
            raise ValueError("the split form is bf16 only")
        y = torch.empty_like(xbc)
        _lib.check(lib.nmt_causal_conv1d_silu_f32(xbc.data_ptr(), w.data_ptr(), bias.data_ptr(), y.data_ptr(), sp, C, S, batch,
                                                  _stream()), "causal_conv1d_silu")
        outs = (y,)
    elif xbc.dtype == torch.bfloat16:
        sizes = tuple(split) if split is not None else (C,)
        if sum(sizes) != C or len(sizes) > 3:
            raise ValueError("split must be up to three sizes that add up to conv_dim")
        outs = tuple(torch.empty(batch, S, n, dtype=xbc.dtype, device=xbc.device) for n in sizes)
        ptrs = [o.data_ptr() for o in outs] + [None] * (3 - len(outs))
        ns = list(sizes) + [0] * (3 - len(sizes))
        _lib.check(lib.nmt_causal_conv1d_silu_split_bf16(xbc.data_ptr(), w.data_ptr(), bias.data_ptr(), ptrs[0], ptrs[1], ptrs[2],
                                                         ns[0], ns[1], ns[2], sp, S, batch, _stream()), "causal_conv1d_silu")
    else:
        raise ValueError("xbc must be bf16 or fp32")
    res = outs if split is not None else outs[0]
    return (res, state) if return_state else res


def causal_conv1d_silu_decode(xbc: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, state: torch.Tensor,
                              split: tuple[int, ...] | None = None):
    """One decode step of the causal conv1d + SiLU: xbc [batch, conv_dim] bf16, state [batch, conv_dim, 3] fp32
    (updated in place).  Returns the bf16 result, as three tensors when split=(n0, n1, n2) is given."""
    if xbc.dim() != 2 or xbc.dtype != torch.bfloat16:
        raise ValueError("xbc must be bf16 [batch, conv_dim]")
    batch, C = xbc.shape
    _dev(xbc, w, bias, state)
    if w.dtype != torch.float32 or bias.dtype != torch.float32 or w.numel() != C * 4 or bias.numel() != C:
        raise ValueError("w must be fp32 [conv_dim, 4] and bias fp32 [conv_dim]")
    if state.dtype != torch.float32 or tuple(state.shape) != (batch, C, 3) or not state.is_contiguous():
        raise ValueError("state must be contiguous fp32 [batch, conv_dim, 3]")
    sizes = tuple(split) if split is not None else (C,)
    if sum(sizes) != C or len(sizes) > 3:
        raise ValueError("split must be up to three sizes that add up to conv_dim")
    outs = [torch.empty(batch, n, dtype=torch.bfloat16, device=xbc.device) for n in sizes]
    ptrs = [o.data_ptr() for o in outs] + [None] * (3 - len(outs))
    ns = list(sizes) + [0] * (3 - len(sizes))
    _lib.check(_lib.load().nmt_causal_conv1d_silu_decode_split_bf16(xbc.data_ptr(), w.data_ptr(), bias.data_ptr(), ptrs[0], ptrs[1],
                                                                    ptrs[2], ns[0], ns[1], ns[2], state.data_ptr(), batch, _stream()),
               "causal_conv1d_silu_decode")
    return outs if split is not None else outs[0]


def gemv_w8a16_gated(y_in: torch.Tensor, gate: torch.Tensor, gnorm_w: torch.Tensor, group_size: int, W: torch.Tensor,
                     w_scale: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """out = W @ (gated_rmsnorm(y_in, gate, group_size) * gnorm_w) * w_scale (+ residual): the Mamba-2 decode block's gated
    norm, out_proj and residual add in one launch, byte-identical to the separate ops."""
    N, K = W.shape
    out = torch.empty(N, dtype=torch.bfloat16, device=y_in.device) if out is None else out
    _dev(y_in, gate, gnorm_w, W, w_scale, out)
    if W.dtype != torch.float8_e4m3fn or any(t.dtype != torch.bfloat16 for t in (y_in, gate, out)) or \
            gnorm_w.dtype != torch.float32 or w_scale.dtype != torch.float32:
        raise ValueError("W must be float8_e4m3fn, y_in / gate / out bf16, gnorm_w / w_scale fp32")
    if y_in.numel() != K or gate.numel() != K or gnorm_w.numel() != K or w_scale.numel() != N or out.numel() != N:
        raise ValueError("shape mismatch")
    _lib.check(_lib.load().nmt_gemv_w8a16_gated(y_in.data_ptr(), gate.data_ptr(), gnorm_w.data_ptr(), float(eps), int(group_size),
                                                W.data_ptr(), w_scale.data_ptr(), residual.data_ptr() if residual is not None else None,
                                                out.data_ptr(), N, K, _stream()), "gemv_w8a16_gated")
    return out


def sdpa_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                s_cache: int, out: torch.Tensor | None = None, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of one query token [H_Q, 128] over the first `s_cache` positions of the caches [H_KV, cap, 128]; then
    k_new / v_new [H_KV, 128] are written to position `s_cache` (the new token does not attend to itself)."""
    H_Q, D = q.shape
    H_KV, cap, _ = k_cache.shape
    out = torch.empty_like(q) if out is None else out
    _dev(q, k_cache, v_cache, k_new, v_new, out)
    if any(t.dtype != torch.bfloat16 for t in (q, k_cache, v_cache, k_new, v_new, out)):
        raise ValueError("all tensors must be bf16")
    lib = _lib.load()
    need = lib.nmt_sdpa_decode_workspace_bytes(int(s_cache), H_Q)
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    elif workspace.numel() * workspace.element_size() < need:
        raise ValueError("workspace too small")
    _lib.check(lib.nmt_sdpa_decode_bf16(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), k_new.data_ptr(),
                                        v_new.data_ptr(), int(s_cache), cap, H_Q, H_KV, D, workspace.data_ptr(), _stream()), "sdpa_decode")
    return out


def ssm_decode_step(x: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor, B: torch.Tensor, C: torch.Tensor, D: torch.Tensor,
                    state: torch.Tensor, dt_bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
                    dt_min: float = 0.0, dt_max: float = 3.4028234663852886e38) -> torch.Tensor:
    """One token of the Mamba-2 recurrence: updates `state` [batch, H, P, N] (fp32) in place and returns y [batch, H * P]
    (bf16).  x [batch, H * P], dt [batch, H], B and C [batch, G, N] are bf16; A_log, D, dt_bias [H] fp32."""
    batch, H, P, N = state.shape
    G = B.shape[-2]
    out = torch.empty(batch, H * P, dtype=torch.bfloat16, device=x.device) if out is None else out
    _dev(x, dt, A_log, B, C, D, state, out)
    if any(t.dtype != torch.bfloat16 for t in (x, dt, B, C, out)) or any(t.dtype != torch.float32 for t in (A_log, D, state)):
        raise ValueError("x, dt, B, C, out must be bf16; A_log, D, state fp32")
    if x.numel() != batch * H * P or dt.numel() != batch * H or B.numel() != batch * G * N or C.numel() != batch * G * N:
        raise ValueError("shape mismatch")
    _lib.check(_lib.load().nmt_ssm_decode_step_bf16(x.data_ptr(), dt.data_ptr(), A_log.data_ptr(), B.data_ptr(), C.data_ptr(),
                                                    D.data_ptr(), dt_bias.data_ptr() if dt_bias is not None else None,
                                                    state.data_ptr(), out.data_ptr(), batch, H, P, N, G, float(dt_min), float(dt_max),
                                                    _stream()), "ssm_decode_step")
    return out


def gemv_w8a16(x: torch.Tensor, W: torch.Tensor, w_scale: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """y[N] = (W[N, K] (e4m3) @ x[K] (bf16)) * w_scale[N], fp32 accumulation, bf16 result: the decode projection."""
    N, K = W.shape
    out = torch.empty(N, dtype=torch.bfloat16, device=x.device) if out is None else out
    _dev(x, W, w_scale, out)
    if W.dtype != torch.float8_e4m3fn or x.dtype != torch.bfloat16 or w_scale.dtype != torch.float32 or out.dtype != torch.bfloat16:
        raise ValueError("W must be float8_e4m3fn, x and out bf16, w_scale fp32")
    if x.numel() != K or w_scale.numel() != N or out.numel() != N:
        raise ValueError("shape mismatch")
    _lib.check(_lib.load().nmt_gemv_w8a16(x.data_ptr(), W.data_ptr(), w_scale.data_ptr(), out.data_ptr(), N, K, _stream()),
               "gemv_w8a16")
    return out


def gemv_w8a16_fused(x: torch.Tensor, W: torch.Tensor, w_scale: torch.Tensor, norm_w: torch.Tensor | None = None,
                     eps: float = 1e-5, activation: str | None = None, residual: torch.Tensor | None = None,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """The decode projection with its neighbours folded in: y = W @ (rmsnorm(x) * norm_w if norm_w is given else x)
    * w_scale, then relu^2 (activation="relu2"), then + residual - one launch, byte-identical to the separate ops."""
    N, K = W.shape
    out = torch.empty(N, dtype=torch.bfloat16, device=x.device) if out is None else out
    _dev(x, W, w_scale, out)
    if W.dtype != torch.float8_e4m3fn or x.dtype != torch.bfloat16 or w_scale.dtype != torch.float32 or out.dtype != torch.bfloat16:
        raise ValueError("W must be float8_e4m3fn, x and out bf16, w_scale fp32")
    if x.numel() != K or w_scale.numel() != N or out.numel() != N:
        raise ValueError("shape mismatch")
    if norm_w is not None and (norm_w.dtype != torch.float32 or norm_w.numel() != K or not norm_w.is_cuda):
        raise ValueError("norm_w must be fp32 [K] on the device")
    if residual is not None and (residual.dtype != torch.bfloat16 or residual.numel() != N or not residual.is_cuda):
        raise ValueError("residual must be bf16 [N] on the device")
    if activation not in (None, "relu2"):
        raise ValueError("activation must be None or 'relu2'")
    _lib.check(_lib.load().nmt_gemv_w8a16_fused(x.data_ptr(), norm_w.data_ptr() if norm_w is not None else None, float(eps),
                                                W.data_ptr(), w_scale.data_ptr(), 1 if activation == "relu2" else 0,
                                                residual.data_ptr() if residual is not None else None, out.data_ptr(), N, K,
                                                _stream()), "gemv_w8a16_fused")
    return out


def _fp8_out(like: torch.Tensor, out: torch.Tensor | None) -> torch.Tensor:
    out = torch.empty(like.shape, dtype=torch.float8_e4m3fn, device=like.device) if out is None else out
    if out.dtype != torch.float8_e4m3fn or out.shape != like.shape:
        raise ValueError("out must be float8_e4m3fn with the input's shape")
    return out


def quantize_fp8(x: torch.Tensor, out: torch.Tensor | None = None, relu2_first: bool = False):
    """(q, scale): per-tensor dynamic e4m3 quantisation, q = e4m3(clamp(x / scale)), scale = max|x| / 448.
    With relu2_first the tensor quantised is relu(x)^2, which is never written out."""
    out = _fp8_out(x, out)
    _dev(x, out)
    if x.dtype != torch.bfloat16:
        raise ValueError("x must be bf16")
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    amax = torch.empty(1, dtype=torch.int32, device=x.device)
    lib = _lib.load()
    fn = lib.nmt_relu2_quant_fp8 if relu2_first else lib.nmt_quantize_fp8
    _lib.check(fn(x.data_ptr(), out.data_ptr(), scale.data_ptr(), amax.data_ptr(), x.numel(), _stream()), "quantize_fp8")
    return out, scale


def fp8_workspace(rows: int, device) -> torch.Tensor:
    """Workspace for rmsnorm_quant_fp8 / add_rmsnorm_quant_fp8 on `rows` rows."""
    return torch.empty(int(_lib.load().nmt_fp8_workspace_bytes(rows)), dtype=torch.uint8, device=device)


def rmsnorm_quant_fp8(x: torch.Tensor, w: torch.Tensor, r: torch.Tensor | None = None, eps: float = EPS,
                      out_res: torch.Tensor | None = None, out: torch.Tensor | None = None,
                      workspace: torch.Tensor | None = None):
    """(q, scale) or, with a residual r, (out_res, q, scale): RMSNorm (after the residual add) fused with the
    per-tensor e4m3 quantisation of its output; the bf16 normed tensor is never written."""
    out = _fp8_out(x, out)
    rows, cols = _rows_cols(x)
    workspace = fp8_workspace(rows, x.device) if workspace is None else workspace
    _dev(x, w, out, workspace)
    if x.dtype != torch.bfloat16 or w.dtype != torch.float32 or w.numel() != cols:
        raise ValueError("x must be bf16 and w fp32 with one entry per column")
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    if r is None:
        _lib.check(lib.nmt_rmsnorm_quant_fp8(x.data_ptr(), w.data_ptr(), out.data_ptr(), scale.data_ptr(),
                                             workspace.data_ptr(), rows, cols, eps, _stream()), "rmsnorm_quant_fp8")
        return out, scale
    out_res = torch.empty_like(x) if out_res is None else out_res
    _dev(r, out_res)
    if r.dtype != x.dtype or r.shape != x.shape or out_res.dtype != x.dtype or out_res.shape != x.shape:
        raise ValueError("r and out_res must match x")
    _lib.check(lib.nmt_add_rmsnorm_quant_fp8(x.data_ptr(), r.data_ptr(), w.data_ptr(), out_res.data_ptr(), out.data_ptr(),
                                             scale.data_ptr(), workspace.data_ptr(), rows, cols, eps, _stream()),
               "add_rmsnorm_quant_fp8")
    return out_res, out, scale


def rmsnorm_gated_quant_fp8(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, group_size: int, eps: float = EPS,
                            out_bf16: torch.Tensor | None = None, out: torch.Tensor | None = None):
    """(out_bf16, q, scale): gated RMSNorm whose kernel also tracks max|out|, followed by the e4m3 quantiser."""
    out_bf16 = torch.empty_like(y) if out_bf16 is None else out_bf16
    out = _fp8_out(y, out)
    _dev(y, z, w, out_bf16, out)
    if y.dtype != torch.bfloat16 or z.dtype != y.dtype or out_bf16.dtype != y.dtype or w.dtype != torch.float32:
        raise ValueError("y, z, out_bf16 must be bf16 and w fp32")
    rows, cols = _rows_cols(y)
    scale = torch.empty(1, dtype=torch.float32, device=y.device)
    amax = torch.empty(1, dtype=torch.int32, device=y.device)
    _lib.check(_lib.load().nmt_rmsnorm_gated_quant_fp8(y.data_ptr(), z.data_ptr(), w.data_ptr(), out_bf16.data_ptr(),
                                                       out.data_ptr(), scale.data_ptr(), amax.data_ptr(), rows, cols,
                                                       int(group_size), eps, _stream()), "rmsnorm_gated_quant_fp8")
    return out_bf16, out, scale


def tune(key: str, value: int) -> None:
    """Sets a launch-shape / variant knob (see nmt_tune_set in include/nemotron_b200.h)."""
    _lib.check(_lib.load().nmt_tune_set(key.encode(), int(value)), f"tune({key})")


def launch_count() -> int:
    return int(_lib.load().nmt_launch_count())
