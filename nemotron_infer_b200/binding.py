"""Drop-in for the hot-path part of the reference's pybind module `nemotron_infer.csrc.binding`.

Same names, argument order and meaning as the reference (binding.cu:59-73,
214-232): every tensor argument is an integer device address (what
`tensor.data_ptr()` returns, engine.py:40-42), sizes are ints, the functions
return None and enqueue asynchronously on the legacy default stream unless
`set_stream` chose another one.  Unlike the reference, which never checks
anything, a rejected argument raises `NemotronB200Error` and launches nothing.

Reference names kept: embedding, rmsnorm, sync, reset_allocator, free_allocator
and the model constants.  Added (the fused forms the reference spreads over two
block calls, and the ops its blocks call internally): add_rmsnorm,
rmsnorm_gated, relu2, add; and fuse_next_norm / fusion_reset / fusion_counters,
the announcement that lets the reference's unchanged blocks (built on the drop-in
headers) fuse the residual add of one layer with the pre-norm of the next.
"""
from __future__ import annotations

from . import _lib

# Model dimensions, compile-time constants in the reference (binding.cu:35-46, 214-226).
HIDDEN = 3136
H, P, N, G, CONV_K = 96, 80, 128, 8, 4
H_Q, H_KV, HEAD = 40, 8, 128
INTER = 12544
VOCAB = 131072
CONV_DIM = H * P + 2 * G * N
IN_PROJ = H * P + CONV_DIM + H
EPS = 1e-5
D_INNER = H * P            # 7680: width of the gated RMSNorm (model/mamba_block.cuh:165,217)

_stream = None             # None = legacy default stream, like every reference call site


def set_stream(stream_ptr: int | None) -> None:
    """Selects the cudaStream_t (as an int) later calls enqueue on; None = legacy default stream."""
    global _stream
    _stream = stream_ptr or None


def set_device(device: int) -> None:
    _lib.check(_lib.load().nmt_set_device(int(device)), "set_device")


def sync() -> None:
    """cudaDeviceSynchronize (binding.cu:62)."""
    _lib.check(_lib.load().nmt_device_synchronize(), "sync")


def reset_allocator() -> None:
    """Kept for call-site compatibility (binding.cu:59): these kernels use no workspace."""


def free_allocator() -> None:
    """Kept for call-site compatibility (binding.cu:61): these kernels own no memory."""


def embedding(table: int, ids: int, out: int, num_tokens: int) -> None:
    """out[bf16, num_tokens, HIDDEN] = table[ids[int64, num_tokens], :] (binding.cu:65-68)."""
    _lib.check(_lib.load().nmt_embedding_bf16_i64(table, ids, out, num_tokens, HIDDEN, 0, None, _stream),
               "embedding")


def embedding_checked(table: int, ids: int, out: int, num_tokens: int, err_flag: int, ids_int32: bool = False) -> None:
    """Same gather with ids range-checked against VOCAB; `err_flag` is a device int32 set to 1 on a bad id."""
    lib = _lib.load()
    fn = lib.nmt_embedding_bf16_i32 if ids_int32 else lib.nmt_embedding_bf16_i64
    _lib.check(fn(table, ids, out, num_tokens, HIDDEN, VOCAB, err_flag, _stream), "embedding_checked")


def rmsnorm(inp: int, out: int, w: int, M: int) -> None:
    """Final / pre-norm RMSNorm over HIDDEN with eps 1e-5 (binding.cu:71-73)."""
    _lib.check(_lib.load().nmt_rmsnorm_bf16(inp, out, w, M, HIDDEN, EPS, _stream), "rmsnorm")


def add_rmsnorm(x: int, r: int, w: int, out_res: int, out: int, M: int) -> None:
    """out_res = x + r (bf16); out = rmsnorm(out_res) * w.  One launch instead of the reference's
    block-tail add (model/mlp_block.cuh:104) plus the next block's rmsnorm (model/mlp_block.cuh:98)."""
    _lib.check(_lib.load().nmt_add_rmsnorm_bf16(x, r, w, out_res, out, M, HIDDEN, EPS, _stream), "add_rmsnorm")


def rmsnorm_gated(y: int, z: int, w: int, out: int, M: int, cols: int = D_INNER, groups: int = G) -> None:
    """Mamba-2 gated RMSNorm as called at model/mamba_block.cuh:217 (cols 7680, 8 groups of 960)."""
    _lib.check(_lib.load().nmt_rmsnorm_gated_bf16(y, z, w, out, M, cols, cols // groups, EPS, _stream),
               "rmsnorm_gated")


def relu2(u: int, out: int, M: int, width: int = INTER) -> None:
    """out = relu(u)^2 over [M, width] (model/mlp_block.cuh:100)."""
    _lib.check(_lib.load().nmt_relu2_bf16(u, out, M * width, _stream), "relu2")


def add(a: int, b: int, out: int, M: int, width: int = HIDDEN) -> None:
    """out = a + b over [M, width] (the residual add, model/mlp_block.cuh:104)."""
    _lib.check(_lib.load().nmt_add_bf16(a, b, out, M * width, _stream), "add")


def fuse_next_norm(next_norm_w: int | None) -> None:
    """Announces, before block i is called, the device address of block i+1's norm weight (None withdraws it).
    The reference's blocks built on include/nemotron_b200_shim then run block i's closing residual add
    (model/mlp_block.cuh:104) and block i+1's pre-norm (model/mlp_block.cuh:98) as one launch; engine.py's layer
    loop (engine.py:262-270) only gains this call.  See nmt_fuse_next_norm in include/nemotron_b200.h."""
    _lib.check(_lib.load().nmt_fuse_next_norm(next_norm_w or None, EPS), "fuse_next_norm")


def fusion_reset() -> None:
    """Forgets an announcement and a pending fused tail (call when a pass is abandoned half way)."""
    _lib.check(_lib.load().nmt_fusion_reset(), "fusion_reset")


def fusion_counters() -> tuple[int, int]:
    """(residual adds that ran fused with the next norm, pre-norms that were skipped) on this thread so far."""
    import ctypes as C
    a, b = C.c_int64(0), C.c_int64(0)
    _lib.check(_lib.load().nmt_fusion_counters(C.byref(a), C.byref(b)), "fusion_counters")
    return a.value, b.value
