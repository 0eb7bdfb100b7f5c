"""CPU-side checks of the C-ABI library: it builds, loads, exports every symbol the header declares,
and rejects bad arguments before touching the GPU.  No kernel is launched here."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nemotron_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nmt_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("nmt_rmsnorm_bf16", "nmt_add_rmsnorm_bf16", "nmt_rmsnorm_gated_bf16", "nmt_relu2_bf16",
                 "nmt_add_bf16", "nmt_embedding_bf16_i64", "nmt_embedding_bf16_i32", "nmt_rmsnorm_f32",
                 "nmt_rmsnorm_gated_f32", "nmt_relu2_f32", "nmt_add_f32"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    from nemotron_infer_b200 import _lib
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(raw, name), f"{name} is declared in include/nemotron_b200.h but not exported"
        assert name in _lib.PROTOTYPES, f"{name} has no ctypes prototype"
    assert b"sm_100a" in built_lib.nmt_version()


def test_library_is_built_for_sm_100a_only():
    from nemotron_infer_b200 import build
    flags = " ".join(build.NVCC_FLAGS)
    assert "arch=compute_100a,code=sm_100a" in flags and flags.count("-gencode") == 1


BUF = 0x7F0000000000     # a well-aligned fake device address; validation never dereferences it


def test_argument_validation_happens_before_any_launch(built_lib):
    L = built_lib
    before = L.nmt_launch_count()
    OK, NULL, ALIGN, SHAPE = 0, 1, 2, 3
    # rows == 0 / n == 0: successful no-op
    assert L.nmt_rmsnorm_bf16(BUF, BUF, BUF, 0, 3136, 1e-5, None) == OK
    assert L.nmt_add_rmsnorm_bf16(BUF, BUF, BUF, BUF, BUF + 64, 0, 3136, 1e-5, None) == OK
    assert L.nmt_relu2_bf16(BUF, BUF, 0, None) == OK
    assert L.nmt_embedding_bf16_i64(BUF, BUF, BUF, 0, 3136, 131072, None, None) == OK
    assert L.nmt_rmsnorm_gated_bf16(BUF, BUF, BUF, BUF, 0, 6144, 768, 1e-5, None) == OK
    # null pointers
    assert L.nmt_rmsnorm_bf16(None, BUF, BUF, 4, 3136, 1e-5, None) == NULL
    assert L.nmt_add_rmsnorm_bf16(BUF, None, BUF, BUF, BUF + 64, 4, 3136, 1e-5, None) == NULL
    assert L.nmt_rmsnorm_gated_bf16(BUF, BUF, None, BUF, 4, 6144, 768, 1e-5, None) == NULL
    assert L.nmt_relu2_bf16(BUF, None, 64, None) == NULL
    assert L.nmt_add_bf16(BUF, None, BUF, 64, None) == NULL
    assert L.nmt_embedding_bf16_i32(BUF, None, BUF, 4, 3136, 131072, None, None) == NULL
    # misaligned bf16 tensors (the reference requires 16-byte alignment, ops/reduce.cuh:134-135)
    assert L.nmt_rmsnorm_bf16(BUF + 2, BUF, BUF, 4, 3136, 1e-5, None) == ALIGN
    assert L.nmt_relu2_bf16(BUF, BUF + 8, 64, None) == ALIGN
    assert L.nmt_embedding_bf16_i64(BUF, BUF + 4, BUF, 4, 3136, 131072, None, None) == ALIGN
    assert L.nmt_rmsnorm_f32(BUF + 1, BUF, BUF, 4, 64, 1e-5, None) == ALIGN
    # shapes: cols % 8, negative sizes, group size that does not divide cols, aliased norm output
    assert L.nmt_rmsnorm_bf16(BUF, BUF, BUF, 4, 3137, 1e-5, None) == SHAPE
    assert L.nmt_rmsnorm_bf16(BUF, BUF, BUF, -1, 3136, 1e-5, None) == SHAPE
    assert L.nmt_relu2_bf16(BUF, BUF, 12, None) == SHAPE
    assert L.nmt_rmsnorm_gated_bf16(BUF, BUF, BUF, BUF, 4, 6144, 1000, 1e-5, None) == SHAPE
    assert L.nmt_embedding_bf16_i64(BUF, BUF, BUF, 4, 3133, 131072, None, None) == SHAPE
    assert L.nmt_add_rmsnorm_bf16(BUF, BUF + 64, BUF, BUF, BUF, 4, 3136, 1e-5, None) == SHAPE
    assert L.nmt_launch_count() == before, "a rejected call must launch nothing"
    for s in range(6):
        assert L.nmt_status_string(s)


def test_tuning_knobs_round_trip(built_lib):
    v = ctypes.c_int(-1)
    assert built_lib.nmt_tune_set(b"ew.unroll", 4) == 0
    assert built_lib.nmt_tune_get(b"ew.unroll", ctypes.byref(v)) == 0 and v.value == 4
    assert built_lib.nmt_tune_set(b"ew.unroll", 0) == 0
    assert built_lib.nmt_tune_set(b"no.such.knob", 1) == 5


def test_binding_mirrors_reference_constants_and_names():
    from nemotron_infer_b200 import binding as B
    # binding.cu:35-46, 214-226
    assert (B.HIDDEN, B.H, B.P, B.N, B.G, B.CONV_K) == (3136, 96, 80, 128, 8, 4)
    assert (B.H_Q, B.H_KV, B.HEAD, B.INTER, B.VOCAB) == (40, 8, 128, 12544, 131072)
    assert B.CONV_DIM == 9728 and B.IN_PROJ == 17504
    for name in ("embedding", "rmsnorm", "sync", "reset_allocator", "free_allocator",
                 "add_rmsnorm", "rmsnorm_gated", "relu2", "add"):
        assert callable(getattr(B, name))


def test_operators_refuse_cpu_tensors(built_lib):
    import torch
    from nemotron_infer_b200 import ops
    x = torch.zeros(2, 3136, dtype=torch.bfloat16)
    w = torch.ones(3136)
    with pytest.raises(ValueError, match="no CPU fallback"):
        ops.rmsnorm(x, w)
    with pytest.raises(ValueError, match="no CPU fallback"):
        ops.relu2(x)


def test_binding_raises_on_rejected_arguments(built_lib):
    from nemotron_infer_b200 import NemotronB200Error, binding as B
    with pytest.raises(NemotronB200Error) as e:
        B.rmsnorm(0, BUF, BUF, 4)
    assert e.value.status == 1
    B.rmsnorm(BUF, BUF, BUF, 0)      # M == 0 is a no-op, like a zero-size grid in the reference


def test_pybind_module_has_the_reference_surface(built_lib):
    """The compiled pybind11 module keeps the reference's names, arity and None return for the hot ops
    (binding.cu:59-73, 214-232) and raises instead of invoking undefined behaviour."""
    from nemotron_infer_b200.pybind import binding as B
    assert (B.HIDDEN, B.INTER, B.VOCAB, B.CONV_DIM, B.IN_PROJ, B.G) == (3136, 12544, 131072, 9728, 17504, 8)
    assert B.embedding(BUF, BUF, BUF, 0) is None          # (table, ids, out, num_tokens)
    assert B.rmsnorm(BUF, BUF, BUF, 0) is None             # (in, out, w, M)
    assert B.reset_allocator() is None and B.free_allocator() is None
    assert B.add_rmsnorm(BUF, BUF + 64, BUF, BUF, BUF + 128, 0) is None
    with pytest.raises(RuntimeError, match="null pointer"):
        B.rmsnorm(0, BUF, BUF, 4)
    with pytest.raises(TypeError):
        B.rmsnorm(BUF, BUF, BUF)                            # same arity as the reference


def test_cross_block_fusion_entry_points_validate_and_count_without_launching(built_lib):
    """The announcement / bookkeeping half of the cross-block fusion needs no device: a misaligned weight is refused,
    NULL withdraws, rows == 0 goes through the head and tail entry points as a no-op, and nothing is counted."""
    L = built_lib
    before = L.nmt_launch_count()
    a, b = ctypes.c_int64(-1), ctypes.c_int64(-1)
    assert L.nmt_fusion_reset() == 0
    assert L.nmt_fusion_counters(ctypes.byref(a), ctypes.byref(b)) == 0
    fused0, skipped0 = a.value, b.value
    assert L.nmt_fuse_next_norm(BUF, 1e-5) == 0
    assert L.nmt_fuse_next_norm(BUF + 4, 1e-5) == 2
    assert L.nmt_fuse_next_norm(None, 1e-5) == 0
    assert L.nmt_fuse_next_norm(BUF, 1e-5) == 0
    assert L.nmt_block_head_rmsnorm_bf16(BUF, BUF, BUF, 0, 3136, 1e-5, None) == 0
    assert L.nmt_block_tail_add_bf16(BUF, BUF, BUF, 0, None) == 0
    assert L.nmt_block_head_rmsnorm_bf16(None, BUF, BUF, 4, 3136, 1e-5, None) == 1
    assert L.nmt_block_tail_add_bf16(BUF, BUF + 2, BUF, 64, None) == 2
    assert L.nmt_fusion_counters(ctypes.byref(a), ctypes.byref(b)) == 0
    assert (a.value, b.value) == (fused0, skipped0)
    assert L.nmt_fusion_reset() == 0
    assert L.nmt_launch_count() == before
