import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


# Every 1-ulp comparison of the parity tests records what it observed here; when the environment variable
# NMT_ULP_REPORT names a file, the list is written there as JSON at the end of the session.
ULP_LOG: list = []


def pytest_sessionfinish(session, exitstatus):
    path = os.environ.get("NMT_ULP_REPORT")
    if path and ULP_LOG:
        import json
        with open(path, "w") as f:
            json.dump(ULP_LOG, f, indent=0)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # A GPU test on a box without a GPU is a configuration error, not a pass.
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if not has_gpu:
        skip = pytest.mark.skip(reason="no CUDA device")
        for it in items:
            if "gpu" in it.keywords:
                it.add_marker(skip)


@pytest.fixture(scope="session")
def built_lib():
    """Builds (if stale) and loads the C-ABI library; fails loudly when it cannot."""
    from nemotron_infer_b200 import _lib, build
    build.build()
    build.build_pybind()
    return _lib.load()


@pytest.fixture(scope="session")
def oracle_c():
    """The scalar C restatement of the reference's test loops (oracle/ref_loops.c)."""
    path = os.path.join(ROOT, "oracle", "_build", "liboracle_c.so")
    if not os.path.exists(path):
        import subprocess
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "oracle"], check=True, stdout=subprocess.DEVNULL)
    lib = ctypes.CDLL(path)
    fp = ctypes.POINTER(ctypes.c_float)
    sz = ctypes.c_size_t
    lib.orc_bf16_round.restype = ctypes.c_float
    lib.orc_bf16_round.argtypes = [ctypes.c_float]
    lib.orc_rmsnorm_f32.argtypes = [fp, fp, fp, sz, sz, ctypes.c_float]
    lib.orc_rmsnorm_bf16.argtypes = [fp, fp, fp, sz, sz, ctypes.c_float]
    lib.orc_gated_f32.argtypes = [fp, fp, fp, fp, sz, sz, sz, ctypes.c_float]
    lib.orc_gated_bf16.argtypes = [fp, fp, fp, fp, sz, sz, sz, ctypes.c_float]
    lib.orc_relu2_f32.argtypes = [fp, fp, sz]
    lib.orc_add_f32.argtypes = [fp, fp, fp, sz]
    lib.orc_embedding_u16.argtypes = [ctypes.POINTER(ctypes.c_uint16), ctypes.POINTER(ctypes.c_int64),
                                      ctypes.POINTER(ctypes.c_uint16), sz, sz]
    return lib


@pytest.fixture(scope="session")
def ref_kernels():
    """The reference's own kernels recompiled for sm_100a (oracle/_ref), or None when not built."""
    path = os.path.join(ROOT, "oracle", "_ref", "libnemotron_ref.so")
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    return lib


def fptr(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


def bf16_from_bits(bits: np.ndarray):
    import torch
    return torch.from_numpy(bits.astype(np.uint16).view(np.int16).copy()).view(torch.bfloat16)
