"""B200 (sm_100a) replacements for nemotron_infer's bandwidth-bound layer kernels.

`binding` mirrors the reference's pybind module (integer device addresses);
`ops` is the same set of operators over torch tensors; `chain` runs the
per-pass op mix of one forward pass.  Everything goes through
libnemotron_b200.so (see include/nemotron_b200.h); build it with
`python -m nemotron_infer_b200.build`.
"""
from ._lib import LIB_PATH, NemotronB200Error, load  # noqa: F401

__all__ = ["LIB_PATH", "NemotronB200Error", "load"]
