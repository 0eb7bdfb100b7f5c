"""A bounded wait that actually runs out, in the harmless form: a self-test kernel waits a few polls on an mbarrier
in its own shared memory that nothing completes.  The timeout must be counted, reported, and leave the context
usable.  Run in a child process, because the counter is per process and every other test asserts that it stays 0."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

CHILD = r'''
import torch
from nemotron_infer_b200 import _lib, ops
lib = _lib.load()
assert lib.nmt_set_device(0) == 0
x = torch.randn(8, 3136, device="cuda").to(torch.bfloat16)
w = torch.ones(3136, device="cuda")
ops.rmsnorm(x, w)
assert lib.nmt_device_wait_timeouts() == 0
flag = torch.zeros(1, dtype=torch.int32, device="cuda")
assert lib.nmt_selftest_wait_runs_out(64, flag.data_ptr(), None) == 0
assert lib.nmt_device_wait_timeouts() == 1, "the run-out wait must be counted"
assert int(flag.item()) == 1
assert lib.nmt_selftest_wait_runs_out(0, None, None) == 3 and lib.nmt_selftest_wait_runs_out(5000, None, None) == 3
# the context is still usable: a product kernel runs and gives the right answer afterwards
y = ops.rmsnorm(x, w)
torch.cuda.synchronize()
ref = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16)
assert (y.float() - ref.float()).abs().max().item() < 0.05
assert lib.nmt_selftest_wait_runs_out(8, None, None) == 0
assert lib.nmt_device_wait_timeouts() == 2
print("WAIT_SELFTEST_OK")
'''


def test_a_wait_that_runs_out_is_counted_and_leaves_the_context_usable(built_lib):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0 and "WAIT_SELFTEST_OK" in r.stdout, r.stdout + r.stderr
