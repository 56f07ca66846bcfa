"""The bounds-check build (-DHQKV_CHECKS) on small cases: the stand-in for a memory checker.

The regular library trusts the index lists of the cache tuple.  The checked build range-checks every index it
takes out of a caller-supplied list before addressing memory with it, counts violations and skips the access.
Here (1) a set of small decode and flush parity cases runs under the checked build in a child process and must
report zero violations, and (2) a cache whose index list holds out-of-range positions must be reported - and
must not fault, the accesses being skipped.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import ctypes, sys
import numpy as np, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
from hqekv_b200 import _lib, synthetic
from hqekv_b200.quant.hqe_matmul import qkv_matmul_hqe_2
assert _lib.lib.hqkv_checks_enabled() == 1, "the checked library is not the one loaded"
dev = torch.device("cuda:0")
def failures(reset=1):
    n = ctypes.c_uint(0)
    _lib.check(_lib.lib.hqkv_check_failures(reset, ctypes.byref(n)))
    return n.value
failures()
# (1) clean cases: flush (plan + build kernels) and decode over every tier kind, ragged residuals, GQA 1/4/8
for batch, nh_q, nh_kv, ctx, res, ratios, evict, group, strat in (
        (1, 8, 2, 4 * 32 + 5, 5, (0.25, 0.25, 0.25, 0.25), 0.0, 32, "uniform_group"),
        (2, 16, 2, 640 + 33, 33, (0.2, 0.4, 0.4), 0.1, 32, "uniform_group"),
        (3, 4, 4, 512 + 16, 16, (0.25, 0.5, 0.25), 0.0, 64, "uniform_group"),
        (1, 32, 8, 1024 + 40, 40, (0.25, 0.25, 0.25, 0.25), 0.125, 32, "high_uniform_group_low_normal_group"),
        (2, 8, 2, 128 * 5 + 100, 100, (0.34, 0.33, 0.33), 0.0, 128, "uniform_group")):
    cfg = synthetic.CacheConfig("chk", batch, nh_q, nh_kv, 128, ctx, res, ratios, evict, group, True, 1, 32)
    cache, q = synthetic.build_cache(cfg, dev, seed=3, times_range=True, quant_strategy=strat)
    w, o = qkv_matmul_hqe_2(q, cache, None, 128, strat, group, group)
    torch.cuda.synchronize()
    assert torch.isfinite(o).all()
n = failures()
assert n == 0, f"{{n}} index violations on well-formed caches"
# (2) an index list with positions beyond the logical length: counted, skipped, no fault
bad = list(cache)
idx = bad[13].clone()            # positions of the 4-bit K tier
idx[:7] = 10 ** 6
bad[13] = idx
w, o = qkv_matmul_hqe_2(q, tuple(bad), None, 128, strat, group, group)
torch.cuda.synchronize()
n = failures()
assert n >= 7, f"out-of-range positions were not reported ({{n}})"
assert float(torch.ones(8, device=dev).sum()) == 8.0
print("checked build ok:", n, "violations reported for the malformed cache")
"""


def test_small_cases_under_the_bounds_check_build(cuda_device):
    from hqekv_b200 import build
    lib = build.CHECKED_LIB_PATH
    if not os.path.exists(lib):
        lib = build.build(checks=True)
    env = dict(os.environ, HQKV_LIB=lib)
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "checked build ok" in r.stdout
