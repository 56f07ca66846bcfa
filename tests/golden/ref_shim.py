"""Import the reference's own Python modules on a CPU-only machine.

Used only by ``make_golden.py`` (the script that produced the committed
``*.npz`` fixtures).  Nothing in the test-suite or the product imports this
module: the reference tree is not available where the GPU tests run.

The reference modules are imported *unmodified*; four stand-ins make them
executable without a GPU:

1. ``fast_hadamard_transform`` (imported at the top of ``model/public_func.py``
   but absent here) becomes an empty module.
2. ``kvhq_gemv`` (the reference's unbuilt CUDA extension) becomes an empty
   module, so ``quant/matmul.py`` imports; none of its functions are called.
3. ``torch.sort`` as seen by ``model/public_func.py`` is forced to ``stable=True``.  The
   reference sorts block keys with the default (unstable) sort, whose order among equal fp16
   keys is unspecified and differs between torch's CPU and CUDA sorts; a stable sort is one of
   the orders it may legally produce, and it makes the fixtures reproducible.
4. The two Triton launch objects of ``quant/pack_unpack.py`` are replaced by
   CPU callables with the same ``kernel[grid](...)`` call shape that perform
   the same bit placement (element i of a word at bits [i*bit, (i+1)*bit)),
   and ``torch.cuda.device(<cpu device>)`` becomes a null context.
"""
import contextlib
import os
import sys
import types

import torch

REFERENCE_ROOT = os.environ.get("HQEKV_REFERENCE_ROOT", "/root/reference")


class _CpuLaunch:
    """Mimics ``triton_kernel[grid](*args, **kwargs)`` with a Python callable."""

    def __init__(self, fn):
        self._fn = fn

    def __getitem__(self, grid):
        return self._fn


def _cpu_pack(bits, intensor, code, n_rows, num_feats, feat_per_int, BLOCK_SIZE_N=128, num_warps=8):
    src = intensor.reshape(n_rows, num_feats // feat_per_int, feat_per_int).to(torch.int64)
    shifts = torch.arange(feat_per_int, dtype=torch.int64) * bits
    words = ((src & 0xFFFFFFFF) << shifts).sum(-1) & 0xFFFFFFFF
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    code.copy_(words.to(torch.int32).reshape(code.shape))


def _cpu_unpack(bits, intensor, data, n_rows, num_feats, feat_per_int, BLOCK_SIZE_N=128, num_warps=8):
    words = intensor.reshape(n_rows, num_feats).to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(feat_per_int, dtype=torch.int64) * bits
    vals = (words.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    data.copy_(vals.reshape(n_rows, num_feats * feat_per_int).to(data.dtype))


def load_reference():
    """Return a namespace with the reference modules of the hot path."""
    if not os.path.isdir(REFERENCE_ROOT):
        raise RuntimeError(f"reference tree not found at {REFERENCE_ROOT}")
    for p in (REFERENCE_ROOT, os.path.join(REFERENCE_ROOT, "quant")):
        if p not in sys.path:
            sys.path.insert(0, p)
    sys.modules.setdefault("fast_hadamard_transform", types.ModuleType("fast_hadamard_transform"))
    sys.modules.setdefault("kvhq_gemv", types.ModuleType("kvhq_gemv"))

    real_device_ctx = torch.cuda.device

    def _device_ctx(dev):
        if torch.device(dev).type == "cpu":
            return contextlib.nullcontext()
        return real_device_ctx(dev)

    torch.cuda.device = _device_ctx

    import pack_unpack  # noqa: E402  (reference module)

    pack_unpack._pack_along_last_dim = _CpuLaunch(_cpu_pack)
    pack_unpack._unpack_along_last_dim = _CpuLaunch(_cpu_unpack)

    from model import public_func  # noqa: E402

    class _TorchStableSort:
        def __getattr__(self, name):
            return getattr(torch, name)

        @staticmethod
        def sort(input, *args, **kwargs):
            kwargs["stable"] = True
            return torch.sort(input, *args, **kwargs)

    public_func.torch = _TorchStableSort()
    import hqe_2  # noqa: E402

    ns = types.SimpleNamespace(pack_unpack=pack_unpack, public_func=public_func, hqe_2=hqe_2)
    return ns
