"""Import the reference's own Python modules on a CPU-only machine.

TEST INFRASTRUCTURE ONLY.  Used by ``tests/golden/make_golden.py`` (the script that produced the committed
``*.npz`` fixtures) and by the CPU arm of ``bench.py`` (``--impl reference``), which times the reference's own
dense reconstruction when a staged copy of its modules exists (``oracle/_ref``, made by ``oracle/build_ref.py``).
Nothing in the product package imports this module.

Where the reference modules are read from: the directory named by ``HQEKV_REFERENCE_ROOT``, else the staged copy
``oracle/_ref`` beside this file; there is no other default.

The reference modules are imported *unmodified*; these stand-ins make them
executable without a GPU:

1. ``fast_hadamard_transform`` (imported at the top of ``model/public_func.py``
   but absent here) becomes an empty module.
2. ``kvhq_gemv`` (the reference's unbuilt CUDA extension) becomes a module with CPU
   callables for the two entry points the live path uses, ``gemv_forward_cuda_uniform_group`` and
   ``gemv_forward_cuda_normalize_group``: same arguments and result shape, the kernels' arithmetic
   (w = scale * code + zero, resp. std * center[code] + mean, in fp32; fp32 accumulation; fp16 result —
   quant/csrc/gemv_cuda_uniform.cu:455-489, gemv_cuda_normal.cu:104-106).  With them the reference's own
   ``qkv_matmul_hqe_2`` and ``LlamaAttention_hqe.forward`` run unmodified on the CPU; what the fixtures
   pin there is the reference's control flow and fp16 intermediate roundings, not its CUDA summation order.
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

STAGED = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
REFERENCE_ROOT = os.environ.get("HQEKV_REFERENCE_ROOT") or STAGED


def available() -> bool:
    """True if the reference modules of the hot path can be found."""
    return os.path.isfile(os.path.join(REFERENCE_ROOT, "quant", "hqe_2.py"))


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


def _cpu_unpack_words(qB, bits):
    """qB int32 [BH, N/fpi, K] (the transposed layout the reference hands its kernels) -> codes [BH, N, K]."""
    fpi = 32 // bits
    words = qB.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(fpi, dtype=torch.int64) * bits).view(1, 1, fpi, 1)
    codes = (words.unsqueeze(2) >> shifts) & ((1 << bits) - 1)          # [BH, N/fpi, fpi, K]
    return codes.reshape(qB.shape[0], qB.shape[1] * fpi, qB.shape[2])


def _cpu_gemv(fA, w, nh_q, nh_kv):
    """fA fp16 [B*nh_q, M, K], w fp32 [B*nh_kv, N, K] -> fp16 [B*nh_q, M, N] with fp32 accumulation."""
    rep = nh_q // nh_kv
    w = w.repeat_interleave(rep, dim=0)
    return torch.matmul(fA.float(), w.transpose(1, 2)).to(torch.float16)


def _cpu_gemv_uniform_group(fA, qB, scales, zeros, bits, group_size, nh_q, nh_kv):
    codes = _cpu_unpack_words(qB, bits).float()                           # [BH, N, K]
    s = scales.float().repeat_interleave(group_size, dim=1)               # [BH, G, K] -> [BH, N, K]
    z = zeros.float().repeat_interleave(group_size, dim=1)
    return _cpu_gemv(fA, s * codes + z, nh_q, nh_kv)


def _cpu_gemv_normalize_group(fA, qB, stds, means, center, bits, group_size, nh_q, nh_kv):
    codes = _cpu_unpack_words(qB, bits)
    c = center.float()[codes]
    s = stds.float().repeat_interleave(group_size, dim=1)
    m = means.float().repeat_interleave(group_size, dim=1)
    return _cpu_gemv(fA, s * c + m, nh_q, nh_kv)


def load_reference_model():
    """The reference's decode function and Llama attention module (imports transformers: slow).
    One more stand-in: ``transformers.utils.LossKwargs``, which newer transformers releases no longer
    export and ``model/llama_hqe.py`` only uses as a base of a typing class."""
    ns = load_reference()
    import transformers.utils as tu
    if not hasattr(tu, "LossKwargs"):
        from typing import TypedDict

        class LossKwargs(TypedDict, total=False):
            pass

        tu.LossKwargs = LossKwargs
    import hqe_matmul  # noqa: E402
    from model import llama_hqe  # noqa: E402
    ns.hqe_matmul, ns.llama_hqe = hqe_matmul, llama_hqe
    return ns


def load_reference():
    """Return a namespace with the reference modules of the hot path."""
    if not available():
        raise RuntimeError(f"reference modules not found under {REFERENCE_ROOT}: set HQEKV_REFERENCE_ROOT to a checkout of "
                           "skywclouds/HqeKV or stage a copy with oracle/build_ref.py")
    for p in (REFERENCE_ROOT, os.path.join(REFERENCE_ROOT, "quant")):
        if p not in sys.path:
            sys.path.insert(0, p)
    sys.modules.setdefault("fast_hadamard_transform", types.ModuleType("fast_hadamard_transform"))
    if "kvhq_gemv" not in sys.modules:
        gemv = types.ModuleType("kvhq_gemv")
        gemv.gemv_forward_cuda_uniform_group = _cpu_gemv_uniform_group
        gemv.gemv_forward_cuda_normalize_group = _cpu_gemv_normalize_group
        sys.modules["kvhq_gemv"] = gemv

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
