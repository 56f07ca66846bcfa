"""Batched GEMV of fp16 activations with one packed tier — same names and argument meaning as
cuda_bmm_fA_qB_uniform_group / cuda_bmm_fA_qB_normal_group in the reference's quant/matmul.py:263-299,
72-95, backed by hqkv_gemv_uniform_group / hqkv_gemv_normal_group (hqekv_b200/csrc/gemv.cu).

The reference flattens (B, nh) and makes transposed contiguous copies of the codes, scales and
zeros on every call before entering its extension; here the operands are read in the layout the
cache stores them in.
"""
import torch

from .._lib import check, lib, ptr, require_cuda, stream_ptr


def _gemv(entry, widths, group_size, fA, qB, scales, zeros, bits):
    """C = fA x dequant(qB) with fp32 accumulation.

    fA     (B, nh_q, 1, K) float16
    qB     (B, nh_kv, K, N // feat_per_int) int32
    scales (B, nh_kv, K, N // group_size) float16
    zeros  (B, nh_kv, K, N // group_size) float16
    Returns C (B, nh_q, 1, N) float16.
    """
    require_cuda(fA, qB, scales, zeros)
    if fA.dim() != 4 or qB.dim() != 4:
        raise ValueError("invalid matrix.")
    B, nh_q, M, K = fA.shape
    if M != 1:
        raise ValueError("invalid matrix.")  # decode only: one query row, as in the reference's kernels
    nh_kv = qB.shape[1]
    if qB.shape[2] != K or bits not in widths:
        raise ValueError("invalid matrix.")
    N = qB.shape[3] * (32 // bits)
    fA, qB, scales, zeros = fA.contiguous(), qB.contiguous(), scales.contiguous(), zeros.contiguous()
    out = torch.empty(B, nh_q, 1, N, dtype=torch.float16, device=fA.device)
    with torch.cuda.device(fA.device):
        check(entry(ptr(fA), ptr(qB), ptr(scales), ptr(zeros), B, nh_q, nh_kv, K, N, group_size, bits, ptr(out),
                    stream_ptr(fA.device)))
    return out


def cuda_bmm_fA_qB_uniform_group(group_size: int, fA: torch.Tensor, qB: torch.Tensor, scales: torch.Tensor,
                                 zeros: torch.Tensor, bits: int) -> torch.Tensor:
    """quant/matmul.py:263-299; shapes as in :func:`_gemv`, bits 8, 4, 2 or 1."""
    return _gemv(lib.hqkv_gemv_uniform_group, (8, 4, 2, 1), group_size, fA, qB, scales, zeros, bits)


def cuda_bmm_fA_qB_normal_group(group_size: int, fA: torch.Tensor, qB: torch.Tensor, stds: torch.Tensor,
                                means: torch.Tensor, bits: int) -> torch.Tensor:
    """quant/matmul.py:72-95 at bits = 1 (Gaussian codebook: std * (+-0.67448974) + mean); wider
    codebooks raise NotImplementedError."""
    if bits != 1:
        raise NotImplementedError("cuda_bmm_fA_qB_normal_group: only bits = 1 is built in hqekv_b200")
    return _gemv(lib.hqkv_gemv_normal_group, (1,), group_size, fA, qB, stds, means, bits)


def _not_built(name):
    def f(*args, **kwargs):
        raise NotImplementedError(f"{name}: this variant of the reference's GEMV wrappers is not built in hqekv_b200 "
                                  "(outlier, un-grouped and token-major paths)")
    f.__name__ = name
    return f


cuda_bmm_fA_qB_normal = _not_built("cuda_bmm_fA_qB_normal")
cuda_bmm_fA_qB_uniform = _not_built("cuda_bmm_fA_qB_uniform")
