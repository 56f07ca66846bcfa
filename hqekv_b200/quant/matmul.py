"""Batched GEMV of fp16 activations with one packed tier — same name and argument meaning as
cuda_bmm_fA_qB_uniform_group in the reference's quant/matmul.py:263-299, backed by
hqkv_gemv_uniform_group (hqekv_b200/csrc/gemv.cu).

The reference flattens (B, nh) and makes transposed contiguous copies of the codes, scales and
zeros on every call before entering its extension; here the operands are read in the layout the
cache stores them in.
"""
import torch

from .._lib import check, lib, ptr, require_cuda, stream_ptr


def cuda_bmm_fA_qB_uniform_group(group_size: int, fA: torch.Tensor, qB: torch.Tensor, scales: torch.Tensor,
                                 zeros: torch.Tensor, bits: int) -> torch.Tensor:
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
    if qB.shape[2] != K or bits not in (8, 4, 2):
        raise ValueError("invalid matrix.")
    N = qB.shape[3] * (32 // bits)
    fA, qB, scales, zeros = fA.contiguous(), qB.contiguous(), scales.contiguous(), zeros.contiguous()
    out = torch.empty(B, nh_q, 1, N, dtype=torch.float16, device=fA.device)
    with torch.cuda.device(fA.device):
        check(lib.hqkv_gemv_uniform_group(ptr(fA), ptr(qB), ptr(scales), ptr(zeros), B, nh_q, nh_kv, K, N, group_size,
                                          bits, ptr(out), stream_ptr(fA.device)))
    return out


def _not_built(name):
    def f(*args, **kwargs):
        raise NotImplementedError(f"{name}: this variant of the reference's GEMV wrappers is not built in hqekv_b200 "
                                  "(outlier, un-grouped, token-major and Gaussian-codebook paths)")
    f.__name__ = name
    return f


cuda_bmm_fA_qB_normal_group = _not_built("cuda_bmm_fA_qB_normal_group")
cuda_bmm_fA_qB_normal = _not_built("cuda_bmm_fA_qB_normal")
cuda_bmm_fA_qB_uniform = _not_built("cuda_bmm_fA_qB_uniform")
