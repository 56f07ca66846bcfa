"""Decode attention over the tiered cache — same name, arguments, results and errors as
qkv_matmul_hqe_2 in the reference's quant/hqe_matmul.py:354-451, in one call into libhqkv
(hqekv_b200/csrc/decode.cu) instead of up to a dozen per-tier GEMV launches with index scatter /
gather copies between them.
"""
from typing import Tuple

import torch

from .._lib import CODEC_NORMAL, CODEC_UNIFORM, HqkvError, check, decode_workspace, lib, ptr, require_cuda, stream_ptr
from ._cache import UNIFORM_STRATEGIES, cached_cache_desc


def qkv_matmul_hqe_2(q: torch.Tensor, past_key_value: Tuple, attention_mask: torch.Tensor, head_dim: int,
                     quant_strategy: str, block_size: int = 32, group_size: int = 32, *, head_sum_out=None):
    """softmax(q K^T / sqrt(d)) V over all tiers and the fp16 residual window.

    ``head_sum_out`` (keyword only, not in the reference's signature): a float16 row of at least L elements that
    receives ``attn_weights.sum(0).sum(0)`` - the importance row last_attn_weights.update would compute from the
    result (model/public_func.py:253-254) - written by the decode call itself.

    q [B, nh_q, 1, D] float16; ``past_key_value`` the 42-slot tuple.  ``attention_mask`` is accepted
    and ignored, as on the reference path (its use is commented out at quant/hqe_matmul.py:431);
    ``head_dim`` is re-derived from the cache as the reference does (:379-404).
    Returns (attn_weights [B, nh_q, 1, L] float16, attn_output [B, nh_q, 1, D] float16).
    Raises ValueError('invalid quant_strategy') / ValueError('invalid past_key_value') like the
    reference.  Under 'uniform_group' all five tiers are uniform-group tiers; under
    'high_uniform_group_low_normal_group' the 1-bit tier is read in the Gaussian-codebook codec
    (slots +2 / +3 hold std / mean; cuda_bmm_fA_qB_normal_group, quant/matmul.py:72-95).
    """
    if quant_strategy not in UNIFORM_STRATEGIES:
        raise ValueError("invalid quant_strategy")
    if len(past_key_value) != 42:
        raise ValueError("invalid past_key_value")
    low_codec = CODEC_UNIFORM if quant_strategy == "uniform_group" else CODEC_NORMAL
    require_cuda(q)
    if q.dtype != torch.float16 or q.dim() != 4 or q.shape[2] != 1:
        raise ValueError("q must be float16 of shape [B, nh_q, 1, head_dim]")
    desc, keep, L, dev = cached_cache_desc(past_key_value, q.shape[1], block_size, group_size, low_codec)
    if dev != q.device or q.shape[0] != desc.B or q.shape[3] != desc.D:
        raise ValueError("q does not match the cache (device, batch or head_dim)")
    q = q.contiguous()
    B, nh_q, D = q.shape[0], q.shape[1], q.shape[3]
    attn_weights = torch.empty(B, nh_q, 1, L, dtype=torch.float16, device=dev)
    attn_output = torch.empty(B, nh_q, 1, D, dtype=torch.float16, device=dev)
    if head_sum_out is not None:
        if (head_sum_out.dtype != torch.float16 or head_sum_out.device != dev or head_sum_out.dim() != 1
                or head_sum_out.numel() < L or head_sum_out.stride(0) != 1):
            raise ValueError("head_sum_out must be a contiguous float16 row of at least L elements on the cache's device")
    if dev.index is None or dev.index == torch.cuda.current_device():
        _launch(desc, q, attn_weights, attn_output, dev, head_sum_out)
    else:
        with torch.cuda.device(dev):
            _launch(desc, q, attn_weights, attn_output, dev, head_sum_out)
    return attn_weights, attn_output


def _launch(desc, q, attn_weights, attn_output, dev, head_sum_out=None):
    need = lib.hqkv_decode_workspace_bytes(desc)
    if need == 0:
        _raise_from_status(lib.hqkv_decode_attention(desc, ptr(q), ptr(attn_weights), ptr(attn_output), None, 0, None))
    st = stream_ptr(dev)
    ws = decode_workspace(dev, need, st)
    if head_sum_out is None:
        rc = lib.hqkv_decode_attention(desc, q.data_ptr(), attn_weights.data_ptr(), attn_output.data_ptr(), ws.data_ptr(),
                                       ws.numel(), st)
    else:
        rc = lib.hqkv_decode_attention_headsum(desc, q.data_ptr(), attn_weights.data_ptr(), attn_output.data_ptr(),
                                               head_sum_out.data_ptr(), ws.data_ptr(), ws.numel(), st)
    if rc:
        _raise_from_status(rc)


def _raise_from_status(rc):
    if rc == -2:
        raise NotImplementedError(lib.hqkv_last_error().decode())
    check(rc)


def qkv_matmul_hqe(q: torch.Tensor, past_key_value: Tuple, attention_mask: torch.Tensor, head_dim: int,
                   quant_strategy: str, block_size: int = 32, group_size: int = 32):
    """quant/hqe_matmul.py:27-92: the variant whose index scatter / gather happens inside the GEMV kernels
    (cuda_bmm_forward_qk_group_hq / cuda_bmm_forward_wv_group_hq) instead of between per-tier launches.  The
    fused decode does exactly that, so this is the same call.  Like the reference it accepts only
    'high_uniform_group_low_normal_group' (:43-47: uniform-group high tiers, Gaussian-codebook 1-bit tier)
    and raises ValueError('invalid quant_strategy') otherwise."""
    if quant_strategy != "high_uniform_group_low_normal_group":
        raise ValueError("invalid quant_strategy")
    return qkv_matmul_hqe_2(q, past_key_value, attention_mask, head_dim, quant_strategy, block_size, group_size)


def qkv_matmul_hqe_1(q: torch.Tensor, past_key_value: Tuple, attention_mask: torch.Tensor, head_dim: int,
                     quant_strategy: str, block_size: int = 32, group_size: int = 32):
    """quant/hqe_matmul.py:94-147: decode over the SEQUENTIAL layout of quant/hqe_1.py - no index lists, the
    logical order is tier order (16, 8, 4, 2, 1 bit) then the residual window; the 1-bit tier is always read in
    the Gaussian-codebook codec (cuda_bmm_forward_qk_group_hq_seq passes std / mean and the centre,
    quant/matmul.py:436-505).  The same fused kernel with identity index lists; ``quant_strategy`` is not looked
    at, as in the reference."""
    if len(past_key_value) != 42:
        raise ValueError("invalid past_key_value")
    from .hqe_1 import sequential_index_lists
    return qkv_matmul_hqe_2(q, sequential_index_lists(past_key_value), attention_mask, head_dim,
                            "high_uniform_group_low_normal_group", block_size, group_size)
