"""Decode attention entry points of the no-eviction flavour - same names and arguments as qkv_matmul /
qkv_matmul_hq in the reference's quant/quant_matmul_hq.py (:23-31, :122-130).

Without eviction the cache's logical length equals kv_seq_len, so both map onto the fused decode of
quant/hqe_matmul.py.  The reference adds ``attention_mask`` to the scaled logits before the softmax (:101,
:164); the fused kernel does the same when a mask is given (hqkv_decode_attention_masked).
"""
import torch

from .._lib import CODEC_NORMAL, CODEC_UNIFORM, check, decode_workspace, lib, require_cuda, stream_ptr
from ._cache import UNIFORM_STRATEGIES, cached_cache_desc
from .hqe_matmul import qkv_matmul_hqe_2


def _masked(q, past_key_value, attention_mask, quant_strategy, block_size, group_size):
    if quant_strategy not in UNIFORM_STRATEGIES:
        raise ValueError("invalid quant_strategy")
    if len(past_key_value) != 42:
        raise ValueError("invalid past_key_value")
    require_cuda(q, attention_mask)
    low_codec = CODEC_UNIFORM if quant_strategy == "uniform_group" else CODEC_NORMAL
    desc, keep, L, dev = cached_cache_desc(past_key_value, q.shape[1], block_size, group_size, low_codec)
    B, nh_q, D = q.shape[0], q.shape[1], q.shape[3]
    m = attention_mask
    if m.dim() != 4 or m.shape[2] != 1 or m.shape[3] != L or m.shape[0] not in (1, B) or m.shape[1] not in (1, nh_q):
        raise ValueError(f"attention_mask must be [B or 1, nh_q or 1, 1, {L}]")
    m = m.to(torch.float16).contiguous()
    b_stride = 0 if m.shape[0] == 1 else m.shape[1] * L
    h_stride = 0 if m.shape[1] == 1 else L
    q = q.contiguous()
    attn_weights = torch.empty(B, nh_q, 1, L, dtype=torch.float16, device=dev)
    attn_output = torch.empty(B, nh_q, 1, D, dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        st = stream_ptr(dev)
        ws = decode_workspace(dev, lib.hqkv_decode_workspace_bytes(desc), st)
        check(lib.hqkv_decode_attention_masked(desc, q.data_ptr(), m.data_ptr(), b_stride, h_stride, attn_weights.data_ptr(),
                                               attn_output.data_ptr(), ws.data_ptr(), ws.numel(), st))
    return attn_weights, attn_output


def _no_mask(attention_mask):
    return attention_mask is None or (not torch.is_tensor(attention_mask) and attention_mask == 0)


def qkv_matmul(q, past_key_value, attention_mask, head_dim, quant_strategy, block_size=32, group_size=32):
    """quant/quant_matmul_hq.py:23-120."""
    if _no_mask(attention_mask):
        return qkv_matmul_hqe_2(q, past_key_value, None, head_dim, quant_strategy, block_size, group_size)
    return _masked(q, past_key_value, attention_mask, quant_strategy, block_size, group_size)


def qkv_matmul_hq(q, past_key_value, attention_mask, head_dim, quant_strategy, block_size=32, group_size=32):
    """quant/quant_matmul_hq.py:122-174 (the variant that calls the fused-index GEMVs): the same fused call."""
    return qkv_matmul(q, past_key_value, attention_mask, head_dim, quant_strategy, block_size, group_size)
