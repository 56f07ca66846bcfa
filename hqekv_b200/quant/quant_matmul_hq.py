"""Decode attention entry points of the no-eviction flavour — same names and arguments as qkv_matmul /
qkv_matmul_hq in the reference's quant/quant_matmul_hq.py (:23-31, :122-130).

Without eviction the cache's logical length equals kv_seq_len, so both map onto the fused decode of
quant/hqe_matmul.py.  The reference adds ``attention_mask`` to the logits (:88); a decode step sees
every cached token, so only an absent / zero mask is accepted here.
"""
import torch

from .hqe_matmul import qkv_matmul_hqe_2


def _check_mask(attention_mask):
    if attention_mask is None or (not torch.is_tensor(attention_mask) and attention_mask == 0):
        return
    raise NotImplementedError("an additive attention mask is not built into the fused decode; pass None or 0 "
                              "(a single-token decode step attends to the whole cache)")


def qkv_matmul(q, past_key_value, attention_mask, head_dim, quant_strategy, block_size=32, group_size=32):
    _check_mask(attention_mask)
    return qkv_matmul_hqe_2(q, past_key_value, None, head_dim, quant_strategy, block_size, group_size)


def qkv_matmul_hq(q, past_key_value, attention_mask, head_dim, quant_strategy, block_size=32, group_size=32):
    _check_mask(attention_mask)
    return qkv_matmul_hqe_2(q, past_key_value, None, head_dim, quant_strategy, block_size, group_size)
