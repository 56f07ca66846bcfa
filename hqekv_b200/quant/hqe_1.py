"""Names of the reference's quant/hqe_1.py that quant/hqe_matmul.py:8 imports.

quant/hqe_1.py keeps every tier in arrival order without index lists (the "sequential" layout read by
qkv_matmul_hqe_1, quant/hqe_matmul.py:94-147).  Its flush (quant/hqe_1.py:314-425) is not on the decode path
of the reference's model files and is not built; the decode over that layout is
(:func:`hqekv_b200.quant.hqe_matmul.qkv_matmul_hqe_1`), and so is the dense reconstruction, which is the
reconstruction of quant/hqe_2.py with identity index lists.
"""
import torch

from . import hqe_2 as _hqe_2
from ._cache import SLOT_K, SLOT_NEW_K, SLOT_V, TIER_BITS


def KV_cache_hqe_1(*args, **kwargs):
    raise NotImplementedError("KV_cache_hqe_1 (quant/hqe_1.py:314): the sequential-layout flush of the reference is "
                              "not built in hqekv_b200; the models flush through quant.hqe_2.KV_cache_hqe_2")


def sequential_index_lists(past_key_value: tuple) -> tuple:
    """The 42-slot tuple with index lists filled in for the sequential layout: tier order 16, 8, 4, 2, 1 bit,
    tokens of a tier in storage order, then the residual window (quant/hqe_matmul.py:138-146)."""
    cache = list(past_key_value)
    for slots in (SLOT_K, SLOT_V):
        at = 0
        for bits in TIER_BITS:
            data = cache[slots[bits]]
            if data is None:
                continue
            if slots is SLOT_K:
                n = data.shape[3] * (1 if bits == 16 else 32 // bits)
            else:
                n = data.shape[2]
            cache[slots[bits] + 1] = torch.arange(at, at + n, dtype=torch.int64, device=data.device)
            at += n
    return tuple(cache)


def KV_cache_reconstruct_hqe(past_key_value: tuple, quant_strategy: str, block_size: int = 32, group_size: int = 32):
    """quant/hqe_1.py:428-520: dense fp16 (K, V) of a sequential-layout cache."""
    return _hqe_2.KV_cache_reconstruct_hqe(sequential_index_lists(past_key_value), quant_strategy, block_size, group_size)
