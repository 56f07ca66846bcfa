"""No-eviction flavour of the flush — same names and arguments as KV_cache_compress /
KV_cache_reconstruct in the reference's quant/hybrid_quant.py (:318-329, :732-737).

That flavour is the ladder of quant/hqe_2.py without the eviction step: five tier counts instead of
six, V always ranked by importance x value range, no importance ring to compact.  It therefore maps
onto the same planning and build kernels with an eviction count of zero.
"""
import torch

from .hqe_2 import KV_cache_hqe_2, KV_cache_reconstruct_hqe


def KV_cache_compress(past_key_value: tuple, compress_length: int, history_length: int, K_sorted_idx: torch.Tensor,
                      K_bit_num: torch.Tensor, V_bit_num: torch.Tensor, token_importance: torch.Tensor,
                      quant_strategy: str, block_size: int = 32, group_size: int = 32):
    """quant/hybrid_quant.py:318-612.  ``K_bit_num`` / ``V_bit_num`` hold five counts (16, 8, 4, 2, 1 bit)."""
    k = [int(v) for v in (K_bit_num.tolist() if hasattr(K_bit_num, "tolist") else K_bit_num)]
    v = [int(x) for x in (V_bit_num.tolist() if hasattr(V_bit_num, "tolist") else V_bit_num)]
    if len(k) != 5 or len(v) != 5:
        raise ValueError("K_bit_num and V_bit_num must hold five counts")
    return KV_cache_hqe_2(past_key_value, compress_length, history_length, K_sorted_idx, k + [0], v + [0],
                          token_importance, quant_strategy, None, block_size, group_size, True)


def KV_cache_reconstruct(past_key_value: tuple, quant_strategy: str, block_size: int = 32, group_size: int = 32):
    """quant/hybrid_quant.py:732-846: dense fp16 (K, V) of the whole cache."""
    return KV_cache_reconstruct_hqe(past_key_value, quant_strategy, block_size, group_size)
