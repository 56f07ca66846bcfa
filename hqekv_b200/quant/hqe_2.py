"""Flush of the fp16 residual window into the tiered cache: evict + tier-assign + re-quantise.

Same names, arguments, results and errors as KV_cache_hqe_2 / KV_cache_reconstruct_hqe in the
reference's quant/hqe_2.py (:456-843, :967-1084).  The reference walks a ladder of up to 30
isin / boolean-mask / torch.cat steps with a host synchronisation in most of them and an
n_tier x n_all equality matrix for the re-ranking; here each side (K, V) is one planning kernel
plus one build kernel per destination tier (hqekv_b200/csrc/policy.cu), with a single device-to-host
copy of ten integers in between to size the new tensors.
"""
import torch

from .._lib import CODEC_NORMAL, CODEC_UNIFORM, TIER_BITS, check, lib, ptr, require_cuda, stream_ptr
from ..model.public_func import calculate_token_range, get_block_token_idx, last_attn_weights
from ._cache import (NUM_SLOTS, SLOT_K, SLOT_NEW_K, SLOT_NEW_V, SLOT_SEQ_LEN, SLOT_V, SLOT_V_TOKEN_NORM,
                     build_flush_src, cache_geometry, tier_tensors, void_p_array)
from .pack_unpack import normal_group_dequantize_unpack_last_dim, uniform_group_dequantize_unpack_last_dim

import ctypes as C

# strategies built here -> codec of the 1-bit tier (every other tier is uniform in both)
_FLUSH_STRATEGIES = {"uniform_group": CODEC_UNIFORM, "high_uniform_group_low_normal_group": CODEC_NORMAL}
_KNOWN_STRATEGIES = ("uniform", "normal", "uniform_group", "normal_group", "high_uniform_group_low_normal_group")


def _as_int_list(x):
    return [int(v) for v in (x.tolist() if hasattr(x, "tolist") else x)]


def _plan_side(cache, side, hist, compress, sorted_idx, bit_num, dev, out_counts):
    """Launch the planning kernel of one side; returns the device buffers it fills."""
    total = hist + compress
    idx_lists = [tier_tensors(cache, b, side)[1] for b in TIER_BITS]
    idx_lists = [None if i is None else i.contiguous() for i in idx_lists]
    n_host = (C.c_int32 * 5)(*[0 if i is None else i.numel() for i in idx_lists])
    counts = _as_int_list(bit_num)
    if len(counts) != 6:
        raise ValueError("bit_num must hold six counts (16, 8, 4, 2, 1 bit, evicted)")
    cum, run = [], 0
    for c in counts:
        run += c
        cum.append(run)
    cum_host = (C.c_int64 * 6)(*cum)
    plan_src = torch.empty(5, total, dtype=torch.int32, device=dev)
    plan_ids = torch.empty(5, total, dtype=torch.int64, device=dev)
    survivors = torch.empty(total, dtype=torch.int64, device=dev)
    ws = torch.empty(lib.hqkv_flush_plan_workspace_bytes(total), dtype=torch.uint8, device=dev)
    sorted_idx = sorted_idx.to(device=dev, dtype=torch.int64).contiguous()
    check(lib.hqkv_flush_plan(void_p_array(idx_lists), n_host, hist, compress, ptr(sorted_idx), cum_host,
                              ptr(plan_src), ptr(plan_ids), ptr(survivors), ptr(out_counts), ptr(ws), ws.numel(),
                              stream_ptr(dev)))
    return plan_src, plan_ids, survivors, (idx_lists, sorted_idx, ws)


def _build_side(cache, side, residual, plan_src, plan_ids, counts, B, H, D, group, dev, low_codec):
    """Build the five destination tiers of one side.  Returns [(data, idx, scale, zero)] * 5."""
    src, keep = build_flush_src(cache, side, residual, low_codec)
    build = lib.hqkv_flush_build_k if side == "K" else lib.hqkv_flush_build_v
    out = []
    for t, bits in enumerate(TIER_BITS):
        n = counts[t]
        if n == 0:
            out.append((None, None, None, None))
            continue
        if bits == 16:
            data = torch.empty((B, H, D, n) if side == "K" else (B, H, n, D), dtype=torch.float16, device=dev)
            scale = zero = None
        elif side == "K":
            data = torch.empty(B, H, D, n * bits // 32, dtype=torch.int32, device=dev)
            scale = torch.empty(B, H, D, n // group, dtype=torch.float16, device=dev)
            zero = torch.empty_like(scale)
        else:
            data = torch.empty(B, H, n, D * bits // 32, dtype=torch.int32, device=dev)
            scale = torch.empty(B, H, n, D // group, dtype=torch.float16, device=dev)
            zero = torch.empty_like(scale)
        check(build(src, B, H, D, group, t, ptr(plan_src[t]), n, ptr(data), ptr(scale), ptr(zero), stream_ptr(dev)))
        out.append((data, plan_ids[t, :n].clone(), scale, zero))
    del keep
    return out


def KV_cache_hqe_2(past_key_value: tuple, compress_length: int, history_length: int, K_sorted_idx: torch.Tensor,
                   K_bit_num: torch.Tensor, V_bit_num: torch.Tensor, token_importance: torch.Tensor,
                   quant_strategy: str, last_weights: last_attn_weights = None, block_size: int = 32,
                   group_size: int = 32, times_range: bool = True):
    """Quantise the first ``compress_length`` tokens of the residual window into the tiers, demote and
    evict cached tokens according to the ranked ids and the six per-tier counts.

    K is quantised in groups of ``block_size`` tokens per channel, V in groups of ``group_size``
    channels per token.  ``token_importance`` must be the array that was ranked for K (it then holds
    importance / block_size, because get_block_token_idx divides its argument in place); V is ranked
    here from it (times the per-token value range when ``times_range``).  ``last_weights`` and
    slot 38 (V_token_norm) are compacted to the V-side survivors.  Returns the new 42-slot tuple.
    quant_strategy 'uniform_group' and 'high_uniform_group_low_normal_group' (1-bit tier in the
    Gaussian-codebook codec, slots +2/+3 then hold std/mean) are built; the other strategy names of the
    reference raise NotImplementedError, unknown names ValueError('invalid quant_strategy').
    """
    if quant_strategy not in _KNOWN_STRATEGIES:
        raise ValueError("invalid quant_strategy")
    if quant_strategy not in _FLUSH_STRATEGIES:
        raise NotImplementedError(f"KV_cache_hqe_2: quant_strategy '{quant_strategy}' needs the un-grouped codec or the "
                                  "Gaussian codebook above 1 bit, which are not built; use 'uniform_group' or "
                                  "'high_uniform_group_low_normal_group'")
    low_codec = _FLUSH_STRATEGIES[quant_strategy]
    if len(past_key_value) != NUM_SLOTS:
        raise ValueError("invalid past_key_value")
    cache = tuple(past_key_value)
    new_K, new_V = cache[SLOT_NEW_K], cache[SLOT_NEW_V]
    if new_K is None or new_V is None:
        raise ValueError("invalid past_key_value")
    require_cuda(new_K, new_V, token_importance)
    compress_length, history_length = int(compress_length), int(history_length)
    dev = new_K.device
    B, H, _, D = new_K.shape
    res_K = new_K[:, :, compress_length:, :].clone()
    res_V = new_V[:, :, compress_length:, :].clone()
    res_K = None if res_K.numel() == 0 else res_K
    res_V = None if res_V.numel() == 0 else res_V
    flush_K = new_K[:, :, :compress_length, :]
    flush_V = new_V[:, :, :compress_length, :]
    total = history_length + compress_length
    block_num = total // block_size

    with torch.cuda.device(dev):
        # V ranking keys: importance (x per-token value range), ranked block-wise (:513-518)
        norm = calculate_token_range(flush_V, cache[SLOT_V_TOKEN_NORM])
        v_keys = token_importance.clone()
        V_sorted_idx = get_block_token_idx(block_size, block_num, v_keys, norm if times_range else None)

        counts_dev = torch.zeros(2, 8, dtype=torch.int32, device=dev)
        kp_src, kp_ids, _, keep_k = _plan_side(cache, "K", history_length, compress_length, K_sorted_idx, K_bit_num,
                                               dev, counts_dev[0])
        vp_src, vp_ids, v_surv, keep_v = _plan_side(cache, "V", history_length, compress_length, V_sorted_idx,
                                                    V_bit_num, dev, counts_dev[1])
        counts = counts_dev.cpu().tolist()  # the one synchronisation of the flush
        outK = _build_side(cache, "K", flush_K, kp_src, kp_ids, counts[0], B, H, D, block_size, dev, low_codec)
        outV = _build_side(cache, "V", flush_V, vp_src, vp_ids, counts[1], B, H, D, group_size, dev, low_codec)
        if counts[1][6]:  # something was evicted on the V side: compact the range vector and the ring
            surv = v_surv[:counts[1][5]]
            norm = norm[surv]
            if last_weights is not None:
                last_weights.eviction(surv)
        del keep_k, keep_v

    out = [None] * NUM_SLOTS
    for t, bits in enumerate(TIER_BITS):
        k, v = SLOT_K[bits], SLOT_V[bits]
        out[k], out[k + 1] = outK[t][0], outK[t][1]
        out[v], out[v + 1] = outV[t][0], outV[t][1]
        if bits < 16:
            out[k + 2], out[k + 3] = outK[t][2], outK[t][3]
            out[v + 2], out[v + 3] = outV[t][2], outV[t][3]
    out[36], out[37] = cache[36], cache[37]
    out[SLOT_V_TOKEN_NORM] = norm
    out[SLOT_NEW_K], out[SLOT_NEW_V] = res_K, res_V
    out[SLOT_SEQ_LEN] = cache[SLOT_SEQ_LEN]
    return tuple(out)


def KV_cache_reconstruct_hqe(past_key_value: tuple, quant_strategy: str, block_size: int = 32, group_size: int = 32):
    """Dense fp16 K and V [B, H, L, D] at logical positions (quant/hqe_2.py:967-1084): every tier
    dequantised with the two-rounding recipe and scattered by its index list.  A checking aid, not
    part of the decode step.  Unlike the reference (:1060) the 4-bit V tier is restored whether or
    not an 8-bit V tier exists."""
    if quant_strategy not in _KNOWN_STRATEGIES:
        raise ValueError("invalid quant_strategy")
    if quant_strategy not in _FLUSH_STRATEGIES:
        raise NotImplementedError(f"KV_cache_reconstruct_hqe: quant_strategy '{quant_strategy}' is not built")
    normal_low = _FLUSH_STRATEGIES[quant_strategy] == CODEC_NORMAL

    def dense_of(data, a, b, group, bits):
        if bits == 1 and normal_low:
            return normal_group_dequantize_unpack_last_dim(data, a, b, group, bits)
        return uniform_group_dequantize_unpack_last_dim(data, a, b, group, bits)

    cache = tuple(past_key_value)
    B, H, D, n, r, dev = cache_geometry(cache)
    L = n + r
    K = torch.zeros(B, H, L, D, dtype=torch.float16, device=dev)
    V = torch.zeros(B, H, L, D, dtype=torch.float16, device=dev)
    for bits in TIER_BITS:
        kd, ki, ks, kz = tier_tensors(cache, bits, "K")
        if kd is not None:
            dense = kd if bits == 16 else dense_of(kd, ks, kz, block_size, bits)
            K[:, :, ki, :] = dense.transpose(2, 3)
        vd, vi, vs, vz = tier_tensors(cache, bits, "V")
        if vd is not None:
            dense = vd if bits == 16 else dense_of(vd, vs, vz, group_size, bits)
            V[:, :, vi, :] = dense
    if r:
        K[:, :, L - r:, :] = cache[SLOT_NEW_K]
        V[:, :, L - r:, :] = cache[SLOT_NEW_V]
    return K, V
