"""CPU oracle for the hybrid mixed-precision KV-cache hot path (numpy).

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA kernels are
compared against; it is imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline legs of ``bench.py`` — never by the product package.

It restates, in numpy and with its own structure, the algorithm of the
reference project skywclouds/HqeKV for that path.  Every function cites the
reference file:line it follows.  Parity pin: the fixtures under
``tests/golden/*.npz`` were produced by executing the reference's own Python
modules (CPU, fp16, seeded) with ``tests/golden/make_golden.py``; the test
``tests/test_oracle_golden.py`` checks this module against every one of them
bit for bit.  The reference ships no golden vectors of its own.

Arithmetic convention (what "one torch op on fp16 tensors" means): operands are
widened to fp32, the operation is done in fp32 and the result is rounded to
nearest-even fp16.  Each helper below spells those roundings out explicitly.
"""
from __future__ import annotations

import math

import numpy as np

F16 = np.float16
F32 = np.float32

TIER_BITS = (16, 8, 4, 2, 1)          # slot order of the quantised tiers in the cache tuple
NUM_SLOTS = 42

# --- slot map of the 42-entry cache tuple (quant/hqe_matmul.py:364-368) -------------------
SLOT_K = {16: 0, 8: 4, 4: 12, 2: 20, 1: 28}      # K payload; +1 idx; (+2 scale, +3 zero) if bits<16
SLOT_V = {16: 2, 8: 8, 4: 16, 2: 24, 1: 32}      # V payload; +1 idx; (+2 scale, +3 zero) if bits<16
SLOT_V_TOKEN_NORM = 38
SLOT_NEW_K = 39
SLOT_NEW_V = 40
SLOT_SEQ_LEN = 41


def _h(x):
    """Round an fp32 array to fp16 (nearest even)."""
    return np.asarray(x, dtype=F32).astype(F16)


def _f(x):
    return np.asarray(x).astype(F32)


# ==========================================================================================
# codec: group quantise + bit-pack, unpack + dequantise
# ==========================================================================================

def pack_last_dim(codes: np.ndarray, bit: int) -> np.ndarray:
    """Pack integer codes along the last axis into int32 words.

    Element i of a word occupies bits [i*bit, (i+1)*bit) — quant/pack_unpack.py:42-51.
    """
    fpi = 32 // bit
    lead, T = codes.shape[:-1], codes.shape[-1]
    if T % fpi:
        raise ValueError("last dimension must be a multiple of 32/bit")
    c = (codes.astype(np.int64) & 0xFFFFFFFF).reshape(*lead, T // fpi, fpi)
    shifts = (np.arange(fpi, dtype=np.int64) * bit)
    words = np.bitwise_or.reduce((c << shifts) & 0xFFFFFFFF, axis=-1)
    return words.astype(np.uint32).view(np.int32)


def unpack_last_dim(words: np.ndarray, bit: int) -> np.ndarray:
    """Inverse of :func:`pack_last_dim`; returns fp16 integers like
    quant/pack_unpack.py:255-297 does."""
    fpi = 32 // bit
    w = words.view(np.uint32).astype(np.int64)
    shifts = (np.arange(fpi, dtype=np.int64) * bit)
    vals = (w[..., None] >> shifts) & ((1 << bit) - 1)
    return vals.reshape(*words.shape[:-1], words.shape[-1] * fpi).astype(F16)


def quantize_codes_last_dim(x: np.ndarray, group_size: int, bit: int):
    """Asymmetric uniform group quantisation along the last axis, fp16 arithmetic with a
    rounding after every step (quant/pack_unpack.py:166-175).

    Returns (codes int32 [..., T], scale f16 [..., T/g], mn f16 [..., T/g]).
    A constant group has scale 0, its quotient 0/0 is NaN and the NaN converts to code 0
    (what the float->int conversion does on the GPU the reference runs on).
    """
    x = np.asarray(x, dtype=F16)
    lead, T = x.shape[:-1], x.shape[-1]
    if T % group_size:
        raise ValueError("last dimension must be a multiple of the group size")
    levels = F32(2 ** bit - 1)
    xg = x.reshape(*lead, T // group_size, group_size)
    mn = xg.min(axis=-1, keepdims=True)
    mx = xg.max(axis=-1, keepdims=True)
    with np.errstate(all="ignore"):
        rng = _h(_f(mx) - _f(mn))                       # (mx - mn) is an fp16 tensor ...
        scale = _h(_f(rng) / levels)                    # ... before the divide (:169)
        t = _h(_f(xg) - _f(mn))                         # data.sub_(mn)          (:171)
        u = _h(_f(t) / _f(scale))                       # data.div_(scale)       (:173)
        u = np.clip(_f(u), F32(0), levels)              # clamp_ keeps NaN       (:175)
        r = np.rint(u)                                  # round_: half to even
        codes = np.where(np.isnan(r), F32(0), r).astype(np.int32)
    return codes.reshape(*lead, T), scale[..., 0], mn[..., 0]


def quantize_pack_last_dim(x: np.ndarray, group_size: int, bit: int):
    """uniform_group_quantize_pack_last_dim — quant/pack_unpack.py:156-193."""
    codes, scale, mn = quantize_codes_last_dim(x, group_size, bit)
    return pack_last_dim(codes, bit), scale, mn


def dequantize_unpack_last_dim(words, scale, mn, group_size: int, bit: int) -> np.ndarray:
    """uniform_group_dequantize_unpack_last_dim — quant/pack_unpack.py:316-333:
    x = half(half(code * scale) + mn), i.e. ``mul_`` then ``add_`` on an fp16 tensor."""
    codes = unpack_last_dim(words, bit)
    lead, T = codes.shape[:-1], codes.shape[-1]
    cg = codes.reshape(*lead, T // group_size, group_size)
    with np.errstate(all="ignore"):
        prod = _h(_f(cg) * _f(scale)[..., None])
        out = _h(_f(prod) + _f(mn)[..., None])
    return out.reshape(*lead, T)


# Gaussian-codebook codec at 1 bit: the low tier of quant_strategy 'high_uniform_group_low_normal_group'.
# Quantile centres norm.ppf(0.25), norm.ppf(0.75) as the reference holds them (float32, then cast to the
# fp16 of std); the decision bounds are [0, inf] (quant/pack_unpack.py:6-14).
NORMAL1_CENTER = np.array([-0.67448974, 0.67448974], dtype=F32)


def normal1_quantize_codes_last_dim(x: np.ndarray, group_size: int):
    """normal_group_quantize_pack_last_dim at bit = 1 before packing — quant/pack_unpack.py:218-253.

    std, mean = torch.std_mean (unbiased) of every group, returned in fp16.  torch's result on fp16
    input equals the exactly computed value rounded once to fp16, which is what float64 gives here.
    data.sub_(mean), data.div_(std) in fp16 with a rounding after each; code = searchsorted([0, inf], v):
    0 for v <= 0, 1 for v > 0.  NaN (a constant group: 0/0) is given code 0.
    Returns (codes int32 [..., T], std f16 [..., T/g], mean f16 [..., T/g])."""
    x = np.asarray(x, dtype=F16)
    lead, T = x.shape[:-1], x.shape[-1]
    if T % group_size:
        raise ValueError("last dimension must be a multiple of the group size")
    xg = x.reshape(*lead, T // group_size, group_size)
    x64 = xg.astype(np.float64)
    with np.errstate(all="ignore"):
        mean64 = x64.sum(axis=-1, keepdims=True) / group_size
        var64 = ((x64 - mean64) ** 2).sum(axis=-1, keepdims=True) / (group_size - 1)
        mean = mean64.astype(F16)
        std = np.sqrt(var64).astype(F16)
        t = _h(_f(xg) - _f(mean))
        v = _h(_f(t) / _f(std))
        codes = (_f(v) > 0).astype(np.int32)  # NaN > 0 is False
    return codes.reshape(*lead, T), std[..., 0], mean[..., 0]


def normal1_quantize_pack_last_dim(x: np.ndarray, group_size: int):
    codes, std, mean = normal1_quantize_codes_last_dim(x, group_size)
    return pack_last_dim(codes, 1), std, mean


def normal1_dequantize_unpack_last_dim(words, std, mean, group_size: int) -> np.ndarray:
    """normal_group_dequantize_unpack_last_dim at bit = 1 — quant/pack_unpack.py:356-376:
    x = half(half(center[code] * std) + mean) with center cast to fp16 first."""
    codes = unpack_last_dim(words, 1).astype(np.int64)
    lead, T = codes.shape[:-1], codes.shape[-1]
    cg = NORMAL1_CENTER.astype(F16)[codes].reshape(*lead, T // group_size, group_size)
    with np.errstate(all="ignore"):
        prod = _h(_f(cg) * _f(std)[..., None])
        out = _h(_f(prod) + _f(mean)[..., None])
    return out.reshape(*lead, T)


# ==========================================================================================
# importance bookkeeping, token range, block ranking
# ==========================================================================================

def _sum_f16_sequential(rows: np.ndarray) -> np.ndarray:
    """Sum fp16 rows over axis 0 with one fp32 accumulator per column, adding the rows in
    index order, and round the total to fp16 once (how a torch fp16 ``sum`` over an outer
    axis accumulates on the CPU)."""
    acc = np.zeros(rows.shape[1:], dtype=F32)
    for r in rows:
        acc = (acc + _f(r)).astype(F32)
    return acc.astype(F16)


def head_sum_probabilities(attn_weights: np.ndarray) -> np.ndarray:
    """Row that the importance ring stores for one decode step: probabilities summed over the
    batch, then over the heads, each sum rounded to fp16 (model/public_func.py:254
    ``attn_weights.sum(0).sum(0)`` with q_len == 1).  Input [B, nh_q, 1, L] fp16."""
    per_head = _sum_f16_sequential(np.asarray(attn_weights, dtype=F16))       # [nh, 1, L]
    return _sum_f16_sequential(per_head)                                      # [1, L]


class ImportanceRing:
    """Rolling buffer of the last ``last_length`` head-summed probability rows
    (class last_attn_weights, model/public_func.py:208-257)."""

    def __init__(self, last_length: int = 20):
        self.last_length = last_length
        self.max_length = 0
        self.kv_seq_len = 0
        self.next_line = 0
        self.weights = None

    def set_max_length(self, max_length: int):
        self.max_length = max_length

    def update(self, attn_weights: np.ndarray):
        attn_weights = np.asarray(attn_weights, dtype=F16)
        if self.weights is None:
            self.weights = np.zeros((self.last_length, self.max_length), dtype=F16)
        q_len = attn_weights.shape[2]
        if q_len > 1:                                           # prefill seeding (:247-252)
            tail = attn_weights if q_len < self.last_length else attn_weights[:, :, -self.last_length:, :]
            rows = _sum_f16_sequential(_sum_f16_sequential(tail))
            self.weights[:rows.shape[0], :rows.shape[1]] = rows
        else:                                                   # one decode step (:253-255)
            rows = head_sum_probabilities(attn_weights)
            self.weights[self.next_line:self.next_line + 1, :rows.shape[1]] = rows
        self.kv_seq_len = rows.shape[1]
        self.next_line = (self.next_line + rows.shape[0]) % self.last_length

    def calculate_token_importance(self) -> np.ndarray:
        """importance = column sum / min(last_length, age) in fp16 (:217-221)."""
        L = self.kv_seq_len
        count = np.arange(L, 0, -1).astype(F16)
        if L > self.last_length:
            count[:-self.last_length] = F16(self.last_length)
        col = _sum_f16_sequential(self.weights[:, :L])
        with np.errstate(all="ignore"):
            return _h(_f(col) / _f(count))

    def eviction(self, reserve_idx: np.ndarray):
        """Compact the columns of the surviving tokens to the front (:228-231)."""
        if self.weights is not None:
            kept = self.weights[:, reserve_idx].copy()
            self.weights[:, :kept.shape[1]] = kept


def token_range(new_V: np.ndarray) -> np.ndarray:
    """Per token: (max_d V - min_d V) in fp16, summed over batch then heads with an fp16
    rounding after each sum (calculate_token_range, model/public_func.py:58-73)."""
    v = np.asarray(new_V, dtype=F16)
    rng = _h(_f(v.max(axis=-1)) - _f(v.min(axis=-1)))       # [B, H, T]
    return _sum_f16_sequential(_sum_f16_sequential(rng))    # [T]


def block_rank(block_size: int, block_num: int, importance: np.ndarray) -> np.ndarray:
    """get_block_token_idx — model/public_func.py:92-106.

    ``importance`` (fp16, length block_num*block_size) is divided IN PLACE by the block
    length, like the reference does to its argument; block key = fp16 sum of the divided
    values; blocks are ordered by descending key, equal keys by ascending block id (the
    reference's sort leaves ties unspecified; this is the order its CPU sort produces).
    Returns the expanded int64 token ids.
    """
    if importance.dtype != F16 or importance.shape != (block_num * block_size,):
        raise ValueError("importance must be fp16 of length block_num*block_size")
    with np.errstate(all="ignore"):
        importance[...] = _h(_f(importance) / F32(block_size))
    keys = _sum_f16_sequential(importance.reshape(block_num, block_size).T)
    order = np.argsort(-_f(keys), kind="stable")
    return (order[:, None].astype(np.int64) * block_size + np.arange(block_size, dtype=np.int64)).reshape(-1)


def make_sum_equal(array: np.ndarray, array_sum: int, start_idx: int = 4) -> np.ndarray:
    """Take the rounding surplus off the lowest tiers first (model/public_func.py:259-268)."""
    sub = int(array.sum()) - int(array_sum)
    for i in range(start_idx, -1, -1):
        if array[i] - sub < 0:
            sub -= int(array[i])
            array[i] = 0
        else:
            array[i] -= sub
            break
    return array


# ==========================================================================================
# flush: evict + tier-assign + re-quantise (KV_cache_hqe_2, quant/hqe_2.py:456-843)
# ==========================================================================================

def _targets(sorted_idx: np.ndarray, bit_num: np.ndarray, total: int) -> np.ndarray:
    """Target of every logical token from the ranked ids and the six counts
    (quant/hqe_2.py:521-538): 0..4 = 16/8/4/2/1-bit tier, 5 = evict, -1 = none."""
    c = np.cumsum(np.asarray(bit_num, dtype=np.int64))
    tgt = np.full(total, -1, dtype=np.int64)
    lo = 0
    for t in range(6):
        hi = int(c[t])
        if hi > lo:
            tgt[sorted_idx[lo:hi]] = t
        lo = max(lo, hi)
    return tgt


def _plan(tier_idx: list, history_length: int, compress_length: int, tgt: np.ndarray):
    """Where every cached token ends up.

    ``tier_idx[t]`` is the id list of tier t (storage order) or None.  A token moves only to
    a tier of strictly fewer bits than it has now (the ladder quant/hqe_2.py:584-659 and
    :737-825 visits destinations 1,2,4,8,16-bit in that order and only looks at sources of
    more bits); new tokens always take their target.  Within a destination the order is:
    what it already held and keeps, then arrivals from the residual (ascending id), then
    from the 16-, 8-, 4-, 2-bit tiers, each in its storage order.

    Returns (dest, evict_any) where dest[t] is a list of (source, positions) pairs with
    source in {-1 (residual), 0..4} and positions indexing that source's storage.
    """
    new_ids = np.arange(history_length, history_length + compress_length, dtype=np.int64)
    sources = [(-1, new_ids)] + [(t, tier_idx[t]) for t in range(5) if tier_idx[t] is not None]
    dest = [[] for _ in range(5)]
    for t in range(5):
        # kept members first
        if tier_idx[t] is not None:
            tg = tgt[tier_idx[t]]
            keep = np.nonzero((tg != 5) & ~((tg > t) & (tg <= 4)))[0]
            if keep.size:
                dest[t].append((t, keep))
        for src, ids in sources:
            if src >= t:                    # only sources of more bits (residual = -1 counts)
                continue
            tg = tgt[ids]
            mv = np.nonzero(tg == t)[0]
            if mv.size:
                dest[t].append((src, mv))
    return dest, bool((tgt == 5).any())


def _ids_of(dest_t, tier_idx, new_ids):
    parts = [(new_ids if s < 0 else tier_idx[s])[pos] for s, pos in dest_t]
    return np.concatenate(parts) if parts else None


def _rerank(id_lists):
    """Replace ids by their rank among all survivors (quant/hqe_2.py:661-671)."""
    present = [x for x in id_lists if x is not None]
    allv = np.sort(np.concatenate(present))
    return [None if x is None else np.searchsorted(allv, x).astype(np.int64) for x in id_lists]


STRATEGIES = ("uniform_group", "high_uniform_group_low_normal_group")


def _low_is_normal(quant_strategy: str) -> bool:
    """Under 'high_uniform_group_low_normal_group' the 1-bit tier alone uses the Gaussian-codebook
    codec (quant/hqe_2.py:488-492: the *_low functions are only ever handed to the 1-bit tier, :588-608,
    :741-762); every other tier and every source of a demotion is uniform."""
    if quant_strategy not in STRATEGIES:
        raise ValueError("invalid quant_strategy")
    return quant_strategy == "high_uniform_group_low_normal_group"


def _requant(values_last_dim: np.ndarray, group: int, bit: int, normal_low: bool = False):
    if bit == 1 and normal_low:
        return normal1_quantize_pack_last_dim(values_last_dim, group)
    return quantize_pack_last_dim(values_last_dim, group, bit)


def flush(cache: tuple, compress_length: int, history_length: int, K_sorted_idx, K_bit_num, V_bit_num,
          token_importance: np.ndarray, quant_strategy: str, ring: ImportanceRing | None = None,
          block_size: int = 32, group_size: int = 32, times_range: bool = True) -> tuple:
    """KV_cache_hqe_2 (quant/hqe_2.py:456-843) for ``quant_strategy`` 'uniform_group' and
    'high_uniform_group_low_normal_group' (1-bit destination tier in the Gaussian-codebook codec).

    K is quantised in groups of ``block_size`` tokens per channel, V in groups of
    ``group_size`` channels per token.  ``token_importance`` is the array the caller already
    passed through :func:`block_rank` for K (so it holds importance/block_size); it is
    divided a second time, in place, when V is ranked — as in the reference.
    """
    normal_low = _low_is_normal(quant_strategy)
    cache = list(cache)
    new_K, new_V = cache[SLOT_NEW_K], cache[SLOT_NEW_V]
    res_K = new_K[:, :, compress_length:, :].copy()
    res_V = new_V[:, :, compress_length:, :].copy()
    res_K = None if res_K.size == 0 else res_K
    res_V = None if res_V.size == 0 else res_V
    new_K = new_K[:, :, :compress_length, :]
    new_V = new_V[:, :, :compress_length, :]
    total = history_length + compress_length
    block_num = total // block_size
    new_ids = np.arange(history_length, total, dtype=np.int64)

    # ---- V ranking keys (:513-518)
    rng_new = token_range(new_V)
    norm = rng_new if cache[SLOT_V_TOKEN_NORM] is None else np.concatenate((cache[SLOT_V_TOKEN_NORM], rng_new))
    if times_range:
        with np.errstate(all="ignore"):
            v_keys = _h(_f(token_importance) * _f(norm))
    else:
        v_keys = token_importance.copy()
    V_sorted_idx = block_rank(block_size, block_num, v_keys)

    # ---- K side ---------------------------------------------------------------------------
    K_idx = [cache[SLOT_K[b] + 1] for b in TIER_BITS]
    tgtK = _targets(np.asarray(K_sorted_idx, dtype=np.int64), K_bit_num, total)
    destK, evictK = _plan(K_idx, history_length, compress_length, tgtK)
    outK = []
    for t, bits in enumerate(TIER_BITS):
        payload, sc, zp = [], [], []
        for src, pos in destK[t]:
            if src == t:                                  # kept: copy codes/scales of whole blocks
                tier = cache[SLOT_K[bits]]
                if bits == 16:
                    payload.append(tier[..., pos])
                else:
                    fpi = 32 // bits
                    blk = pos.reshape(-1, block_size)[:, 0] // block_size
                    wcols = (blk[:, None] * (block_size // fpi) + np.arange(block_size // fpi)).reshape(-1)
                    payload.append(tier[..., wcols])
                    sc.append(cache[SLOT_K[bits] + 2][..., blk])
                    zp.append(cache[SLOT_K[bits] + 3][..., blk])
                continue
            # arrivals: bring to fp16 channel-major [B,H,D,n]
            if src < 0:
                dense = np.swapaxes(new_K[:, :, pos, :], 2, 3)
            elif TIER_BITS[src] == 16:
                dense = cache[SLOT_K[16]][..., pos]
            else:
                sb = TIER_BITS[src]
                fpi = 32 // sb
                blk = pos.reshape(-1, block_size)[:, 0] // block_size
                wcols = (blk[:, None] * (block_size // fpi) + np.arange(block_size // fpi)).reshape(-1)
                dense = dequantize_unpack_last_dim(cache[SLOT_K[sb]][..., wcols], cache[SLOT_K[sb] + 2][..., blk],
                                                   cache[SLOT_K[sb] + 3][..., blk], block_size, sb)
            if bits == 16:
                payload.append(np.ascontiguousarray(dense))
            else:
                w, s, z = _requant(dense, block_size, bits, normal_low)
                payload.append(w); sc.append(s); zp.append(z)
        ids = _ids_of(destK[t], K_idx, new_ids)
        outK.append((np.concatenate(payload, axis=3) if payload else None, ids,
                     np.concatenate(sc, axis=3) if sc else None, np.concatenate(zp, axis=3) if zp else None))
    if evictK:
        ranked = _rerank([o[1] for o in outK])
        outK = [(o[0], r, o[2], o[3]) for o, r in zip(outK, ranked)]

    # ---- V side ---------------------------------------------------------------------------
    V_idx = [cache[SLOT_V[b] + 1] for b in TIER_BITS]
    tgtV = _targets(V_sorted_idx, V_bit_num, total)
    destV, evictV = _plan(V_idx, history_length, compress_length, tgtV)
    # survivors compact the range vector and the ring (:727-735)
    survivors = np.nonzero(tgtV != 5)[0]
    norm = norm[survivors]
    if ring is not None:
        ring.eviction(survivors)
    outV = []
    for t, bits in enumerate(TIER_BITS):
        payload, sc, zp = [], [], []
        for src, pos in destV[t]:
            if src == t:
                payload.append(cache[SLOT_V[bits]][:, :, pos, :])
                if bits < 16:
                    sc.append(cache[SLOT_V[bits] + 2][:, :, pos, :])
                    zp.append(cache[SLOT_V[bits] + 3][:, :, pos, :])
                continue
            if src < 0:
                dense = new_V[:, :, pos, :]
            elif TIER_BITS[src] == 16:
                dense = cache[SLOT_V[16]][:, :, pos, :]
            else:
                sb = TIER_BITS[src]
                dense = dequantize_unpack_last_dim(cache[SLOT_V[sb]][:, :, pos, :], cache[SLOT_V[sb] + 2][:, :, pos, :],
                                                   cache[SLOT_V[sb] + 3][:, :, pos, :], group_size, sb)
            if bits == 16:
                payload.append(np.ascontiguousarray(dense))
            else:
                w, s, z = _requant(dense, group_size, bits, normal_low)
                payload.append(w); sc.append(s); zp.append(z)
        ids = _ids_of(destV[t], V_idx, new_ids)
        outV.append((np.concatenate(payload, axis=2) if payload else None, ids,
                     np.concatenate(sc, axis=2) if sc else None, np.concatenate(zp, axis=2) if zp else None))
    if evictV:
        ranked = _rerank([o[1] for o in outV])
        outV = [(o[0], r, o[2], o[3]) for o, r in zip(outV, ranked)]

    out = [None] * NUM_SLOTS
    for t, bits in enumerate(TIER_BITS):
        k, v = SLOT_K[bits], SLOT_V[bits]
        out[k], out[k + 1] = outK[t][0], outK[t][1]
        out[v], out[v + 1] = outV[t][0], outV[t][1]
        if bits < 16:
            out[k + 2], out[k + 3] = outK[t][2], outK[t][3]
            out[v + 2], out[v + 3] = outV[t][2], outV[t][3]
    out[SLOT_V_TOKEN_NORM] = norm
    out[SLOT_NEW_K], out[SLOT_NEW_V] = res_K, res_V
    out[SLOT_SEQ_LEN] = cache[SLOT_SEQ_LEN]
    return tuple(out)


# ==========================================================================================
# dense reconstruction and fp32 decode attention
# ==========================================================================================

def cache_dims(cache: tuple):
    """(B, nh_kv, head_dim, n_quantised_tokens, residual_len) from the V payloads
    (quant/hqe_matmul.py:379-404)."""
    B = H = D = None
    n = 0
    for bits in TIER_BITS:
        v = cache[SLOT_V[bits]]
        if v is not None:
            B, H = v.shape[0], v.shape[1]
            n += v.shape[2]
            D = v.shape[3] * (1 if bits == 16 else 32 // bits)
    r = 0
    if cache[SLOT_NEW_V] is not None:
        B, H, r, D = cache[SLOT_NEW_V].shape
    if n + r == 0:
        raise ValueError("invalid past_key_value")
    return B, H, D, n, r


def reconstruct(cache: tuple, block_size: int = 32, group_size: int = 32, quant_strategy: str = "uniform_group"):
    """Dense fp16 K and V [B,H,L,D] at logical positions (KV_cache_reconstruct_hqe,
    quant/hqe_2.py:967-1084), every tier dequantised with the two-rounding recipe."""
    normal_low = _low_is_normal(quant_strategy)

    def tier_dense(words, a, b, group, bits):
        if bits == 1 and normal_low:
            return normal1_dequantize_unpack_last_dim(words, a, b, group)
        return dequantize_unpack_last_dim(words, a, b, group, bits)

    B, H, D, n, r = cache_dims(cache)
    L = n + r
    K = np.zeros((B, H, L, D), dtype=F16)
    V = np.zeros((B, H, L, D), dtype=F16)
    for bits in TIER_BITS:
        k, v = SLOT_K[bits], SLOT_V[bits]
        if cache[k] is not None:
            dense = cache[k] if bits == 16 else tier_dense(cache[k], cache[k + 2], cache[k + 3], block_size, bits)
            K[:, :, cache[k + 1], :] = np.swapaxes(dense, 2, 3)
        if cache[v] is not None:
            dense = cache[v] if bits == 16 else tier_dense(cache[v], cache[v + 2], cache[v + 3], group_size, bits)
            V[:, :, cache[v + 1], :] = dense
    if r:
        K[:, :, L - r:, :] = cache[SLOT_NEW_K]
        V[:, :, L - r:, :] = cache[SLOT_NEW_V]
    return K, V


def reconstruct_fp32(cache: tuple, block_size: int = 32, group_size: int = 32,
                     quant_strategy: str = "uniform_group"):
    """Dense fp32 K and V with the dequantisation the reference's GEMV kernels do in registers:
    w = scale * code + zero evaluated in fp32 from the fp16 scale and zero, no fp16 rounding
    (quant/csrc/gemv_cuda_uniform.cu:465-467); for the Gaussian-codebook 1-bit tier
    w = std * center[code] + mean with the float32 centres (quant/csrc/gemv_cuda_normal.cu:104-106)."""
    normal_low = _low_is_normal(quant_strategy)
    B, H, D, n, r = cache_dims(cache)
    L = n + r
    K = np.zeros((B, H, L, D), dtype=F32)
    V = np.zeros((B, H, L, D), dtype=F32)

    def deq(words, scale, zero, group, bits):
        codes = unpack_last_dim(words, bits)
        codes = NORMAL1_CENTER[codes.astype(np.int64)] if (bits == 1 and normal_low) else _f(codes)
        lead, T = codes.shape[:-1], codes.shape[-1]
        cg = codes.reshape(*lead, T // group, group)
        return (cg * _f(scale)[..., None] + _f(zero)[..., None]).astype(F32).reshape(*lead, T)

    for bits in TIER_BITS:
        k, v = SLOT_K[bits], SLOT_V[bits]
        if cache[k] is not None:
            dense = _f(cache[k]) if bits == 16 else deq(cache[k], cache[k + 2], cache[k + 3], block_size, bits)
            K[:, :, cache[k + 1], :] = np.swapaxes(dense, 2, 3)
        if cache[v] is not None:
            dense = _f(cache[v]) if bits == 16 else deq(cache[v], cache[v + 2], cache[v + 3], group_size, bits)
            V[:, :, cache[v + 1], :] = dense
    if r:
        K[:, :, L - r:, :] = _f(cache[SLOT_NEW_K])
        V[:, :, L - r:, :] = _f(cache[SLOT_NEW_V])
    return K, V


def decode_attention(q: np.ndarray, cache: tuple, head_dim: int | None = None, block_size: int = 32,
                     group_size: int = 32, dequant: str = "fp32", quant_strategy: str = "uniform_group"):
    """fp32-accumulated dequant-matmul decode attention: softmax(q K^T / sqrt(d)) V, everything in
    fp32.  This is the quantity qkv_matmul_hqe_2 (quant/hqe_matmul.py:354-451) approximates with
    fp16 intermediates.  ``dequant='fp32'`` dequantises as the reference's CUDA kernels do
    (:func:`reconstruct_fp32`); ``'fp16'`` uses the dense fp16 reconstruction of
    KV_cache_reconstruct_hqe (:func:`reconstruct`).  q [B, nh_q, 1, D] fp16.
    Returns (weights fp32 [B,nh_q,1,L], out fp32 [B,nh_q,1,D])."""
    K, V = (reconstruct_fp32 if dequant == "fp32" else reconstruct)(cache, block_size, group_size, quant_strategy)
    B, H, L, D = K.shape
    nh_q = q.shape[1]
    rep = nh_q // H
    qf = _f(q).reshape(B, H, rep, D)
    logits = np.matmul(qf, np.swapaxes(_f(K), 2, 3)) / F32(math.sqrt(head_dim or D))     # [B,H,rep,L]
    logits = logits - logits.max(axis=-1, keepdims=True)
    p = np.exp(logits, dtype=F32)
    p = p / p.sum(axis=-1, keepdims=True, dtype=F32)
    out = np.matmul(p, _f(V))
    return p.reshape(B, nh_q, 1, L), out.reshape(B, nh_q, 1, D)


def decode_attention_fp16_flow(q: np.ndarray, cache: tuple, block_size: int = 32, group_size: int = 32,
                               quant_strategy: str = "uniform_group"):
    """qkv_matmul_hqe_2 with the reference's fp16 intermediates (quant/hqe_matmul.py:405-451): every tier's
    q.K^T is an fp32-accumulated GEMV rounded to fp16 and scattered into an fp16 row, the row is divided by
    sqrt(head_dim) in fp16, softmax runs in fp32 and is rounded to fp16, and the tiers' p.V products (each
    rounded to fp16) are added into an fp16 output one after the other in tier order 16, 8, 4, 2, 1, residual.
    Returns (weights f16 [B,nh_q,1,L], out f16 [B,nh_q,1,D]).  Used to pin the oracle against decode outputs
    produced by the reference's own function; the parity target of the CUDA path is :func:`decode_attention`."""
    normal_low = _low_is_normal(quant_strategy)
    B, H, D, n, r = cache_dims(cache)
    L = n + r
    nh_q = q.shape[1]
    rep = nh_q // H
    qf = _f(q).reshape(B, H, rep, D)

    def dense32(words, a, b, group, bits):
        codes = unpack_last_dim(words, bits)
        cg = NORMAL1_CENTER[codes.astype(np.int64)] if (bits == 1 and normal_low) else _f(codes)
        lead, T = cg.shape[:-1], cg.shape[-1]
        cg = cg.reshape(*lead, T // group, group)
        return (cg * _f(a)[..., None] + _f(b)[..., None]).astype(F32).reshape(*lead, T)

    logits = np.zeros((B, H, rep, L), dtype=F16)
    for bits in TIER_BITS:
        k = SLOT_K[bits]
        if cache[k] is None:
            continue
        Kd = _f(cache[k]) if bits == 16 else dense32(cache[k], cache[k + 2], cache[k + 3], block_size, bits)  # [B,H,D,n]
        logits[..., cache[k + 1]] = _h(np.matmul(qf, Kd))
    if r:
        logits[..., L - r:] = _h(np.matmul(qf, np.swapaxes(_f(cache[SLOT_NEW_K]), 2, 3)))
    with np.errstate(all="ignore"):
        logits = _h(_f(logits) / F32(D ** 0.5))
    x = _f(logits)
    x = x - x.max(axis=-1, keepdims=True)
    e = np.exp(x, dtype=F32)
    p = _h(e / e.sum(axis=-1, keepdims=True, dtype=F32))
    out = np.zeros((B, H, rep, D), dtype=F16)
    for bits in TIER_BITS:
        v = SLOT_V[bits]
        if cache[v] is None:
            continue
        Vd = _f(cache[v]) if bits == 16 else dense32(cache[v], cache[v + 2], cache[v + 3], group_size, bits)  # [B,H,n,D]
        out = _h(_f(out) + _f(_h(np.matmul(_f(p[..., cache[v + 1]]), Vd))))
    if r:
        out = _h(_f(out) + _f(_h(np.matmul(_f(p[..., L - r:]), _f(cache[SLOT_NEW_V])))))
    return p.reshape(B, nh_q, 1, L), out.reshape(B, nh_q, 1, D)


def gemv_dequant(fA: np.ndarray, qB: np.ndarray, scales: np.ndarray, zeros: np.ndarray, group_size: int,
                 bits: int) -> np.ndarray:
    """C = fA x dequant(qB) with fp32 accumulation — what cuda_bmm_fA_qB_uniform_group
    (quant/matmul.py:263-299) computes through bgemv_kernel_uniform_group_*
    (quant/csrc/gemv_cuda_uniform.cu:455-489: w = scale*code + zero in fp32).
    fA [B,nh_q,M,K] f16; qB [B,nh_kv,K,N/fpi] i32; scales/zeros [B,nh_kv,K,N/g] f16.
    Returns fp32 [B,nh_q,M,N]."""
    codes = _f(unpack_last_dim(qB, bits))
    B, H, Kd, N = codes.shape
    w = codes.reshape(B, H, Kd, N // group_size, group_size) * _f(scales)[..., None] + _f(zeros)[..., None]
    w = w.reshape(B, H, Kd, N)
    nh_q, M = fA.shape[1], fA.shape[2]
    a = _f(fA).reshape(B, H, (nh_q // H) * M, Kd)
    return np.matmul(a, w).reshape(B, nh_q, M, N)


def gemv_dequant_normal1(fA: np.ndarray, qB: np.ndarray, stds: np.ndarray, means: np.ndarray,
                         group_size: int) -> np.ndarray:
    """C = fA x dequant(qB) over a Gaussian-codebook 1-bit tier with fp32 accumulation — what
    cuda_bmm_fA_qB_normal_group (quant/matmul.py:72-95) computes through the kernels of
    quant/csrc/gemv_cuda_normal.cu (:104-106: w = std * center[code] + mean in fp32, float32 centres).
    Shapes as in :func:`gemv_dequant`."""
    c = NORMAL1_CENTER[unpack_last_dim(qB, 1).astype(np.int64)]
    B, H, Kd, N = c.shape
    w = c.reshape(B, H, Kd, N // group_size, group_size) * _f(stds)[..., None] + _f(means)[..., None]
    w = w.reshape(B, H, Kd, N).astype(F32)
    nh_q, M = fA.shape[1], fA.shape[2]
    a = _f(fA).reshape(B, H, (nh_q // H) * M, Kd)
    return np.matmul(a, w).reshape(B, nh_q, M, N)
