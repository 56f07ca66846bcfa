"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations
(decode attention over a Llama-3.1-8B / Qwen3-8B shaped cache).  Real prompts and model weights are
not available offline; these stand in for them.  Used by bench.py, the smoke test and the GPU tests.
"""
import math
import torch

from .model.public_func import get_block_token_idx, make_sum_equal
from .quant.hqe_2 import KV_cache_hqe_2


from .configs import CONFIGS, CacheConfig, tier_counts  # noqa: F401  (re-exported: the workload definitions)


def make_kv(cfg: CacheConfig, device, seed: int, heads=None):
    """K, V [B, H, context, D] fp16 ~ N(0,1) (K with 4 outlier channels per head x10 if configured) and
    q [B, nh_q_local, 1, D].  ``heads`` = (first kv head, number of kv heads) restricts to a head shard;
    the values of a head do not depend on the shard it is generated in."""
    h0, nh = heads if heads is not None else (0, cfg.nh_kv)
    rep = cfg.nh_q // cfg.nh_kv
    K = torch.empty(cfg.batch, nh, cfg.context, cfg.head_dim, dtype=torch.float16, device=device)
    V = torch.empty_like(K)
    q = torch.empty(cfg.batch, nh * rep, 1, cfg.head_dim, dtype=torch.float16, device=device)
    for i in range(nh):
        gen = torch.Generator(device=device)
        gen.manual_seed(seed * 1000003 + (h0 + i))
        k = torch.randn(cfg.batch, cfg.context, cfg.head_dim, generator=gen, device=device)
        v = torch.randn(cfg.batch, cfg.context, cfg.head_dim, generator=gen, device=device)
        qq = torch.randn(cfg.batch, rep, 1, cfg.head_dim, generator=gen, device=device)
        if cfg.k_outliers:
            ch = torch.randperm(cfg.head_dim, generator=gen, device=device)[:4]
            k[:, :, ch] *= 10
        K[:, i], V[:, i] = k.half(), v.half()
        q[:, i * rep:(i + 1) * rep] = qq.half()
    return K, V, q


def synthetic_importance(cfg: CacheConfig, device, seed: int, length: int, K: torch.Tensor = None):
    """Token importance of ``length`` tokens as fp16.

    'random' (default): mean of 8 random softmax rows with the peakedness of real attention; it depends on the
    seed only, so every rank of a head-sharded run ranks identically.
    'qk' (the single-layer configuration): what the importance ring would hold after 8 decode steps with random
    queries - softmax(q.K^T / sqrt(d)) over the first ``length`` tokens of ``K`` [B, H, T, D], summed over batch
    and query heads per step and averaged over the 8 steps."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 7919 + 17)
    if cfg.importance == "qk":
        assert K is not None and K.shape[1] == cfg.nh_kv, "the q.K^T importance needs all kv heads of K"
        rep = cfg.nh_q // cfg.nh_kv
        q = torch.randn(8, cfg.batch, cfg.nh_kv, rep, cfg.head_dim, generator=gen, device=device).half().float()
        logits = torch.einsum("sbhrd,bhtd->sbhrt", q, K[:, :, :length].float()) / math.sqrt(cfg.head_dim)
        rows = torch.softmax(logits, dim=-1).sum(dim=(1, 2, 3))   # [8, length]: one head-summed row per step
        return rows.sum(0).div_(8).half()
    logits = torch.randn(8, length, generator=gen, device=device) * 2.0
    return torch.softmax(logits, dim=-1).sum(0).div_(8).half()


def build_cache(cfg: CacheConfig, device, seed: int = 0, heads=None, times_range: bool = False,
                quant_strategy: str = None):
    """Prefill-shaped K/V -> one flush through KV_cache_hqe_2 -> (cache tuple, q).  With
    ``times_range=False`` K and V are ranked identically, so every rank of a head-sharded run selects
    the same blocks without exchanging value ranges."""
    quant_strategy = quant_strategy or cfg.strategy
    K, V, q = make_kv(cfg, device, seed, heads)
    flushed = cfg.context - cfg.residual
    counts = tier_counts(cfg)
    imp = synthetic_importance(cfg, device, seed, flushed, K)
    ids = get_block_token_idx(cfg.group, flushed // cfg.group, imp)
    cache = (None,) * 39 + (K, V, cfg.context)
    bit_num = torch.tensor(counts, dtype=torch.int32)
    cache = KV_cache_hqe_2(cache, flushed, 0, ids, bit_num, bit_num.clone(), imp, quant_strategy, None, cfg.group,
                           cfg.group, times_range)
    return cache, q


def cache_bytes(cache, nh_q: int):
    """Algorithmic bytes one decode step reads from this cache: packed codes, scales, zeros and the
    fp16 payloads of K and V of every tier plus the residual window (index lists and the probability
    row are not counted)."""
    total = 0
    for i, item in enumerate(cache[:36]):
        if item is None or not torch.is_tensor(item):
            continue
        if item.dtype == torch.int64:      # index lists
            continue
        total += item.numel() * item.element_size()
    for i in (39, 40):
        if cache[i] is not None:
            total += cache[i].numel() * cache[i].element_size()
    return total


def logical_length(cache):
    n = sum(cache[s].numel() for s in (1, 5, 13, 21, 29) if cache[s] is not None)
    return n + (cache[39].shape[2] if cache[39] is not None else 0)
