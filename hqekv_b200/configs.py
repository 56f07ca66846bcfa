"""Benchmark configurations of the decode path: shapes, tier shares and the six token counts of the flush that
builds each cache.  Pure Python (no CUDA library is loaded): both arms of bench.py and the tests read the same
definitions from here.
"""
from dataclasses import dataclass


def make_sum_equal_list(array, array_sum: int, start_idx: int = 4):
    """Take the rounding surplus off the lowest tiers first - make_sum_equal of the reference's
    model/public_func.py:259-268 on a plain list of ints."""
    array = list(array)
    sub = sum(array) - array_sum
    for i in range(start_idx, -1, -1):
        if array[i] - sub < 0:
            sub -= array[i]
            array[i] = 0
        else:
            array[i] -= sub
            break
    return array


@dataclass
class CacheConfig:
    name: str
    batch: int
    nh_q: int
    nh_kv: int
    head_dim: int
    context: int          # tokens seen before the decode step
    residual: int         # fp16 residual window kept after the flush
    ratios: tuple         # share of the SURVIVING quantised tokens in the 8-, 4-, 2-bit tiers
    evict: float          # share of the flushed tokens that is evicted
    group: int            # K block / group size and V group size
    k_outliers: bool      # 4 random K channels per head scaled x10
    layers: int = 1
    fp16_tokens: int = 0  # tokens kept in the 16-bit tier (the reference's models keep 64)
    strategy: str = "uniform_group"   # or 'high_uniform_group_low_normal_group' (1-bit tier = Gaussian codebook)
    importance: str = "random"        # 'random': softmax of random logits; 'qk': softmax(q.K^T) of 8 random queries over the cache's own K


CONFIGS = {
    # single layer, CPU-checkable
    "cfg0": CacheConfig("cfg0-llama-1layer-4k", 1, 32, 8, 128, 4096, 128, (0.25, 0.50, 0.25), 0.10, 32, True, 1,
                        importance="qk"),
    # Llama-3.1-8B decode at 32k context (the configuration the headline metric is quoted on)
    "cfg1": CacheConfig("cfg1-llama3.1-8b-32k", 1, 32, 8, 128, 32768, 128, (0.20, 0.40, 0.40), 0.10, 32, False, 32),
    # Qwen3-8B, batch 8, 16k, group 64, no eviction
    "cfg2": CacheConfig("cfg2-qwen3-8b-b8-16k", 8, 32, 8, 128, 16384, 128, (0.25, 0.50, 0.25), 0.0, 64, True, 36),
    # long-context sizing, heads sharded over 8 GPUs
    "cfg3": CacheConfig("cfg3-llama3.1-8b-b4-128k", 4, 32, 8, 128, 131072, 256, (0.10, 0.25, 0.65), 0.30, 32, False, 32),
    # the setting the reference's own model files run (pred_long_bench_hq.py:135-141): 64 fp16 tokens, no 8-bit
    # tier, equal 4 / 2 / 1-bit shares with the 1-bit tier in the Gaussian codebook, a quarter evicted
    "cfgm": CacheConfig("cfgm-llama3.1-8b-32k-model-shares", 1, 32, 8, 128, 32768, 128, (0.0, 1 / 3, 1 / 3, 1 / 3), 0.25,
                        32, False, 32, 64, "high_uniform_group_low_normal_group"),
}


def tier_counts(cfg: CacheConfig):
    """Six token counts (16, 8, 4, 2, 1 bit, evicted), multiples of the block size, for one flush of
    everything but the residual window.  Eviction takes round(evict * blocks) blocks; the survivors
    split by ``ratios`` with the rounding surplus taken off the lowest tier first."""
    block = cfg.group
    flushed = cfg.context - cfg.residual
    assert flushed % block == 0, "context - residual must be a multiple of the block size"
    nblocks = flushed // block
    ev = int(round(nblocks * cfg.evict))
    f16 = min(cfg.fp16_tokens // block, nblocks - ev)
    keep = nblocks - ev - f16
    one = round(keep * cfg.ratios[3]) if len(cfg.ratios) > 3 else 0  # optional uniform 1-bit share
    raw = [0, round(keep * cfg.ratios[0]), round(keep * cfg.ratios[1]), round(keep * cfg.ratios[2]), one]
    raw = make_sum_equal_list(raw, keep, start_idx=4 if one else 3)
    counts = [int(v) * block for v in raw] + [ev * block]
    counts[0] = f16 * block
    assert sum(counts) == flushed
    return counts
