"""End-to-end decode throughput of a decoder stack on the tiered cache (random-init weights, synthetic input).

    python -m hqekv_b200.model.bench_model --model llama31-8b --ctx 32768 --steps 64

Prefills ``ctx`` synthetic hidden-state rows through every layer (dense causal attention, ring seeding, first
flush), then decodes ``steps`` tokens one at a time, each step feeding the previous step's output row back in;
every 32nd step every layer flushes its residual window.  The dense parts of a decode step (norms, projections,
rotary, MLP) are replayed from CUDA graphs unless ``--no-graphs``; the cache-facing calls are issued eagerly.  Prints one JSON line: decode tokens/s over all steps
(flush steps included), the same without the flush steps, prefill seconds, and the cache footprint against an
fp16 cache.  Timed with CUDA events on the current stream; weights are random (no checkpoint is read), so the
numbers measure the runtime, not a model's quality.
"""
import argparse
import json
import os
import time

import torch

from .decoder import LLAMA31_8B, QWEN3_8B, DecoderConfig, GraphedDecodeStep, HqeDecoder, init_like_pretrained

MODELS = {"llama31-8b": LLAMA31_8B, "qwen3-8b": QWEN3_8B}
# tier mixes handed to the layers from outside instead of the model files' own shares:
# name -> (shares of the surviving tokens in the 8 / 4 / 2-bit tiers, share of the newly flushed tokens evicted)
TIER_MIXES = {"cfg1": ((0.20, 0.40, 0.40), 0.10), "cfg2": ((0.25, 0.50, 0.25), 0.0)}


def external_counts(schedule, mix):
    """(shares, K counts, V counts) for the flush that is due: the cached + new tokens split by ``mix`` into the
    8 / 4 / 2-bit tiers after evicting a share of the NEW blocks (tokens only ever move down, so asking for the
    same shares of a growing total keeps the tiers at those shares)."""
    from .attention_hqe import BLOCK
    from .public_func import make_sum_equal
    ratios, evict = TIER_MIXES[mix]
    compress, total, blocks = schedule.lengths()
    ev = int(round(evict * (compress // BLOCK)))
    keep = blocks - ev
    raw = torch.tensor([0] + [round(keep * r) for r in ratios] + [0], dtype=torch.int32, device="cpu")
    raw = make_sum_equal(raw, keep, start_idx=3)
    counts = torch.cat((raw, torch.tensor([ev], dtype=torch.int32))) * BLOCK
    shares = counts.float() / total
    return shares, counts, counts.clone()


def cache_nbytes(caches):
    total = 0
    for c in caches:
        for t in c[:41]:
            if torch.is_tensor(t):
                total += t.numel() * t.element_size()
    return total


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=sorted(MODELS), default="llama31-8b")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the model's)")
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--strategy", default="high_uniform_group_low_normal_group")
    ap.add_argument("--no-graphs", action="store_true", help="issue the dense parts of a decode step eagerly")
    ap.add_argument("--tiers", choices=["model"] + sorted(TIER_MIXES), default="model",
                    help="model: the shares the reference's model files derive (64 fp16 tokens, 4/2/1-bit, eviction); "
                         "cfg1 / cfg2: 8/4/2-bit mixes of the benchmark configurations, handed in as auxiliary parameters")
    args = ap.parse_args(argv)
    # every flush re-allocates every tier a little larger than before: segments that can grow keep the caching
    # allocator from fragmenting into driver allocations (read when the allocator first runs)
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    if not torch.cuda.is_available():
        raise SystemExit("bench_model needs a GPU")
    dev = torch.device("cuda", torch.cuda.current_device())
    base = MODELS[args.model]
    cfg = DecoderConfig(**{**base.__dict__, "quant_strategy": args.strategy,
                           "num_layers": args.layers or base.num_layers})
    torch.set_default_dtype(torch.float16)
    try:
        with torch.device(dev):
            model = HqeDecoder(cfg)
    finally:
        torch.set_default_dtype(torch.float32)
    init_like_pretrained(model, 0)
    model.eval()
    gen = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(args.batch, args.ctx, cfg.hidden_size, generator=gen, device=dev, dtype=torch.float16)
    total_steps = args.warmup + args.steps
    model.start_sequence(args.ctx + total_steps + 1)
    with torch.no_grad():
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        sched = model.layers[0].self_attn.schedule

        def aux_for(n_new):
            """Counts for the flush this call will trigger (None: none is due, or the layers derive their own)."""
            if args.tiers == "model" or sched.current_length + n_new < 32:
                return None
            sched.append(n_new)
            try:
                return external_counts(sched, args.tiers)
            finally:
                sched.append(-n_new)

        h, caches = model(x, None, 0, aux_for(args.ctx))
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        del x
        row = h[:, -1:, :].contiguous()
        del h
        pos = args.ctx
        step = model if args.no_graphs else GraphedDecodeStep(model, args.batch)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(total_steps + 1)]
        flushed = []
        ev[0].record()
        for s in range(total_steps):
            before = model.layers[0].self_attn.history_reserve_length
            row, caches = step(row, caches, pos, aux_for(1))
            pos += 1
            flushed.append(model.layers[0].self_attn.history_reserve_length != before)
            ev[s + 1].record()
        torch.cuda.synchronize()
    ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(total_steps)]
    timed, timed_flush = ms[args.warmup:], flushed[args.warmup:]
    plain = [m for m, f in zip(timed, timed_flush) if not f]
    att = model.layers[0].self_attn
    cached_tokens = att.history_reserve_length + att.current_length
    fp16_bytes = 2 * 2 * args.batch * cfg.num_kv_heads * cfg.head_dim * pos * cfg.num_layers
    out = {
        "metric": "end_to_end_decode_tokens_per_s", "unit": "tokens/s",
        "value": round(args.batch * len(timed) / (sum(timed) / 1e3), 2),
        "value_without_flush_steps": round(args.batch * len(plain) / (sum(plain) / 1e3), 2) if plain else None,
        "ms_per_step_median": round(sorted(timed)[len(timed) // 2], 3),
        "ms_flush_step_mean": round(sum(m for m, f in zip(timed, timed_flush) if f) / max(1, sum(timed_flush)), 3),
        "ms_flush_steps": [round(m, 1) for m, f in zip(timed, timed_flush) if f],
        "flush_steps": int(sum(timed_flush)), "steps": len(timed), "warmup": args.warmup,
        "prefill_s": round(prefill_s, 3),
        "config": {"model": args.model, "layers": cfg.num_layers, "batch": args.batch, "context": args.ctx,
                   "strategy": args.strategy, "tiers": args.tiers,
                   "dense_parts": "eager" if args.no_graphs else "cuda graphs", "shares_evict_4_2_1": [cfg.bit_0, cfg.bit_4, cfg.bit_2, cfg.bit_1]},
        "cached_tokens": cached_tokens, "positions": pos,
        "cache_bytes": cache_nbytes(caches), "fp16_cache_bytes": fp16_bytes,
        "data": "synthetic hidden states, random-init weights", "dtype": "f16",
    }
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
