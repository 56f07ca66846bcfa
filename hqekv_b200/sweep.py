"""Kernel microbench sweep of the fused decode and of quantise+pack.

    python -m hqekv_b200.sweep [--out sweep.jsonl] [--quick]

For every point (context, tier mix, group size, batch) a model-shaped stack of 32 layer caches is built
(8 kv heads x head_dim 128, GQA 4, fp16 N(0,1) data, K with outlier channels, residual 128, no eviction)
and the whole decode call and each of its two passes alone are replayed from CUDA graphs and timed with CUDA
events.  Reported per point: microseconds per layer, achieved GB/s on the algorithmic bytes and the
fraction of the measured copy bandwidth.  Small contexts fit the 126 MB L2 across layers; the line says
so (`working_set_MB_per_gpu`).  One JSON object per line.

Under torch.distributed.run with N ranks (one per GPU) the 8 kv heads of every point are split over the ranks, as
the decode path shards them; a point's time is the maximum over the ranks (device-timed, all-reduced), its bytes
are the whole job's.  The microbench is the kernels alone, so no output exchange is part of it:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29541 \
        -m hqekv_b200.sweep --out sweep_n8.jsonl --ctxs 32768 --mixes mixed,all2 --batches 1,8,32,64
"""
import argparse
import json
import os
import sys

import torch

from . import synthetic
from ._lib import check, lib, ptr, stream_ptr
from .quant._cache import build_cache_desc
from .quant.pack_unpack import uniform_group_quantize_pack_last_dim

TIER_MIXES = {"all8": (1.0, 0.0, 0.0), "all4": (0.0, 1.0, 0.0), "all2": (0.0, 0.0, 1.0), "all1": (0.0, 0.0, 0.0, 1.0),
              "mixed": (0.25, 0.5, 0.25),
              # trailing "n": quant_strategy 'high_uniform_group_low_normal_group' (1-bit tier = Gaussian codebook)
              "all1n": (0.0, 0.0, 0.0, 1.0), "mixed1n": (0.25, 0.25, 0.25, 0.25)}


def _strategy(mix):
    return "high_uniform_group_low_normal_group" if mix.endswith("n") else "uniform_group"


def _graph_time(fn, reps):
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def decode_point(dev, ctx, mix, group, batch, layers, peak_gbs, world=1):
    """One point on this rank's share of the heads (8 / world kv heads, 32 / world query heads)."""
    cfg = synthetic.CacheConfig(f"sweep-ctx{ctx}-{mix}-g{group}-b{batch}", batch, 32 // world, 8 // world, 128, ctx, 128,
                                TIER_MIXES[mix], 0.0, group, True, layers)
    items = []
    for layer in range(layers):
        cache, q = synthetic.build_cache(cfg, dev, seed=layer % 4, quant_strategy=_strategy(mix))
        desc, keep, L, _ = build_cache_desc(cache, cfg.nh_q, group, group, 1 if mix.endswith("n") else 0)
        ws = torch.zeros(lib.hqkv_decode_workspace_bytes(desc), dtype=torch.uint8, device=dev)
        w = torch.empty(batch, cfg.nh_q, 1, L, dtype=torch.float16, device=dev)
        o = torch.empty(batch, cfg.nh_q, 1, 128, dtype=torch.float16, device=dev)
        items.append((desc, keep, cache, q, ws, w, o))
    nbytes = synthetic.cache_bytes(items[0][2], cfg.nh_q) * world  # the whole job's bytes per layer

    def run(phase):
        st = stream_ptr(dev)
        for desc, _, _, q, ws, w, o in items:
            check(lib.hqkv_decode_attention_phases(desc, ptr(q), ptr(w), ptr(o), ptr(ws), ws.numel(), phase, st))

    run(3)
    out = {"kind": "decode", "n_gpus": world, "context": ctx, "tiers": mix, "group": group, "batch": batch, "layers": layers,
           "cache_MB_per_layer": nbytes / 1e6, "working_set_MB_per_gpu": nbytes * layers / 1e6 / world}
    # the whole call (two launches per layer) and each of its passes alone
    for phase, name in ((3, "step"), (1, "k_pass"), (2, "v_pass")):
        us = _graph_time(lambda: run(phase), 5) * 1e3 / layers
        if world > 1:  # the slowest rank's time
            t = torch.tensor([us], device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            us = float(t.item())
        b = nbytes / 2 if phase < 3 else nbytes
        out[f"{name}_us"] = us
        out[f"{name}_GBps"] = b / us / 1e3
        out[f"{name}_frac"] = b / us / 1e3 / (peak_gbs * world)  # of the N GPUs' combined copy bandwidth
    out["tokens_per_s"] = batch / (out["step_us"] * 1e-6 * layers) if layers == 32 else None
    return out


def quantize_point(dev, tokens, bit, group, peak_gbs):
    x = torch.randn(1, 8, tokens, 128, device=dev).half()
    out = {"kind": "quantize_pack", "tokens": tokens, "bits": bit, "group": group}
    for name, view in (("v_rows", x), ("k_cols", x.transpose(2, 3))):
        ms = _graph_time(lambda: uniform_group_quantize_pack_last_dim(view, group, bit), 10)
        nbytes = x.numel() * (2 + bit / 8 + 4 / group)
        out[f"{name}_us"] = ms * 1e3
        out[f"{name}_GBps"] = nbytes / ms / 1e6
        out[f"{name}_frac"] = nbytes / ms / 1e6 / peak_gbs
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="sweep.jsonl")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--mixes", default="", help="comma-separated tier mixes instead of the default set, e.g. all1,all1n")
    ap.add_argument("--ctxs", default="", help="comma-separated context lengths instead of the default set")
    ap.add_argument("--batches", default="", help="comma-separated batch sizes instead of 1,8,32")
    ap.add_argument("--groups", default="", help="comma-separated group sizes instead of the default set")
    ap.add_argument("--quantize-only", action="store_true", help="skip the decode points")
    ap.add_argument("--quantize-tokens", default="", help="comma-separated token counts of the quantise+pack points")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        if 8 % world:
            sys.exit("the 8 kv heads of the sweep split over 1, 2, 4 or 8 ranks")
        torch.distributed.init_process_group("nccl", device_id=dev)
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks))["hbm_gbs"]) if os.path.exists(peaks) else 6650.0
    os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    ctxs = (1024 + 128, 4096, 32768) if args.quick else (1024 + 128, 4096, 16384, 32768, 131072)
    if args.ctxs:
        ctxs = tuple(int(c) for c in args.ctxs.split(","))
    mixes = ("mixed",) if args.quick else ("all8", "all4", "all2", "all1", "mixed")
    if args.mixes:
        mixes = tuple(args.mixes.split(","))
    batches = tuple(int(b) for b in args.batches.split(",")) if args.batches else (1, 8, 32)
    groups = tuple(int(g) for g in args.groups.split(",")) if args.groups else ((32,) if args.quick else (32, 128))
    points = []
    for ctx in (() if args.quantize_only else ctxs):
        for mix in mixes:
            for group in groups:
                for batch in batches:
                    shares = TIER_MIXES[mix] + (0.0,) * (4 - len(TIER_MIXES[mix]))
                    avg_bits = sum(sh * b for sh, b in zip(shares, (8, 4, 2, 1)))
                    per_layer = batch * 8 * ctx * 2 * (16 * avg_bits + 512 / group) / world   # bytes on one GPU
                    if per_layer * 32 > 100e9 or (batch >= 32 and ctx > 16384 * world and not args.batches):
                        continue
                    points.append((ctx, mix, group, batch))
    with open(args.out if rank == 0 else os.devnull, "w") as f:
        for ctx, mix, group, batch in points:
            r = decode_point(dev, ctx, mix, group, batch, 32, peak, world)
            if rank == 0:
                f.write(json.dumps(r) + "\n")
                f.flush()
                print(json.dumps(r), flush=True)
            torch.cuda.empty_cache()
        if world > 1:  # quantise+pack is a per-GPU kernel: measured at one GPU only
            torch.distributed.barrier()
            torch.cuda.synchronize()
            return 0
        q_tokens = (tuple(int(t) for t in args.quantize_tokens.split(",")) if args.quantize_tokens
                    else (4096, 32768) if args.quick else (1024, 8192, 32768, 131072))
        for tokens in q_tokens:
            for bit in (8, 4, 2):
                r = quantize_point(dev, tokens, bit, 32, peak)
                f.write(json.dumps(r) + "\n")
                print(json.dumps(r), flush=True)


if __name__ == "__main__":
    sys.exit(main())
