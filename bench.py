#!/usr/bin/env python
"""Decode-attention throughput of the hybrid mixed-precision KV cache on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-cuda] [--workload cfg1]

One "step" = the attention of one decode step of the whole model: for every layer, the fused decode
(q.K^T, softmax, p.V over the 8/4/2-bit tiers and the fp16 residual window: two kernel launches) over that
layer's own cache.  Default workload (N=1): Llama-3.1-8B shape, 32 layers, batch 1, context 32768, 10 % evicted,
20/40/40 % of the rest in 8/4/2-bit, group 32, residual 128, synthetic N(0,1) data.  The 32 caches
total ~1.2 GB, ten times the 126 MB L2, so every step streams its cache from HBM.

N > 1 (launched by torch.distributed.run): kv heads are sharded over the ranks (strong scaling); each
layer's per-head outputs are exchanged by flagged peer stores from the decode kernel (--peer-gather; an NCCL
all-gather per layer with 'off').

Prints ONE JSON line on rank 0.  Keys beside the contract's: `value` is the median over `timed_windows` windows
of exactly --steps steps each (a window is repeated until about a second has been timed); `e2e` the same
metric through the public Python operator with q coming from and the outputs going to pinned host memory every
step; `roofline` per kernel (algorithmic bytes / CUDA-event time against the measured copy bandwidth, DRAM
traffic from an ncu capture); `cpu_baseline` the reference's CPU path on the host cores (one layer, scaled);
`parity` the errors of the timed workload's first layer against the fp32 oracle; `build_id` the stamp of the
library that ran; `importance_row_exchange_us` (N > 1) the other exchange of the sharded path, timed alone.

--impl reference: the reference's own CPU implementation of the path on the host cores, no GPU and no CUDA library
(rank 0 alone under torchrun).  --impl reference-cuda: the reference's own CUDA extension, where it has been built
into baseline/_ref, on the same cache tuples.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode-attn tokens/sec at 32k ctx"
UNIT = "tokens/s"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the default workload (one cfg1 layer), from one ncu
# capture of the two kernels (cold caches: logits and index lists are read from DRAM there, in the chained run they
# are L2 hits).  Only valid for that workload on one GPU; other workloads report null.
NCU_TRAFFIC_BYTES = {"k_pass_kernel": 19390464, "v_pass_kernel": 23248128}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"],
                    help="reference: the reference's CPU path on the host cores; reference-cuda: the reference's own CUDA "
                         "kernels (needs baseline/_ref, see baseline/build_ref.py), one GPU")
    ap.add_argument("--workload", default="cfg1")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = the workload's)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--max-windows", type=int, default=200,
                    help="the timed window of --steps steps is repeated until about a second has been timed, at most "
                         "this many times (1 for a run under a profiler)")
    ap.add_argument("--peer-gather", choices=["off", "flagged", "barrier"], default="flagged",
                    help="multi-GPU: the decode kernel stores its rows into the peers' buffers (symmetric memory) "
                         "instead of an NCCL all-gather per layer: 'flagged' = values travel with the call number, "
                         "'barrier' = plain stores + cross-GPU barrier")
    return ap.parse_args()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region (read-only query)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# -------------------------------------------------------------------------------------------------
# CPU arm: the reference's own pure-PyTorch path on the host cores (or its numpy restatement)
# -------------------------------------------------------------------------------------------------
def cpu_threads():
    return os.cpu_count() or 1


def build_cache_on_host(cfg, seed=0):
    """One layer's cache of the workload built WITHOUT the CUDA library: seeded K, V, q with the configuration's
    distributions, ranked and flushed by the numpy oracle.  Returns (cache tuple of numpy arrays, q)."""
    import numpy as np
    import torch
    from hqekv_b200 import configs
    from oracle import hqkv_oracle as O
    g = torch.Generator().manual_seed(seed)
    shape = (cfg.batch, cfg.nh_kv, cfg.context, cfg.head_dim)
    K = torch.randn(shape, generator=g)
    V = torch.randn(shape, generator=g)
    if cfg.k_outliers:
        for h in range(cfg.nh_kv):
            K[:, h][:, :, torch.randperm(cfg.head_dim, generator=g)[:4]] *= 10
    q = torch.randn(cfg.batch, cfg.nh_q, 1, cfg.head_dim, generator=g).half().numpy()
    K, V = K.half().numpy(), V.half().numpy()
    flushed = cfg.context - cfg.residual
    counts = np.array(configs.tier_counts(cfg))
    imp = torch.softmax(torch.randn(8, flushed, generator=g) * 2.0, dim=-1).sum(0).div_(8).half().numpy()
    ids = O.block_rank(cfg.group, flushed // cfg.group, imp.copy())
    cache = (None,) * 39 + (K, V, cfg.context)
    return O.flush(cache, flushed, 0, ids, counts, counts.copy(), imp, cfg.strategy, None, cfg.group, cfg.group, False), q


def cpu_layer_timer(cache_host, q_host, cfg):
    """Returns (fn, kind, cores): fn() runs ONE layer's decode attention on the host - dense dequantisation of every
    tier + fp32 softmax(q K^T / sqrt(d)) V, the path the reference offers without its CUDA extension.
    kind 'reference': the reference's own KV_cache_reconstruct_hqe (quant/hqe_2.py:967-1084), imported unmodified
    from the staged copy oracle/_ref through oracle/ref_shim.py, + torch fp32 attention, all host threads.
    kind 'port': the numpy oracle (same arithmetic restated), kv heads spread over the host threads."""
    import numpy as np
    import torch
    from oracle import ref_shim
    threads = cpu_threads()
    if ref_shim.available():
        ref = ref_shim.load_reference()
        torch.set_num_threads(threads)
        cache_t = tuple(torch.from_numpy(np.ascontiguousarray(x)) if isinstance(x, np.ndarray) else x for x in cache_host)
        q_t = torch.from_numpy(q_host)
        H = cfg.nh_kv
        rep = cfg.nh_q // H

        def run():
            K, V = ref.hqe_2.KV_cache_reconstruct_hqe(cache_t, cfg.strategy, cfg.group, cfg.group)
            qf = q_t.float().view(cfg.batch, H, rep, cfg.head_dim)
            logits = torch.matmul(qf, K.float().transpose(2, 3)) / (cfg.head_dim ** 0.5)
            p = torch.softmax(logits, dim=-1)
            return torch.matmul(p, V.float())
        return run, "reference", threads

    from concurrent.futures import ThreadPoolExecutor
    from oracle import hqkv_oracle as O
    H = cfg.nh_kv
    rep = cfg.nh_q // H
    workers = min(H, threads)

    def head_slice(h):
        out = []
        for i, item in enumerate(cache_host):
            out.append(item if (item is None or i == 41 or item.ndim < 4) else item[:, h:h + 1])
        return tuple(out), q_host[:, h * rep:(h + 1) * rep]

    def one(h):
        c, qq = head_slice(h)
        return O.decode_attention(qq, c, None, cfg.group, cfg.group, dequant="fp16", quant_strategy=cfg.strategy)

    def run():
        with ThreadPoolExecutor(workers) as ex:
            return list(ex.map(one, range(H)))
    return run, "port", workers


def time_cpu_layer(cache_host, q_host, cfg, layers, reps):
    """cpu_baseline record: one layer timed `reps` times after one warm-up, scaled to the layers of a step."""
    run, kind, cores = cpu_layer_timer(cache_host, q_host, cfg)
    run()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        run()
        ts.append(time.perf_counter() - t0)
    per_layer = statistics.median(ts)
    value = cfg.batch / (per_layer * layers)
    sample = (f"one layer of {cfg.name} (all {cfg.nh_kv} kv heads) timed {reps} times on the host after one warm-up, "
              f"median {per_layer:.3f} s, scaled x{layers} layers to a full step")
    return {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample,
            "extrapolated_from_layers": 1, "seconds_per_layer": per_layer}


def first_layer_parity(cache_host, q_host, w_gpu, o_gpu, cfg, heads=2):
    """Errors of the timed workload's first layer against the fp32 oracle (the checker), on the first `heads` kv heads
    to bound the host time: largest |out - oracle| / max |oracle| per head (bound 2e-3) and the largest relative error
    of a probability beyond the fp16 subnormal quantum (bound 2^-9)."""
    import numpy as np
    from oracle import hqkv_oracle as O
    rep = cfg.nh_q // cfg.nh_kv
    heads = min(heads, cfg.nh_kv)
    c = tuple(item if (item is None or i == 41 or item.ndim < 4) else item[:, :heads] for i, item in enumerate(cache_host))
    ow, oo = O.decode_attention(q_host[:, :heads * rep], c, None, cfg.group, cfg.group, quant_strategy=cfg.strategy)
    o = o_gpu[:, :heads * rep].astype(np.float32)
    w = w_gpu[:, :heads * rep].astype(np.float32)
    out_rel = float((np.abs(o - oo).max(axis=-1) / np.abs(oo).max(axis=-1)).max())
    w_rel = float((np.maximum(np.abs(w - ow) - 2.0 ** -24, 0) / np.maximum(ow, 1e-30)).max())
    return {"checked": f"layer 0, kv heads 0..{heads - 1}, against the fp32 oracle", "attn_output_max_rel_err": out_rel,
            "attn_output_bound": 2e-3, "attn_weights_max_rel_err": w_rel, "attn_weights_bound": 2.0 ** -9,
            "ok": bool(out_rel <= 2e-3 and w_rel <= 2.0 ** -9)}


def workload_config(cfg, layers, world, cached_tokens, cache_bytes):
    return {"workload": cfg.name, "layers": layers, "batch": cfg.batch, "context": cfg.context,
            "q_heads": cfg.nh_q, "kv_heads": cfg.nh_kv, "head_dim": cfg.head_dim, "group": cfg.group,
            "residual": cfg.residual, "evicted_frac": cfg.evict, "tier_ratio_8_4_2": list(cfg.ratios),
            "fp16_tokens": cfg.fp16_tokens, "quant_strategy": cfg.strategy,
            "parallelism": f"kv-head-shard x{world}" if world > 1 else "single-gpu",
            "l2": "one step streams layers x cache bytes (>> 126 MB L2); no flush needed",
            "cached_tokens": cached_tokens, "cache_bytes_per_layer_per_gpu": cache_bytes}


def host_cache_stats(cache_host, cfg):
    """(logical length, algorithmic bytes) of a host cache tuple: the figures the GPU arm reports for its caches."""
    import numpy as np
    L = sum(cache_host[s].size for s in (1, 5, 13, 21, 29) if cache_host[s] is not None)
    L += cache_host[39].shape[2] if cache_host[39] is not None else 0
    nbytes = sum(x.nbytes for i, x in enumerate(cache_host[:36]) if isinstance(x, np.ndarray) and x.dtype != np.int64)
    nbytes += sum(cache_host[i].nbytes for i in (39, 40) if cache_host[i] is not None)
    return L, nbytes


def host_cache_stats_of_config(cfg):
    """(logical length, algorithmic bytes per layer) of a configuration's cache, from its token counts alone."""
    from hqekv_b200 import configs
    counts = configs.tier_counts(cfg)
    L = sum(counts[:5]) + cfg.residual
    per_head = 0
    for n, bits in zip(counts[:5], (16, 8, 4, 2, 1)):
        per_head += 2 * n * 256 if bits == 16 else 2 * n * (16 * bits + 512 // cfg.group)
    per_head += cfg.residual * 512
    return L, per_head * cfg.batch * cfg.nh_kv


def run_reference_cpu(args, cfg, layers, world):
    """The reference arm: the reference's CPU path for this workload.  Loads neither the CUDA library nor a GPU."""
    cache_host, q_host = build_cache_on_host(cfg, seed=0)
    L, nbytes = host_cache_stats(cache_host, cfg)
    rec = time_cpu_layer(cache_host, q_host, cfg, layers, max(1, min(args.steps, 5)))
    step_s = rec["seconds_per_layer"] * layers
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, layers, max(world, args.gpus), L, nbytes // max(world, args.gpus)),
        "cpu_baseline": rec,
        "e2e": {"value": rec["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def load_reference_cuda():
    """The reference's own quant/hqe_matmul.py on top of its own kvhq_gemv extension, from baseline/_ref (built by
    baseline/build_ref.py; nothing of this package is on that path).  Returns (module, None) or (None, reason)."""
    import glob
    import types
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not glob.glob(os.path.join(ref, "quant", "kvhq_gemv*.so")):
        return None, "baseline/_ref holds no kvhq_gemv extension (python baseline/build_ref.py --reference <checkout>)"
    sys.modules.setdefault("fast_hadamard_transform", types.ModuleType("fast_hadamard_transform"))  # imported, not used here
    sys.path[:0] = [ref, os.path.join(ref, "quant")]
    try:
        import hqe_matmul as ref_hm
    except Exception as e:  # a missing dependency of the reference's environment
        return None, f"the reference modules do not import here: {type(e).__name__}: {e}"
    return ref_hm, None


def run_reference_cuda(args, cfg, layers, config):
    """Time the reference's unmodified qkv_matmul_hqe_2 (per-tier transposes + kvhq_gemv launches + torch softmax,
    quant/hqe_matmul.py:354-451) on the same cache tuples this package's flush builds, and compare its outputs with
    this package's decode of the same tuple."""
    import torch
    ref_hm, why = load_reference_cuda()
    if ref_hm is None:
        print(json.dumps({"impl": "reference-cuda", "unavailable": why}))
        return
    from hqekv_b200 import synthetic
    from hqekv_b200.quant.hqe_matmul import qkv_matmul_hqe_2
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    caches, qs = [], []
    for layer in range(layers):
        cache, q = synthetic.build_cache(cfg, dev, seed=layer)
        caches.append(cache)
        qs.append(q)
    torch.cuda.synchronize()

    def step():
        return [ref_hm.qkv_matmul_hqe_2(qs[i], caches[i], None, cfg.head_dim, cfg.strategy, cfg.group, cfg.group)
                for i in range(layers)]

    for _ in range(max(args.warmup, 3)):
        outs = step()
    torch.cuda.synchronize()
    # agreement with this package's decode on the first layer (the reference rounds logits and per-tier partial
    # outputs to fp16, so it is the looser of the two against an fp32 oracle)
    w_ref, o_ref = outs[0]
    w_our, o_our = qkv_matmul_hqe_2(qs[0], caches[0], None, cfg.head_dim, cfg.strategy, cfg.group, cfg.group)
    torch.cuda.synchronize()
    rel = float(((o_ref.float() - o_our.float()).abs().amax(-1) / o_our.float().abs().amax(-1)).max())
    wdiff = float((w_ref.float() - w_our.float()).abs().max())
    agreement = {"attn_output_max_rel_diff": rel, "attn_weights_max_abs_diff": wdiff}
    if w_ref.shape[-1] <= 8192:
        # small enough for the checker: the oracle's restatement of the reference's fp16 flow (per-tier GEMV rounded to
        # fp16, fp16 scaling, fp32 softmax rounded to fp16, per-tier partial outputs rounded to fp16) against what the
        # reference's kernels really return
        from oracle import hqkv_oracle as O
        host = tuple(x.cpu().numpy() if torch.is_tensor(x) else x for x in caches[0])
        fw, fo = O.decode_attention_fp16_flow(qs[0].cpu().numpy(), host, cfg.group, cfg.group, cfg.strategy)
        fo_t, fw_t = torch.from_numpy(fo).float().to(dev), torch.from_numpy(fw).float().to(dev)
        agreement["vs_fp16_flow_oracle"] = {
            "attn_output_max_rel_diff": float(((o_ref.float() - fo_t).abs().amax(-1) / fo_t.abs().amax(-1)).max()),
            "attn_weights_max_abs_diff": float((w_ref.float() - fw_t).abs().max())}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = max(args.steps, 20)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms_per_step = e0.elapsed_time(e1) / steps
    value = cfg.batch / (ms_per_step * 1e-3)
    print(json.dumps({
        "impl": "reference-cuda", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": config,
        "note": "the reference's own CUDA extension (kvhq_gemv, built for sm_100 from its sources) driven by its own "
                "quant/hqe_matmul.py:qkv_matmul_hqe_2, eager launches on the default stream, CUDA events around "
                f"{steps} steps of {layers} layers",
        "agreement_with_this_package": agreement}))


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # convenience: relaunch under torch.distributed.run
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29531"),
               os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))

    from hqekv_b200 import configs
    cfg = configs.CONFIGS[args.workload]
    layers = args.layers or cfg.layers

    # ---------------------------------------------------------------------------------------------
    # reference arm: the reference's CPU path on the host cores; rank 0 alone, no GPU, no CUDA library
    # ---------------------------------------------------------------------------------------------
    if args.impl == "reference":
        if rank == 0:
            run_reference_cpu(args, cfg, layers, world)
        return

    import numpy as np
    import torch
    from hqekv_b200 import build
    build.build()
    from hqekv_b200 import synthetic
    from hqekv_b200._lib import check, lib, ptr, stream_ptr
    build_id = lib.hqkv_build_id().decode()
    if not os.environ.get("HQKV_LIB") and build_id != build.source_id():
        raise SystemExit(f"libhqkv.so was built from other sources (stamp {build_id}, sources {build.source_id()})")
    from hqekv_b200.quant._cache import build_cache_desc
    from hqekv_b200.quant.hqe_matmul import qkv_matmul_hqe_2

    if args.impl == "reference-cuda":
        if rank == 0:
            L0, nbytes0 = host_cache_stats_of_config(cfg)
            run_reference_cuda(args, cfg, layers, workload_config(cfg, layers, 1, L0, nbytes0))
        return

    # ---------------------------------------------------------------------------------------------
    # our arm
    # ---------------------------------------------------------------------------------------------
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this package has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        assert cfg.nh_kv % world == 0, "kv heads must divide over the ranks"
    heads_per_rank = cfg.nh_kv // world
    shard = (rank * heads_per_rank, heads_per_rank)
    rep = cfg.nh_q // cfg.nh_kv
    nh_q_local = heads_per_rank * rep

    # one cache per layer (distinct memory), seeded per layer
    caches, qs = [], []
    for layer in range(layers):
        cache, q = synthetic.build_cache(cfg, dev, seed=layer, heads=shard)
        caches.append(cache)
        qs.append(q)
    torch.cuda.synchronize()
    L = synthetic.logical_length(caches[0])
    bytes_per_layer = synthetic.cache_bytes(caches[0], nh_q_local)
    config = workload_config(cfg, layers, world, L, bytes_per_layer)

    gathered = [torch.empty(world, cfg.batch, nh_q_local, 1, cfg.head_dim, dtype=torch.float16, device=dev)
                for _ in range(layers)] if world > 1 else None

    # Multi-GPU exchange of the per-head outputs.  Default: the decode kernel stores its rows, each pair of
    # values in one 8-byte word with the call number, into every peer's receive buffer and a bounded
    # unpack kernel follows (sharding.FlaggedPeerGather).  --peer-gather barrier: plain stores + cross-GPU
    # barrier; off: NCCL all-gather per layer, also the fallback when symmetric memory is not available
    # or the result differs from NCCL's on the first layer (checked every run).
    peer = None
    exchange = None
    if world > 1 and args.peer_gather != "off":
        try:
            from hqekv_b200.sharding import FlaggedPeerGather, PeerGather
            peer = (PeerGather if args.peer_gather == "barrier" else FlaggedPeerGather)(
                max(layers, 2), cfg.batch, nh_q_local, cfg.head_dim, dev)
            _, o_ref = qkv_matmul_hqe_2(qs[0], caches[0], None, cfg.head_dim, cfg.strategy, cfg.group, cfg.group)
            dist.all_gather_into_tensor(gathered[0], o_ref)
            _, got = peer.decode(0, qs[0], caches[0], cfg.group, cfg.group, cfg.strategy)
            torch.cuda.synchronize()
            ok = torch.tensor([int(torch.equal(got, gathered[0]) and peer.status() == 0)], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) != 1:
                raise RuntimeError("peer-store gather differs from the NCCL all-gather")
        except Exception as e:
            if rank == 0:
                print(f"[bench] peer-store gather unavailable ({type(e).__name__}: {e}); using NCCL all-gather", file=sys.stderr)
            peer = None
    if world > 1:
        exchange = (f"peer stores from the decode kernel ({args.peer_gather})" if peer else "nccl all_gather per layer")
    # the other exchange of the sharded path: the head-summed probability row that feeds the ranking, once per
    # layer-step over NCCL (sharding.reduce_importance_row); timed here on its own, outside the step
    importance_row_us = None
    if world > 1:
        from hqekv_b200.sharding import reduce_importance_row
        part = torch.rand(cfg.context, dtype=torch.float32, device=dev)
        for _ in range(3):
            reduce_importance_row(part)
        torch.cuda.synchronize()
        dist.barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(20):
            reduce_importance_row(part)
        r1.record()
        torch.cuda.synchronize()
        t = torch.tensor([r0.elapsed_time(r1) / 20 * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        importance_row_us = float(t.item())

    def decode_layer(i, q):
        if peer is not None:
            w, g = peer.decode(i, q, caches[i], cfg.group, cfg.group, cfg.strategy)
            return g[rank]
        w, o = qkv_matmul_hqe_2(q, caches[i], None, cfg.head_dim, cfg.strategy, cfg.group, cfg.group)
        if world > 1:
            dist.all_gather_into_tensor(gathered[i], o)
        return o

    def step_device():
        return [decode_layer(i, qs[i]) for i in range(layers)]

    use_graph = not args.no_graph
    graph = None
    for _ in range(2):
        step_device()
    torch.cuda.synchronize()
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_device()
                with torch.cuda.graph(graph, stream=side):
                    graph_outs = step_device()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
        except Exception as e:  # capture can fail with some NCCL configurations: fall back to eager launches
            if rank == 0:
                print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); launching eagerly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    launch = "cuda_graph" if graph is not None else "eager"

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step_device()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()

    def timed_window(step_fn):
        """EXACTLY args.steps steps between two events, a barrier + synchronize on both sides; max over ranks."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(args.steps):
            step_fn()
        e1.record()
        barrier()
        ms_ = e0.elapsed_time(e1)
        if world > 1:
            t_ = torch.tensor([ms_], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            ms_ = float(t_.item())
        return ms_

    def timed_median(step_fn):
        """A window of a few milliseconds is fragile: the window is repeated until about a second has been timed
        (at most 200 times, the same count on every rank) and the median window is reported."""
        first = timed_window(step_fn)
        n = max(1, min(args.max_windows, int(1000.0 / max(first, 1e-3))))
        windows = sorted([first] + [timed_window(step_fn) for _ in range(n - 1)])
        return windows[len(windows) // 2], len(windows)

    ms, n_windows = timed_median(run_step)
    clocks = sampler.stop() if rank == 0 else None
    if peer is not None and peer.status() != 0:
        raise RuntimeError(f"rank {rank}: a cross-GPU barrier gave up waiting for rank {peer.status() - 1}")
    ms_per_step = ms / args.steps
    value = cfg.batch / (ms_per_step * 1e-3)

    # ---- end to end through the public call: the step's inputs (q of every layer) start in pinned host
    #      memory, the step's results (attn_output of every layer) end there
    q_host = torch.stack([q.cpu() for q in qs]).pin_memory()          # [layers, B, nh_q, 1, D]
    q_dev = torch.empty_like(q_host, device=dev)
    out_host = torch.empty(layers, cfg.batch, nh_q_local, 1, cfg.head_dim, dtype=torch.float16).pin_memory()

    def enqueue_e2e():
        q_dev.copy_(q_host, non_blocking=True)
        outs = []
        for i in range(layers):
            outs.append(decode_layer(i, q_dev[i]))
        out_host.copy_(torch.stack(outs), non_blocking=True)

    # The way a serving loop drives the operator: the step's host->device copies, the public call for
    # every layer and the device->host copies are captured once into a CUDA graph and replayed per
    # step (eager Python launches cost more host time per layer than the two kernels take on the GPU;
    # that figure is reported beside it).
    e2e_graph = None
    if use_graph:
        try:
            enqueue_e2e()
            torch.cuda.synchronize()
            e2e_graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(e2e_graph, stream=side):
                    enqueue_e2e()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
        except Exception as e:
            if rank == 0:
                print(f"[bench] e2e graph capture failed ({type(e).__name__}: {e}); launching eagerly", file=sys.stderr)
            e2e_graph = None
            torch.cuda.synchronize()

    def time_e2e(step_fn):
        for _ in range(3):
            step_fn()
        return timed_median(step_fn)[0]

    def step_e2e_eager():
        enqueue_e2e()
        torch.cuda.synchronize()  # the host reads the step's result

    def step_e2e_graph():
        e2e_graph.replay()
        torch.cuda.synchronize()

    eager_ms = time_e2e(step_e2e_eager)
    e2e_ms = time_e2e(step_e2e_graph) if e2e_graph is not None else eager_ms
    e2e_value = cfg.batch / (e2e_ms / args.steps * 1e-3)
    q_bytes = qs[0].numel() * 2
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": layers * q_bytes,
           "d2h_bytes_per_step": layers * q_bytes, "ms_per_step": e2e_ms / args.steps,
           "launch": "cuda_graph" if e2e_graph is not None else "eager",
           "eager_value": cfg.batch / (eager_ms / args.steps * 1e-3),
           "note": "per step: q of all layers copied from pinned host memory in one transfer, the public operator "
                   "called per layer, all attn_outputs copied back to pinned host memory in one transfer, one host "
                   "synchronisation; the cache is resident state. value: the "
                   "step replayed from a CUDA graph; eager_value: the same calls issued from Python every step"}

    # ---- per-kernel timing for the roofline: each phase launched alone over all layers (own scratch each)
    peak, peak_kind = load_peaks()
    descs = []
    for i in range(layers):
        desc, keep, Ld, _ = build_cache_desc(caches[i], nh_q_local, cfg.group, cfg.group, 0 if cfg.strategy == "uniform_group" else 1)
        need = lib.hqkv_decode_workspace_bytes(desc)
        ws = torch.zeros(need, dtype=torch.uint8, device=dev)
        w = torch.empty(cfg.batch, nh_q_local, 1, Ld, dtype=torch.float16, device=dev)
        o = torch.empty(cfg.batch, nh_q_local, 1, cfg.head_dim, dtype=torch.float16, device=dev)
        descs.append((desc, keep, ws, w, o))
    def run_phase(phase):
        st = stream_ptr(dev)
        for i in range(layers):
            desc, _, ws, w, o = descs[i]
            check(lib.hqkv_decode_attention_phases(desc, ptr(qs[i]), ptr(w), ptr(o), ptr(ws), ws.numel(), phase, st))

    # one launch costs less GPU time than a Python call takes, so the launches of all layers are replayed
    # from a CUDA graph back to back and the event time is divided by the number of launches: the K pass
    # alone, the V pass alone (on the logits the K pass left), and the pair as the call issues it.
    kernel_ms = {}
    reps = max(3, min(args.steps, 10))
    for phase, name in ((1, "k_pass_kernel"), (2, "v_pass_kernel"), (3, "k_pass_kernel+v_pass_kernel")):
        run_phase(3)
        torch.cuda.synchronize()
        pg = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(pg, stream=side):
                run_phase(phase)
        torch.cuda.current_stream().wait_stream(side)
        pg.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            pg.replay()
        b.record()
        torch.cuda.synchronize()
        kernel_ms[name] = a.elapsed_time(b) / ((reps) * layers)
    # algorithmic bytes per launch: K side and V side of one layer's cache on this GPU
    k_bytes = sum(c.numel() * c.element_size() for s in (0, 4, 6, 7, 12, 14, 15, 20, 22, 23, 28, 30, 31) if (c := caches[0][s]) is not None)
    k_bytes += caches[0][39].numel() * 2 if caches[0][39] is not None else 0
    kernels = []
    for name, nbytes in (("k_pass_kernel", k_bytes), ("v_pass_kernel", bytes_per_layer - k_bytes),
                         ("k_pass_kernel+v_pass_kernel", bytes_per_layer)):
        achieved = nbytes / (kernel_ms[name] * 1e-3) / 1e9
        kernels.append({"kernel": name, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                        "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(name) if (args.workload == "cfg1" and world == 1 and not args.layers) else None,
                        "algorithmic_bytes_per_launch": nbytes, "us_per_launch": kernel_ms[name] * 1e3,
                        "peak_source": peak_kind})
    dominant = max(kernels[:2], key=lambda k: k["us_per_launch"])  # the slower of the two kernels
    roofline = {k: dominant[k] for k in ("bound", "achieved", "peak", "unit", "frac", "traffic")}
    roofline.update({"kernel": dominant["kernel"], "peak_source": peak_kind, "kernels": kernels,
                     "frac_of_8TBps_nominal": dominant["achieved"] / 8000.0,
                     "whole_step_GBps": bytes_per_layer * layers / (ms_per_step * 1e-3) / 1e9,
                     "whole_step_frac": bytes_per_layer * layers / (ms_per_step * 1e-3) / 1e9 / peak})

    # ---- CPU baseline on rank 0, N=1: one layer of the same workload through the same host path the reference arm times
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cache_host = tuple(x.cpu().numpy() if torch.is_tensor(x) else x for x in caches[0])
        cpu_baseline = time_cpu_layer(cache_host, qs[0].cpu().numpy(), cfg, layers, 3)
    parity = None
    if rank == 0 and world == 1:
        w0, o0 = qkv_matmul_hqe_2(qs[0], caches[0], None, cfg.head_dim, cfg.strategy, cfg.group, cfg.group)
        cache_host = tuple(x.cpu().numpy() if torch.is_tensor(x) else x for x in caches[0])
        parity = first_layer_parity(cache_host, qs[0].cpu().numpy(), w0.cpu().numpy(), o0.cpu().numpy(), cfg)

    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "timed_windows": n_windows,
            "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16-in/f32-acc",
            "data": "synthetic", "config": config, "launch": launch, "exchange": exchange,
            "importance_row_exchange_us": importance_row_us, "clocks": clocks, "e2e": e2e,
            "gpu_launches": args.steps * layers * (3 if (peer is not None and args.peer_gather == "flagged") else 2),
            "roofline": roofline, "cpu_baseline": cpu_baseline, "parity": parity, "build_id": build_id,
            "tokens_per_sec_per_gpu": value / world}), flush=True)
    if world > 1:
        # Leave without tearing the communicator down: destroying a process group whose collectives
        # were captured into CUDA graphs that are still alive can block forever at interpreter exit.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
