"""Generate the golden fixtures in this directory by EXECUTING THE REFERENCE.

Run once, where a checkout of the reference is available (point ``HQEKV_REFERENCE_ROOT`` at it):

    python tests/golden/make_golden.py [fixture names; none = all]

It imports the reference's own ``quant/pack_unpack.py``, ``model/public_func.py``,
``quant/hqe_2.py``, ``quant/hqe_matmul.py`` and ``model/llama_hqe.py`` through ``oracle/ref_shim.py`` (CPU, fp16) and stores seeded inputs together with
the outputs the reference produced as ``*.npz`` files.  The tests read only the ``.npz``
files; the reference is not needed to run them.

Inputs avoid constant quantisation groups (scale 0 -> NaN code), whose integer conversion
differs between x86 and the GPU the reference targets.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ref_shim  # noqa: E402

ref = ref_shim.load_reference_model()
pu, pf, hq, hm = ref.pack_unpack, ref.public_func, ref.hqe_2, ref.hqe_matmul


def npy(t):
    return None if t is None else t.detach().cpu().numpy()


ONLY = set(sys.argv[1:])      # fixture names to (re)write; none given = all


def save(name, **arrays):
    if ONLY and name not in ONLY:
        return
    arrays = {k: v for k, v in arrays.items() if v is not None}
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}.npz: {os.path.getsize(path) / 1024:.1f} KiB, {len(arrays)} arrays")


def outlier_K(gen, B, H, T, D):
    K = torch.randn(B, H, T, D, generator=gen)
    for h in range(H):
        ch = torch.randperm(D, generator=gen)[:4]
        K[:, h, :, ch] *= 10
    return K.half()


# ------------------------------------------------------------------------------------------
# 1. codec known-answer tests: every bit width x group size, V-like and K-like shapes
# ------------------------------------------------------------------------------------------
def codec_cases():
    gen = torch.Generator().manual_seed(1234)
    out = {}
    n = 0
    for bit in (8, 4, 2, 1):
        for g in (32, 64, 128):
            # V layout: [B,H,T,D] groups along D
            x = torch.randn(2, 2, 5, 128, generator=gen).half()
            code, scale, mn = pu.uniform_group_quantize_pack_last_dim(x.clone(), g, bit)
            deq = pu.uniform_group_dequantize_unpack_last_dim(code, scale, mn, g, bit)
            out.update({f"c{n}_x": npy(x), f"c{n}_code": npy(code), f"c{n}_scale": npy(scale), f"c{n}_mn": npy(mn),
                        f"c{n}_deq": npy(deq), f"c{n}_meta": np.array([bit, g, 0])})
            n += 1
            # K layout: token-major source viewed channel-major [B,H,D,T], groups along T, outlier channels
            T = 2 * g
            k = outlier_K(gen, 1, 2, T, 128)
            kt = k.transpose(2, 3)
            code, scale, mn = pu.uniform_group_quantize_pack_last_dim(kt, g, bit)
            deq = pu.uniform_group_dequantize_unpack_last_dim(code, scale, mn, g, bit)
            out.update({f"c{n}_x": npy(kt.contiguous()), f"c{n}_code": npy(code), f"c{n}_scale": npy(scale),
                        f"c{n}_mn": npy(mn), f"c{n}_deq": npy(deq), f"c{n}_meta": np.array([bit, g, 1])})
            n += 1
    # extreme magnitudes (fp16 max / tiny) and exact .5 rounding ties
    x = torch.zeros(1, 1, 4, 32).half()
    x[0, 0, 0] = torch.linspace(-30000, 32000, 32).half()
    x[0, 0, 1] = torch.linspace(0, 6e-5, 32).half()
    x[0, 0, 2] = torch.arange(32).half() * 0.5            # scale 0.5 at 5 bit-ish: ties at 8 bit below
    x[0, 0, 3] = torch.arange(32).half() * 127.5 / 31
    for bit in (8, 4, 2):
        code, scale, mn = pu.uniform_group_quantize_pack_last_dim(x.clone(), 32, bit)
        deq = pu.uniform_group_dequantize_unpack_last_dim(code, scale, mn, 32, bit)
        out.update({f"c{n}_x": npy(x), f"c{n}_code": npy(code), f"c{n}_scale": npy(scale), f"c{n}_mn": npy(mn),
                    f"c{n}_deq": npy(deq), f"c{n}_meta": np.array([bit, 32, 0])})
        n += 1
    out["count"] = np.array(n)
    save("codec", **out)


# ------------------------------------------------------------------------------------------
# 1b. Gaussian-codebook codec at 1 bit (the low tier of 'high_uniform_group_low_normal_group')
# ------------------------------------------------------------------------------------------
def normal_codec_cases():
    gen = torch.Generator().manual_seed(4321)
    out = {}
    n = 0
    for g in (32, 64, 128):
        x = (torch.randn(2, 2, 5, 128, generator=gen) * 1.7 + 0.3).half()
        code, std, mean = pu.normal_group_quantize_pack_last_dim(x.clone(), g, 1)
        deq = pu.normal_group_dequantize_unpack_last_dim(code, std, mean, g, 1)
        out.update({f"c{n}_x": npy(x), f"c{n}_code": npy(code), f"c{n}_std": npy(std), f"c{n}_mean": npy(mean),
                    f"c{n}_deq": npy(deq), f"c{n}_meta": np.array([1, g, 0])})
        n += 1
        T = 2 * g
        k = outlier_K(gen, 1, 2, T, 128)
        kt = k.transpose(2, 3)
        code, std, mean = pu.normal_group_quantize_pack_last_dim(kt.contiguous(), g, 1)
        deq = pu.normal_group_dequantize_unpack_last_dim(code, std, mean, g, 1)
        out.update({f"c{n}_x": npy(kt.contiguous()), f"c{n}_code": npy(code), f"c{n}_std": npy(std),
                    f"c{n}_mean": npy(mean), f"c{n}_deq": npy(deq), f"c{n}_meta": np.array([1, g, 1])})
        n += 1
    # values that straddle the group mean closely, and tiny magnitudes
    x = torch.zeros(1, 1, 3, 32).half()
    x[0, 0, 0] = (1.0 + torch.arange(32) * 9.765625e-4).half()
    x[0, 0, 1] = torch.linspace(-6e-5, 6e-5, 32).half()
    x[0, 0, 2] = (torch.randn(32, generator=gen) * 300).half()
    code, std, mean = pu.normal_group_quantize_pack_last_dim(x.clone(), 32, 1)
    deq = pu.normal_group_dequantize_unpack_last_dim(code, std, mean, 32, 1)
    out.update({f"c{n}_x": npy(x), f"c{n}_code": npy(code), f"c{n}_std": npy(std), f"c{n}_mean": npy(mean),
                f"c{n}_deq": npy(deq), f"c{n}_meta": np.array([1, 32, 0])})
    n += 1
    out["count"] = np.array(n)
    out["center_f32"] = pu.normal_quantiles_center[1].numpy()
    out["upper_f32"] = pu.normal_quantiles_upper_bound[1].numpy()
    save("codec_normal", **out)


# ------------------------------------------------------------------------------------------
# 2. importance ring, token range, block ranking
# ------------------------------------------------------------------------------------------
def ranking_cases():
    gen = torch.Generator().manual_seed(77)
    out = {}
    L = 32 * 40
    ring = pf.last_attn_weights()
    ring.set_max_length(L + 64)
    prefill = torch.softmax(torch.randn(1, 8, 24, L, generator=gen) * 2, -1).half()
    ring.update(prefill)
    out["prefill_w"] = npy(prefill)
    out["ring_after_prefill"] = npy(ring.weights.clone())
    steps = []
    for s in range(5):
        w = torch.softmax(torch.randn(2, 8, 1, L + s + 1, generator=gen) * 2, -1).half()
        ring.update(w)
        steps.append(w)
        out[f"step_w{s}"] = npy(w)
    out["ring_after_steps"] = npy(ring.weights.clone())
    out["ring_next_line"] = np.array(ring.next_line)
    imp = ring.calculate_token_importance()
    out["importance"] = npy(imp)
    work = imp[:L].clone()
    ids = pf.get_block_token_idx(32, L // 32, work)
    out["rank_ids"] = npy(ids)
    out["rank_importance_after"] = npy(work)
    # realistic long-context magnitudes (probabilities ~1/L -> fp16 subnormal keys, many ties)
    L2 = 32 * 256
    imp2 = (torch.rand(L2, generator=gen) * 2e-3).half()
    out["imp2"] = npy(imp2)
    w2 = imp2.clone()
    out["rank2_ids"] = npy(pf.get_block_token_idx(32, L2 // 32, w2))
    out["rank2_after"] = npy(w2)
    w3 = w2.clone()                                         # second division, as on the V side
    out["rank3_ids"] = npy(pf.get_block_token_idx(32, L2 // 32, w3))
    # token range
    v = torch.randn(2, 4, 37, 128, generator=gen).half()
    out["range_v"] = npy(v)
    out["range_out"] = npy(pf.calculate_token_range(v, None))
    arr = torch.tensor([3, 0, 7, 9, 1, 2], dtype=torch.int32)
    out["mse_in"] = npy(arr.clone())
    out["mse_out"] = npy(pf.make_sum_equal(arr.clone(), 20))
    save("ranking", **out)


# ------------------------------------------------------------------------------------------
# 3. flush sequences through KV_cache_hqe_2, then the dense reconstruction
# ------------------------------------------------------------------------------------------
def dump_cache(prefix, cache, out):
    for i, item in enumerate(cache):
        if item is None:
            continue
        out[f"{prefix}_{i}"] = np.array(item) if isinstance(item, int) else npy(item)


def flush_sequence(name, seed, B, H, steps, times_range, block=32, group=32, strategy="uniform_group"):
    """steps: list of (n_new_tokens, bit_num[6]); the first entry is the prefill."""
    gen = torch.Generator().manual_seed(seed)
    D = 128
    out = {"meta": np.array([B, H, D, block, group, int(times_range), len(steps)])}
    ring = pf.last_attn_weights()
    ring.set_max_length(4096)
    cache = None
    hist = 0
    cur = 0
    seq = 0
    for si, (n_new, bit_num) in enumerate(steps):
        k = outlier_K(gen, B, H, n_new, D)
        v = torch.randn(B, H, n_new, D, generator=gen).half()
        seq += n_new
        cur += n_new
        if cache is None:
            cache = (None,) * 39 + (k, v, seq)
        else:
            nk = torch.cat((cache[-3], k), dim=2) if cache[-3] is not None else k
            nv = torch.cat((cache[-2], v), dim=2) if cache[-2] is not None else v
            cache = cache[:-3] + (nk, nv, seq)
        L = hist + cur
        # a few decode-step probability rows so the ring holds realistic importances
        for _ in range(3):
            ring.update(torch.softmax(torch.randn(B, 4 * H, 1, L, generator=gen) * 3, -1).half())
        compress = cur - cur % block
        total = hist + compress
        imp = ring.calculate_token_importance()
        sort_imp = imp[:total].clone()
        out[f"s{si}_importance_in"] = npy(sort_imp.clone())
        K_ids = pf.get_block_token_idx(block, total // block, sort_imp)
        bn = torch.tensor(bit_num, dtype=torch.int32)
        assert int(bn.sum()) == total, (int(bn.sum()), total)
        dump_cache(f"s{si}_in", cache, out)
        out[f"s{si}_args"] = np.array([compress, hist])
        out[f"s{si}_K_ids"] = npy(K_ids)
        out[f"s{si}_bit_num"] = npy(bn)
        out[f"s{si}_importance_ranked"] = npy(sort_imp.clone())
        out[f"s{si}_ring_in"] = npy(ring.weights.clone())
        cache = hq.KV_cache_hqe_2(cache, compress, hist, K_ids, bn, bn.clone(), sort_imp, strategy, ring,
                                  block, group, times_range)
        dump_cache(f"s{si}_out", cache, out)
        # one decode step over the new cache through the reference's own qkv_matmul_hqe_2 (CPU stand-in GEMV)
        qgen = torch.Generator().manual_seed(seed * 1000 + si)
        q = torch.randn(B, 4 * H, 1, D, generator=qgen).half()
        aw, ao = hm.qkv_matmul_hqe_2(q, cache, None, D, strategy, block, group)
        out[f"s{si}_q"], out[f"s{si}_attn_weights"], out[f"s{si}_attn_output"] = npy(q), npy(aw), npy(ao)
        out[f"s{si}_ring_out"] = npy(ring.weights.clone())
        out[f"s{si}_importance_after"] = npy(sort_imp.clone())
        hist += compress - bit_num[5]
        cur -= compress
        ring.kv_seq_len = hist + cur          # the next update() overwrites this anyway
    rk, rv = hq.KV_cache_reconstruct_hqe(cache, strategy, block, group)
    out["strategy"] = np.array(strategy)
    out["recon_K"] = npy(rk)
    out["recon_V"] = npy(rv)
    save(name, **out)


# ------------------------------------------------------------------------------------------
# 4. the attention module that drives the cache: LlamaAttention_hqe.forward, prefill + decode steps
# ------------------------------------------------------------------------------------------
def rotary(positions, head_dim, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = positions.float().unsqueeze(-1) * inv
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos().half(), ang.sin().half()


def attention_module_case(name, seed, strategy, B, hidden, nh, nkv, prefill, steps, shares):
    """Run the reference's attention layer (eager prefill, then one token at a time) on seeded hidden states
    and record, per call: the input, the layer output, the tier counts it derived when it flushed, and the
    lengths / tier sizes afterwards."""
    from transformers.models.llama.configuration_llama import LlamaConfig
    cfg = LlamaConfig(hidden_size=hidden, num_attention_heads=nh, num_key_value_heads=nkv, head_dim=128,
                      intermediate_size=2 * hidden, num_hidden_layers=1, attention_bias=False, attention_dropout=0.0)
    cfg._attn_implementation = "eager"
    cfg.quant_strategy, cfg.times_range = strategy, True
    cfg.bit_0, cfg.bit_4, cfg.bit_2, cfg.bit_1 = shares
    gen = torch.Generator().manual_seed(seed)
    attn = ref.llama_hqe.LlamaAttention_hqe(cfg, 0)
    out = {"meta": np.array([B, hidden, nh, nkv, prefill, steps]), "shares": np.array(shares, dtype=np.float64),
           "strategy": np.array(strategy)}
    with torch.no_grad():
        for pname in ("q_proj", "k_proj", "v_proj", "o_proj"):
            w = getattr(attn, pname).weight
            w.copy_(torch.randn(w.shape, generator=gen) * w.shape[1] ** -0.5)
        attn = attn.half()
        for pname in ("q_proj", "k_proj", "v_proj", "o_proj"):
            out[f"w_{pname}"] = npy(getattr(attn, pname).weight)
        attn.last_weights.set_max_length(prefill + steps)
        cache, aux = None, None
        pos = 0
        for call in range(steps + 1):
            S = prefill if call == 0 else 1
            x = torch.randn(B, S, hidden, generator=gen).half()
            cos, sin = rotary(torch.arange(pos, pos + S).unsqueeze(0).expand(B, S), 128)
            mask = None
            if call == 0:
                mask = torch.full((S, S), torch.finfo(torch.float16).min, dtype=torch.float16).triu(1).view(1, 1, S, S)
            y, _, cache, aux_out = attn(x, (cos, sin), mask, past_key_value=cache, auxiliary_parameters=None, use_cache=True)
            pos += S
            out[f"c{call}_x"], out[f"c{call}_y"] = npy(x), npy(y)
            if aux_out is not None:
                out[f"c{call}_ratio"], out[f"c{call}_bit_num"] = npy(aux_out[0]), npy(aux_out[1])
            sizes = [0 if cache[i] is None else cache[i].numel() for i in (1, 5, 13, 21, 29, 3, 9, 17, 25, 33)]
            out[f"c{call}_state"] = np.array([attn.current_length, attn.history_reserve_length, cache[41]] + sizes)
    save(name, **out)


def main():
    codec_cases()
    normal_codec_cases()
    ranking_cases()
    # totals: 256 | 224+96=320 | 288+64=352
    flush_sequence("flush_a", 11, 1, 2,
                   [(262, [64, 32, 64, 64, 0, 32]), (96, [64, 32, 64, 96, 32, 32]), (64, [64, 0, 64, 128, 64, 32])],
                   times_range=True)
    # no eviction at all, batch 2, K and V ranked identically
    flush_sequence("flush_b", 12, 2, 1,
                   [(130, [32, 32, 32, 32, 0, 0]), (64, [32, 32, 64, 64, 0, 0])], times_range=False)
    # group 64 (block 64 for K), heavier eviction
    flush_sequence("flush_c", 13, 1, 2,
                   [(256 + 5, [64, 64, 64, 0, 0, 64]), (128, [64, 0, 64, 64, 64, 64])], times_range=True,
                   block=64, group=64)
    # 1-bit tier in the Gaussian-codebook codec: arrivals from the residual and from every higher tier
    flush_sequence("flush_n", 14, 1, 2,
                   [(262, [64, 32, 64, 32, 32, 32]), (96, [64, 32, 32, 96, 64, 32]), (64, [32, 32, 64, 96, 96, 32])],
                   times_range=True, strategy="high_uniform_group_low_normal_group")
    flush_sequence("flush_n64", 15, 2, 1,
                   [(256 + 7, [64, 64, 64, 0, 64, 0]), (128, [64, 0, 64, 64, 128, 64])], times_range=True,
                   block=64, group=64, strategy="high_uniform_group_low_normal_group")
    # the attention layer around the cache: prefill 420 tokens (two blocks evicted), 75 decode steps (three more flushes)
    attention_module_case("attn_llama_n", 21, "high_uniform_group_low_normal_group", 2, 256, 2, 1, 420, 75,
                          (0.25, 0.25, 0.25, 0.25))
    attention_module_case("attn_llama_u", 22, "uniform_group", 1, 512, 4, 1, 200, 40, (0.1, 0.4, 0.3, 0.2))


if __name__ == "__main__":
    main()
