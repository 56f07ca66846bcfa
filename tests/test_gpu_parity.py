"""GPU parity tests: the CUDA path, called through the C ABI (ctypes -> libhqkv.so), against the numpy
oracle and against the golden fixtures produced by the reference's own code.

Bit-exact: packed words, fp16 scale/zero, dequantised values, ranked ids, importance, value ranges,
every slot of a flushed cache.  Tolerance (stated where used): attention outputs within 2e-3 of the
fp32-accumulated dequant-matmul oracle, relative to the largest output magnitude of the head.
"""
import numpy as np
import pytest
import torch

from conftest import golden_cache, load_golden
from oracle import hqkv_oracle as O

pytestmark = pytest.mark.gpu

ATTN_REL_TOL = 2e-3        # max |out - oracle| / max |oracle| per head
# Probabilities are returned in fp16 (subnormal below 6.1e-5, quantum 2^-24).  The kernel carries the logits in
# fp32 (q * scale enters the tensor pipe exactly, as hi + lo), so a probability differs from the fp32 oracle's by
# its final rounding to fp16 (half an ulp, 2^-11 relative) plus the fp32 accumulation noise of the logit.  That
# noise is largest for 1-bit tiers with groups of 64 / 128 tokens, where code * scale and the zero term are two
# large sums that nearly cancel: measured 1.4e-3 relative there, below 1e-3 everywhere else.  Bound: TWO fp16
# ulps (2^-9).  (The reference rounds the logits themselves to fp16, which is an order of magnitude coarser.)
WEIGHT_ABS_TOL = 2.0 ** -24
WEIGHT_REL_TOL = 2.0 ** -9
MEASURED = {"attn_rel": 0.0, "weight_rel": 0.0}   # largest errors seen over the whole module, reported at the end


def dev_cache(cache_np, device):
    out = []
    for i, item in enumerate(cache_np):
        if item is None or i == 41:
            out.append(item)
        else:
            out.append(torch.from_numpy(np.ascontiguousarray(item)).to(device))
    return tuple(out)


def host_cache(cache_t):
    return tuple(x.cpu().numpy() if torch.is_tensor(x) else x for x in cache_t)


def bits_equal(a, b, what):
    if a is None or b is None:
        assert a is None and b is None, f"{what}: one side is None"
        return
    a = a.cpu().numpy() if torch.is_tensor(a) else np.asarray(a)
    b = b.cpu().numpy() if torch.is_tensor(b) else np.asarray(b)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    assert a.dtype == b.dtype, f"{what}: dtype {a.dtype} vs {b.dtype}"
    if a.dtype == np.float16:
        a, b = a.view(np.uint16), b.view(np.uint16)
    bad = np.argwhere(a != b)
    assert bad.size == 0, f"{what}: {len(bad)} mismatches, first at {bad[0].tolist()}: {a[tuple(bad[0])]} vs {b[tuple(bad[0])]}"


@pytest.fixture(scope="module")
def ops(cuda_device):
    from hqekv_b200.model import public_func
    from hqekv_b200.quant import hqe_2, hqe_matmul, matmul, pack_unpack
    import types
    return types.SimpleNamespace(pu=pack_unpack, pf=public_func, hqe_2=hqe_2, hm=hqe_matmul, mm=matmul)


# ---------------------------------------------------------------------------------------------
# codec
# ---------------------------------------------------------------------------------------------
def test_codec_golden(ops, cuda_device):
    z = load_golden("codec")
    for n in range(int(z["count"])):
        bit, g, klike = (int(v) for v in z[f"c{n}_meta"])
        x = torch.from_numpy(z[f"c{n}_x"]).to(cuda_device)
        if klike:  # feed the transposed view of a token-major tensor, as the flush does for K
            x = x.transpose(2, 3).contiguous().transpose(2, 3)
        keep = x.clone()
        code, scale, mn = ops.pu.uniform_group_quantize_pack_last_dim(x, g, bit)
        assert torch.equal(x, keep), "quantiser modified its input"
        bits_equal(code, z[f"c{n}_code"], f"case {n} code (bit {bit} g {g} klike {klike})")
        bits_equal(scale, z[f"c{n}_scale"], f"case {n} scale")
        bits_equal(mn, z[f"c{n}_mn"], f"case {n} mn")
        deq = ops.pu.uniform_group_dequantize_unpack_last_dim(code, scale, mn, g, bit)
        bits_equal(deq, z[f"c{n}_deq"], f"case {n} dequantised")


@pytest.mark.parametrize("bit", [8, 4, 2, 1])
@pytest.mark.parametrize("group", [32, 64, 128])
def test_codec_random_vs_oracle(ops, cuda_device, bit, group):
    rng = np.random.default_rng(100 * bit + group)
    # row path, unaligned rows included (T = 3 groups), and the column (K) path
    x = (rng.standard_normal((2, 3, 7, 3 * group)) * 3).astype(np.float16)
    xt = torch.from_numpy(x).to(cuda_device)
    code, scale, mn = ops.pu.uniform_group_quantize_pack_last_dim(xt, group, bit)
    oc, os_, om = O.quantize_pack_last_dim(x, group, bit)
    bits_equal(code, oc, "row path code")
    bits_equal(scale, os_, "row path scale")
    bits_equal(mn, om, "row path mn")
    k = (rng.standard_normal((2, 2, 2 * group, 128)) * np.where(rng.random(128) < 0.05, 10, 1)).astype(np.float16)
    kt = torch.from_numpy(k).to(cuda_device).transpose(2, 3)
    code, scale, mn = ops.pu.uniform_group_quantize_pack_last_dim(kt, group, bit)
    oc, os_, om = O.quantize_pack_last_dim(np.ascontiguousarray(np.swapaxes(k, 2, 3)), group, bit)
    bits_equal(code, oc, "column path code")
    bits_equal(scale, os_, "column path scale")
    bits_equal(mn, om, "column path mn")
    deq = ops.pu.uniform_group_dequantize_unpack_last_dim(code, scale, mn, group, bit)
    bits_equal(deq, O.dequantize_unpack_last_dim(oc, os_, om, group, bit), "dequantised")


@pytest.mark.parametrize("bit", [8, 4, 2, 1])
def test_codec_column_path_ragged_tiles(ops, cuda_device, bit):
    """The tiled column kernel (groups of 32, tiles of 8 groups x 128 channels) on shapes that leave partial tiles
    both ways: 11 and 19 groups, 96 and 200 channels, several (batch, head) planes; bit-exact with the oracle."""
    rng = np.random.default_rng(300 + bit)
    for groups, ch in ((11, 96), (19, 200), (8, 128)):
        k = (rng.standard_normal((2, 3, 32 * groups, ch)) * np.where(rng.random(ch) < 0.05, 10, 1)).astype(np.float16)
        kt = torch.from_numpy(k).to(cuda_device).transpose(2, 3)
        code, scale, mn = ops.pu.uniform_group_quantize_pack_last_dim(kt, 32, bit)
        oc, os_, om = O.quantize_pack_last_dim(np.ascontiguousarray(np.swapaxes(k, 2, 3)), 32, bit)
        bits_equal(code, oc, f"{groups} groups x {ch} channels: code")
        bits_equal(scale, os_, f"{groups} groups x {ch} channels: scale")
        bits_equal(mn, om, f"{groups} groups x {ch} channels: mn")


def test_codec_constant_group_and_roundtrip(ops, cuda_device):
    x = torch.full((1, 1, 2, 64), 3.5, dtype=torch.float16, device=cuda_device)
    x[0, 0, 1, :32] = torch.arange(32, device=cuda_device).half()
    code, scale, mn = ops.pu.uniform_group_quantize_pack_last_dim(x, 32, 4)
    oc, os_, om = O.quantize_pack_last_dim(x.cpu().numpy(), 32, 4)
    bits_equal(code, oc, "constant-group code")
    bits_equal(scale, os_, "constant-group scale")
    rng = np.random.default_rng(5)
    for bit in (8, 4, 2, 1):
        codes = rng.integers(0, 2 ** bit, size=(2, 3, 4, 64), dtype=np.int32)
        words = ops.pu.pack_along_last_dim(torch.from_numpy(codes).to(cuda_device), bit)
        bits_equal(words, O.pack_last_dim(codes, bit), f"pack {bit}")
        back = ops.pu.unpack_along_last_dim(words, bit)
        bits_equal(back, codes.astype(np.float16), f"unpack {bit}")


def test_codec_full_size_roundtrip_property(ops, cuda_device):
    """At the benchmark's full flush size (32k tokens x 8 heads) the dequantised values must lie
    within about half a quantisation step of the input: 0.5 from the rounding to a code, up to 0.0625
    more because the quotient is itself rounded to fp16 before that (ulp 0.125 above 128), plus the
    two fp16 roundings of the dequantiser (about 1e-3 of |x| each)."""
    gen = torch.Generator(device=cuda_device).manual_seed(3)
    x = torch.randn(1, 8, 32640, 128, generator=gen, device=cuda_device).half()
    for bit in (8, 4, 2):
        code, scale, mn = ops.pu.uniform_group_quantize_pack_last_dim(x, 32, bit)
        deq = ops.pu.uniform_group_dequantize_unpack_last_dim(code, scale, mn, 32, bit)
        step = scale.float().repeat_interleave(32, dim=-1)
        err = (deq.float() - x.float()).abs()
        rng = step * (2 ** bit - 1)          # (x - mn) and code*scale reach the group's range: their fp16 ulp
        bound = 0.57 * step + 2e-3 * rng + 1e-3 * x.float().abs() + 1e-3
        assert bool((err <= bound).all()), f"bit {bit}: worst excess {(err - bound).max().item():.3e}"
        kt = x.transpose(2, 3)
        code_k, scale_k, mn_k = ops.pu.uniform_group_quantize_pack_last_dim(kt, 32, bit)
        code_c, scale_c, mn_c = ops.pu.uniform_group_quantize_pack_last_dim(kt.contiguous(), 32, bit)
        assert torch.equal(code_k, code_c) and torch.equal(scale_k, scale_c) and torch.equal(mn_k, mn_c)


# ---------------------------------------------------------------------------------------------
# importance ring, value range, block ranking
# ---------------------------------------------------------------------------------------------
def test_ring_and_ranking_golden(ops, cuda_device):
    z = load_golden("ranking")
    L = z["prefill_w"].shape[-1]
    ring = ops.pf.last_attn_weights()
    ring.set_max_length(L + 64)
    ring.update(torch.from_numpy(z["prefill_w"]).to(cuda_device))
    bits_equal(ring.weights, z["ring_after_prefill"], "ring after prefill")
    for s in range(5):
        ring.update(torch.from_numpy(z[f"step_w{s}"]).to(cuda_device))
    bits_equal(ring.weights, z["ring_after_steps"], "ring after steps")
    assert ring.next_line == int(z["ring_next_line"])
    imp = ring.calculate_token_importance()
    bits_equal(imp, z["importance"], "importance")
    work = imp[:L].clone()
    ids = ops.pf.get_block_token_idx(32, L // 32, work)
    bits_equal(ids, z["rank_ids"], "ranked ids")
    bits_equal(work, z["rank_importance_after"], "importance after the in-place divide")
    w = torch.from_numpy(z["imp2"]).to(cuda_device)
    bits_equal(ops.pf.get_block_token_idx(32, w.numel() // 32, w), z["rank2_ids"], "ranking with ties")
    bits_equal(w, z["rank2_after"], "rank2 importance")
    bits_equal(ops.pf.get_block_token_idx(32, w.numel() // 32, w), z["rank3_ids"], "ranking, second divide")
    bits_equal(ops.pf.calculate_token_range(torch.from_numpy(z["range_v"]).to(cuda_device), None), z["range_out"],
               "token range")


def test_ranking_full_size_properties(ops, cuda_device):
    """4088 blocks (the 128k-context case): output is a permutation, keys are non-increasing along it,
    equal keys keep ascending block order."""
    gen = torch.Generator(device=cuda_device).manual_seed(9)
    n = 4088
    imp = (torch.rand(n * 32, generator=gen, device=cuda_device) * 1e-4).half()
    ref = imp.clone().cpu().numpy()
    ids = ops.pf.get_block_token_idx(32, n, imp)
    want = O.block_rank(32, n, ref)
    bits_equal(ids, want, "ranking at 4088 blocks")
    bits_equal(imp, ref, "divided importance")


# ---------------------------------------------------------------------------------------------
# flush
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["flush_a", "flush_b", "flush_c", "flush_n", "flush_n64"])
def test_flush_golden_sequences(ops, cuda_device, name):
    """flush_n / flush_n64: quant_strategy 'high_uniform_group_low_normal_group' (1-bit tier in the
    Gaussian-codebook codec, fed from the residual and from every higher tier)."""
    z = load_golden(name)
    strategy = str(z["strategy"]) if "strategy" in z else "uniform_group"
    B, H, D, block, group, times_range, nsteps = (int(v) for v in z["meta"])
    cache = None
    for s in range(nsteps):
        cin = golden_cache(z, f"s{s}_in")
        if cache is None:
            cache = dev_cache(cin, cuda_device)
        else:  # carry our own tiers forward, take the grown residual window from the fixture
            cache = cache[:39] + dev_cache(cin, cuda_device)[39:]
        compress, hist = (int(v) for v in z[f"s{s}_args"])
        imp = torch.from_numpy(z[f"s{s}_importance_in"].copy()).to(cuda_device)
        ids = ops.pf.get_block_token_idx(block, (hist + compress) // block, imp)
        bits_equal(ids, z[f"s{s}_K_ids"], f"{name} step {s} K ids")
        ring = ops.pf.last_attn_weights()
        ring.weights = torch.from_numpy(z[f"s{s}_ring_in"].copy()).to(cuda_device)
        bn = torch.from_numpy(z[f"s{s}_bit_num"])
        cache = ops.hqe_2.KV_cache_hqe_2(cache, compress, hist, ids, bn, bn.clone(), imp, strategy, ring, block,
                                         group, bool(times_range))
        want = golden_cache(z, f"s{s}_out")
        for i in range(41):
            bits_equal(cache[i], want[i], f"{name} step {s} slot {i}")
        assert cache[41] == want[41]
        bits_equal(ring.weights, z[f"s{s}_ring_out"], f"{name} step {s} ring")
    K, V = ops.hqe_2.KV_cache_reconstruct_hqe(cache, strategy, block, group)
    oK, oV = O.reconstruct(host_cache(cache), block, group, strategy)
    bits_equal(K, oK, f"{name} reconstructed K")
    bits_equal(V, oV, f"{name} reconstructed V")


def test_normal_codec_1bit_golden(ops, cuda_device):
    """Gaussian-codebook codec at 1 bit: std, mean, packed codes and dequantised values bit for bit against
    the reference's output; row layout and the transposed (K) view."""
    z = load_golden("codec_normal")
    for n in range(int(z["count"])):
        bit, g, klayout = (int(v) for v in z[f"c{n}_meta"])
        x = torch.from_numpy(z[f"c{n}_x"]).to(cuda_device)
        if klayout:  # hand the kernel the transposed view of a token-major tensor, as the flush does
            x = x.transpose(2, 3).contiguous().transpose(2, 3)
        code, std, mean = ops.pu.normal_group_quantize_pack_last_dim(x, g, 1)
        bits_equal(std, z[f"c{n}_std"], f"normal case {n} std")
        bits_equal(mean, z[f"c{n}_mean"], f"normal case {n} mean")
        bits_equal(code, z[f"c{n}_code"], f"normal case {n} codes")
        deq = ops.pu.normal_group_dequantize_unpack_last_dim(code, std, mean, g, 1)
        bits_equal(deq, z[f"c{n}_deq"], f"normal case {n} dequantised")
    # random cross-check against the oracle at a larger size
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((2, 3, 64, 256)) * 2 + 0.5).astype(np.float16)
    oc, os_, om = O.normal1_quantize_pack_last_dim(x, 64)
    code, std, mean = ops.pu.normal_group_quantize_pack_last_dim(torch.from_numpy(x).to(cuda_device), 64, 1)
    bits_equal(std, os_, "normal random std"); bits_equal(mean, om, "normal random mean"); bits_equal(code, oc, "normal random codes")
    with pytest.raises(NotImplementedError):
        ops.pu.normal_group_quantize_pack_last_dim(torch.from_numpy(x).to(cuda_device), 64, 2)


def test_flush_errors(ops, cuda_device):
    k = torch.zeros(1, 1, 32, 128, dtype=torch.float16, device=cuda_device)
    cache = (None,) * 39 + (k, k.clone(), 32)
    imp = torch.zeros(32, dtype=torch.float16, device=cuda_device)
    ids = torch.arange(32, device=cuda_device)
    with pytest.raises(ValueError, match="invalid quant_strategy"):
        ops.hqe_2.KV_cache_hqe_2(cache, 32, 0, ids, [0, 32, 0, 0, 0, 0], [0, 32, 0, 0, 0, 0], imp, "bogus")
    with pytest.raises(NotImplementedError):
        ops.hqe_2.KV_cache_hqe_2(cache, 32, 0, ids, [0, 32, 0, 0, 0, 0], [0, 32, 0, 0, 0, 0], imp, "normal_group")
    with pytest.raises(ValueError, match="invalid past_key_value"):
        ops.hqe_2.KV_cache_hqe_2(cache[:41], 32, 0, ids, [0, 32, 0, 0, 0, 0], [0, 32, 0, 0, 0, 0], imp, "uniform_group")


# ---------------------------------------------------------------------------------------------
# decode attention
# ---------------------------------------------------------------------------------------------
def check_attention(ops, cache_t, q, block, group, what, strategy="uniform_group"):
    w, out = ops.hm.qkv_matmul_hqe_2(q, cache_t, None, q.shape[-1], strategy, block, group)
    torch.cuda.synchronize()
    ow, oo = O.decode_attention(q.cpu().numpy(), host_cache(cache_t), None, block, group, quant_strategy=strategy)
    out_f = out.float().cpu().numpy()
    assert out_f.shape == oo.shape and w.shape == ow.shape, what
    assert np.isfinite(out_f).all(), f"{what}: non-finite output"
    per_head = np.abs(out_f - oo).max(axis=-1) / np.abs(oo).max(axis=-1)
    assert per_head.max() <= ATTN_REL_TOL, f"{what}: attention output rel err {per_head.max():.3e} > {ATTN_REL_TOL}"
    w_f = w.float().cpu().numpy()
    werr = np.abs(w_f - ow)
    excess = werr - (WEIGHT_ABS_TOL + WEIGHT_REL_TOL * ow)
    k = int(excess.argmax())
    assert excess.flat[k] <= 0, \
        f"{what}: probability {w_f.flat[k]:.6e} vs oracle {ow.flat[k]:.6e} (error {werr.flat[k]:.3e}, allowed " \
        f"{WEIGHT_ABS_TOL + WEIGHT_REL_TOL * ow.flat[k]:.3e}); largest error {werr.max():.3e} at p={ow.flat[werr.argmax()]:.3e}"
    assert abs(w_f.sum(-1) - 1).max() < 2e-2, f"{what}: probabilities do not sum to 1"
    MEASURED["attn_rel"] = max(MEASURED["attn_rel"], float(per_head.max()))
    MEASURED["weight_rel"] = max(MEASURED["weight_rel"], float((np.maximum(werr - WEIGHT_ABS_TOL, 0) / np.maximum(ow, 1e-30)).max()))
    return per_head.max()


@pytest.mark.parametrize("name", ["flush_a", "flush_b", "flush_c", "flush_n", "flush_n64"])
def test_decode_on_golden_caches(ops, cuda_device, name):
    """Every flush step of the fixtures gives a cache with a different set of present/absent tiers (the
    uniform 1-bit tier included), K and V ranked differently (flush_a/c), batch 2 (flush_b), group 64
    (flush_c); flush_n / flush_n64 hold the 1-bit tier in the Gaussian-codebook codec."""
    z = load_golden(name)
    strategy = str(z["strategy"]) if "strategy" in z else "uniform_group"
    B, H, D, block, group, _, nsteps = (int(v) for v in z["meta"])
    gen = torch.Generator(device=cuda_device).manual_seed(1)
    for s in range(nsteps):
        cache_np = golden_cache(z, f"s{s}_out")
        for rep in (1, 4, 8):
            q = torch.randn(B, rep * H, 1, D, generator=gen, device=cuda_device).half()
            check_attention(ops, dev_cache(cache_np, cuda_device), q, block, group, f"{name} step {s} rep {rep}", strategy)
        # the reference's own qkv_matmul_hqe_2 on this cache (fixture: fp16 intermediates, fp32-accumulating CPU
        # stand-in for its GEMV extension): agreement to the accuracy of that fp16 flow (5e-3 of the largest output)
        q = torch.from_numpy(z[f"s{s}_q"]).to(cuda_device)
        w, out = ops.hm.qkv_matmul_hqe_2(q, dev_cache(cache_np, cuda_device), None, D, strategy, block, group)
        ro = z[f"s{s}_attn_output"].astype(np.float32)
        got = out.float().cpu().numpy()
        assert (np.abs(got - ro).max(-1) <= 5e-3 * np.abs(ro).max(-1)).all(), f"{name} step {s}: vs reference decode output"
        assert np.abs(w.float().cpu().numpy() - z[f"s{s}_attn_weights"].astype(np.float32)).max() <= 2.5e-3


def test_decode_cfg0_vs_oracle(ops, cuda_device):
    """Single-layer Llama-3.1-8B-shaped case: ctx 4096, 32/8 heads, group 32, 10 % evicted, 25/50/25 % in
    the 8/4/2-bit tiers, residual 128, K with outlier channels."""
    from hqekv_b200 import synthetic
    cfg = synthetic.CONFIGS["cfg0"]
    for times_range in (False, True):
        cache, q = synthetic.build_cache(cfg, cuda_device, seed=0, times_range=times_range)
        assert synthetic.logical_length(cache) == 4096 - 12 * 32
        err = check_attention(ops, cache, q, cfg.group, cfg.group, f"cfg0 times_range={times_range}")
        # twice in a row: the scratch counters must be left clean
        w1, o1 = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", cfg.group, cfg.group)
        w2, o2 = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", cfg.group, cfg.group)
        assert torch.equal(o1, o2) and torch.equal(w1, w2), "decode is not deterministic call to call"


def test_decode_cfg0_flush_matches_oracle_flush(ops, cuda_device):
    """The cache that the CUDA flush builds for cfg0 equals the oracle's flush of the same inputs."""
    from hqekv_b200 import synthetic
    cfg = synthetic.CONFIGS["cfg0"]
    K, V, q = synthetic.make_kv(cfg, cuda_device, 0)
    flushed = cfg.context - cfg.residual
    counts = synthetic.tier_counts(cfg)
    imp = synthetic.synthetic_importance(cfg, cuda_device, 0, flushed, K)
    imp_np = imp.cpu().numpy().copy()
    ids = ops.pf.get_block_token_idx(cfg.group, flushed // cfg.group, imp)
    ids_np = O.block_rank(cfg.group, flushed // cfg.group, imp_np)
    bits_equal(ids, ids_np, "cfg0 ranked ids")
    cache = (None,) * 39 + (K, V, cfg.context)
    got = ops.hqe_2.KV_cache_hqe_2(cache, flushed, 0, ids, counts, list(counts), imp, "uniform_group", None, 32, 32, True)
    want = O.flush(host_cache(cache), flushed, 0, ids_np, np.array(counts), np.array(counts), imp_np, "uniform_group",
                   None, 32, 32, True)
    for i in range(41):
        bits_equal(got[i], want[i], f"cfg0 flush slot {i}")


def test_decode_full_size_properties(ops, cuda_device):
    """Llama-3.1-8B at 32k context (one layer of the benchmark workload): the fused decode must agree
    with fp32 attention over the dense reconstruction of the same cache, computed with torch on the
    GPU (the reconstruction's dequantiser is pinned bit-exactly above), within the same 2e-3."""
    from hqekv_b200 import synthetic
    cfg = synthetic.CONFIGS["cfg1"]
    cache, q = synthetic.build_cache(cfg, cuda_device, seed=1)
    L = synthetic.logical_length(cache)
    assert L == 32768 - 102 * 32
    w, out = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", 32, 32)
    Kd, Vd = ops.hqe_2.KV_cache_reconstruct_hqe(cache, "uniform_group", 32, 32)
    qf = q.float().view(1, 8, 4, 128)
    logits = torch.matmul(qf, Kd.float().transpose(2, 3)) / (128 ** 0.5)
    p = torch.softmax(logits, dim=-1)
    ref = torch.matmul(p, Vd.float()).view(1, 32, 1, 128)
    rel = ((out.float() - ref).abs().amax(-1) / ref.abs().amax(-1)).max().item()
    assert rel <= ATTN_REL_TOL, f"32k decode rel err {rel:.3e}"
    pw = p.view(1, 32, 1, L)
    # (this reference dequantises K to fp16 with two roundings, which moves a logit by ~1e-3: the bound on the
    # probabilities is the looser one that goes with it; the one-ulp bound is checked against the fp32 oracle)
    assert bool(((w.float() - pw).abs() <= WEIGHT_ABS_TOL + 1e-2 * pw).all())


def test_decode_cfg1_layer_vs_oracle(ops, cuda_device):
    """One layer of the benchmark workload (Llama-3.1-8B shape, 29 504 cached tokens, 8 kv heads) against the
    numpy oracle itself - fp32 dequantisation, fp32 attention - at the same 2e-3 / one-ulp bounds."""
    from hqekv_b200 import synthetic
    cfg = synthetic.CONFIGS["cfg1"]
    cache, q = synthetic.build_cache(cfg, cuda_device, seed=2)
    check_attention(ops, cache, q, cfg.group, cfg.group, "cfg1 layer vs oracle")


def test_decode_cfg2_heads_vs_oracle(ops, cuda_device):
    """The batch-8 configuration (Qwen3-8B shape: context 16384, group 64, no eviction, 25/50/25 % in 8/4/2 bit, K
    with outlier channels) on two of its kv heads (eight query heads), against the numpy oracle."""
    from hqekv_b200 import synthetic
    c2 = synthetic.CONFIGS["cfg2"]
    cfg = synthetic.CacheConfig("cfg2-two-heads", c2.batch, 8, 2, 128, c2.context, c2.residual, c2.ratios, c2.evict,
                                c2.group, c2.k_outliers, 1)
    cache, q = synthetic.build_cache(cfg, cuda_device, seed=4, times_range=True)
    assert synthetic.logical_length(cache) == 16384
    check_attention(ops, cache, q, cfg.group, cfg.group, "cfg2 two heads vs oracle")


def test_decode_batch64_vs_oracle(ops, cuda_device):
    """Batch 64 x 8 kv heads = 512 (batch, kv head) pairs (the largest batch of the kernel sweep), context 1024."""
    from hqekv_b200 import synthetic
    cfg = synthetic.CacheConfig("sweep-b64", 64, 32, 8, 128, 1024 + 24, 24, (0.25, 0.5, 0.25), 0.0, 32, True, 1)
    cache, q = synthetic.build_cache(cfg, cuda_device, seed=6)
    check_attention(ops, cache, q, 32, 32, "batch 64")


def test_decode_errors(ops, cuda_device):
    q = torch.zeros(1, 4, 1, 128, dtype=torch.float16, device=cuda_device)
    with pytest.raises(ValueError, match="invalid quant_strategy"):
        ops.hm.qkv_matmul_hqe_2(q, (None,) * 42, None, 128, "bogus")
    with pytest.raises(ValueError, match="invalid past_key_value"):
        ops.hm.qkv_matmul_hqe_2(q, (None,) * 42, None, 128, "uniform_group")


# ---------------------------------------------------------------------------------------------
# stand-alone GEMV
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("bits", [8, 4, 2, 1])
def test_gemv_uniform_group_vs_oracle(ops, cuda_device, bits):
    """Both uses of cuda_bmm_fA_qB_uniform_group: q.K^T of a tier (K = head_dim rows, N = tokens) and
    p.V of a tier (K = tokens, N = head_dim).  Tolerance: 2e-3 of the largest output (fp16 result)."""
    rng = np.random.default_rng(bits)
    for (K, N, g) in ((128, 32 * 9, 32), (32 * 7, 128, 32), (128, 128, 64)):
        x = rng.standard_normal((2, 2, K, N)).astype(np.float16)
        code, scale, mn = O.quantize_pack_last_dim(x, g, bits)
        fA = rng.standard_normal((2, 8, 1, K)).astype(np.float16)
        want = O.gemv_dequant(fA, code, scale, mn, g, bits)
        got = ops.mm.cuda_bmm_fA_qB_uniform_group(g, *(torch.from_numpy(a).to(cuda_device) for a in (fA, code, scale, mn)),
                                                  bits)
        err = np.abs(got.float().cpu().numpy() - want).max() / np.abs(want).max()
        assert err <= 2e-3, f"gemv bits {bits} K {K} N {N}: rel err {err:.3e}"


@pytest.mark.parametrize("rep", [1, 4, 8])
def test_gemv_normal_group_vs_oracle(ops, cuda_device, rep):
    """cuda_bmm_fA_qB_normal_group at 1 bit (Gaussian codebook), both operand shapes, GQA 1 / 4 / 8."""
    rng = np.random.default_rng(40 + rep)
    for (K, N, g) in ((128, 32 * 9, 32), (32 * 7, 128, 32), (128, 128, 64), (64, 256, 128)):
        x = (rng.standard_normal((2, 2, K, N)) * 1.5 + 0.25).astype(np.float16)
        code, std, mean = O.normal1_quantize_pack_last_dim(x, g)
        fA = rng.standard_normal((2, 2 * rep, 1, K)).astype(np.float16)
        want = O.gemv_dequant_normal1(fA, code, std, mean, g)
        got = ops.mm.cuda_bmm_fA_qB_normal_group(g, *(torch.from_numpy(a).to(cuda_device) for a in (fA, code, std, mean)), 1)
        err = np.abs(got.float().cpu().numpy() - want).max() / np.abs(want).max()
        assert err <= 2e-3, f"normal gemv rep {rep} K {K} N {N}: rel err {err:.3e}"
    with pytest.raises(NotImplementedError):
        ops.mm.cuda_bmm_fA_qB_normal_group(32, *(torch.from_numpy(a).to(cuda_device) for a in (fA, code, std, mean)), 2)


# ---------------------------------------------------------------------------------------------
# sweep: uniform and mixed tiers x group size x batch x GQA ratio (shapes of the kernel microbench)
# ---------------------------------------------------------------------------------------------
SWEEP_RATIOS = {"all8": (1.0, 0.0, 0.0), "all4": (0.0, 1.0, 0.0), "all2": (0.0, 0.0, 1.0), "mixed": (0.25, 0.5, 0.25),
                "all1": (0.0, 0.0, 0.0, 1.0), "mixed1": (0.25, 0.25, 0.25, 0.25)}


@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("tiers", ["all8", "all4", "all2", "mixed", "all1", "mixed1"])
def test_decode_sweep_vs_oracle(ops, cuda_device, tiers, group):
    """Context 1024 + a ragged residual, batch 1 and 3, GQA 4 and 8, K with outlier channels, K and V
    ranked differently (times_range): the fused decode against the fp32 oracle, tolerance 2e-3."""
    from hqekv_b200 import synthetic
    for batch, nh_q, nh_kv, evict in ((1, 32, 8, 0.0), (3, 16, 2, 0.125)):
        cfg = synthetic.CacheConfig(f"sweep-{tiers}-g{group}", batch, nh_q, nh_kv, 128, 1024 + 40, 40,
                                    SWEEP_RATIOS[tiers], evict, group, True, 1)
        cache, q = synthetic.build_cache(cfg, cuda_device, seed=group + batch, times_range=True)
        check_attention(ops, cache, q, group, group, f"{cfg.name} B{batch} {nh_q}/{nh_kv}")


@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("tiers", ["all1", "mixed1"])
def test_decode_normal_low_tier_vs_oracle(ops, cuda_device, tiers, group):
    """quant_strategy 'high_uniform_group_low_normal_group': the 1-bit tier (all of the cache, or a quarter of
    it beside 8/4/2-bit tiers) in the Gaussian-codebook codec, written by the flush and read by the fused
    decode; flushed tiers bit for bit against the oracle's flush, attention against the fp32 oracle at 2e-3."""
    from hqekv_b200 import synthetic
    strategy = "high_uniform_group_low_normal_group"
    for batch, nh_q, nh_kv, evict in ((1, 32, 8, 0.0), (3, 16, 2, 0.125), (2, 2, 2, 0.0)):
        cfg = synthetic.CacheConfig(f"normal-{tiers}-g{group}", batch, nh_q, nh_kv, 128, 1024 + 40, 40,
                                    SWEEP_RATIOS[tiers], evict, group, True, 1)
        cache, q = synthetic.build_cache(cfg, cuda_device, seed=group + batch, times_range=True, quant_strategy=strategy)
        assert cache[28] is not None and cache[32] is not None
        Kd, Vd = ops.hqe_2.KV_cache_reconstruct_hqe(cache, strategy, group, group)
        oK, oV = O.reconstruct(host_cache(cache), group, group, strategy)
        bits_equal(Kd, oK, f"{cfg.name} reconstructed K")
        bits_equal(Vd, oV, f"{cfg.name} reconstructed V")
        check_attention(ops, cache, q, group, group, f"{cfg.name} B{batch} {nh_q}/{nh_kv}", strategy)
    # the same 1-bit payload read as a uniform tier gives a different answer: the codec flag is honoured
    w_u, o_u = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", group, group)
    w_n, o_n = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, strategy, group, group)
    assert not torch.equal(o_u, o_n)


@pytest.mark.parametrize("case", [
    # name, batch, nh_q, nh_kv, context, residual, ratios (8/4/2/1-bit), evict, group
    ("one-block-per-tier", 1, 8, 2, 4 * 32 + 5, 5, (0.25, 0.25, 0.25, 0.25), 0.0, 32),
    ("single-8bit-block-ragged-residual", 2, 4, 2, 32 + 7, 7, (1.0, 0.0, 0.0), 0.0, 32),
    ("gqa-2", 1, 8, 4, 640 + 33, 33, (0.2, 0.4, 0.4), 0.1, 32),
    ("mha", 2, 4, 4, 512 + 16, 16, (0.25, 0.5, 0.25), 0.0, 64),
    ("many-heads-short", 32, 32, 8, 160 + 1, 1, (0.2, 0.4, 0.4), 0.0, 32),
    ("group128-tiles-straddle-groups", 1, 32, 8, 128 * 9 + 100, 100, (0.34, 0.33, 0.33), 0.0, 128),
])
def test_decode_edge_shapes(ops, cuda_device, case):
    """Shapes at the edges of the tiling: tiers of a single block, a residual of 1..100 tokens, GQA ratios 1 and
    2, 256 (batch, kv head) pairs, tiles that cover part of a 128-token scale group.  Against the fp32 oracle."""
    from hqekv_b200 import synthetic
    name, batch, nh_q, nh_kv, ctx, res, ratios, evict, group = case
    cfg = synthetic.CacheConfig(name, batch, nh_q, nh_kv, 128, ctx, res, ratios, evict, group, True, 1)
    cache, q = synthetic.build_cache(cfg, cuda_device, seed=7, times_range=True)
    check_attention(ops, cache, q, group, group, name)


def test_decode_long_context_shard_properties(ops, cuda_device):
    """One kv head of the 128k-context case (what one of 8 GPUs holds per head, batch 1): 10/25/65 % in
    8/4/2-bit, 30 % evicted, residual 256.  Checked against torch fp32 attention over the dense
    reconstruction on the GPU, tolerance 2e-3; the probabilities must sum to 1."""
    from hqekv_b200 import synthetic
    cfg = synthetic.CONFIGS["cfg3"]
    cfg1 = synthetic.CacheConfig("cfg3-one-head", 1, 4, 1, 128, cfg.context, cfg.residual, cfg.ratios, cfg.evict,
                                 cfg.group, False, 1)
    cache, q = synthetic.build_cache(cfg1, cuda_device, seed=3)
    L = synthetic.logical_length(cache)
    assert L == 131072 - 1226 * 32
    w, out = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", 32, 32)
    Kd, Vd = ops.hqe_2.KV_cache_reconstruct_hqe(cache, "uniform_group", 32, 32)
    logits = torch.matmul(q.float().view(1, 1, 4, 128), Kd.float().transpose(2, 3)) / (128 ** 0.5)
    p = torch.softmax(logits, dim=-1)
    ref = torch.matmul(p, Vd.float()).view(1, 4, 1, 128)
    rel = ((out.float() - ref).abs().amax(-1) / ref.abs().amax(-1)).max().item()
    assert rel <= ATTN_REL_TOL, f"128k decode rel err {rel:.3e}"
    assert (w.float().sum(-1) - 1).abs().max().item() < 2e-2


# ---------------------------------------------------------------------------------------------
# the attention layer around the cache
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["attn_llama_n", "attn_llama_u"])
def test_attention_layer_against_reference_layer(ops, cuda_device, name):
    """HqeAttention with the reference layer's weights on the reference layer's inputs: prefill, then one token
    per call, flushing whenever 32 tokens are unquantised.  Exact: the tier counts of every flush, the lengths
    and the size of every tier after every call (so the same blocks were ranked into the same tiers, evicted
    blocks included).  Layer output: 1e-2 of the largest output of the call (fp16 GEMMs on different hardware,
    and the reference's decode rounds per-tier logits to fp16)."""
    from hqekv_b200.model.attention_hqe import HqeAttention, rotary_tables, causal_mask
    z = load_golden(name)
    B, hidden, nh, nkv, prefill, steps = (int(v) for v in z["meta"])
    attn = HqeAttention(hidden, nh, nkv, 128, str(z["strategy"]), True, *(float(v) for v in z["shares"]))
    with torch.no_grad():
        for pname in ("q_proj", "k_proj", "v_proj", "o_proj"):
            getattr(attn, pname).weight.copy_(torch.from_numpy(z[f"w_{pname}"]).float())
    attn = attn.half().to(cuda_device)
    attn.set_max_length(prefill + steps)
    cache, pos, worst = None, 0, 0.0
    with torch.no_grad():
        for call in range(steps + 1):
            S = prefill if call == 0 else 1
            x = torch.from_numpy(z[f"c{call}_x"]).to(cuda_device)
            cos, sin = rotary_tables(torch.arange(pos, pos + S).unsqueeze(0).expand(B, S), 128, 10000.0)
            mask = causal_mask(S, S, torch.float16, cuda_device) if call == 0 else None
            y, _, cache, aux = attn(x, (cos.to(cuda_device), sin.to(cuda_device)), mask, cache, None)
            pos += S
            if f"c{call}_bit_num" in z.files:
                assert aux is not None and np.array_equal(aux[1].cpu().numpy(), z[f"c{call}_bit_num"]), f"{name} call {call}"
            else:
                assert aux is None
            sizes = [0 if cache[i] is None else cache[i].numel() for i in (1, 5, 13, 21, 29, 3, 9, 17, 25, 33)]
            state = [attn.current_length, attn.history_reserve_length, cache[41]] + sizes
            assert state == [int(v) for v in z[f"c{call}_state"]], f"{name} call {call}: state {state}"
            want = z[f"c{call}_y"].astype(np.float32)
            err = np.abs(y.float().cpu().numpy() - want).max() / np.abs(want).max()
            worst = max(worst, err)
            assert err <= 1e-2, f"{name} call {call}: layer output rel err {err:.3e}"
    assert cache[28] is not None or cache[20] is not None


def test_decoder_stack_shares_tier_counts_and_matches_dense_attention(ops, cuda_device):
    """Two-layer decoder (Qwen3 flavour: q/k RMSNorm) on the tiered cache: every layer flushes with the first
    layer's tier counts, the caches account for every position, and a decode step's attention equals dense fp32
    attention over the reconstructed cache of that layer (2e-3)."""
    from hqekv_b200.model.decoder import DecoderConfig, HqeDecoder, init_like_pretrained
    cfg = DecoderConfig(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=2, num_kv_heads=1, qk_norm=True,
                        rope_theta=10000.0)
    model = init_like_pretrained(HqeDecoder(cfg).half().to(cuda_device), 3).eval()
    gen = torch.Generator(device=cuda_device).manual_seed(5)
    ctx, steps, B = 300, 70, 2
    model.start_sequence(ctx + steps)
    with torch.no_grad():
        h, caches = model(torch.randn(B, ctx, 256, generator=gen, device=cuda_device).half(), None, 0)
        row = h[:, -1:, :]
        for s in range(steps):
            row, caches = model(row, caches, ctx + s)
            assert torch.isfinite(row).all()
    a0, a1 = model.layers[0].self_attn, model.layers[1].self_attn
    assert (a0.current_length, a0.history_reserve_length) == (a1.current_length, a1.history_reserve_length)
    for c, a in zip(caches, (a0, a1)):
        sizes_k = sum(0 if c[i] is None else c[i].numel() for i in (1, 5, 13, 21, 29))
        sizes_v = sum(0 if c[i] is None else c[i].numel() for i in (3, 9, 17, 25, 33))
        assert sizes_k == sizes_v == a.history_reserve_length and c[39].shape[2] == a.current_length
        assert c[41] == ctx + steps
    assert a0.history_reserve_length < ctx + steps - a0.current_length          # something was evicted
    assert caches[0][28] is not None                                            # the Gaussian-codebook tier is in use
    # the same steps with the dense parts replayed from CUDA graphs: a twin model is fed the eager model's rows
    # step by step (the recurrence through random weights amplifies rounding noise, so the runs are compared
    # call by call, not after 70 free-running steps)
    import copy
    from hqekv_b200.model.decoder import GraphedDecodeStep
    twin = copy.deepcopy(model)
    for m in (model, twin):
        m.start_sequence(ctx + steps)
    gen2 = torch.Generator(device=cuda_device).manual_seed(5)
    with torch.no_grad():
        x0 = torch.randn(B, ctx, 256, generator=gen2, device=cuda_device).half()
        h, caches = model(x0, None, 0)
        _, caches_g = twin(x0, None, 0)
        step = GraphedDecodeStep(twin, B)
        row = h[:, -1:, :]
        for s in range(steps):
            nxt, caches = model(row, caches, ctx + s)
            nxt_g, caches_g = step(row, caches_g, ctx + s)
            err = (nxt_g.float() - nxt.float()).abs().max() / nxt.float().abs().max()
            assert err <= 1e-2, f"graphed decode step {s}: rel err {err:.3e}"
            row = nxt
    for cg, ce in zip(caches_g, caches):
        assert [None if t is None else tuple(t.shape) for t in cg[:41]] == [None if t is None else tuple(t.shape) for t in ce[:41]]
    # one more attention call on layer 1's cache against dense attention over its reconstruction
    q = torch.randn(B, 2, 1, 128, generator=gen, device=cuda_device).half()
    check_attention(ops, caches[1], q, 32, 32, "decoder layer 1 cache", cfg.quant_strategy)



def test_zz_report_measured_maxima():
    """Not a check of its own: prints the largest errors the decode checks of this module measured (run with -s
    to see them) and asserts they are within the documented bounds."""
    print(f"\nmeasured maxima: attention output rel err {MEASURED['attn_rel']:.3e} (bound {ATTN_REL_TOL}), "
          f"probability rel err beyond the subnormal quantum {MEASURED['weight_rel']:.3e} (bound {WEIGHT_REL_TOL:.3e})")
    assert MEASURED["attn_rel"] <= ATTN_REL_TOL and MEASURED["weight_rel"] <= WEIGHT_REL_TOL
