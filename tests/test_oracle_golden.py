"""Pin the numpy oracle against outputs of the reference's own code (tests/golden/*.npz,
produced by tests/golden/make_golden.py).  Everything here is bit-exact."""
import numpy as np
import pytest

from conftest import golden_cache, load_golden
from oracle import hqkv_oracle as O


def same(a, b, what=""):
    if a is None or b is None:
        assert a is None and b is None, f"{what}: one side is None"
        return
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    assert a.dtype == b.dtype, f"{what}: dtype {a.dtype} vs {b.dtype}"
    if a.dtype.kind == "f":
        assert np.array_equal(a.view(np.uint16 if a.dtype == np.float16 else np.uint32),
                              b.view(np.uint16 if b.dtype == np.float16 else np.uint32)), f"{what}: bits differ"
    else:
        assert np.array_equal(a, b), f"{what}: values differ"


def test_codec_known_answers():
    z = load_golden("codec")
    for n in range(int(z["count"])):
        bit, g, _ = z[f"c{n}_meta"]
        x = z[f"c{n}_x"]
        code, scale, mn = O.quantize_pack_last_dim(x, int(g), int(bit))
        same(code, z[f"c{n}_code"], f"case {n} code")
        same(scale, z[f"c{n}_scale"], f"case {n} scale")
        same(mn, z[f"c{n}_mn"], f"case {n} mn")
        same(O.dequantize_unpack_last_dim(code, scale, mn, int(g), int(bit)), z[f"c{n}_deq"], f"case {n} deq")


def test_pack_unpack_roundtrip():
    rng = np.random.default_rng(0)
    for bit in (8, 4, 2, 1):
        codes = rng.integers(0, 2 ** bit, size=(3, 5, 64), dtype=np.int32)
        words = O.pack_last_dim(codes, bit)
        assert words.dtype == np.int32 and words.shape == (3, 5, 64 * bit // 32)
        assert np.array_equal(O.unpack_last_dim(words, bit).astype(np.int32), codes)


def test_constant_group_gives_code_zero():
    x = np.full((1, 1, 1, 32), 3.5, dtype=np.float16)
    code, scale, mn = O.quantize_pack_last_dim(x, 32, 4)
    assert scale[0, 0, 0, 0] == 0 and mn[0, 0, 0, 0] == np.float16(3.5)
    assert not code.any()


def test_importance_ring_and_ranking():
    z = load_golden("ranking")
    L = z["prefill_w"].shape[-1]
    ring = O.ImportanceRing()
    ring.set_max_length(L + 64)
    ring.update(z["prefill_w"])
    same(ring.weights, z["ring_after_prefill"], "ring after prefill")
    for s in range(5):
        ring.update(z[f"step_w{s}"])
    same(ring.weights, z["ring_after_steps"], "ring after steps")
    assert ring.next_line == int(z["ring_next_line"])
    imp = ring.calculate_token_importance()
    same(imp, z["importance"], "importance")
    work = imp[:L].copy()
    ids = O.block_rank(32, L // 32, work)
    same(ids, z["rank_ids"], "ranked ids")
    same(work, z["rank_importance_after"], "importance after in-place divide")


def test_ranking_with_subnormal_keys_and_ties():
    z = load_golden("ranking")
    w = z["imp2"].copy()
    same(O.block_rank(32, w.size // 32, w), z["rank2_ids"], "rank2")
    same(w, z["rank2_after"], "rank2 importance")
    same(O.block_rank(32, w.size // 32, w), z["rank3_ids"], "rank3 (second divide)")


def test_token_range_and_make_sum_equal():
    z = load_golden("ranking")
    same(O.token_range(z["range_v"]), z["range_out"], "token range")
    same(O.make_sum_equal(z["mse_in"].copy(), 20), z["mse_out"], "make_sum_equal")


@pytest.mark.parametrize("name", ["flush_a", "flush_b", "flush_c", "flush_n", "flush_n64"])
def test_flush_sequence(name):
    z = load_golden(name)
    strategy = str(z["strategy"]) if "strategy" in z else "uniform_group"
    B, H, D, block, group, times_range, nsteps = (int(v) for v in z["meta"])
    cache = None
    for s in range(nsteps):
        cin = golden_cache(z, f"s{s}_in")
        if cache is not None:                      # the oracle's own previous output feeds the next flush
            for i in range(39):
                same(cache[i], cin[i], f"{name} step {s} carried slot {i}")
        compress, hist = (int(v) for v in z[f"s{s}_args"])
        imp = z[f"s{s}_importance_in"].copy()
        ids = O.block_rank(block, (hist + compress) // block, imp)
        same(ids, z[f"s{s}_K_ids"], f"{name} step {s} K ids")
        same(imp, z[f"s{s}_importance_ranked"], f"{name} step {s} ranked importance")
        ring = O.ImportanceRing()
        ring.weights = z[f"s{s}_ring_in"].copy()
        cache = O.flush(cin, compress, hist, ids, z[f"s{s}_bit_num"], z[f"s{s}_bit_num"].copy(), imp,
                        strategy, ring, block, group, bool(times_range))
        want = golden_cache(z, f"s{s}_out")
        for i in range(41):
            same(cache[i], want[i], f"{name} step {s} slot {i}")
        assert cache[41] == want[41]
        same(ring.weights, z[f"s{s}_ring_out"], f"{name} step {s} ring")
        same(imp, z[f"s{s}_importance_after"], f"{name} step {s} importance after flush")
    K, V = O.reconstruct(cache, block, group, strategy)
    same(K, z["recon_K"], f"{name} reconstructed K")
    want_V = z["recon_V"].copy()
    if cache[8] is None and cache[16] is not None:
        # quant/hqe_2.py:1060 guards the 4-bit V scatter with "eight_V is not None", so the
        # reference leaves those rows zero when the 8-bit tier is empty; the oracle fills them.
        assert not want_V[:, :, cache[17], :].any()
        want_V[:, :, cache[17], :] = V[:, :, cache[17], :]
    same(V, want_V, f"{name} reconstructed V")


def test_flush_rejects_unknown_strategy():
    with pytest.raises(ValueError, match="invalid quant_strategy"):
        O.flush((None,) * 42, 0, 0, None, None, None, None, "nope")


def test_normal_codec_1bit_matches_reference_fixtures():
    """Gaussian-codebook codec at 1 bit (std / mean / codes / dequantised values) against the reference's output."""
    z = load_golden("codec_normal")
    assert np.array_equal(z["center_f32"], O.NORMAL1_CENTER) and z["upper_f32"][0] == 0 and np.isinf(z["upper_f32"][1])
    for n in range(int(z["count"])):
        bit, g, _ = (int(v) for v in z[f"c{n}_meta"])
        assert bit == 1
        code, std, mean = O.normal1_quantize_pack_last_dim(z[f"c{n}_x"], g)
        assert np.array_equal(std.view(np.uint16), z[f"c{n}_std"].view(np.uint16)), f"case {n}: std"
        assert np.array_equal(mean.view(np.uint16), z[f"c{n}_mean"].view(np.uint16)), f"case {n}: mean"
        assert np.array_equal(code, z[f"c{n}_code"]), f"case {n}: packed codes"
        deq = O.normal1_dequantize_unpack_last_dim(code, std, mean, g)
        assert np.array_equal(deq.view(np.uint16), z[f"c{n}_deq"].view(np.uint16)), f"case {n}: dequantised"


@pytest.mark.parametrize("name", ["flush_n", "flush_n64"])
def test_decode_oracle_reads_normal_low_tier(name):
    """The fp32 decode oracle under 'high_uniform_group_low_normal_group': dequantising the 1-bit tier in
    registers (float32 centres) and attending over the reference's own dense reconstruction agree to fp16
    accuracy, and reading the same payload as a uniform tier does not."""
    z = load_golden(name)
    B, H, D, block, group, _, nsteps = (int(v) for v in z["meta"])
    strategy = str(z["strategy"])
    cache = golden_cache(z, f"s{nsteps - 1}_out")
    assert cache[28] is not None and cache[32] is not None
    rng = np.random.default_rng(3)
    q = rng.standard_normal((B, 4 * H, 1, D)).astype(np.float16)
    w32, o32 = O.decode_attention(q, cache, None, block, group, "fp32", strategy)
    w16, o16 = O.decode_attention(q, cache, None, block, group, "fp16", strategy)
    assert np.abs(o32 - o16).max() <= 2e-3 * np.abs(o32).max()
    K, V = O.reconstruct(cache, block, group, strategy)
    same(K, z["recon_K"], f"{name} K")
    wu, ou = O.decode_attention(q, cache, None, block, group, "fp32", "uniform_group")
    assert np.abs(ou - o32).max() > 1e-2 * np.abs(o32).max()


@pytest.mark.parametrize("name", ["flush_a", "flush_b", "flush_c", "flush_n", "flush_n64"])
def test_decode_oracle_against_reference_decode_outputs(name):
    """attn_weights / attn_output the reference's own qkv_matmul_hqe_2 returned for every cache of the flush
    sequences (its CUDA GEMV replaced by an fp32-accumulating CPU stand-in).  The oracle's restatement of the
    reference's fp16 flow must agree to within one fp16 ulp of a logit and be identical in at least 95 % of the probabilities (summation order is the only freedom); the fp32 oracle,
    which is the parity target of the CUDA path, must agree to the accuracy of that fp16 flow."""
    z = load_golden(name)
    B, H, D, block, group, _, nsteps = (int(v) for v in z["meta"])
    strategy = str(z["strategy"])
    for s in range(nsteps):
        cache = golden_cache(z, f"s{s}_out")
        q = z[f"s{s}_q"]
        rw = z[f"s{s}_attn_weights"].astype(np.float32)
        ro = z[f"s{s}_attn_output"].astype(np.float32)
        w, o = O.decode_attention_fp16_flow(q, cache, block, group, strategy)
        w, o = w.astype(np.float32), o.astype(np.float32)
        # one fp16 ulp of a row's largest logit (summation order) moves all its probabilities by up to 0.4 %
        assert (np.abs(w - rw) <= 2.0 ** -8 * rw + 2.0 ** -24).all(), f"{name} step {s}: weights"
        assert (w != rw).mean() <= 0.05 and (o != ro).mean() <= 0.15, f"{name} step {s}: too many one-ulp differences"
        assert np.abs(o - ro).max() <= 1e-3 * np.abs(ro).max(), f"{name} step {s}: output"
        w32, o32 = O.decode_attention(q, cache, None, block, group, "fp32", strategy)
        assert (np.abs(o32 - ro).max(-1) <= 5e-3 * np.abs(o32).max(-1)).all(), f"{name} step {s}: fp32 oracle vs reference flow"
        assert np.abs(w32 - rw).max() <= 2.5e-3, f"{name} step {s}: fp32 probabilities vs reference flow"
