"""GPU parity tests of the other callers of the decode path: the fused-index and sequential-layout entry
points (qkv_matmul_hqe, qkv_matmul_hqe_1), the two halves as operators (cuda_bmm_forward_qk_group_hq /
cuda_bmm_forward_wv_group_hq and their _seq forms), the no-eviction flavour (hybrid_quant, quant_matmul_hq),
the kvhq_gemv shim in the reference's transposed operand layout, and the bounded waits of the cross-GPU
exchange.  Everything is called through the C ABI and compared with the numpy oracle.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import hqkv_oracle as O
from test_gpu_parity import ATTN_REL_TOL, bits_equal, check_attention, host_cache

pytestmark = pytest.mark.gpu

NORMAL = "high_uniform_group_low_normal_group"


@pytest.fixture(scope="module")
def ops(cuda_device):
    import types
    from hqekv_b200.model import public_func
    from hqekv_b200.quant import hqe_1, hqe_2, hqe_matmul, hybrid_quant, kvhq_gemv, matmul, pack_unpack, quant_matmul_hq
    return types.SimpleNamespace(pu=pack_unpack, pf=public_func, hqe_1=hqe_1, hqe_2=hqe_2, hm=hqe_matmul, mm=matmul,
                                 hq=hybrid_quant, qm=quant_matmul_hq, gemv=kvhq_gemv)


def small_cache(cuda_device, strategy, batch=2, nh_q=8, nh_kv=2, group=32, seed=11, evict=0.125, residual=40):
    from hqekv_b200 import synthetic
    cfg = synthetic.CacheConfig("callers", batch, nh_q, nh_kv, 128, 1024 + residual, residual, (0.25, 0.25, 0.25, 0.25),
                                evict, group, True, 1, 64)
    return synthetic.build_cache(cfg, cuda_device, seed=seed, times_range=True, quant_strategy=strategy)


def drop_index_lists(cache):
    out = list(cache)
    for s in (1, 3, 5, 9, 13, 17, 21, 25, 29, 33):
        out[s] = None
    return tuple(out)


def test_qkv_matmul_hqe_is_the_fused_call(ops, cuda_device):
    """qkv_matmul_hqe (index scatter / gather inside the kernels): same result as qkv_matmul_hqe_2 under the one
    strategy it accepts, the reference's ValueError for any other."""
    cache, q = small_cache(cuda_device, NORMAL)
    w, o = ops.hm.qkv_matmul_hqe(q, cache, None, 128, NORMAL, 32, 32)
    w2, o2 = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, NORMAL, 32, 32)
    assert torch.equal(w, w2) and torch.equal(o, o2)
    check_attention(ops, cache, q, 32, 32, "qkv_matmul_hqe", NORMAL)
    with pytest.raises(ValueError, match="invalid quant_strategy"):
        ops.hm.qkv_matmul_hqe(q, cache, None, 128, "uniform_group", 32, 32)


@pytest.mark.parametrize("group", [32, 64])
def test_qkv_matmul_hqe_1_sequential_layout(ops, cuda_device, group):
    """qkv_matmul_hqe_1: no index lists, logical order = tier order then the residual window; the 1-bit tier in
    the Gaussian codebook.  Against the fp32 oracle on the same cache with identity index lists."""
    cache, q = small_cache(cuda_device, NORMAL, group=group, evict=0.0)
    seq = drop_index_lists(cache)
    w, out = ops.hm.qkv_matmul_hqe_1(q, seq, None, 128, "anything", group, group)
    torch.cuda.synchronize()
    ident = ops.hqe_1.sequential_index_lists(seq)
    ow, oo = O.decode_attention(q.cpu().numpy(), host_cache(ident), None, group, group, quant_strategy=NORMAL)
    rel = (np.abs(out.float().cpu().numpy() - oo).max(-1) / np.abs(oo).max(-1)).max()
    assert rel <= ATTN_REL_TOL, f"sequential decode rel err {rel:.3e}"
    assert np.abs(w.float().cpu().numpy() - ow).max() <= 2e-3
    Kd, Vd = ops.hqe_1.KV_cache_reconstruct_hqe(seq, NORMAL, group, group)
    oK, oV = O.reconstruct(host_cache(ident), group, group, NORMAL)
    bits_equal(Kd, oK, "sequential reconstruction K")
    bits_equal(Vd, oV, "sequential reconstruction V")
    with pytest.raises(NotImplementedError):
        ops.hqe_1.KV_cache_hqe_1()


def _tier_args(cache, side, with_idx):
    """Positional tier arguments of cuda_bmm_forward_{qk,wv}_group_hq(_seq) from a cache tuple."""
    base = {"K": (0, 4, 12, 20, 28), "V": (2, 8, 16, 24, 32)}[side]
    args = [cache[base[0]]] + ([cache[base[0] + 1]] if with_idx else [])
    for s in base[1:]:
        args += [cache[s]] + ([cache[s + 1]] if with_idx else []) + [cache[s + 2], cache[s + 3]]
    return args


@pytest.mark.parametrize("sequential", [False, True])
def test_forward_qk_and_wv_group_hq(ops, cuda_device, sequential):
    """The K half and the V half as operators: raw q.K^T at logical positions (fp16) and sum_t w_t V_t for given
    weights, against fp32 products over the oracle's fp32 dequantisation.  Tolerance 2e-3 of the largest value of
    the row (the results are fp16)."""
    cache, q = small_cache(cuda_device, NORMAL, evict=0.0 if sequential else 0.125)
    H = cache[40].shape[1]
    if sequential:
        cache_l = drop_index_lists(cache)
        ref_cache = ops.hqe_1.sequential_index_lists(cache_l)
        qk = ops.mm.cuda_bmm_forward_qk_group_hq_seq(32, H, q, *_tier_args(cache_l, "K", False), cache[39])
    else:
        ref_cache = cache
        qk = ops.mm.cuda_bmm_forward_qk_group_hq(32, H, q, *_tier_args(cache, "K", True), cache[39])
    torch.cuda.synchronize()
    Kf, Vf = O.reconstruct_fp32(host_cache(ref_cache), 32, 32, NORMAL)
    B, _, L, D = Kf.shape
    rep = q.shape[1] // H
    qf = q.float().cpu().numpy().reshape(B, H, rep, D)
    want = np.matmul(qf, np.swapaxes(Kf, 2, 3)).reshape(B, H * rep, 1, L)
    got = qk.float().cpu().numpy()
    assert got.shape == want.shape
    err = np.abs(got - want).max(-1) / np.abs(want).max(-1)
    assert err.max() <= 2e-3, f"qk_group_hq rel err {err.max():.3e}"
    # the same call twice, then a full decode on the same stream: the scratch is left clean
    w1, o1 = ops.hm.qkv_matmul_hqe_2(q, ref_cache, None, 128, NORMAL, 32, 32)
    gen = torch.Generator(device=cuda_device).manual_seed(5)
    p = torch.softmax(torch.randn(B, H * rep, 1, L, generator=gen, device=cuda_device) * 2, dim=-1).half()
    if sequential:
        wv = ops.mm.cuda_bmm_forward_wv_group_hq_seq(32, H, p, *_tier_args(cache_l, "V", False), cache[40])
    else:
        wv = ops.mm.cuda_bmm_forward_wv_group_hq(32, H, p, *_tier_args(cache, "V", True), cache[40])
    torch.cuda.synchronize()
    pf = p.float().cpu().numpy().reshape(B, H, rep, L)
    want = np.matmul(pf, Vf).reshape(B, H * rep, 1, D)
    got = wv.float().cpu().numpy()
    err = np.abs(got - want).max(-1) / np.abs(want).max(-1)
    assert err.max() <= 2e-3, f"wv_group_hq rel err {err.max():.3e}"
    w2, o2 = ops.hm.qkv_matmul_hqe_2(q, ref_cache, None, 128, NORMAL, 32, 32)
    assert torch.equal(o1, o2) and torch.equal(w1, w2)
    with pytest.raises(ValueError, match="invalid matrix"):
        ops.mm.cuda_bmm_forward_qk_group_hq(32, H, q, *([None] * 18), None)


@pytest.mark.parametrize("batch,nh_q,nh_kv", [(1, 32, 8), (2, 8, 2), (8, 32, 8)])
def test_decode_writes_the_importance_row(ops, cuda_device, batch, nh_q, nh_kv):
    """qkv_matmul_hqe_2(head_sum_out=row): the row equals last_attn_weights.update on the returned probabilities
    bit for bit (emitted by the V pass up to B * nh_q = 64, by one more launch beyond), the other results are those
    of the plain call, and consecutive calls do not disturb one another (the arrival counters return to zero)."""
    cache, q = small_cache(cuda_device, "uniform_group", batch=batch, nh_q=nh_q, nh_kv=nh_kv)
    w0, o0 = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group")
    L = w0.shape[-1]
    want = ops.pf.last_attn_weights(last_length=4)
    want.set_max_length(L + 8)
    got = ops.pf.last_attn_weights(last_length=4)
    got.set_max_length(L + 8)
    for step in range(3):
        want.update(w0)
        row = got.decode_row(cuda_device)
        w, o = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", head_sum_out=row)
        got.advance(w.shape[-1])
        assert torch.equal(w, w0) and torch.equal(o, o0), f"step {step}: results differ from the plain call"
    torch.cuda.synchronize()
    bits_equal(got.weights, want.weights.cpu().numpy(), "ring rows written by the decode call")
    assert got.next_line == want.next_line and got.kv_seq_len == want.kv_seq_len
    # the row against the oracle's rounding order on the same probabilities
    ref = O.head_sum_probabilities(w0.cpu().numpy())
    bits_equal(got.weights[0, :L], ref.reshape(-1), "importance row vs oracle")
    with pytest.raises(ValueError, match="head_sum_out"):
        ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", head_sum_out=row[: L - 1])


def test_hybrid_quant_compress_is_the_flush_without_eviction(ops, cuda_device):
    """KV_cache_compress (five counts) builds the same tuple as KV_cache_hqe_2 with an eviction count of zero -
    every slot bit for bit against the oracle's flush - and KV_cache_reconstruct returns the oracle's dense cache."""
    from hqekv_b200 import synthetic
    cfg = synthetic.CacheConfig("hq", 2, 8, 2, 128, 512 + 20, 20, (0.25, 0.5, 0.25), 0.0, 32, True, 1, 32)
    K, V, q = synthetic.make_kv(cfg, cuda_device, 3)
    flushed = cfg.context - cfg.residual
    counts = synthetic.tier_counts(cfg)
    assert counts[5] == 0
    imp = synthetic.synthetic_importance(cfg, cuda_device, 3, flushed)
    imp_np = imp.cpu().numpy().copy()
    ids = ops.pf.get_block_token_idx(32, flushed // 32, imp)
    ids_np = O.block_rank(32, flushed // 32, imp_np)
    cache = (None,) * 39 + (K, V, cfg.context)
    five = torch.tensor(counts[:5], dtype=torch.int32)
    got = ops.hq.KV_cache_compress(cache, flushed, 0, ids, five, five.clone(), imp, "uniform_group", 32, 32)
    want = O.flush(host_cache(cache), flushed, 0, ids_np, np.array(counts), np.array(counts), imp_np, "uniform_group",
                   None, 32, 32, True)
    for i in range(41):
        bits_equal(got[i], want[i], f"KV_cache_compress slot {i}")
    Kd, Vd = ops.hq.KV_cache_reconstruct(got, "uniform_group", 32, 32)
    oK, oV = O.reconstruct(want, 32, 32, "uniform_group")
    bits_equal(Kd, oK, "KV_cache_reconstruct K")
    bits_equal(Vd, oV, "KV_cache_reconstruct V")
    with pytest.raises(ValueError):
        ops.hq.KV_cache_compress(cache, flushed, 0, ids, counts, counts, imp, "uniform_group", 32, 32)  # six counts


def test_quant_matmul_hq_entry_points(ops, cuda_device):
    """qkv_matmul / qkv_matmul_hq of the no-eviction flavour against the fp32 oracle, without a mask and with an
    additive mask over the cached positions (quant/quant_matmul_hq.py:101,164: attn_weights += attention_mask)."""
    cache, q = small_cache(cuda_device, "uniform_group", evict=0.0)
    L = sum(cache[s].numel() for s in (1, 5, 13, 21, 29) if cache[s] is not None) + cache[39].shape[2]
    for fn in (ops.qm.qkv_matmul, ops.qm.qkv_matmul_hq):
        w, out = fn(q, cache, None, 128, "uniform_group", 32, 32)
        torch.cuda.synchronize()
        ow, oo = O.decode_attention(q.cpu().numpy(), host_cache(cache), None, 32, 32)
        rel = (np.abs(out.float().cpu().numpy() - oo).max(-1) / np.abs(oo).max(-1)).max()
        assert rel <= ATTN_REL_TOL
        assert np.abs(w.float().cpu().numpy() - ow).max() <= 2e-3
    # additive mask: -inf on a third of the positions, a finite bias elsewhere
    gen = torch.Generator(device=cuda_device).manual_seed(9)
    mask = torch.randn(q.shape[0], 1, 1, L, generator=gen, device=cuda_device).half()
    mask[..., ::3] = float("-inf")
    w, out = ops.qm.qkv_matmul(q, cache, mask, 128, "uniform_group", 32, 32)
    torch.cuda.synchronize()
    Kf, Vf = O.reconstruct_fp32(host_cache(cache), 32, 32, "uniform_group")
    B, H, _, D = Kf.shape
    rep = q.shape[1] // H
    qf = q.float().cpu().numpy().reshape(B, H, rep, D)
    logits = np.matmul(qf, np.swapaxes(Kf, 2, 3)) / np.float32(np.sqrt(D)) + mask.float().cpu().numpy().reshape(B, 1, 1, L)
    logits = logits - logits.max(-1, keepdims=True)
    p = np.exp(logits)
    p /= p.sum(-1, keepdims=True)
    want = np.matmul(p, Vf).reshape(B, H * rep, 1, D)
    rel = (np.abs(out.float().cpu().numpy() - want).max(-1) / np.abs(want).max(-1)).max()
    assert rel <= 3e-3, f"masked decode rel err {rel:.3e}"   # logits pass through fp16 once on this path
    assert float(w[..., ::3].abs().max()) == 0.0


@pytest.mark.parametrize("bits", [8, 4, 2])
def test_kvhq_gemv_shim_transposed_layout(ops, cuda_device, bits):
    """kvhq_gemv.gemv_forward_cuda_uniform_group with operands as quant/matmul.py:285-298 hands them over
    (codes [B*nh_kv, N/fpi, K], scales / zeros [B*nh_kv, N/group, K], activations [B*nh_q, 1, K])."""
    rng = np.random.default_rng(bits)
    B, nh_q, nh_kv, K, N, g = 2, 8, 2, 128, 32 * 6, 32
    x = rng.standard_normal((B, nh_kv, K, N)).astype(np.float16)
    code, scale, mn = O.quantize_pack_last_dim(x, g, bits)
    fA = rng.standard_normal((B, nh_q, 1, K)).astype(np.float16)
    want = O.gemv_dequant(fA, code, scale, mn, g, bits)
    t = lambda a: torch.from_numpy(a).to(cuda_device)
    kern = t(code).reshape(B * nh_kv, K, -1).transpose(1, 2).contiguous()
    sc = t(scale).reshape(B * nh_kv, K, -1).transpose(1, 2).contiguous()
    zp = t(mn).reshape(B * nh_kv, K, -1).transpose(1, 2).contiguous()
    got = ops.gemv.gemv_forward_cuda_uniform_group(t(fA).reshape(B * nh_q, 1, K), kern, sc, zp, bits, g, nh_q, nh_kv)
    assert got.shape == (B * nh_q, 1, N)
    err = np.abs(got.float().cpu().numpy().reshape(want.shape) - want).max() / np.abs(want).max()
    assert err <= 2e-3
    # the Gaussian-codebook sibling at 1 bit
    code1, std, mean = O.normal1_quantize_pack_last_dim(x, g)
    want1 = O.gemv_dequant_normal1(fA, code1, std, mean, g)
    k1 = t(code1).reshape(B * nh_kv, K, -1).transpose(1, 2).contiguous()
    s1 = t(std).reshape(B * nh_kv, K, -1).transpose(1, 2).contiguous()
    m1 = t(mean).reshape(B * nh_kv, K, -1).transpose(1, 2).contiguous()
    got1 = ops.gemv.gemv_forward_cuda_normalize_group(t(fA).reshape(B * nh_q, 1, K), k1, s1, m1, None, 1, g, nh_q, nh_kv)
    err = np.abs(got1.float().cpu().numpy().reshape(want1.shape) - want1).max() / np.abs(want1).max()
    assert err <= 2e-3


# ---------------------------------------------------------------------------------------------
# bounded waits of the cross-GPU exchange, on ONE GPU: a wait that nobody answers must run out, record
# which rank was missing and leave the context usable
# ---------------------------------------------------------------------------------------------
def test_peer_unpack_wait_runs_out(cuda_device):
    from hqekv_b200._lib import lib, stream_ptr
    entries, world = 64, 2
    recv = torch.zeros(world * entries, 2, dtype=torch.int32, device=cuda_device)   # nobody writes it
    plain = torch.full((world * entries,), -1, dtype=torch.int32, device=cuda_device)
    state = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    rc = lib.hqkv_peer_unpack(recv.data_ptr(), plain.data_ptr(), 0, world, entries, state.data_ptr(), 100,
                              stream_ptr(cuda_device))
    assert rc == 0, lib.hqkv_last_error().decode()
    torch.cuda.synchronize()
    assert state.tolist() == [1, 2], "call number advanced, status = 1 + the missing rank"
    assert torch.ones(4, device=cuda_device).sum().item() == 4.0   # the context still works


def test_peer_barrier_wait_runs_out(cuda_device):
    from hqekv_b200._lib import lib, stream_ptr
    pad0 = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    pad1 = torch.zeros(8, dtype=torch.int32, device=cuda_device)   # stands in for the peer's pad; nobody signals ours
    state = torch.zeros(2, dtype=torch.int32, device=cuda_device)
    pads = (C.c_void_p * 2)(pad0.data_ptr(), pad1.data_ptr())
    rc = lib.hqkv_peer_barrier(pads, 0, 2, state.data_ptr(), 100, stream_ptr(cuda_device))
    assert rc == 0, lib.hqkv_last_error().decode()
    torch.cuda.synchronize()
    assert state.tolist() == [1, 2]
    assert pad1[0].item() == 1, "our arrival was signalled to the peer's pad"


def test_flagged_exchange_loopback(ops, cuda_device):
    """The flagged peer stores of the decode kernel and the unpack kernel, with the 'peer' receive buffer on the
    same GPU: rank 0 stores into the buffer a rank 1 polls; three consecutive calls over two rotating slots.
    The unpacked rows equal the plain decode output bit for bit, the call number advances, the status stays 0."""
    from hqekv_b200._lib import CODEC_UNIFORM, lib, stream_ptr
    from hqekv_b200.quant._cache import build_cache_desc
    cache, q = small_cache(cuda_device, "uniform_group", batch=1)
    desc, keep, L, dev = build_cache_desc(cache, q.shape[1], 32, 32, CODEC_UNIFORM)
    need = lib.hqkv_decode_workspace_bytes(desc)
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    B, nh_q, D = q.shape[0], q.shape[1], 128
    entries = B * nh_q * D // 2
    st = stream_ptr(dev)
    w_ref, o_ref = ops.hm.qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", 32, 32)
    send_state = torch.zeros(2, dtype=torch.int32, device=dev)    # rank 0's call number (the sender's flag source)
    recv_state = torch.zeros(2, dtype=torch.int32, device=dev)    # rank 1's
    slots = [torch.zeros(2 * entries, 2, dtype=torch.int32, device=dev) for _ in range(2)]   # rank 1's receive buffers
    for call in range(3):
        recv = slots[call % 2]
        w = torch.empty(B, nh_q, 1, L, dtype=torch.float16, device=dev)
        o = torch.empty(B, nh_q, 1, D, dtype=torch.float16, device=dev)
        peers = (C.c_void_p * 1)(recv.data_ptr())   # rank 0's entries start at word 0 of rank 1's buffer
        rc = lib.hqkv_decode_attention_gather_flagged(desc, q.data_ptr(), w.data_ptr(), o.data_ptr(), ws.data_ptr(),
                                                      ws.numel(), peers, 1, send_state.data_ptr(), st)
        assert rc == 0, lib.hqkv_last_error().decode()
        send_state[0] += 1   # the sender's own unpack would advance it; here rank 0 has no unpack launch
        gathered = torch.zeros(2 * entries, dtype=torch.int32, device=dev)
        rc = lib.hqkv_peer_unpack(recv.data_ptr(), gathered.data_ptr(), 1, 2, entries, recv_state.data_ptr(), 1 << 20, st)
        assert rc == 0, lib.hqkv_last_error().decode()
        torch.cuda.synchronize()
        assert recv_state.tolist() == [call + 1, 0]
        got = gathered[:entries].view(torch.float16).view(B, nh_q, 1, D)
        assert torch.equal(got, o) and torch.equal(o, o_ref) and torch.equal(w, w_ref), f"call {call}"
