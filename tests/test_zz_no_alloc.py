"""The allocation-free decode entry point (hqkv_decode_attention_static).

Some users of the library cannot call cudaMalloc when they need attention: a server that has handed
all GPU memory to its own pool, a latency-critical loop that must not allocate after start-up, a
binding without a device allocator.  For them the library carries its decode scratch in a fixed
16 MiB array on the device.  This test drives that entry point through the C ABI, twice in a row
(the array is shared and keeps the previous call's contents), and compares with the regular entry
point that takes caller-provided scratch.  It also checks that an oversized cache is refused.

The file name makes pytest collect it after every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

ATTN_REL_TOL = 2e-3  # the tolerance the decode parity tests use; the two paths run the same kernels


def test_static_scratch_decode_matches_regular_entry_point(cuda_device):
    from hqekv_b200 import synthetic
    from hqekv_b200._lib import lib, ptr, stream_ptr
    from hqekv_b200.quant._cache import build_cache_desc
    from hqekv_b200.quant.hqe_matmul import qkv_matmul_hqe_2

    cfg = synthetic.CONFIGS["cfg0"]
    assert lib.hqkv_decode_static_scratch_bytes() == 16 << 20
    with torch.cuda.device(cuda_device):
        for seed in (0, 1):  # two calls in a row, different caches: nothing may leak from one to the next
            cache, q = synthetic.build_cache(cfg, cuda_device, seed=seed, times_range=bool(seed))
            w_ref, o_ref = qkv_matmul_hqe_2(q, cache, None, 128, "uniform_group", cfg.group, cfg.group)
            desc, keep, L, _ = build_cache_desc(cache, q.shape[1], cfg.group, cfg.group)
            w = torch.full_like(w_ref, float("nan"))
            o = torch.full_like(o_ref, float("nan"))
            rc = lib.hqkv_decode_attention_static(desc, ptr(q), ptr(w), ptr(o), stream_ptr(cuda_device))
            assert rc == 0, lib.hqkv_last_error().decode()
            torch.cuda.synchronize()
            assert torch.isfinite(o).all() and torch.isfinite(w).all()
            rel = ((o.float() - o_ref.float()).abs().amax(-1) / o_ref.float().abs().amax(-1)).max().item()
            assert rel <= ATTN_REL_TOL, f"call {seed}: static-scratch output differs by {rel:.3e}"
            assert (w.float() - w_ref.float()).abs().max().item() <= ATTN_REL_TOL
            del keep


def test_static_scratch_refuses_oversized_cache(cuda_device):
    from hqekv_b200._lib import CacheDesc, lib
    desc = CacheDesc()
    desc.B, desc.H, desc.nh_q, desc.D, desc.group_k, desc.group_v, desc.n_new = 8, 8, 32, 128, 32, 32, 128
    desc.new_k = desc.new_v = 256                      # never dereferenced: the size check comes first
    t = desc.tier[2]
    t.bits, t.n_k, t.n_v = 4, 32768, 32768
    for f in ("k_data", "k_scale", "k_zero", "k_idx", "v_data", "v_scale", "v_zero", "v_idx"):
        setattr(t, f, 256)
    assert lib.hqkv_decode_workspace_bytes(desc) > lib.hqkv_decode_static_scratch_bytes()
    rc = lib.hqkv_decode_attention_static(desc, 256, 256, 256, None)
    assert rc == -3
    assert b"built-in array" in lib.hqkv_last_error()
