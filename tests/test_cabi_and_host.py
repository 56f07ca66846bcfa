"""CPU-only checks: the C-ABI library loads and exports every symbol include/hqkv.h declares, argument
validation works without a GPU (it runs before any CUDA call), the host-side logic (tuple slot map,
tier counts, error conventions) behaves like the reference's, and nothing falls back to a CPU path."""
import ctypes
import sys
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from hqekv_b200 import build
    build.build()
    from hqekv_b200 import _lib
    return _lib


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "hqkv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hqkv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) >= 18
    raw = ctypes.CDLL(lib.LIB_PATH)
    for name in names:
        assert hasattr(raw, name), f"{name} is declared in include/hqkv.h but not exported"
    assert set(names) == set(lib.EXPORTED_SYMBOLS), "ctypes signature table and header disagree"
    assert lib.lib.hqkv_version() >= 100


def test_argument_validation_needs_no_gpu(lib):
    L = lib.lib
    assert L.hqkv_quantize_pack(None, 4, 32, 4, 32, 32, 1, 32, 3, None, None, None, None) == -1
    assert b"bits" in L.hqkv_last_error()
    assert L.hqkv_quantize_pack(None, 4, 48, 4, 48, 48, 1, 32, 4, None, None, None, None) == -1
    assert b"multiple of the group" in L.hqkv_last_error()
    assert L.hqkv_quantize_pack(None, 0, 32, 1, 32, 32, 1, 32, 4, None, None, None, None) == 0   # empty input
    assert L.hqkv_gemv_uniform_group(None, None, None, None, 1, 4, 3, 128, 128, 32, 4, None, None) == -1
    assert L.hqkv_block_rank(None, None, 32, 9000, None, None) == -1
    assert L.hqkv_decode_workspace_bytes(None) == 0
    desc = lib.CacheDesc()
    desc.B, desc.H, desc.nh_q, desc.D, desc.group_k, desc.group_v = 1, 8, 32, 64, 32, 32
    assert L.hqkv_decode_attention(desc, None, None, None, None, 0, None) == -1
    assert b"head dim" in L.hqkv_last_error()
    desc.D = 128
    assert L.hqkv_decode_attention(desc, None, None, None, None, 0, None) == -1
    assert b"empty" in L.hqkv_last_error()
    desc.tier[4].bits, desc.tier[4].n_k, desc.tier[4].n_v = 1, 32, 32
    assert L.hqkv_decode_attention(desc, None, None, None, None, 0, None) == -1      # 1-bit tier: null pointers
    assert b"pointers are null" in L.hqkv_last_error()


def test_gaussian_codebook_entry_points_validate_without_gpu(lib):
    """The 1-bit Gaussian-codebook tier: codec flags are checked before any device work."""
    L = lib.lib
    assert L.hqkv_gemv_normal_group(None, None, None, None, 1, 4, 1, 128, 128, 32, 2, None, None) == -1
    assert b"1 bit only" in L.hqkv_last_error()
    assert L.hqkv_gemv_normal_group(None, None, None, None, 1, 4, 1, 128, 128, 32, 1, None, None) == -1
    assert b"null pointer" in L.hqkv_last_error()
    assert L.hqkv_normal1_quantize_pack(None, 4, 48, 4, 48, 48, 1, 32, None, None, None, None) == -1
    assert b"multiple of the group" in L.hqkv_last_error()
    assert L.hqkv_normal1_quantize_pack(None, 0, 32, 1, 32, 32, 1, 32, None, None, None, None) == 0     # empty input
    assert L.hqkv_normal1_dequantize_unpack(None, None, None, 4, 64, 48, None, None) == -1
    src = lib.FlushSrc()
    src.low_codec = 7
    assert L.hqkv_flush_build_v(src, 1, 1, 128, 32, 4, None, 32, None, None, None, None) == -1
    assert b"low_codec" in L.hqkv_last_error()
    desc = lib.CacheDesc()
    desc.B, desc.H, desc.nh_q, desc.D, desc.group_k, desc.group_v = 1, 8, 32, 128, 32, 32
    desc.tier[3].bits, desc.tier[3].n_k, desc.tier[3].n_v, desc.tier[3].codec = 2, 32, 32, lib.CODEC_NORMAL
    assert L.hqkv_decode_attention(desc, None, None, None, None, 0, None) == -1
    assert b"codec" in L.hqkv_last_error()


def test_peer_entry_points_validate_without_gpu(lib):
    """kv-head sharding entry points: argument checks run before anything touches a device."""
    import ctypes as C
    L = lib.lib
    desc = lib.CacheDesc()
    desc.B, desc.H, desc.nh_q, desc.D, desc.group_k, desc.group_v = 1, 8, 32, 128, 32, 32
    peers = (C.c_void_p * 8)()
    assert L.hqkv_decode_attention_gather(desc, None, None, None, None, 0, peers, 8, None, 0, 0, None, 0, None) == -1
    assert b"at most 7 peers" in L.hqkv_last_error()
    assert L.hqkv_decode_attention_gather(desc, None, None, None, None, 0, peers, 2, None, 0, 0, None, 0, None) == -1
    assert b"peer output 0 is null" in L.hqkv_last_error()
    pads = (C.c_void_p * 2)()
    assert L.hqkv_peer_barrier(pads, 2, 2, None, 1000, None) == -1      # rank out of range
    assert b"bad rank/world" in L.hqkv_last_error()
    assert L.hqkv_peer_barrier(pads, 0, 2, None, 1000, None) == -1      # no state block
    assert L.hqkv_peer_barrier(pads, 0, 2, C.c_void_p(4096), 0, None) == -1  # spin limit must be positive: waits are bounded
    assert L.hqkv_decode_attention_gather_flagged(desc, None, None, None, None, 0, peers, 0, None, None) == -1
    assert b"1..7 peers" in L.hqkv_last_error()
    assert L.hqkv_peer_unpack(None, None, 0, 2, 256, None, 1000, None) == -1
    assert b"null or misaligned" in L.hqkv_last_error()
    assert L.hqkv_peer_unpack(C.c_void_p(4096), C.c_void_p(4096), 0, 2, 256, C.c_void_p(4096), 0, None) == -1  # bounded waits only


def test_library_is_stamped_with_its_sources(lib):
    """hqkv_build_id() is the hash of the sources the binary was compiled from; the build script reads the same stamp
    out of the file and rebuilds on a mismatch."""
    from hqekv_b200 import build
    stamp = lib.lib.hqkv_build_id().decode()
    assert len(stamp) == 16 and stamp == build.library_id(lib.LIB_PATH)
    if not os.environ.get("HQKV_LIB"):
        assert stamp == build.source_id() and not build.needs_build()


def test_workspace_size_of_the_benchmark_cache(lib):
    """Llama-3.1-8B at 32k: 5888/11744/11744 tokens in the 8/4/2-bit tiers + 128 residual."""
    desc = lib.CacheDesc()
    desc.B, desc.H, desc.nh_q, desc.D, desc.group_k, desc.group_v, desc.n_new = 1, 8, 32, 128, 32, 32, 128
    dummy = ctypes.c_void_p(256)
    desc.new_k, desc.new_v = 256, 256
    for t, n in ((1, 5888), (2, 11744), (3, 11744)):
        tier = desc.tier[t]
        tier.bits, tier.n_k, tier.n_v = (16, 8, 4, 2, 1)[t], n, n
        for f in ("k_data", "k_scale", "k_zero", "k_idx", "v_data", "v_scale", "v_zero", "v_idx"):
            setattr(tier, f, 256)
    need = lib.lib.hqkv_decode_workspace_bytes(desc)
    L = 5888 + 11744 * 2 + 128
    assert need >= lib.WS_HEADER_BYTES + 32 * L * 4
    assert lib.lib.hqkv_decode_workspace_zero_bytes(desc) == lib.WS_HEADER_BYTES
    assert need < 16 << 20
    del dummy


def test_ops_refuse_cpu_tensors(lib):
    from hqekv_b200.quant import hqe_matmul, pack_unpack
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        pack_unpack.uniform_group_quantize_pack_last_dim(torch.zeros(1, 1, 1, 32, dtype=torch.float16), 32, 4)
    cache = (None,) * 39 + (torch.zeros(1, 1, 4, 128, dtype=torch.float16),) * 2 + (4,)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        hqe_matmul.qkv_matmul_hqe_2(torch.zeros(1, 4, 1, 128, dtype=torch.float16), cache, None, 128, "uniform_group")


def test_error_conventions_match_the_reference(lib):
    from hqekv_b200.quant import hqe_2, hqe_matmul
    q = torch.zeros(1, 4, 1, 128, dtype=torch.float16)
    with pytest.raises(ValueError, match="invalid quant_strategy"):
        hqe_matmul.qkv_matmul_hqe_2(q, (None,) * 42, None, 128, "nope")
    with pytest.raises(ValueError, match="invalid quant_strategy"):
        hqe_2.KV_cache_hqe_2((None,) * 42, 0, 0, None, None, None, None, "nope")
    with pytest.raises(ValueError, match="invalid quant_strategy"):
        hqe_2.KV_cache_reconstruct_hqe((None,) * 42, "nope")


def test_reference_import_names(lib):
    import hqekv_b200
    hqekv_b200.install_reference_names()
    import hqe_matmul
    import quant.hqe_2
    from model.public_func import get_block_token_idx, last_attn_weights  # noqa: F401
    from pack_unpack import uniform_group_quantize_pack_last_dim  # noqa: F401
    import kvhq_gemv
    assert quant.hqe_2.KV_cache_hqe_2.__module__ == "hqekv_b200.quant.hqe_2"
    assert hqe_matmul.qkv_matmul_hqe_2.__module__ == "hqekv_b200.quant.hqe_matmul"
    assert callable(kvhq_gemv.gemv_forward_cuda_uniform_group)


# The project-import statements of the reference's model files, verbatim: model/llama_hqe.py:20-25 (the
# Llama fork also imports fast_hadamard_transform at :20) and model/qwen3_hqe.py:21-25.
_LLAMA_HQE_IMPORTS = """
import fast_hadamard_transform
from model.public_func import (get_block_token_idx, make_sum_equal, last_attn_weights)

from quant.hqe import KV_cache_hqe
from quant.hqe_2 import KV_cache_hqe_2
from quant.hqe_matmul import qkv_matmul_hqe, qkv_matmul_hqe_2
"""
_QWEN3_HQE_IMPORTS = """
from model.public_func import (get_block_token_idx, make_sum_equal, last_attn_weights)

from quant.hqe import KV_cache_hqe
from quant.hqe_2 import KV_cache_hqe_2
from quant.hqe_matmul import qkv_matmul_hqe, qkv_matmul_hqe_2
"""
# quant/hqe_matmul.py:5-24 of the reference (for a user who keeps that file and swaps only the modules under it)
_HQE_MATMUL_IMPORTS = """
from model.public_func import last_attn_weights

from hqe import KV_cache_hqe
from hqe_1 import KV_cache_hqe_1, KV_cache_reconstruct_hqe

from matmul import (cuda_bmm_fA_qB_uniform_group,
                    cuda_bmm_forward_qk_group_hq,
                    cuda_bmm_forward_qk_group_hq_seq,
                    cuda_bmm_forward_qk_uniform_group_token,
                    cuda_bmm_forward_wv_group_hq,
                    cuda_bmm_forward_wv_group_hq_seq,
                    cuda_bmm_forward_wv_group_outlier_hq,
                    cuda_bmm_fA_qB_uniform_group_outlier,
                    cuda_bmm_fA_qB_wv_uniform_group,
                    cuda_bmm_fA_qB_wv_uniform_group_outlier,
                    cuda_bmm_fA_qB_normal_group,
                    cuda_bmm_fA_qB_normal_group_outlier,
                    cuda_bmm_forward_qk_normal_group_token,
                    cuda_bmm_fA_qB_wv_normal_group_outlier)
"""


@pytest.mark.parametrize("text", [_LLAMA_HQE_IMPORTS, _QWEN3_HQE_IMPORTS, _HQE_MATMUL_IMPORTS],
                         ids=["llama_hqe", "qwen3_hqe", "hqe_matmul"])
def test_reference_files_import_lines_resolve(lib, text):
    """After install_reference_names() the import statements of the reference's own files run unchanged
    (fast_hadamard_transform is a third-party package of the reference's environment: an empty stand-in)."""
    import types
    import hqekv_b200
    hqekv_b200.install_reference_names()
    sys.modules.setdefault("fast_hadamard_transform", types.ModuleType("fast_hadamard_transform"))
    ns = {}
    exec(text, ns)
    for name in ("KV_cache_hqe",):
        assert ns[name].__module__.startswith("hqekv_b200.")
    if "KV_cache_hqe_2" in ns:
        assert ns["KV_cache_hqe_2"].__module__ == "hqekv_b200.quant.hqe_2"
        assert ns["qkv_matmul_hqe"].__module__ == "hqekv_b200.quant.hqe_matmul"
    with pytest.raises(NotImplementedError):
        ns["KV_cache_hqe"]()  # imported by the model files, never called by them


def test_importance_ring_refuses_rows_longer_than_its_capacity(lib):
    """A probability row longer than the ring's rows (or a ring whose max length was never set) must raise before
    any kernel is launched: the head-sum kernel writes L halfs into a ring row."""
    from hqekv_b200.model.public_func import last_attn_weights
    ring = last_attn_weights()
    w = torch.zeros(1, 4, 1, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="ring is sized for 0"):
        ring.update(w)
    ring.set_max_length(32)
    with pytest.raises(ValueError, match="ring is sized for 32"):
        ring.update(w)
    ring.set_max_length(64)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):   # fits: now only the CPU tensor is refused
        ring.update(w)


def test_tier_counts_of_the_configurations(lib):
    from hqekv_b200 import synthetic
    assert synthetic.tier_counts(synthetic.CONFIGS["cfg0"]) == [0, 896, 1792, 896, 0, 384]
    assert synthetic.tier_counts(synthetic.CONFIGS["cfg1"]) == [0, 5888, 11744, 11744, 0, 3264]
    c3 = synthetic.tier_counts(synthetic.CONFIGS["cfg3"])
    assert c3 == [0, 286 * 32, 716 * 32, 1860 * 32, 0, 1226 * 32]
    c2 = synthetic.tier_counts(synthetic.CONFIGS["cfg2"])
    assert sum(c2) == 16384 - 128 and c2[5] == 0 and all(v % 64 == 0 for v in c2)


def test_make_sum_equal_matches_oracle(lib):
    from hqekv_b200.model.public_func import make_sum_equal
    from oracle import hqkv_oracle as O
    rng = np.random.default_rng(0)
    for _ in range(50):
        arr = rng.integers(0, 40, size=6)
        target = int(arr.sum()) - int(rng.integers(0, 10))
        a = make_sum_equal(torch.tensor(arr, dtype=torch.int32), target)
        b = O.make_sum_equal(arr.copy(), target)
        assert a.tolist() == b.tolist()


@pytest.mark.parametrize("name", ["attn_llama_n", "attn_llama_u"])
def test_tier_schedule_matches_reference_layer(name):
    """The data-independent flush arithmetic of the attention layer (shares -> six token counts, lengths
    before and after every flush) against what the reference's LlamaAttention_hqe derived, call by call."""
    from conftest import load_golden
    from hqekv_b200.model.attention_hqe import TierSchedule
    z = load_golden(name)
    B, hidden, nh, nkv, prefill, steps = (int(v) for v in z["meta"])
    sch = TierSchedule(*(float(v) for v in z["shares"]))
    flushes = 0
    for call in range(steps + 1):
        sch.append(prefill if call == 0 else 1)
        if sch.due():
            ratio, bit_num = sch.counts()
            assert np.array_equal(bit_num.numpy(), z[f"c{call}_bit_num"]), f"{name} call {call}"
            assert np.array_equal(ratio.numpy(), z[f"c{call}_ratio"]), f"{name} call {call}: shares"
            sch.commit(int(bit_num[-1]), True)
            flushes += 1
        else:
            assert f"c{call}_bit_num" not in z.files
        assert [sch.current_length, sch.history_reserve_length] == [int(v) for v in z[f"c{call}_state"][:2]], f"{name} call {call}"
    assert flushes >= 2
