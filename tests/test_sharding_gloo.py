"""World-size-2 checks of the head-sharding exchange logic on CPU (gloo): shard assignment, cache
slicing, reassembly of gathered head outputs, and the rank-ordered importance reduction that must
give every rank the same bits."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import hqkv_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hqekv_b200 import sharding
        nh_kv, rep, B, D, L = 4, 4, 2, 128, 96
        gen = torch.Generator().manual_seed(5)
        q = torch.randn(B, nh_kv * rep, 1, D, generator=gen).half()
        full_out = torch.randn(B, nh_kv * rep, 1, D, generator=gen).half()
        probs = torch.softmax(torch.randn(B, nh_kv * rep, 1, L, generator=gen) * 3, -1).half()
        first, count = sharding.head_shard(rank, world, nh_kv)
        assert (first, count) == (rank * 2, 2)
        # query / output shards line up with the kv-head shard
        q_local = sharding.shard_query(q, first, count, nh_kv)
        assert torch.equal(q_local, q[:, first * rep:(first + count) * rep])
        out_local = full_out[:, first * rep:(first + count) * rep].contiguous()
        gathered = sharding.gather_head_outputs(out_local)
        assert torch.equal(gathered, full_out), "gathered outputs are not in head order"
        # cache slicing keeps replicated slots and slices per-head ones
        cache = [None] * 42
        cache[8] = torch.arange(B * nh_kv * 5 * 32, dtype=torch.int32).reshape(B, nh_kv, 5, 32)
        cache[9] = torch.arange(5)
        cache[10] = torch.ones(B, nh_kv, 5, 4).half()
        cache[38] = torch.ones(5).half()
        cache[39] = torch.randn(B, nh_kv, 3, D, generator=gen).half()
        cache[41] = 8
        sc = sharding.shard_cache(tuple(cache), first, count)
        assert torch.equal(sc[8], cache[8][:, first:first + count]) and sc[8].is_contiguous()
        assert torch.equal(sc[9], cache[9]) and torch.equal(sc[38], cache[38]) and sc[41] == 8
        assert sc[39].shape == (B, count, 3, D)
        # importance row: per-rank fp32 partials over the local heads, rank-ordered total
        local = probs[:, first * rep:(first + count) * rep].float().sum(0).sum(0).reshape(L)
        row = sharding.reduce_importance_row(local)
        rows = [torch.empty_like(row) for _ in range(world)]
        dist.all_gather(rows, row)
        assert all(torch.equal(rows[0], r) for r in rows), "ranks disagree on the importance row"
        want = probs.float().sum(0).sum(0).reshape(L)
        assert torch.allclose(row.float(), want, rtol=2e-3, atol=1e-6)
        # errors
        try:
            sharding.head_shard(rank, 3, 4)
            raise AssertionError("uneven sharding accepted")
        except ValueError:
            pass
        open(os.path.join(tmpdir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_head_sharding_world_size_2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")


def test_sharded_attention_equals_full_attention_in_the_oracle():
    """Head sharding is exact for attention: the oracle run on two head shards and concatenated equals
    the oracle run on all heads (no cross-head term exists in the math)."""
    from conftest import golden_cache, load_golden
    from hqekv_b200 import sharding
    z = load_golden("flush_a")
    cache = golden_cache(z, "s0_out")
    tcache = tuple(torch.from_numpy(np.ascontiguousarray(x)) if isinstance(x, np.ndarray) else x for x in cache)
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 8, 1, 128)).astype(np.float16)
    _, full = O.decode_attention(q, cache)
    parts = []
    for r in range(2):
        first, count = sharding.head_shard(r, 2, 2)
        sc = sharding.shard_cache(tcache, first, count)
        sc_np = tuple(x.numpy() if torch.is_tensor(x) else x for x in sc)
        ql = sharding.shard_query(torch.from_numpy(q), first, count, 2).numpy()
        parts.append(O.decode_attention(ql, sc_np)[1])
    assert np.array_equal(np.concatenate(parts, axis=1), full)
