"""KV-head sharding of the decode path over the GPUs of one node.

Every kernel of the path treats (batch, kv head) as an outer batch index, so a rank that holds the
kv heads [first, first+count) of every tier runs exactly the single-GPU code on its slice.  Two
things cross ranks:

  * the per-head attention outputs, all-gathered once per layer-step (B * nh_q * 128 fp16 values);
  * the importance row (a sum over ALL heads) that feeds block ranking, which has to be identical
    on every rank: each rank contributes the fp32 sum over its own heads, the partial rows are
    gathered and added in rank order, and the total is rounded to fp16 once.

Index lists, per-token value ranges and tier counts are head-independent and replicated.
The functions below take any torch.distributed process group (NCCL on the GPUs, gloo in the CPU
tests of the exchange logic).
"""
import torch
import torch.distributed as dist

_HEAD_DIM_SLOTS = tuple(i for i in range(36) if i not in (1, 3, 5, 9, 13, 17, 21, 25, 29, 33)) + (39, 40)


def head_shard(rank: int, world: int, nh_kv: int):
    """(first kv head, number of kv heads) of a rank; kv heads must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank/world out of range")
    if nh_kv % world:
        raise ValueError(f"{nh_kv} kv heads do not divide over {world} ranks")
    per = nh_kv // world
    return rank * per, per


def shard_cache(cache: tuple, first: int, count: int):
    """Slice every per-head tensor of a 42-slot cache tuple to kv heads [first, first+count)."""
    if len(cache) != 42:
        raise ValueError("invalid past_key_value")
    out = list(cache)
    for i in _HEAD_DIM_SLOTS:
        t = out[i]
        if t is not None and torch.is_tensor(t) and t.dim() == 4:
            out[i] = t[:, first:first + count].contiguous()
    return tuple(out)


def shard_query(q: torch.Tensor, first: int, count: int, nh_kv: int):
    """Query heads that attend to kv heads [first, first+count) (GQA: nh_q/nh_kv consecutive each)."""
    rep = q.shape[1] // nh_kv
    return q[:, first * rep:(first + count) * rep].contiguous()


def gather_head_outputs(out_local: torch.Tensor, group=None, buffer: torch.Tensor = None):
    """All-gather per-rank attention outputs [B, nh_q/world, 1, D] into [B, nh_q, 1, D] (head order =
    rank order).  ``buffer`` ([world, B, nh_q/world, 1, D]) can be passed to avoid the allocation."""
    world = dist.get_world_size(group)
    B, nh_local, one, D = out_local.shape
    if buffer is None:
        buffer = torch.empty((world,) + tuple(out_local.shape), dtype=out_local.dtype, device=out_local.device)
    # the output is the concatenation of the ranks' tensors along dim 0 (the shape every backend accepts)
    dist.all_gather_into_tensor(buffer.view(world * B, nh_local, one, D), out_local.contiguous(), group=group)
    return buffer.permute(1, 0, 2, 3, 4).reshape(B, world * nh_local, one, D)


def reduce_importance_row(partial_f32: torch.Tensor, group=None):
    """Head-summed probability row from per-rank fp32 partial sums [L]: gathered, added in rank order
    (the same order on every rank, so every rank gets the same bits), rounded to fp16 once."""
    world = dist.get_world_size(group)
    flat = partial_f32.contiguous().float().reshape(-1)
    parts = torch.empty(world * flat.numel(), dtype=torch.float32, device=flat.device)
    dist.all_gather_into_tensor(parts, flat, group=group)
    parts = parts.view((world,) + tuple(partial_f32.shape))
    total = parts[0].clone()
    for r in range(1, world):
        total += parts[r]
    return total.half()
