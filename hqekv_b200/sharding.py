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


class PeerGather:
    """All-gather of the per-rank attention outputs done by the decode kernel itself.

    ``slots`` gathered buffers ``[world, B, nh_q/world, 1, D]`` (one per layer of a step, so that a
    layer's rows stay valid until the same layer of the next step) live in symmetric memory: every
    rank can store into every other rank's copy.  :meth:`decode` runs the fused decode with the peers'
    addresses of this rank's block (``hqkv_decode_attention_gather``: the kernel's last CTAs write the
    output rows locally and over NVLink to all peers, and the CTA that finishes last runs a bounded
    cross-GPU barrier), after which ``self.buffers[slot]`` holds all ranks' rows on every rank.  Everything is stream-ordered
    kernel launches with fixed arguments, so a step can be captured into a CUDA graph.

    Needs torch's symmetric memory (CUDA IPC between the GPUs of one node); construct it inside a
    try block and fall back to :func:`gather_head_outputs` (NCCL) when it is not available.
    """

    def __init__(self, slots: int, batch: int, nh_q_local: int, head_dim: int, device, group=None,
                 max_spins: int = 4_000_000):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm_mem
        from ._lib import lib  # fails loudly without the CUDA library
        self._lib, self._C = lib, C
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world - 1 > 7:
            raise ValueError("at most 8 ranks")
        block = batch * nh_q_local * head_dim
        self._block = block
        self._all = symm_mem.empty(slots * self.world * block, dtype=torch.float16, device=device)
        self._all.zero_()
        self._hdl = symm_mem.rendezvous(self._all, group)
        self.buffers = [self._all[s * self.world * block:(s + 1) * self.world * block]
                        .view(self.world, batch, nh_q_local, 1, head_dim) for s in range(slots)]
        # where THIS rank's block of slot s starts inside peer p's buffer
        base = [int(p) for p in self._hdl.buffer_ptrs]
        self._peers = [p for p in range(self.world) if p != self.rank]
        self._peer_args = []
        for s in range(slots):
            arr = (C.c_void_p * max(len(self._peers), 1))()
            for i, p in enumerate(self._peers):
                arr[i] = base[p] + 2 * ((s * self.world + self.rank) * block)
            self._peer_args.append(arr)
        # arrival counters: `world` 32-bit words in every rank's signal pad, away from the first words,
        # which torch's own symmetric-memory collectives use
        pad_off = 1024 if int(getattr(self._hdl, "signal_pad_size", 0)) >= 1024 + 4 * self.world else 0
        pads = (C.c_void_p * self.world)()
        for r in range(self.world):
            pads[r] = int(self._hdl.signal_pad_ptrs[r]) + pad_off
        self._pads = pads
        self._state = torch.zeros(4, dtype=torch.int32, device=device)  # call number, status, finished heads
        self._max_spins = max_spins
        # nobody may signal before every rank has zeroed its buffers and built its tables
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def local_block(self, slot: int) -> torch.Tensor:
        """This rank's rows inside its own gathered buffer ([B, nh_q/world, 1, D])."""
        return self.buffers[slot][self.rank]

    def decode(self, slot: int, q: torch.Tensor, past_key_value: tuple, block_size: int, group_size: int,
               quant_strategy: str = "uniform_group"):
        """Fused decode of this rank's heads; returns (attn_weights_local, gathered [world, B, nh_q/world, 1, D])."""
        from ._lib import CODEC_NORMAL, CODEC_UNIFORM, check, decode_workspace, stream_ptr
        from .quant._cache import cached_cache_desc
        low_codec = CODEC_UNIFORM if quant_strategy == "uniform_group" else CODEC_NORMAL
        desc, keep, L, dev = cached_cache_desc(past_key_value, q.shape[1], block_size, group_size, low_codec)
        q = q.contiguous()
        weights = torch.empty(q.shape[0], q.shape[1], 1, L, dtype=torch.float16, device=dev)
        out = self.local_block(slot)
        ws = decode_workspace(dev, self._lib.hqkv_decode_workspace_bytes(desc))
        st = stream_ptr(dev)
        check(self._lib.hqkv_decode_attention_gather(desc, q.data_ptr(), weights.data_ptr(), out.data_ptr(), ws.data_ptr(),
                                                     ws.numel(), self._peer_args[slot], len(self._peers), self._pads,
                                                     self.rank, self.world, self._state.data_ptr(), self._max_spins, st))
        return weights, self.buffers[slot]

    def status(self) -> int:
        """0, or 1 + the rank that some barrier gave up waiting for (synchronises the device)."""
        return int(self._state[1].item())


class FlaggedPeerGather:
    """The low-latency form of :class:`PeerGather`: values travel with the call number in 8-byte words.

    Per slot a RECEIVE buffer of ``world * entries`` 8-byte words lives in symmetric memory; the decode
    kernel of every rank stores {two fp16 values, call number} words into the peers' receive buffers
    (``hqkv_decode_attention_gather_flagged``), and ``hqkv_peer_unpack`` on every rank polls its own
    receive buffer, bounded, and writes the plain gathered tensor ``[world, B, nh_q/world, 1, D]``.
    No fence, signal or collective is involved; both launches have fixed arguments (CUDA-graph safe).
    A slot is reused only one full round of slots later, so ``slots`` must be at least 2.
    """

    def __init__(self, slots: int, batch: int, nh_q_local: int, head_dim: int, device, group=None,
                 max_spins: int = 4_000_000):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm_mem
        from ._lib import lib  # fails loudly without the CUDA library
        if slots < 2:
            raise ValueError("at least two slots: a receive buffer is reused only after the peers unpacked it")
        self._lib = lib
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if not 2 <= self.world <= 8:
            raise ValueError("2 to 8 ranks")
        block = batch * nh_q_local * head_dim
        self._entries = block // 2
        words = slots * self.world * self._entries * 2  # int32 words
        self._recv = symm_mem.empty(words, dtype=torch.int32, device=device)
        self._recv.zero_()
        self._hdl = symm_mem.rendezvous(self._recv, group)
        self.buffers = [torch.zeros(self.world, batch, nh_q_local, 1, head_dim, dtype=torch.float16, device=device)
                        for _ in range(slots)]
        base = [int(p) for p in self._hdl.buffer_ptrs]
        self._peers = [p for p in range(self.world) if p != self.rank]
        self._peer_args, self._recv_ptr = [], []
        for s in range(slots):
            arr = (C.c_void_p * len(self._peers))()
            for i, p in enumerate(self._peers):
                arr[i] = base[p] + 8 * ((s * self.world + self.rank) * self._entries)
            self._peer_args.append(arr)
            self._recv_ptr.append(base[self.rank] + 8 * (s * self.world * self._entries))
        self._state = torch.zeros(2, dtype=torch.int32, device=device)  # call number, status
        self._max_spins = max_spins
        torch.cuda.synchronize(device)
        dist.barrier(group)  # nobody sends before every receive buffer is zero

    def decode(self, slot: int, q: torch.Tensor, past_key_value: tuple, block_size: int, group_size: int,
               quant_strategy: str = "uniform_group"):
        """Fused decode of this rank's heads; returns (attn_weights_local, gathered [world, B, nh_q/world, 1, D])."""
        from ._lib import CODEC_NORMAL, CODEC_UNIFORM, check, decode_workspace, stream_ptr
        from .quant._cache import cached_cache_desc
        low_codec = CODEC_UNIFORM if quant_strategy == "uniform_group" else CODEC_NORMAL
        desc, keep, L, dev = cached_cache_desc(past_key_value, q.shape[1], block_size, group_size, low_codec)
        q = q.contiguous()
        weights = torch.empty(q.shape[0], q.shape[1], 1, L, dtype=torch.float16, device=dev)
        gathered = self.buffers[slot]
        out = gathered[self.rank]
        ws = decode_workspace(dev, self._lib.hqkv_decode_workspace_bytes(desc))
        st = stream_ptr(dev)
        check(self._lib.hqkv_decode_attention_gather_flagged(desc, q.data_ptr(), weights.data_ptr(), out.data_ptr(),
                                                             ws.data_ptr(), ws.numel(), self._peer_args[slot],
                                                             len(self._peers), self._state.data_ptr(), st))
        check(self._lib.hqkv_peer_unpack(self._recv_ptr[slot], gathered.data_ptr(), self.rank, self.world, self._entries,
                                         self._state.data_ptr(), self._max_spins, st))
        return weights, gathered

    def status(self) -> int:
        """0, or 1 + the rank that some unpack gave up waiting for (synchronises the device)."""
        return int(self._state[1].item())
