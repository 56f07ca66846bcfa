"""Attention module that drives the tiered cache: the caller of the decode path.

Restates, with plain torch modules and no dependency on a transformers release, what
``LlamaAttention_hqe.forward`` (model/llama_hqe.py:96-251) and ``Qwen3Attention_hqe.forward``
(model/qwen3_hqe.py:116-279, the same with an RMSNorm on every q / k head before the rotary embedding)
do around the path this package implements:

* prefill: dense causal attention; the probabilities of the last 20 queries seed the importance ring;
  the cache tuple starts as 39 empty slots + (K, V, length);
* decode: the new K / V row is appended to the fp16 residual window and ``qkv_matmul_hqe_2`` attends
  over all tiers; the head-summed probability row goes into the ring;
* whenever 32 or more tokens are unquantised: rank blocks by importance, derive the six tier counts
  from the configured shares (:class:`TierSchedule`), and flush with ``KV_cache_hqe_2``.

Signature and results of ``forward`` are the reference's: ``(attn_output, attn_weights | None,
past_key_value, auxiliary_parameters)`` where ``auxiliary_parameters = (compress_ratio, K_bit_num,
V_bit_num)`` is computed by the first layer of a model and handed to the others.
"""
from typing import Optional, Tuple

import torch
from torch import nn

from ..quant.hqe_2 import KV_cache_hqe_2
from ..quant.hqe_matmul import qkv_matmul_hqe_2
from .public_func import get_block_token_idx, last_attn_weights, make_sum_equal

BLOCK = 32          # tokens per ranking block = K group = V group on this path (model/llama_hqe.py:208,230)
FP16_TOKENS = 64    # tokens the 16-bit tier keeps (model/llama_hqe.py:217)
SEED_QUERIES = 20   # prefill queries whose probabilities seed the ring (model/llama_hqe.py:124)


class TierSchedule:
    """The data-independent part of the flush decision (model/llama_hqe.py:58-80, 205-241): how many
    tokens are unquantised, how many are cached, and from the configured shares (``bit_0`` evicted,
    ``bit_4`` / ``bit_2`` / ``bit_1`` in the 4 / 2 / 1-bit tiers; 64 tokens in fp16, none in 8 bits) the six
    counts ``[16, 8, 4, 2, 1 bit, evicted]`` of the next flush.  All arithmetic is float32 tensor
    arithmetic in the reference's order of operations, because the rounding decides block counts."""

    def __init__(self, bit_0: float, bit_4: float, bit_2: float, bit_1: float):
        # host-side bookkeeping: CPU tensors whatever the default device is
        self.ratio_e_0 = torch.tensor([bit_0], dtype=torch.float32, device="cpu")
        self.ratio_e = self.ratio_e_0.clone()
        self.ratio_q = torch.tensor([bit_4, bit_2, bit_1], dtype=torch.float32, device="cpu")
        self.current_length = 0           # tokens in the fp16 residual window
        self.history_reserve_length = 0   # tokens in the tiers

    def append(self, n_tokens: int):
        self.current_length += n_tokens

    def due(self) -> bool:
        return self.current_length >= BLOCK

    def lengths(self):
        """(compress_length, total_length, block_num) of a flush that is due."""
        compress = self.current_length - self.current_length % BLOCK
        total = self.history_reserve_length + compress
        return compress, total, total // BLOCK

    def counts(self):
        """(compress_ratio, bit_num): shares and token counts of the flush that is due."""
        _, total, block_num = self.lengths()
        head = torch.tensor([FP16_TOKENS / total, 0], dtype=torch.float32, device="cpu")
        ratio = torch.cat((head, self.ratio_q, self.ratio_e))
        ratio[2:] = (1 - ratio[0]) * ratio[2:]
        bit_num = torch.round(block_num * ratio).to(torch.int)
        bit_num = make_sum_equal(bit_num, block_num)
        bit_num *= BLOCK
        return ratio, bit_num

    def commit(self, evicted: int, rescale: bool):
        """Account for a finished flush; ``rescale``: this layer owns the shares (no auxiliary parameters
        were handed in), so the eviction share is re-based on the tokens the next flush will add."""
        compress, _, _ = self.lengths()
        self.history_reserve_length += compress - evicted
        self.current_length -= compress
        if rescale:
            nxt = (self.history_reserve_length + BLOCK) // BLOCK * BLOCK
            add = nxt - self.history_reserve_length
            self.ratio_e = (add * self.ratio_e_0) / (self.history_reserve_length + add)
            self.ratio_q = (1 - self.ratio_e) * self.ratio_q / self.ratio_q.sum()

    def reset(self):
        self.ratio_e = self.ratio_e_0.clone()
        self.current_length = 0
        self.history_reserve_length = 0


class HeadRMSNorm(nn.Module):
    """RMSNorm over the last dimension with fp32 statistics (Qwen3's q_norm / k_norm, Llama's layer norms)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        dt = x.dtype
        x = x.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * x.to(dt)


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary(q, k, cos, sin):
    """q, k [B, heads, S, D]; cos, sin [B, S, D] (the half-split rotary layout of Llama / Qwen3)."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def rotary_tables(positions: torch.Tensor, head_dim: int, theta: float = 500000.0, dtype=torch.float16):
    """cos, sin [B, S, D] for integer positions [B, S]."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    ang = positions.float().unsqueeze(-1) * inv
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def causal_mask(q_len: int, kv_len: int, dtype, device):
    """Additive mask [1, 1, q_len, kv_len] for queries that are the last q_len of kv_len positions."""
    i = torch.arange(kv_len - q_len, kv_len, device=device).unsqueeze(1)
    j = torch.arange(kv_len, device=device).unsqueeze(0)
    m = torch.zeros(q_len, kv_len, dtype=dtype, device=device)
    return m.masked_fill(j > i, torch.finfo(dtype).min).view(1, 1, q_len, kv_len)


class HqeAttention(nn.Module):
    """One attention layer with the tiered KV cache.

    ``quant_strategy``: 'uniform_group' or 'high_uniform_group_low_normal_group'; ``times_range``: rank V
    blocks by importance x value range.  ``qk_norm=True`` gives the Qwen3 flavour.  Per-sequence state
    (ring, lengths, shares) lives on the module as in the reference; call :meth:`reset` between sequences
    and :meth:`set_max_length` before the prefill."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int = 128,
                 quant_strategy: str = "high_uniform_group_low_normal_group", times_range: bool = True,
                 bit_0: float = 0.25, bit_4: float = 0.25, bit_2: float = 0.25, bit_1: float = 0.25,
                 qk_norm: bool = False, rms_eps: float = 1e-6, bias: bool = False):
        super().__init__()
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.num_key_value_groups = num_heads // num_kv_heads
        self.scaling = head_dim ** -0.5
        self.quant_strategy, self.times_range = quant_strategy, times_range
        self.q_proj = nn.Linear(hidden_size, num_heads * head_dim, bias=bias)
        self.k_proj = nn.Linear(hidden_size, num_kv_heads * head_dim, bias=bias)
        self.v_proj = nn.Linear(hidden_size, num_kv_heads * head_dim, bias=bias)
        self.o_proj = nn.Linear(num_heads * head_dim, hidden_size, bias=bias)
        self.q_norm = HeadRMSNorm(head_dim, rms_eps) if qk_norm else None
        self.k_norm = HeadRMSNorm(head_dim, rms_eps) if qk_norm else None
        self.schedule = TierSchedule(bit_0, bit_4, bit_2, bit_1)
        self.last_weights = last_attn_weights(last_length=SEED_QUERIES)

    # -- per-sequence state ---------------------------------------------------------------------
    def reset(self):
        self.schedule.reset()
        self.last_weights.reset()

    def set_max_length(self, max_length: int):
        self.last_weights.set_max_length(max_length)

    @property
    def current_length(self):
        return self.schedule.current_length

    @property
    def history_reserve_length(self):
        return self.schedule.history_reserve_length

    # -- pieces ---------------------------------------------------------------------------------
    def _project(self, hidden_states, position_embeddings):
        B, S, _ = hidden_states.shape
        shape = (B, S, -1, self.head_dim)
        q = self.q_proj(hidden_states).view(shape)
        k = self.k_proj(hidden_states).view(shape)
        v = self.v_proj(hidden_states).view(shape).transpose(1, 2)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        cos, sin = position_embeddings
        q, k = apply_rotary(q, k, cos, sin)
        return q, k, v

    def _prefill(self, q, k, v, attention_mask):
        """Dense causal attention for the output; probabilities of the last SEED_QUERIES queries (fp32 softmax,
        rounded to the activations' dtype) for the ring — what the reference's flash branch computes
        (model/llama_hqe.py:141-166); its eager branch (:168-182) produces the same rows inside a full
        [S, S] matrix."""
        B, nh, S, Dh = q.shape
        rep = self.num_key_value_groups
        out = nn.functional.scaled_dot_product_attention(q, k, v, is_causal=S > 1, scale=self.scaling, enable_gqa=rep > 1)
        tail = min(S, SEED_QUERIES)
        # query heads of one kv head are adjacent: [B, kv, rep * tail, D] x [B, kv, D, S]
        qt = q[:, :, -tail:, :].reshape(B, self.num_kv_heads, rep * tail, Dh)
        scores = (torch.matmul(qt, k.transpose(2, 3)) * self.scaling).view(B, nh, tail, S)
        if attention_mask is not None:
            scores = scores + attention_mask[:, :, -tail:, :]
            scores = torch.max(scores, torch.tensor(torch.finfo(scores.dtype).min, device=scores.device))
        weights = nn.functional.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
        return weights, out

    def _flush(self, past_key_value, auxiliary_parameters):
        sch = self.schedule
        compress, total, block_num = sch.lengths()
        importance = self.last_weights.calculate_token_importance()
        own_shares = auxiliary_parameters is None
        if own_shares:
            ratio, k_bits = sch.counts()
            v_bits = k_bits.clone()
        else:
            ratio, k_bits, v_bits = auxiliary_parameters
        evicted = int(k_bits[-1])
        ranked = importance[:total].clone()
        k_ids = get_block_token_idx(BLOCK, block_num, ranked)
        past_key_value = KV_cache_hqe_2(past_key_value, compress, sch.history_reserve_length, k_ids, k_bits, v_bits,
                                        ranked, self.quant_strategy, self.last_weights, BLOCK, BLOCK, self.times_range)
        sch.commit(evicted, own_shares)
        return past_key_value, (ratio, k_bits, v_bits)

    # -- the layer ------------------------------------------------------------------------------
    def attend(self, q, k, v, attention_mask=None, past_key_value=None, auxiliary_parameters=None):
        """Everything between the projections: cache append, attention, ring update, flush when due.
        q [B, nh, S, D], k / v [B, nkv, S, D] already normalised and rotated.  Returns (context [B, S, nh*D],
        attn_weights, past_key_value, auxiliary_parameters)."""
        B, _, S, _ = q.shape
        kv_seq_len = S
        self.schedule.append(S)
        if past_key_value is not None:
            kv_seq_len += past_key_value[-1]
            new_k = k if past_key_value[-3] is None else torch.cat((past_key_value[-3], k), dim=2)
            new_v = v if past_key_value[-2] is None else torch.cat((past_key_value[-2], v), dim=2)
            past_key_value = tuple(past_key_value[:-3]) + (new_k, new_v, kv_seq_len)
            attn_weights, attn_output = qkv_matmul_hqe_2(q, past_key_value, attention_mask, self.head_dim,
                                                         self.quant_strategy, BLOCK, BLOCK)
        else:
            attn_weights, attn_output = self._prefill(q, k, v, attention_mask)
            past_key_value = (None,) * 39 + (k, v, kv_seq_len)
        context = attn_output.transpose(1, 2).reshape(B, S, self.num_heads * self.head_dim)

        # The ring row of the step: one more launch over the probabilities just written (still in L2).  The decode
        # call can write the row itself (qkv_matmul_hqe_2(head_sum_out=...)), one launch less, but measured slower
        # at batch 1: the last CTA to finish a chunk then gathers that chunk's 16 k probabilities alone, while this
        # launch spreads the same gathers over the whole GPU (37.5 against 26.4 us per layer at 32 k context).
        self.last_weights.update(attn_weights)
        if self.schedule.due():
            past_key_value, auxiliary_parameters = self._flush(past_key_value, auxiliary_parameters)
        else:
            auxiliary_parameters = None
        return context, attn_weights, past_key_value, auxiliary_parameters

    def forward(self, hidden_states: torch.Tensor, position_embeddings: Tuple[torch.Tensor, torch.Tensor],
                attention_mask: Optional[torch.Tensor] = None, past_key_value: Optional[tuple] = None,
                auxiliary_parameters: Optional[tuple] = None, output_attentions: bool = False, use_cache: bool = True):
        q, k, v = self._project(hidden_states, position_embeddings)
        context, attn_weights, past_key_value, auxiliary_parameters = self.attend(q, k, v, attention_mask, past_key_value,
                                                                                 auxiliary_parameters)
        return self.o_proj(context), (attn_weights if output_attentions else None), \
            (past_key_value if use_cache else None), auxiliary_parameters
