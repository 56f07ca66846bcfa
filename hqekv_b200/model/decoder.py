"""Decoder stack around :class:`HqeAttention`: the model-level caller of the decode path.

Plain torch restatement of what ``LlamaDecoderLayer_hqe`` / ``LlamaModel_hqe``
(model/llama_hqe.py:255-440) and their Qwen3 twins do with the attention layer: pre-norm residual
blocks (RMSNorm -> attention -> RMSNorm -> SwiGLU MLP), one cache tuple per layer, and the
``auxiliary_parameters`` (tier counts) of the first layer handed to all the others so that every layer
flushes with the same counts (:407-430).  Weights are whatever the caller loads; nothing here depends on
a transformers release.
"""
from dataclasses import dataclass
from typing import List, Optional

import torch
from torch import nn

from .attention_hqe import HeadRMSNorm, HqeAttention, rotary_tables


@dataclass
class DecoderConfig:
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    qk_norm: bool = False          # Qwen3: RMSNorm on every q / k head
    vocab_size: int = 0            # 0: no embedding / lm_head (hidden states in, hidden states out)
    quant_strategy: str = "high_uniform_group_low_normal_group"
    times_range: bool = True
    bit_0: float = 0.25
    bit_4: float = 0.25
    bit_2: float = 0.25
    bit_1: float = 0.25


LLAMA31_8B = DecoderConfig()
QWEN3_8B = DecoderConfig(intermediate_size=12288, num_layers=36, rms_eps=1e-6, rope_theta=1000000.0, qk_norm=True)


class SwiGLU(nn.Module):
    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        return self.down_proj(nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class HqeDecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.self_attn = HqeAttention(cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.quant_strategy,
                                      cfg.times_range, cfg.bit_0, cfg.bit_4, cfg.bit_2, cfg.bit_1, cfg.qk_norm, cfg.rms_eps)
        self.mlp = SwiGLU(cfg.hidden_size, cfg.intermediate_size)
        self.input_layernorm = HeadRMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.post_attention_layernorm = HeadRMSNorm(cfg.hidden_size, cfg.rms_eps)

    def forward(self, hidden_states, position_embeddings, attention_mask, past_key_value, auxiliary_parameters):
        h, _, past_key_value, auxiliary_parameters = self.self_attn(
            self.input_layernorm(hidden_states), position_embeddings, attention_mask, past_key_value, auxiliary_parameters)
        hidden_states = hidden_states + h
        hidden_states = hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))
        return hidden_states, past_key_value, auxiliary_parameters


class HqeDecoder(nn.Module):
    """Stack of decoder layers with per-layer tiered caches.  ``forward(inputs, caches, position)`` takes token
    ids [B, S] (``vocab_size > 0``) or hidden states [B, S, hidden]; returns (logits or hidden states, caches)."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size) if cfg.vocab_size else None
        self.layers = nn.ModuleList(HqeDecoderLayer(cfg) for _ in range(cfg.num_layers))
        self.norm = HeadRMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False) if cfg.vocab_size else None

    def start_sequence(self, max_length: int):
        """Forget the previous sequence and size the importance rings (model/llama_hqe.py:557, 691-695)."""
        for layer in self.layers:
            layer.self_attn.reset()
            layer.self_attn.set_max_length(max_length)

    def forward(self, inputs: torch.Tensor, caches: Optional[List[tuple]] = None, position: int = 0,
                auxiliary_parameters: Optional[tuple] = None):
        """``auxiliary_parameters``: (shares, K counts, V counts) to flush with instead of the counts the first
        layer derives from its configured shares (the reference's layers accept them the same way)."""
        x = self.embed_tokens(inputs) if self.embed_tokens is not None else inputs
        B, S, _ = x.shape
        pos = torch.arange(position, position + S, device=x.device).unsqueeze(0).expand(B, S)
        rope = rotary_tables(pos, self.cfg.head_dim, self.cfg.rope_theta, x.dtype)
        caches = [None] * len(self.layers) if caches is None else list(caches)
        aux = auxiliary_parameters  # None: the first layer derives the tier counts, the others reuse them
        for i, layer in enumerate(self.layers):
            x, caches[i], aux = layer(x, rope, None, caches[i], aux)
        x = self.norm(x)
        return (self.lm_head(x) if self.lm_head is not None else x), caches


class GraphedDecodeStep:
    """Single-token decode of an :class:`HqeDecoder` with the dense parts replayed from CUDA graphs.

    Between two layers' cache accesses everything has static shapes: o_proj + residual + norm + MLP of layer
    i and norm + q/k/v projections + rotary of layer i+1.  Each such segment is captured once into a CUDA
    graph over static buffers; per layer the host then issues one graph replay plus the cache-facing calls
    (append to the residual window, ``qkv_matmul_hqe_2``, ring update, the flush when it is due), whose
    shapes change from step to step.  Results are those of ``HqeDecoder.forward`` on a [B, 1, hidden] input.

    ``fused=True`` (default) also shortens the dense parts themselves: the q / k / v projection weights of a layer
    are moved into one matrix (the three ``nn.Linear`` weights become views of it), likewise gate / up, so a
    single-row step runs two wide GEMVs instead of five narrow ones; RMSNorm is one fused kernel; the rotary
    embedding is applied to q and k together as x * cos + roll(x, D/2) * (+-sin)."""

    def __init__(self, model: HqeDecoder, batch: int, fused: bool = True):
        cfg, self.model = model.cfg, model
        self.fused = fused
        p = next(model.parameters())
        dev, dt = p.device, p.dtype
        z = lambda *shape: torch.zeros(*shape, device=dev, dtype=dt)  # noqa: E731
        n = len(model.layers)
        self.x = z(batch, 1, cfg.hidden_size) if model.embed_tokens is None else None
        self.ids = torch.zeros(batch, 1, dtype=torch.long, device=dev) if model.embed_tokens is not None else None
        self.h = z(batch, 1, cfg.hidden_size)            # residual stream
        self.cos, self.sin = z(batch, 1, cfg.head_dim), z(batch, 1, cfg.head_dim)
        self.q = [z(batch, cfg.num_heads, 1, cfg.head_dim) for _ in range(n)]
        self.k = [z(batch, cfg.num_kv_heads, 1, cfg.head_dim) for _ in range(n)]
        self.v = [z(batch, cfg.num_kv_heads, 1, cfg.head_dim) for _ in range(n)]
        self.ctx = [z(batch, 1, cfg.num_heads * cfg.head_dim) for _ in range(n)]
        self.out = z(batch, 1, cfg.vocab_size or cfg.hidden_size)
        self.pos = torch.zeros(batch, 1, dtype=torch.long, device=dev)
        self.sin_signed = z(batch, 1, 1, cfg.head_dim)
        self.wqkv, self.wgu, self.qk_weight = [], [], []
        if fused:
            for layer in model.layers:
                self._fuse(layer)
        self.graphs = []
        self._capture()

    @torch.no_grad()
    def _fuse(self, layer):
        """Move q/k/v (and gate/up) weights into one matrix each; the Linear modules keep working on views."""
        a, m = layer.self_attn, layer.mlp
        for mods, store in (((a.q_proj, a.k_proj, a.v_proj), self.wqkv), ((m.gate_proj, m.up_proj), self.wgu)):
            w = torch.cat([x.weight for x in mods], dim=0)
            at = 0
            for x in mods:
                n = x.weight.shape[0]
                x.weight = nn.Parameter(w[at:at + n], requires_grad=False)
                at += n
            store.append(w)
        if a.q_norm is not None:  # per-head RMSNorm weights of the q heads, then of the k heads
            self.qk_weight.append(torch.cat((a.q_norm.weight.expand(a.num_heads, -1),
                                             a.k_norm.weight.expand(a.num_kv_heads, -1)), dim=0).contiguous())
        else:
            self.qk_weight.append(None)

    @staticmethod
    def _norm(x, mod):
        return nn.functional.rms_norm(x, (x.shape[-1],), mod.weight, mod.eps)

    def _pre(self, i):
        layer = self.model.layers[i]
        a = layer.self_attn
        if not self.fused:
            q, k, v = a._project(layer.input_layernorm(self.h), (self.cos, self.sin))
            self.q[i].copy_(q)
            self.k[i].copy_(k)
            self.v[i].copy_(v)
            return
        B, nh, nkv, D = self.h.shape[0], a.num_heads, a.num_kv_heads, a.head_dim
        qkv = nn.functional.linear(self._norm(self.h, layer.input_layernorm), self.wqkv[i]).view(B, 1, nh + 2 * nkv, D)
        qk = qkv[:, :, :nh + nkv]
        if self.qk_weight[i] is not None:
            qk = nn.functional.rms_norm(qk, (D,), None, a.q_norm.eps) * self.qk_weight[i]
        qk = qk * self.cos.unsqueeze(2) + torch.roll(qk, D // 2, -1) * self.sin_signed
        self.q[i].copy_(qk[:, :, :nh].transpose(1, 2))
        self.k[i].copy_(qk[:, :, nh:].transpose(1, 2))
        self.v[i].copy_(qkv[:, :, nh + nkv:].transpose(1, 2))

    def _post(self, i):
        layer = self.model.layers[i]
        self.h.add_(layer.self_attn.o_proj(self.ctx[i]))
        if not self.fused:
            self.h.add_(layer.mlp(layer.post_attention_layernorm(self.h)))
            return
        g, u = nn.functional.linear(self._norm(self.h, layer.post_attention_layernorm), self.wgu[i]).chunk(2, dim=-1)
        self.h.add_(layer.mlp.down_proj(nn.functional.silu(g) * u))

    def _segment(self, s):
        n = len(self.model.layers)
        if s == 0:
            m = self.model
            self.h.copy_(m.embed_tokens(self.ids) if m.embed_tokens is not None else self.x)
            cos, sin = rotary_tables(self.pos, m.cfg.head_dim, m.cfg.rope_theta, self.h.dtype)
            self.cos.copy_(cos)
            self.sin.copy_(sin)
            half = m.cfg.head_dim // 2  # rotate_half(x) = roll(x, D/2) with the first half negated
            self.sin_signed.copy_(torch.cat((-sin[..., :half], sin[..., half:]), dim=-1).unsqueeze(2))
        else:
            self._post(s - 1)
        if s < n:
            self._pre(s)
        else:
            y = self._norm(self.h, self.model.norm) if self.fused else self.model.norm(self.h)
            self.out.copy_(self.model.lm_head(y) if self.model.lm_head is not None else y)

    @torch.no_grad()
    def _capture(self):
        n = len(self.model.layers)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # library workspaces and autotuning happen outside the capture
            for s in range(n + 1):
                self._segment(s)
        torch.cuda.current_stream().wait_stream(side)
        pool = None
        for s in range(n + 1):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool):
                self._segment(s)
            pool = g.pool()
            self.graphs.append(g)

    @torch.no_grad()
    def __call__(self, inputs: torch.Tensor, caches: List[tuple], position: int,
                 auxiliary_parameters: Optional[tuple] = None):
        (self.ids if self.ids is not None else self.x).copy_(inputs)
        self.pos.fill_(position)
        caches = list(caches)
        aux = auxiliary_parameters
        self.graphs[0].replay()
        for i, layer in enumerate(self.model.layers):
            k, v = self.k[i], self.v[i]
            if caches[i][-3] is None:  # an empty residual window would adopt the static rows as its storage
                k, v = k.clone(), v.clone()
            ctx, _, caches[i], aux = layer.self_attn.attend(self.q[i], k, v, None, caches[i], aux)
            self.ctx[i].copy_(ctx)
            self.graphs[i + 1].replay()
        return self.out.clone(), caches


def init_like_pretrained(model: nn.Module, seed: int = 0):
    """Random weights with the scale of a trained transformer (projection rows of unit norm in expectation),
    drawn on the module's device: stands in for a checkpoint where none can be loaded."""
    gen = torch.Generator(device=next(model.parameters()).device).manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 2:
                p.copy_(torch.randn(p.shape, generator=gen, device=p.device, dtype=torch.float32).mul_(p.shape[1] ** -0.5))
    return model
