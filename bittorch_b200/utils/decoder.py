"""LLaMA-style ternary decoder: the caller of the ternary linear layers in a language model.

The reference's Python package stops at the layer; its only transformer is the browser runtime
(js/src/models/TernaryTransformer.ts).  This module restates that model's structure on top of the
layers of this package so that the kernels can be driven the way a model drives them (prefill over a
prompt, then one token at a time against a key/value cache):

* pre-norm blocks: ``x += attn(rmsnorm(x)); x += swiglu(rmsnorm(x))`` (TernaryTransformer.ts:366-464);
* RMSNorm with eps 1e-5 inside the square root (js/src/core/RMSNorm.ts:10-38);
* rotary embedding, theta 1e4, pairing element i with i + head_dim/2 (js/src/core/RoPE.ts:10-92),
  applied to the queries and to the keys as they enter the cache;
* grouped-query attention with one fused key/value projection whose output is ``[K | V]``
  (TernaryTransformer.ts:553-600);
* SwiGLU: ``w_down(silu(w_gate(x)) * w_up(x))`` (:520-550);
* every projection a bias-free ternary linear; embedding ``tok``, final ``norm`` and ``head`` in floating point;
* parameter names of the runtime's checkpoint (:141-188): ``tok.weight``, ``blocks.{i}.norm1.weight``,
  ``blocks.{i}.attn.{q_proj,kv_proj,proj}``, ``blocks.{i}.norm2.weight``, ``blocks.{i}.mlp.{w_gate,w_up,w_down}``,
  ``norm.weight``, ``head.weight``; after ``to_inference()`` the ternary layers hold ``weight_packed`` / ``scale``.

The layers are built as ``TernaryLinear`` (trainable masters; ``backend="python"`` runs anywhere);
``to_inference()`` swaps them for packed ``TernaryLinearInference`` layers on a CUDA device.

Two ways to run a single-token step: ``forward(tokens, cache, pos0)`` with the position as a Python integer
(shapes grow with the position), and ``decode_step(tokens, cache, pos)`` with the position in a device tensor and
every shape fixed (attention runs over the whole cache under a mask), which is what a CUDA graph can replay:
``GreedyDecodeGraph`` captures one such step, the arg-max and the position increment, so that a decoded token
costs one graph launch and no host synchronisation.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ..nn import TernaryLinear, TernaryLinearInference

NORM_EPS = 1e-5
ROPE_THETA = 10000.0


@dataclass
class DecoderConfig:
    vocab_size: int
    dim: int
    n_layers: int
    n_heads: int
    ffn_dim: int
    max_seq_len: int
    n_kv_heads: Optional[int] = None          # defaults to n_heads (TernaryTransformer.ts:116)
    threshold_factor: float = 0.05
    backend: str = "auto"
    one_weight_copy: bool = True              # inference form: keep only the tiled copy of every projection on the device
    fused_elementwise: bool = True            # inference form, integer path: residual add + RMSNorm and SiLU * up run inside the quantizer kernels

    def __post_init__(self) -> None:
        if self.n_kv_heads is None:
            self.n_kv_heads = self.n_heads
        if self.dim % self.n_heads or self.n_heads % self.n_kv_heads or (self.dim // self.n_heads) % 2:
            raise ValueError("dim must divide into an even head size and n_heads into n_kv_heads groups")

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads


class RMSNorm(nn.Module):
    """``x / sqrt(mean(x^2) + eps) * weight`` (js/src/core/RMSNorm.ts:10-38)."""

    def __init__(self, dim: int) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: Tensor) -> Tensor:
        xf = x.float()
        rms = torch.sqrt(xf.pow(2).mean(dim=-1, keepdim=True) + NORM_EPS)
        return ((xf / rms) * self.weight.float()).to(x.dtype)


def rope_tables(max_seq_len: int, head_dim: int, device=None) -> Tuple[Tensor, Tensor]:
    """cos / sin of ``pos * theta^(-2i/head_dim)``, shape [max_seq_len, head_dim/2] (js/src/core/RoPE.ts:25-49)."""
    half = head_dim // 2
    freq = 1.0 / torch.pow(torch.tensor(ROPE_THETA, dtype=torch.float64), torch.arange(half, dtype=torch.float64) * 2 / head_dim)
    angle = torch.arange(max_seq_len, dtype=torch.float64)[:, None] * freq[None, :]
    return angle.cos().float().to(device), angle.sin().float().to(device)


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor, pos0: int) -> Tensor:
    """x: [B, H, T, head_dim]; rotates (x[i], x[i + half]) by the angle of position pos0 + t (RoPE.ts:65-92)."""
    t = x.shape[2]
    half = x.shape[3] // 2
    c = cos[pos0:pos0 + t][None, None].to(x.dtype)
    s = sin[pos0:pos0 + t][None, None].to(x.dtype)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def apply_rope_at(x: Tensor, cos: Tensor, sin: Tensor, pos: Tensor) -> Tensor:
    """x: [B, H, 1, head_dim]; as ``apply_rope`` for the single position held in the device tensor ``pos`` [1]."""
    half = x.shape[3] // 2
    c = cos.index_select(0, pos)[None, None].to(x.dtype)             # [1, 1, 1, half]
    s = sin.index_select(0, pos)[None, None].to(x.dtype)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def fuse_inference_columns(layers, share: bool = False) -> TernaryLinearInference:
    """Packed layers that read the same input, as ONE layer with their output columns side by side.  Columns of a
    packed ternary layer are independent (own bytes, own scale; the activation quantizer depends on the input
    only), so the fused layer's outputs are the members' outputs concatenated, bit for bit - and a decode step
    pays one dependent kernel launch instead of one per member.

    ``share`` (every member's width a multiple of the 16-column tile): the fused layer and its members end up
    with ONE device copy of the weights between them.  The tiled layout is column-block major, so the fused tiled
    buffer is the members' tiled buffers one after the other; the members become compact modules whose tiled
    buffers are views into it, and nobody keeps a public packed buffer (state dicts rebuild it)."""
    k = layers[0].in_features
    if any(l.in_features != k for l in layers):
        raise ValueError("fused layers must read the same input")
    scale = torch.cat([l.scale for l in layers])
    bias = None
    if any(l.bias is not None for l in layers):
        bias = torch.cat([l.bias if l.bias is not None else torch.zeros_like(l.scale) for l in layers])
    n = sum(l.out_features for l in layers)
    if share and all(l.out_features % 16 == 0 for l in layers):
        parts = [l._derived()[0] for l in layers]               # each member's tiled buffer (built now if need be)
        tiled = torch.cat(parts)
        fused = TernaryLinearInference(k, n, torch.empty(0, dtype=torch.uint8, device=scale.device), scale, bias)
        fused.compact(tiled)
        offset = 0
        for l, part in zip(layers, parts):
            view = tiled[offset:offset + part.numel()]
            if l._compact:
                l._tiled, l._derived_key = view, None
            else:
                l.compact(view)
            offset += part.numel()
    else:
        wp = torch.cat([l.public_packed() for l in layers], dim=1).contiguous()
        fused = TernaryLinearInference(k, n, wp, scale, bias)
    fused.verify_buffers = False          # private copies: nobody else can write them
    return fused


class _FusedColumns:
    """Runs packed sibling layers as one (``fuse_inference_columns``), rebuilt when a member's buffers change.
    Not a submodule: the members keep their names and buffers in the state dict."""

    def __init__(self, *layers, share: bool = False) -> None:
        self.layers = layers
        self.share = share                    # one device copy of the weights for the fused layer and its members
        self._key = None
        self._fused: Optional[TernaryLinearInference] = None

    @property
    def usable(self) -> bool:
        return all(isinstance(l, TernaryLinearInference) for l in self.layers)

    def _members_key(self):
        from ..nn.ternary_linear_cuda import capturing, content_fingerprint

        key = tuple((l.weight_packed.data_ptr(), l.weight_packed._version, l.scale.data_ptr(), l.scale._version)
                    for l in self.layers)
        if all(l.verify_buffers for l in self.layers) and not capturing():
            # writes through .data leave addresses and versions alone: compare sampled contents too
            watched = [t for l in self.layers for t in ((l.scale,) if l._compact else (l.weight_packed, l.scale))]
            return key + content_fingerprint(*watched)
        if self._key is not None:
            return key + self._key[len(key):]
        return key

    def fused(self) -> TernaryLinearInference:
        """The fused layer, rebuilt if a member changed."""
        if self._members_key() != self._key:
            self._fused = fuse_inference_columns(self.layers, share=self.share)
            self._key = self._members_key()                   # after fusing: sharing replaces the members' buffers
        return self._fused

    def __call__(self, x: Tensor):
        return torch.split(self.fused()(x), [l.out_features for l in self.layers], dim=-1)


class Attention(nn.Module):
    def __init__(self, cfg: DecoderConfig) -> None:
        super().__init__()
        self.cfg = cfg
        kv_dim = cfg.n_kv_heads * cfg.head_dim
        mk = lambda i, o: TernaryLinear(i, o, bias=False, threshold_factor=cfg.threshold_factor, backend=cfg.backend)
        self.q_proj = mk(cfg.dim, cfg.dim)
        self.kv_proj = mk(cfg.dim, 2 * kv_dim)           # output [K | V], heads contiguous inside each half
        self.proj = mk(cfg.dim, cfg.dim)
        self._fused: Optional[_FusedColumns] = None

    def fused_columns(self) -> _FusedColumns:
        if self._fused is None or self._fused.layers != (self.q_proj, self.kv_proj):
            self._fused = _FusedColumns(self.q_proj, self.kv_proj, share=self.cfg.one_weight_copy)
        return self._fused

    def _heads(self, q: Tensor, kv: Tensor, b: int, t: int):
        """flat projections -> q [B, H, T, hd], k and v [B, Hkv, T, hd] (not yet rotated)."""
        cfg = self.cfg
        q = q.reshape(b, t, cfg.n_heads, cfg.head_dim).transpose(1, 2)
        kv = kv.reshape(b, t, 2, cfg.n_kv_heads, cfg.head_dim)
        return q, kv[:, :, 0].transpose(1, 2), kv[:, :, 1].transpose(1, 2)

    def _qkv(self, x: Tensor):
        b, t, _ = x.shape
        fused = self.fused_columns()
        if fused.usable:                                 # packed layers: one launch for both projections
            q, kv = fused(x)
        else:
            q, kv = self.q_proj(x), self.kv_proj(x)
        return self._heads(q, kv, b, t)

    def _attend(self, q: Tensor, k: Tensor, v: Tensor, cache: Tuple[Tensor, Tensor], pos0: int, cos: Tensor,
                sin: Tensor) -> Tensor:
        """Rotary embedding, cache update and causal attention for T tokens at positions pos0 .. -> [B, T, dim]."""
        cfg = self.cfg
        b, _, t, hd = q.shape
        nh, nkv = cfg.n_heads, cfg.n_kv_heads
        q = apply_rope(q, cos, sin, pos0)
        k_cache, v_cache = cache                                                 # [B, Hkv, max_seq_len, hd]
        k_cache[:, :, pos0:pos0 + t] = apply_rope(k, cos, sin, pos0).to(k_cache.dtype)   # keys are stored rotated
        v_cache[:, :, pos0:pos0 + t] = v.to(v_cache.dtype)
        keys = k_cache[:, :, :pos0 + t].to(q.dtype)
        vals = v_cache[:, :, :pos0 + t].to(q.dtype)
        # query at position pos0 + i sees keys 0 .. pos0 + i; query head h reads key/value head h // group
        # (enable_gqa).  The two common cases need no mask tensor: a pass from position 0 is plain causal
        # attention, a single token sees every key there is.
        if t == 1:
            mask, causal = None, False
        elif pos0 == 0:
            mask, causal = None, True
        else:
            mask, causal = torch.ones(t, pos0 + t, dtype=torch.bool, device=q.device).tril(diagonal=pos0), False
        out = F.scaled_dot_product_attention(q, keys, vals, attn_mask=mask, is_causal=causal, scale=1.0 / math.sqrt(hd),
                                             enable_gqa=nkv != nh)
        return out.transpose(1, 2).reshape(b, t, cfg.dim)

    def _attend_fixed(self, q: Tensor, k: Tensor, v: Tensor, cache: Tuple[Tensor, Tensor], pos: Tensor, cos: Tensor,
                      sin: Tensor) -> Tensor:
        """The same for ONE token per sequence at the position in the device tensor ``pos`` [1] (int64), with every
        shape independent of the position: the new key/value go into the cache with ``index_copy_`` and the query
        attends over the WHOLE cache with the positions after ``pos`` masked out.  The query heads of one key/value
        head are batched against it ([B, Hkv, group, hd] x [B, Hkv, S, hd]), so grouped-query attention copies
        nothing.  -> [B, 1, dim]"""
        cfg = self.cfg
        b = q.shape[0]
        hd, nh, nkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
        q = apply_rope_at(q, cos, sin, pos)
        k_cache, v_cache = cache
        k_cache.index_copy_(2, pos, apply_rope_at(k, cos, sin, pos).to(k_cache.dtype))
        v_cache.index_copy_(2, pos, v.to(v_cache.dtype))
        seq = k_cache.shape[2]
        qg = q.reshape(b, nkv, nh // nkv, hd)                                    # query head h = kv head * group + g
        scores = torch.matmul(qg, k_cache.to(q.dtype).transpose(2, 3)) * (1.0 / math.sqrt(hd))     # [B, Hkv, group, S]
        visible = torch.arange(seq, device=q.device) <= pos                      # [S]
        scores = scores.float().masked_fill(~visible, float("-inf"))
        out = torch.matmul(torch.softmax(scores, dim=-1).to(q.dtype), v_cache.to(q.dtype))          # [B, Hkv, group, hd]
        return out.reshape(b, 1, cfg.dim)

    def forward(self, x: Tensor, cache: Tuple[Tensor, Tensor], pos0: int, cos: Tensor, sin: Tensor) -> Tensor:
        q, k, v = self._qkv(x)
        return self.proj(self._attend(q, k, v, cache, pos0, cos, sin))

    def decode_step(self, x: Tensor, cache: Tuple[Tensor, Tensor], pos: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        """One token per sequence (x [B, 1, dim]) at the position in the device tensor ``pos``: fixed shapes."""
        q, k, v = self._qkv(x)
        return self.proj(self._attend_fixed(q, k, v, cache, pos, cos, sin))


class SwiGLU(nn.Module):
    def __init__(self, cfg: DecoderConfig) -> None:
        super().__init__()
        mk = lambda i, o: TernaryLinear(i, o, bias=False, threshold_factor=cfg.threshold_factor, backend=cfg.backend)
        self.w_gate = mk(cfg.dim, cfg.ffn_dim)
        self.w_up = mk(cfg.dim, cfg.ffn_dim)
        self.w_down = mk(cfg.ffn_dim, cfg.dim)
        self.cfg = cfg
        self._fused: Optional[_FusedColumns] = None

    def fused_columns(self) -> _FusedColumns:
        if self._fused is None or self._fused.layers != (self.w_gate, self.w_up):
            self._fused = _FusedColumns(self.w_gate, self.w_up, share=self.cfg.one_weight_copy)
        return self._fused

    def forward(self, x: Tensor) -> Tensor:
        fused = self.fused_columns()
        if fused.usable:                                 # packed layers: one launch for gate and up
            gate, up = fused(x)
        else:
            gate, up = self.w_gate(x), self.w_up(x)
        return self.w_down(F.silu(gate) * up)


class Block(nn.Module):
    def __init__(self, cfg: DecoderConfig) -> None:
        super().__init__()
        self.norm1 = RMSNorm(cfg.dim)
        self.attn = Attention(cfg)
        self.norm2 = RMSNorm(cfg.dim)
        self.mlp = SwiGLU(cfg)

    def forward(self, x: Tensor, cache, pos0: int, cos: Tensor, sin: Tensor) -> Tensor:
        x = x + self.attn(self.norm1(x), cache, pos0, cos, sin)
        return x + self.mlp(self.norm2(x))

    def decode_step(self, x: Tensor, cache, pos: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        x = x + self.attn.decode_step(self.norm1(x), cache, pos, cos, sin)
        return x + self.mlp(self.norm2(x))

    def fused_elementwise_ok(self) -> bool:
        """The block can run with its elementwise steps inside the quantizer kernels: every projection packed, the
        integer activation path selected."""
        from .._ext import require_ext

        layers = (self.attn.q_proj, self.attn.kv_proj, self.attn.proj, self.mlp.w_gate, self.mlp.w_up, self.mlp.w_down)
        return (self.attn.cfg.fused_elementwise and all(isinstance(l, TernaryLinearInference) for l in layers)
                and require_ext().activation_mode() == "int8")

    def forward_fused(self, x: Tensor, delta: Optional[Tensor], cache, pos, cos: Tensor, sin: Tensor, fixed: bool):
        """The block with its elementwise steps fused into the activation quantizer, so that every packed layer but
        ``proj`` starts from int8 rows (``bt_add_rmsnorm_quant``, ``bt_silu_mul_quant``):

            x += delta; q8 = quant(norm1(x))  ->  q, kv = [q_proj | kv_proj](q8)  ->  attention  ->  a = proj(.)
            x += a;     q8 = quant(norm2(x))  ->  gu = [w_gate | w_up](q8)  ->  h8 = quant(silu(gate) * up)  ->  d = w_down(h8)

        ``x`` [B, T, dim] is the residual stream, updated IN PLACE; ``delta`` is what the previous block's MLP still
        owes it (None for the first block).  Returns (x, d): the caller (next block, or the final norm) adds d.
        ``fixed``: one token at the position in the device tensor ``pos``; else T tokens from the integer ``pos``."""
        from .._ext import require_ext

        C = require_ext()
        b, t, d = x.shape
        x2d = x.view(b * t, d)
        xq, sx, xsum = C.add_rmsnorm_quant(x2d, None if delta is None else delta.reshape(b * t, d), self.norm1.weight, NORM_EPS)
        attn = self.attn
        qkv = attn.fused_columns().fused().forward_quantized(xq, sx, xsum, x.dtype)
        q, k, v = attn._heads(qkv[:, :attn.q_proj.out_features], qkv[:, attn.q_proj.out_features:], b, t)
        out = attn._attend_fixed(q, k, v, cache, pos, cos, sin) if fixed else attn._attend(q, k, v, cache, pos, cos, sin)
        a = attn.proj(out)
        xq, sx, xsum = C.add_rmsnorm_quant(x2d, a.reshape(b * t, d), self.norm2.weight, NORM_EPS)
        gate_up = self.mlp.fused_columns().fused().forward_quantized(xq, sx, xsum, x.dtype)     # [M, gate | up]
        hq, sh, hsum = C.silu_mul_quant(gate_up)
        down = self.mlp.w_down.forward_quantized(hq, sh, hsum, x.dtype)
        return x, down.view(b, t, d)


class TernaryDecoder(nn.Module):
    """Token ids -> logits, with a key/value cache for one-token-at-a-time decoding."""

    def __init__(self, cfg: DecoderConfig) -> None:
        super().__init__()
        self.cfg = cfg
        self.tok = nn.Embedding(cfg.vocab_size, cfg.dim)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.dim)
        self.head = nn.Linear(cfg.dim, cfg.vocab_size, bias=False)
        cos, sin = rope_tables(cfg.max_seq_len, cfg.head_dim)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def new_cache(self, batch: int, dtype: Optional[torch.dtype] = None) -> List[Tuple[Tensor, Tensor]]:
        cfg = self.cfg
        dev = self.tok.weight.device
        dtype = dtype or self.tok.weight.dtype
        shape = (batch, cfg.n_kv_heads, cfg.max_seq_len, cfg.head_dim)
        return [(torch.zeros(shape, dtype=dtype, device=dev), torch.zeros(shape, dtype=dtype, device=dev)) for _ in self.blocks]

    def forward(self, tokens: Tensor, cache: Optional[list] = None, pos0: int = 0, last_only: bool = False) -> Tensor:
        """tokens: [B, T] ids at positions pos0 .. pos0+T-1 -> logits [B, T, vocab]; ``cache`` (from ``new_cache``)
        is filled in place; without one the call is a stand-alone pass over the whole sequence.  ``last_only``: the
        final norm and the head run on the last position alone -> [B, 1, vocab] (what a prefill needs)."""
        b, t = tokens.shape
        if pos0 + t > self.cfg.max_seq_len:
            raise ValueError(f"positions up to {pos0 + t} exceed max_seq_len={self.cfg.max_seq_len}")
        if cache is None:
            if pos0 != 0:
                raise ValueError("a pass that does not start at position 0 needs the cache of the earlier positions")
            cache = self.new_cache(b)
        x = self.tok(tokens)
        if self._fused_blocks():
            return self._run_fused(x, cache, pos0, fixed=False, last_only=last_only)
        for block, layer_cache in zip(self.blocks, cache):
            x = block(x, layer_cache, pos0, self.rope_cos, self.rope_sin)
        return self.head(self.norm(x[:, -1:] if last_only else x))

    def _fused_blocks(self) -> bool:
        return len(self.blocks) > 0 and all(block.fused_elementwise_ok() for block in self.blocks)

    def _run_fused(self, x: Tensor, cache: list, pos, fixed: bool, last_only: bool = False) -> Tensor:
        x = x.contiguous()                                     # the embedding's output: a fresh tensor, updated in place
        delta = None
        for block, layer_cache in zip(self.blocks, cache):
            x, delta = block.forward_fused(x, delta, layer_cache, pos, self.rope_cos, self.rope_sin, fixed)
        if last_only:
            x, delta = x[:, -1:], delta[:, -1:]
        return self.head(self.norm(x + delta))

    def decode_step(self, tokens: Tensor, cache: list, pos: Tensor) -> Tensor:
        """tokens [B, 1] at the position held in the device tensor ``pos`` [1] (int64) -> logits [B, 1, vocab].
        Same result as ``forward(tokens, cache, int(pos))``, with shapes that do not depend on the position."""
        x = self.tok(tokens)
        if self._fused_blocks():
            return self._run_fused(x, cache, pos, fixed=True)
        for block, layer_cache in zip(self.blocks, cache):
            x = block.decode_step(x, layer_cache, pos, self.rope_cos, self.rope_sin)
        return self.head(self.norm(x))

    @torch.no_grad()
    def generate_greedy(self, prompt: Tensor, new_tokens: int) -> Tensor:
        """Prefill over ``prompt`` [B, T], then ``new_tokens`` greedy steps against the cache -> [B, T + new_tokens]."""
        b, t = prompt.shape
        cache = self.new_cache(b)
        out = [prompt]
        nxt = self.forward(prompt, cache, 0, last_only=True)[:, -1].argmax(dim=-1, keepdim=True)
        for i in range(new_tokens):
            out.append(nxt)
            if i + 1 < new_tokens:
                nxt = self.forward(nxt, cache, t + i)[:, -1].argmax(dim=-1, keepdim=True)
        return torch.cat(out, dim=1)

    def to_inference(self) -> "TernaryDecoder":
        """Replaces every ternary projection by its packed inference form (2-bit weights, fused kernels); the
        model must be on a CUDA device.  ``tok``, the norms and ``head`` stay in floating point."""
        from .convert import convert_linear_layers

        convert_linear_layers(self, skip_names=["head"], inplace=True)
        if self.cfg.one_weight_copy:
            # proj and w_down run on their own: drop their public buffers now; the fused pairs (q/kv, gate/up) share
            # one tiled buffer with their members the first time they run
            for block in self.blocks:
                block.attn.proj.compact()
                block.mlp.w_down.compact()
        return self


class GreedyDecodeGraph:
    """Greedy decoding with one CUDA-graph launch per token.

    The captured step reads the current tokens [B, 1] and the position from device buffers, runs
    ``TernaryDecoder.decode_step``, writes the arg-max back into the token buffer and advances the position, so
    consecutive replays decode consecutive tokens without the host looking at any result.  ``history`` [B,
    max_seq_len] receives every token at its position.  The model must be in its inference form on a CUDA device.
    """

    def __init__(self, model: TernaryDecoder, batch: int, cache: Optional[list] = None, capture=None) -> None:
        self.model = model
        dev = model.tok.weight.device
        self.cache = cache if cache is not None else model.new_cache(batch)
        self.tokens = torch.zeros((batch, 1), dtype=torch.long, device=dev)
        self.pos = torch.zeros((1,), dtype=torch.long, device=dev)
        self.history = torch.zeros((batch, model.cfg.max_seq_len), dtype=torch.long, device=dev)
        self.graph = None
        self._host_pos = 0
        self._capture = capture if capture is not None else _capture_cuda_graph

    @torch.no_grad()
    def _step(self) -> None:
        self.history.index_copy_(1, self.pos, self.tokens)
        logits = self.model.decode_step(self.tokens, self.cache, self.pos)
        self.tokens.copy_(logits[:, -1].argmax(dim=-1, keepdim=True))
        self.pos.add_(1)

    def start(self, tokens: Tensor, pos0: int) -> None:
        """Set the tokens [B, 1] to feed next and their position; captures the graph on first use.  The capture's
        warm-up calls run the step at ``pos0`` itself (they write scratch keys/values into that one cache slot, which
        the first real step overwrites before anything reads it)."""
        if not (0 <= pos0 < self.model.cfg.max_seq_len):
            raise ValueError(f"position {pos0} is outside the cache (max_seq_len={self.model.cfg.max_seq_len})")

        def reset() -> None:
            self.tokens.copy_(tokens)
            self.pos.fill_(pos0)

        reset()
        if self.graph is None:
            self.graph = self._capture(self._step, reset)
            reset()
        self._host_pos = pos0

    def run(self, steps: int) -> None:
        """Decode ``steps`` tokens: ``steps`` graph launches, nothing else."""
        if self.graph is None:
            raise RuntimeError("call start() first")
        if self._host_pos + steps > self.model.cfg.max_seq_len:
            raise ValueError(f"{steps} steps from position {self._host_pos} exceed max_seq_len={self.model.cfg.max_seq_len}")
        for _ in range(steps):
            self.graph.replay()
        self._host_pos += steps


def _capture_cuda_graph(step_fn, reset, warm: int = 3):
    """Runs ``step_fn`` a few times on a side stream (first calls build caches and must not be captured), calling
    ``reset`` after each, then captures one call into a CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warm):
            step_fn()
            reset()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step_fn()
    return graph
