"""Softmax attention with grouped key/value heads, key and value sizes of their own, projection biases, a rotation of
part of every query and key head, and an optional sliding window.

    q = W_q h + b_q, k = W_k h + b_k, v = W_v h + b_v            (one product; float32 results)
    the first rot.dims entries of every query and key head rotated by position (a "qk" position part, or none)
    score(i, j) = (q_i · k_j) · scale,  j ≤ i, and i − j < window where there is a window
    out = W_o · concat_h softmax_j(score) v_j

Queries and keys have `dim` entries a head, values `vdim`; query head h reads key/value head h // (heads / kv_heads).
Rotation angles, scores and softmax are float32; keys and values lie in the paged cache in the activation dtype.

The mixer is written in three stages so that another mixer can run it beside a second branch on the same input:
`in_weight` / `in_bias` (the rows of the input product), `core(proj, merged, …, factor)` (from the product's float32
result to the merged heads, times a factor, in the activation dtype; both may be column ranges of wider rows), and
`out_weight`.  `forward` chains the three."""
from __future__ import annotations

import torch

from ..cache import KVNeed
from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("mixer", "window_attention")
class WindowAttention:
    def __init__(self, w_q, w_k, w_v, w_out, *, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 b_q=None, b_k=None, b_v=None, window: int = 0, rotary=None):
        H, G = int(n_heads), int(n_kv_heads)
        if H <= 0 or G <= 0 or H % G != 0:
            raise ValueError(f"window attention: {H} heads cannot share {G} key/value heads")
        if tuple(w_q.shape)[0] != H * dim or tuple(w_k.shape)[0] != G * dim or tuple(w_v.shape)[0] != G * vdim:
            raise ValueError("window attention: W_q is [heads·dim, width], W_k [kv_heads·dim, width], W_v [kv_heads·vdim, width]")
        if w_out.shape[1] != H * vdim:
            raise ValueError("window attention: the output projection does not take the merged heads")
        if max(dim, vdim) > ops.WINDOW_HEAD_MAX:
            raise ValueError(f"window attention: head sizes {dim} and {vdim} are above the {ops.WINDOW_HEAD_MAX} the kernels take")
        if rotary is not None and (getattr(rotary, "where", None) != "qk" or rotary.dims > dim):
            raise ValueError("window attention: the rotation acts on queries and keys and on at most a head's entries")
        if window < 0:
            raise ValueError("window attention: a window is positive, or 0 for none")
        biases = (b_q, b_k, b_v)
        if any(b is not None for b in biases) and any(b is None for b in biases):
            raise ValueError("window attention: biases for all three projections or for none")
        self.n_heads, self.n_kv_heads, self.dim, self.vdim = H, G, int(dim), int(vdim)
        self.scale, self.window, self.rotary = float(scale), int(window), rotary
        self.q_off, self.k_off, self.v_off = 0, H * dim, H * dim + G * dim
        self.in_weight = torch.cat([w_q, w_k, w_v], dim=0).contiguous()
        self.in_bias = torch.cat([b.float() for b in biases]).contiguous() if b_q is not None else None
        self.in_width = self.in_weight.shape[0]
        self.out_weight = w_out
        self.merged_width = H * vdim

    def cache_need(self):
        kind = "window" if self.window > 0 else "full"
        return KVNeed(self.n_kv_heads, self.dim, kind, self.window, v_dim=self.vdim if self.vdim != self.dim else 0)

    fuses_norm = False
    leaves_row_stats = False

    def kernels(self, act_dtype: torch.dtype, block_tokens: int) -> dict:
        return ops.attention_window_kind(act_dtype, self.dim, self.vdim, self.n_heads, self.n_kv_heads)

    def core(self, proj, merged, ctx: StepContext, view, writes_cache: bool = True, factor: float = 1.0) -> None:
        T, H, G = ctx.n_tokens, self.n_heads, self.n_kv_heads
        q = ctx.ws.get("window_q", T, H * self.dim, ctx.act_dtype)
        freq = self.rotary.inv_freq if self.rotary is not None else None
        rot = self.rotary.dims if self.rotary is not None else 0
        ops.qkv_rope_append(proj, self.q_off, self.k_off, self.v_off, freq, rot, q, view.k, view.v, view.block_table, ctx.tok_slot,
                            ctx.tok_pos, T, H, G, self.dim, self.vdim, writes_cache, ctx.dev_err)
        ops.attention_window_step(q, view.k, view.v, view.block_table, merged, ctx, H, G, self.dim, self.vdim, self.scale,
                                  self.window, factor)

    def forward(self, h, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True, accumulate: bool = True) -> None:
        T = ctx.n_tokens
        proj = ctx.ws.get("window_in_proj", T, self.in_width, torch.float32)
        ops.linear(h, self.in_weight, self.in_bias, proj)
        merged = ctx.ws.get("attn_out", T, self.merged_width, ctx.act_dtype)
        self.core(proj, merged, ctx, view, writes_cache)
        ops.linear(merged, self.out_weight, None, x, residual=x if accumulate else None)
