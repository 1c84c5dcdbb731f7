"""Two mixers side by side on the same input: out = left_scale · left(h) + right_scale · right(h).

Both branches must be written in stages (`in_weight`, `in_bias`, `core`, `out_weight`; see parts/window_attention.py and
parts/state_space.py).  Their input products are one product, their cores write side by side into one matrix of merged
rows (each times its scale, before the rounding to the activation dtype), and the two output projections are one
product over the concatenated rows: W_o,left (s_l · m_l) + W_o,right (s_r · m_r) = [W_o,left | W_o,right] [s_l m_l ; s_r m_r].
What the branches keep per sequence is a tuple of their needs."""
from __future__ import annotations

import torch

from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("mixer", "parallel")
class ParallelMixer:
    fuses_norm = False
    leaves_row_stats = False

    def __init__(self, left, right, *, left_scale: float = 1.0, right_scale: float = 1.0):
        for b in (left, right):
            for name in ("in_weight", "core", "out_weight", "merged_width", "in_width"):
                if not hasattr(b, name):
                    raise ValueError(f"parallel mixer: {type(b).__name__} is not written in stages (no {name})")
        if left.out_weight.shape[0] != right.out_weight.shape[0] or left.in_weight.shape[1] != right.in_weight.shape[1]:
            raise ValueError("parallel mixer: the branches read and write rows of different widths")
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.in_weight = torch.cat([left.in_weight, right.in_weight], dim=0).contiguous()
        self.in_bias = None
        if left.in_bias is not None or right.in_bias is not None:
            dev = self.in_weight.device
            zeros = lambda n: torch.zeros(n, dtype=torch.float32, device=dev)   # noqa: E731
            self.in_bias = torch.cat([left.in_bias if left.in_bias is not None else zeros(left.in_width),
                                      right.in_bias if right.in_bias is not None else zeros(right.in_width)]).contiguous()
        self.out_weight = torch.cat([left.out_weight, right.out_weight], dim=1).contiguous()
        self.in_width = left.in_width + right.in_width
        self.merged_width = left.merged_width + right.merged_width

    def cache_need(self):
        needs = tuple(n for n in (self.left.cache_need(), self.right.cache_need()))
        return needs

    def kernels(self, act_dtype: torch.dtype, block_tokens: int) -> dict:
        for b in (self.left, self.right):
            if hasattr(b, "kernels"):
                return b.kernels(act_dtype, block_tokens)
        return {"prompt": "none", "decode": "none"}

    def forward(self, h, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True, accumulate: bool = True) -> None:
        T, ws = ctx.n_tokens, ctx.ws
        proj = ws.get("parallel_in_proj", T, self.in_width, torch.float32)
        ops.linear(h, self.in_weight, self.in_bias, proj)
        merged = ws.get("parallel_merged", T, self.merged_width, ctx.act_dtype)
        nl, ml = self.left.in_width, self.left.merged_width
        self.left.core(proj[:, :nl], merged[:, :ml], ctx, view.parts[0], writes_cache, self.left_scale)
        self.right.core(proj[:, nl:], merged[:, ml:], ctx, view.parts[1], writes_cache, self.right_scale)
        ops.linear(merged, self.out_weight, None, x, residual=x if accumulate else None)
