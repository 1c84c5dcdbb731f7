"""A feed-forward of routed experts.

Every token takes the `top` experts with the largest router logits z = h·W_routerᵀ + b (float32 sums; ties go to the
lower index), weighted by the softmax over the chosen logits alone.  An expert is a gated feed-forward without biases,
W_down (silu(W_gate h) · (W_up h)).  A shared expert of the same form, if there is one, runs for every token and is
added, multiplied by sigmoid(w_sg · h), one number per token.

Nothing is decided on the host: the router's kernel counts each expert's rows, the tokens' inputs are copied into a
buffer sorted by expert, and two grouped products (each row block with its expert's matrix) run over it with the gate
between them; a last kernel sums each token's experts with their weights.  So a step with this part launches the same
kernels whatever the tokens choose, and can be captured and replayed.  The shared gate's logit rides in the router's
product as one more row.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("feed_forward", "routed_experts")
class RoutedExperts:
    def __init__(self, w_router, b_router, w_gate, w_up, w_down, *, top: int, shared=None):
        """w_router [E, width], b_router [E] float32 or None; w_gate, w_up [E, ff, width], w_down [E, width, ff];
        shared: None or (w_gate [ffs, width], w_up [ffs, width], w_down [width, ffs], w_sg [1, width] or None)."""
        E, width = w_router.shape
        if w_gate.shape != w_up.shape or w_gate.shape[0] != E or w_gate.shape[2] != width:
            raise ValueError("routed experts: the experts' gate and up matrices are [experts, ff, width]")
        ff = w_gate.shape[1]
        if tuple(w_down.shape) != (E, width, ff):
            raise ValueError("routed experts: the experts' down matrices are [experts, width, ff]")
        if not (0 < top <= min(E, 32)):
            raise ValueError(f"routed experts: a token takes 1…min(32, {E}) experts, not {top}")
        self.n_experts, self.top, self.width, self.ff = E, int(top), width, ff
        self.w_gate_up = torch.cat([w_gate, w_up], dim=1).contiguous()          # [E, 2·ff, width]
        self.w_down = w_down.contiguous()
        self.shared = None
        self.shared_gate = False
        w_r = w_router
        b_r = b_router if b_router is not None else torch.zeros(E, dtype=torch.float32, device=w_router.device)
        if shared is not None:
            s_gate, s_up, s_down, s_sg = shared
            if s_gate.shape != s_up.shape or s_gate.shape[1] != width or tuple(s_down.shape) != (width, s_gate.shape[0]):
                raise ValueError("routed experts: the shared expert's matrices do not chain")
            self.shared = (torch.cat([s_gate, s_up], dim=0).contiguous(), s_down.contiguous(), s_gate.shape[0])
            if s_sg is not None:
                if tuple(s_sg.shape) != (1, width):
                    raise ValueError("routed experts: the shared expert's gate is one row of the model's width")
                w_r = torch.cat([w_router, s_sg.to(w_router.dtype)], dim=0)
                b_r = torch.cat([b_r, torch.zeros(1, dtype=torch.float32, device=b_r.device)])
                self.shared_gate = True
        # One product of the input gives the router's logits (with the shared gate's) and, for few rows (a decode
        # step), behind them the shared expert's gate and up rows, all float32; with many rows the shared expert's
        # are a product of their own in the activation dtype, half the bytes.
        self.n_logits = w_r.shape[0]
        if self.shared is not None:
            w_gu = self.shared[0]
            self.w_in = torch.cat([w_r, w_gu], dim=0).contiguous()
            self.b_in = torch.cat([b_r, torch.zeros(w_gu.shape[0], dtype=torch.float32, device=b_r.device)]).contiguous()
        else:
            self.w_in, self.b_in = w_r.contiguous(), b_r.contiguous()

    fuses_norm = False
    leaves_row_stats = False

    def forward(self, h, x: torch.Tensor, ctx: StepContext, norm=None, accumulate: bool = True) -> None:
        T, ws, act = ctx.n_tokens, ctx.ws, ctx.act_dtype
        E, top, width, ff = self.n_experts, self.top, self.width, self.ff
        P = T * top
        shared_apart = self.shared is not None and T > ops.SKINNY_MAX_ROWS
        n_in = self.n_logits if shared_apart else self.w_in.shape[0]
        inp = ws.get("moe_in_proj", T, n_in, torch.float32)
        ops.linear(h, self.w_in[:n_in], self.b_in[:n_in], inp)
        z = inp
        ids = ws.get("moe_ids", T, top, torch.int32)
        rank = ws.get("moe_rank", T, top, torch.int32)
        row_of = ws.get("moe_row_of", T, top, torch.int32)
        wts = ws.get("moe_weights", T, top, torch.float32)
        gate = ws.get("moe_shared_gate", T, 1, torch.float32) if self.shared_gate else None
        counts = ws.get_zeroed("moe_counts", E, torch.int32)
        offsets = ws.get("moe_offsets", 1, E + 1, torch.int32)
        ops.moe_route(z, E, top, self.shared_gate, ctx.tok_slot, ids, wts, rank, gate, counts, T)
        ops.moe_plan(counts, offsets, E)
        rows = ws.get("moe_sorted", P, width, act)
        ops.moe_gather(h, ids, rank, offsets, rows, row_of, T, top)
        u = ws.get("moe_gate_up", P, 2 * ff, act)
        ops.linear_grouped(rows, self.w_gate_up, u, offsets, P)
        a = ws.get("moe_inner", P, ff, act)
        ops.gate_mul(u[:, :ff], u[:, ff:], a, "silu", P, ff)
        out = ws.get("moe_expert_out", P, width, torch.float32)
        ops.linear_grouped(a, self.w_down, out, offsets, P)
        shared_out = None
        if self.shared is not None:
            w_gu, w_d, ffs = self.shared
            sa = ws.get("moe_shared_inner", T, ffs, act)
            if shared_apart:
                su = ws.get("moe_shared_gate_up", T, 2 * ffs, act)
                ops.linear(h, w_gu, None, su)
                ops.gate_mul(su[:, :ffs], su[:, ffs:], sa, "silu", T, ffs)
            else:
                at = self.n_logits
                ops.gate_mul(inp[:, at:at + ffs], inp[:, at + ffs:at + 2 * ffs], sa, "silu", T, ffs)
            shared_out = ws.get("moe_shared_out", T, width, torch.float32)
            ops.linear(sa, w_d, None, shared_out)
        ops.moe_combine(out, row_of, wts, top, shared_out, gate, x, T, residual=x if accumulate else None)
