"""A selective state-space mixer with a matrix state per head (the "state-space duality" form).

With inner = heads · vdim, N = state, G = groups, one product of the input gives [z: inner | x: inner | B: G·N | C: G·N |
dt: heads].  x, B and C pass a short causal convolution per channel (taps − 1 earlier inputs, zeros before a sequence's
start), a bias and x·sigmoid(x).  Per head h (group h // (heads / groups)), token by token,

    dt ← softplus(dt + dt_bias_h),   S ← exp(−exp(A_log_h) · dt) · S + dt · B xᵀ,   y = Sᵀ C + D_h · x,

S being N × vdim and zero at a sequence's start.  The heads' y, multiplied by z·sigmoid(z), go through an RMS norm in
`norm_groups` equal parts with a weight, then W_o.  The recurrence, its step sizes and decays, the gate and the norm
are float32 in every engine.

Per sequence the mixer keeps the heads' states and the convolution's last taps − 1 inputs: one float32 state row, held
twice (`StateNeed((2, n))`; the kernels say which copy a step reads and which it writes).

Like the attention mixers that can run beside another branch, it is written as `in_weight`, `core(proj, merged, …,
factor)` and `out_weight`; `forward` chains them."""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..csrc import ops
from .context import StepContext
from .registry import register_part


@register_part("mixer", "state_space")
class StateSpaceMixer:
    def __init__(self, w_in, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, w_out, *, n_heads: int, vdim: int, n_state: int,
                 n_groups: int, norm_groups: int, eps: float):
        Hs, P, N, G = int(n_heads), int(vdim), int(n_state), int(n_groups)
        inner = Hs * P
        channels = inner + 2 * G * N
        if Hs <= 0 or G <= 0 or Hs % G != 0:
            raise ValueError(f"state-space mixer: {Hs} heads cannot share {G} groups")
        if w_in.shape[0] != 2 * inner + 2 * G * N + Hs:
            raise ValueError(f"state-space mixer: the input product has {w_in.shape[0]} rows, {2 * inner + 2 * G * N + Hs} expected")
        if conv_w.dim() != 2 or conv_w.shape[0] != channels or conv_b.shape[0] != channels:
            raise ValueError(f"state-space mixer: the convolution covers {channels} channels")
        if not (1 <= conv_w.shape[1] <= ops.SSD_MAX_TAPS):
            raise ValueError(f"state-space mixer: {conv_w.shape[1]} taps are not in 1…{ops.SSD_MAX_TAPS}")
        if any(t.numel() != Hs for t in (dt_bias, a_log, d_skip)):
            raise ValueError("state-space mixer: dt_bias, A_log and D have one number per head")
        if norm_w.shape[0] != inner or norm_groups < 1 or inner % norm_groups != 0 or w_out.shape[1] != inner:
            raise ValueError("state-space mixer: the norm and the output projection take the heads' merged values")
        if P > ops.SSD_MAX_VDIM or N > ops.SSD_MAX_STATE:
            raise ValueError(f"state-space mixer: a state of {N} rows by {P} columns is above the {ops.SSD_MAX_STATE} by "
                             f"{ops.SSD_MAX_VDIM} the kernels take")
        self.n_heads, self.vdim, self.n_state, self.n_groups = Hs, P, N, G
        self.norm_groups, self.eps = int(norm_groups), float(eps)
        self.inner, self.channels, self.taps = inner, channels, int(conv_w.shape[1])
        self.in_weight, self.in_bias, self.in_width = w_in, None, w_in.shape[0]
        self.conv_w, self.conv_b = conv_w.float().contiguous(), conv_b.float().contiguous()
        self.dt_bias, self.a_log, self.d_skip = dt_bias.float().contiguous(), a_log.float().contiguous(), d_skip.float().contiguous()
        self.norm_w, self.out_weight, self.merged_width = norm_w, w_out, inner
        self.z_off, self.x_off, self.dt_off = 0, inner, inner + channels
        self.conv_off = Hs * N * P                                   # where the kept inputs begin in a state row
        self.state_row = self.conv_off + (self.taps - 1) * channels

    def cache_need(self):
        return StateNeed((2, self.state_row), torch.float32)

    fuses_norm = False
    leaves_row_stats = False

    def core(self, proj, merged, ctx: StepContext, view, writes_cache: bool = True, factor: float = 1.0) -> None:
        if not writes_cache:
            raise ValueError("state-space mixer: a layer cannot read another layer's state")
        T, ws = ctx.n_tokens, ctx.ws
        xbc = ws.get("ssd_xbc", T, self.channels, torch.float32)
        ops.ssd_conv(proj, self.x_off, self.conv_w, self.conv_b, view.state, self.conv_off, ctx.seq_slot, ctx.seq_start, ctx.seq_pos0,
                     xbc, ctx.n_seqs, ctx.max_new)
        y = ws.get("ssd_y", T, self.inner, torch.float32)
        ops.ssd_scan_step(xbc, proj, self.dt_off, self.dt_bias, self.a_log, self.d_skip, view.state, ctx, y, self.n_heads,
                          self.n_groups, self.n_state, self.vdim)
        ops.ssd_gate_norm(y, proj, self.z_off, self.norm_w, self.norm_groups, self.eps, factor, merged, T)

    def forward(self, h, x: torch.Tensor, ctx: StepContext, view, writes_cache: bool = True, accumulate: bool = True) -> None:
        T = ctx.n_tokens
        proj = ctx.ws.get("ssd_in_proj", T, self.in_width, torch.float32)
        ops.linear(h, self.in_weight, None, proj)
        merged = ctx.ws.get("ssd_merged", T, self.merged_width, ctx.act_dtype)
        self.core(proj, merged, ctx, view, writes_cache)
        ops.linear(merged, self.out_weight, None, x, residual=x if accumulate else None)
