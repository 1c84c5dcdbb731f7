"""Token embedding and the head that turns the last hidden rows into logits."""
from __future__ import annotations

import torch

from ..csrc import ops
from .context import StepContext


class TokenEmbedding:
    """x[t] = weight[token[t]], fused with a position encoding that acts at the embedding
    (reference: include/model/ops.hpp:615-626, include/model/transformer.hpp:340)."""

    def __init__(self, weight: torch.Tensor, position=None, norm=None, scale: float = 1.0, streams: int = 1):
        """norm: a norm part applied to the embedded rows in place (float32), or None.  scale: a factor on every
        embedded row.  streams: how many copies of the row the residual starts with (a residual carried in several
        streams, see parts/block.py); the rows this part writes are `out_width` = streams · width wide."""
        self.weight = weight
        self.norm = norm
        self.vocab_size, self.width = weight.shape
        self.scale, self.streams = float(scale), int(streams)
        if self.streams < 1:
            raise ValueError("TokenEmbedding: at least one stream")
        if (self.scale != 1.0 or self.streams != 1) and (norm is not None or getattr(position, "where", None) == "embedding"):
            raise ValueError("TokenEmbedding: a scaled or copied embedding takes no norm and no position table")
        self.out_width = self.width * self.streams
        if position is not None and getattr(position, "where", None) == "embedding":
            if position.table.shape[1] != self.width or position.table.dtype != weight.dtype:
                raise ValueError("TokenEmbedding: the position table does not match the embedding")
            self.position = position
        else:
            self.position = None

    @property
    def leaves_row_stats(self) -> bool:
        """The rows are written by a kernel that is handed the step's row statistics (see parts/block.py); a norm
        behind it rewrites them."""
        return self.norm is None and self.scale == 1.0 and self.streams == 1

    def emit_decode(self, program, x: torch.Tensor) -> None:
        if self.scale != 1.0 or self.streams != 1:
            from .program import NotFusable
            raise NotFusable("a scaled or copied embedding is not an operation of the decode program")
        if self.norm is not None:
            from .program import NotFusable
            raise NotFusable("an embedding with a norm behind it is not an operation of the decode program")
        program.embed(self.weight, self.position.table if self.position is not None else None, x)

    def __call__(self, ctx: StepContext, x: torch.Tensor) -> torch.Tensor:
        if self.scale != 1.0 or self.streams != 1:
            ctx.ws.row_stats.forget()
            ops.embed_streams(self.weight, ctx.tokens, x, self.streams, self.scale, ctx.dev_err)
            return x
        table = self.position.table if self.position is not None else None
        ops.embed(self.weight, table, ctx.tokens, ctx.tok_pos if table is not None else None, x, ctx.dev_err,
                  stats=ctx.ws.row_stats)
        if self.norm is not None:
            ctx.ws.row_stats.forget()
            self.norm(x, x)
        return x


class LMHead:
    """logits = h · weightᵀ, float32, no bias; a tied head is given the embedding's weight
    (reference: include/model/transformer.hpp:413-414, :298-300).  With `softcap` = c the logits are then squashed,
    c · tanh(logits / c)."""

    def __init__(self, weight: torch.Tensor, softcap: float | None = None):
        self.weight = weight
        self.vocab_size, self.width = weight.shape
        if softcap is not None and not softcap > 0.0:
            raise ValueError(f"LMHead: a soft cap of {softcap} is not positive")
        self.softcap = float(softcap) if softcap is not None else None

    def emit_decode(self, program, x: torch.Tensor, norm, logits: torch.Tensor) -> None:
        """logits = norm(x) · weightᵀ for every row of the program."""
        from .program import NotFusable, norm_terms
        if self.softcap is not None:
            raise NotFusable("a head with a soft cap is not an operation of the decode program")
        program.product(x, self.weight, None, logits, norm=norm_terms(norm))

    def __call__(self, h: torch.Tensor, logits: torch.Tensor, n_rows: int) -> torch.Tensor:
        ops.linear(h, self.weight, None, logits, rows=n_rows)
        if self.softcap is not None:
            ops.softcap(logits, n_rows, self.softcap)
        return logits
