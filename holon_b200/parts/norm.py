"""RMSNorm: x · rsqrt(mean(x²) + eps) · (weight + offset), all in 32-bit, one rounding at the end
(std/holon_std/ops/units.py:16-35; formula std/holon_std/ops/reference.py:7-18).

DynamicTanh: tanh(alpha · x) · weight + bias, no statistics of the row at all."""
from __future__ import annotations

import torch

from .base import BuildContext, Part, Residual


class RMSNorm(Part):
    def __init__(self, ctx: BuildContext, *, eps: float, dim: int, offset: float = 0.0) -> None:
        super().__init__()
        self.ctx, self.eps, self.dim, self.offset = ctx, float(eps), dim, float(offset)
        self.weight = self.add_param("weight", (dim,), "gain")

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """The norm of the rows of `x` [rows, dim] (engine dtype or 32-bit), as a new tensor of the engine's dtype."""
        out = self.ctx.empty(*x.shape)
        self.ctx.kernels.rmsnorm(out, x, self.weight.tensor, self.eps, self.offset)
        return out

    def add(self, stream: Residual) -> torch.Tensor:
        """Adds the stream's pending output into it and returns the norm of the sum; or, where the product before
        has done both, the rows it left (base.Scaled)."""
        if getattr(stream, "delta_by", None) is not None:
            raise RuntimeError("rmsnorm: the pending output must pass a norm of its own first; this norm adds it as it is")
        if stream.normed is not None:
            rows, by, stream.normed, stream.normed_by = stream.normed, stream.normed_by, None, None
            if by is self:
                return rows                                # (made for another norm: dropped, the stream itself is whole)
        out = self.ctx.empty(*stream.h.shape)
        self.ctx.kernels.add_rmsnorm(out, stream.h, stream.delta, self.weight.tensor, self.eps, self.offset, None)
        stream.delta = None
        return out

    def gather(self, stream: Residual, index: torch.Tensor) -> torch.Tensor:
        """The norm of rows `index` of the stream (pending output included); the stream is left as it is."""
        out = self.ctx.empty(index.shape[0], self.dim)
        self.ctx.kernels.add_rmsnorm(out, stream.h, stream.delta, self.weight.tensor, self.eps, self.offset, index)
        return out


class DynamicTanh(Part):
    """A norm without mean or variance: tanh(alpha · x) · weight + bias, element by element, with one stored number
    `alpha`; 32-bit arithmetic, one rounding at the end. A block may leave a part's output pending on the stream
    together with the norm it passes before it is added (`Residual.delta`, `Residual.delta_by`); `add` and `gather`
    fold both in."""

    def __init__(self, ctx: BuildContext, *, dim: int, eps: float = 0.0) -> None:
        super().__init__()
        self.ctx, self.dim, self.eps, self.offset = ctx, dim, float(eps), 0.0
        self.weight = self.add_param("weight", (dim,), "coef")
        self.bias = self.add_param("bias", (dim,), "coef")
        self.alpha = self.add_param("alpha", (), "coef")

    def triple(self):
        return self.alpha.tensor, self.weight.tensor, self.bias.tensor

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """The norm of the rows of `x` [rows, dim] (engine dtype or 32-bit), as a new tensor of the engine's dtype."""
        out = self.ctx.empty(*x.shape)
        self.ctx.kernels.dyt_add_norm(None, x, None, out, self.triple(), None)
        return out

    @staticmethod
    def _pending(stream: Residual):
        by = getattr(stream, "delta_by", None)
        if stream.delta is not None and by is None:
            raise RuntimeError("dyt: a pending output without the norm it passes; this norm adds only what a "
                               "sandwich block left")
        return stream.delta, (by.triple() if by is not None else None)

    def add(self, stream: Residual) -> torch.Tensor:
        """Adds the stream's pending output (under its own norm) into it and returns the norm of the sum."""
        y, post = self._pending(stream)
        out = self.ctx.empty(*stream.h.shape)
        self.ctx.kernels.dyt_add_norm(stream.h, y, post, out, self.triple(), None)
        stream.delta = stream.delta_by = None
        return out

    def gather(self, stream: Residual, index: torch.Tensor) -> torch.Tensor:
        """The norm of rows `index` of the stream (pending output included); the stream is left as it is."""
        y, post = self._pending(stream)
        out = self.ctx.empty(index.shape[0], self.dim)
        self.ctx.kernels.dyt_add_norm(stream.h, y, post, out, self.triple(), index)
        return out

    def add_shifted(self, stream: Residual, mix: torch.Tensor, carried: torch.Tensor, rows) -> torch.Tensor:
        """`add`, and each token's normed row n_t blended with the one before it: n_t + (n_(t-1) − n_t) · mix, in the
        same kernel and in 32-bit. `carried` float32 [slots, dim] holds, per request, the normed row of the last token
        of its step before (zeros at admission) and receives this step's."""
        y, post = self._pending(stream)
        out = self.ctx.empty(*stream.h.shape)
        # with a pending output the sums go to a new tensor: a token's block also reads the row before its own
        into = stream.h if y is None else self.ctx.empty(*stream.h.shape, dtype=torch.float32)
        self.ctx.kernels.dyt_shift(out, into, stream.h, y, post, self.triple(), mix, carried, rows)
        stream.h, stream.delta, stream.delta_by = into, None, None
        return out

    def add_then(self, stream: Residual, y: torch.Tensor, then: "DynamicTanh") -> torch.Tensor:
        """stream += this norm of `y`; returns the norm `then` of the sum (one kernel)."""
        out = self.ctx.empty(*stream.h.shape)
        self.ctx.kernels.dyt_add_norm(stream.h, y, self.triple(), out, then.triple(), None)
        return out
