"""Pre-norm residual block: h += mixer(input_norm(h)); h += ffn(post_norm(h))
(std/holon_std/blocks/units.py:8-25). The sums are folded into the next norm's kernel: the block leaves the
feed-forward's output pending on the stream. For the few rows of a decode step sum and norm move one kernel further
up, into the product that ends the mixer or the feed-forward (base.Link, base.Scaled).

OutNorm: the norm stands on a sublayer's OUTPUT, and the sublayers read the stream itself: x ← x + N(mixer(x)), then
x ← x + N(ffn(x)). With `average` = n the block ends with an average over depth: with X_0 the embedding's rows and X_j
what the j-th block before left (before ITS averaging), what goes on is Σ_j c[j] X_j over the n results so far, c the
block's stored `depth` coefficients. The results of a step's blocks wait on the step (`step.shared`), 32-bit.

Sandwich: a norm before and behind each sublayer, x ← x + N1b(mixer(N1(x))), then x ← x + N2b(ffn(N2(x))). With `shift`
the mixer reads each token's normed row blended with the row of the token before, m_t = n_t + (n_(t−1) − n_t) · mix with a
stored vector `shift` (zeros before a sequence's first token); the last normed row of a request's step is kept per
request and cache entry (a `SlotState` the block declares, `block.shift`). The feed-forward's output stays pending on the
stream together with its norm, and the next block's first kernel (or the model's last norm) adds it.
"""
from __future__ import annotations

import torch

from ..config.spec import PartRef
from .base import BuildContext, Link, Part, Residual, SlotState


class PreNorm(Part):
    def __init__(self, ctx: BuildContext, *, layer: int, hidden: int, mixer: PartRef, ffn: PartRef | None,
                 norm: PartRef) -> None:
        super().__init__()
        self.ctx = ctx
        self.input_norm = self.add_child("input_norm", ctx.part(norm, dim=hidden))
        self.mixer = self.add_child("mixer", ctx.part(mixer, layer=layer, hidden=hidden))
        self.post_norm = self.ffn = None                             # (a layer may have a mixer only)
        if ffn is not None:
            self.post_norm = self.add_child("post_norm", ctx.part(norm, dim=hidden))
            self.ffn = self.add_child("ffn", ctx.part(ffn, layer=layer, hidden=hidden))

    def forward(self, stream: Residual, step, cache, after=None) -> Residual:
        """`after`: the block that runs next (None: none, or unknown). For the few rows of a decode step the
        product that ends the mixer does the residual sum and the post norm in its epilogue, and the one that ends
        the feed-forward the sum and `after`'s input norm (see base.Link), where the part that reads those rows can
        take them unscaled."""
        x = self.input_norm.add(stream)
        if self.ffn is None:
            stream.delta = self.mixer.forward(x, step, cache)
            return stream
        step.link = self._offer(stream, step, self.post_norm, self.ffn)
        stream.delta = self.mixer.forward(x, step, cache)
        step.link = None                                             # (an offer nobody took lapses)
        x = self.post_norm.add(stream)
        step.link = self._offer(stream, step, getattr(after, "input_norm", None), getattr(after, "mixer", None))
        stream.delta = self.ffn.forward(x, step)
        step.link = None
        return stream

    def _offer(self, stream, step, norm, reader):
        can = getattr(self.ctx.kernels, "can_link", None)
        if can is None or not getattr(reader, "takes_scaled", False) or not hasattr(norm, "weight"):
            return None
        return Link(stream, norm) if can(step.rows.n_tokens, stream.h.shape[1], norm) else None


class OutNorm(Part):
    """`average`: how many results this block averages (its own included; None: no averaging). `results`: how many the
    step's blocks leave in all, the embedding's rows included (the first block of a step makes room for them)."""

    KEY = "outnorm"                # step.shared: {"x": the stream's rows as the sublayers read them, "hist", "n"}

    def __init__(self, ctx: BuildContext, *, layer: int, hidden: int, mixer: PartRef, ffn: PartRef | None, norm: PartRef,
                 average: int | None = None, results: int = 0) -> None:
        super().__init__()
        if average is not None and not 1 <= average <= results:
            raise ValueError(f"outnorm: an average over {average} of {results} results")
        self.ctx, self.average, self.results = ctx, average, results
        self.mixer_norm = self.add_child("mixer_norm", ctx.part(norm, dim=hidden))
        self.mixer = self.add_child("mixer", ctx.part(mixer, layer=layer, hidden=hidden))
        self.ffn_norm = self.ffn = None
        if ffn is not None:
            self.ffn_norm = self.add_child("ffn_norm", ctx.part(norm, dim=hidden))
            self.ffn = self.add_child("ffn", ctx.part(ffn, layer=layer, hidden=hidden))
        self.coef = self.add_param("depth", (average,), "coef") if average is not None else None

    def _rows(self, t: int, hidden: int):
        """A place for the stream's rows in the engine's dtype (None where that is 32-bit: the stream itself is read)."""
        return None if self.ctx.dtype == torch.float32 else self.ctx.empty(t, hidden)

    def forward(self, stream: Residual, step, cache, after=None) -> Residual:
        k, ctx = self.ctx.kernels, self.ctx
        t, hidden = stream.h.shape
        if stream.delta is not None:                                     # (what a block of another kind left pending)
            k.sum_into(stream.h, [(stream.delta, 1.0)])
            stream.delta = None
        stream.normed = stream.normed_by = None
        state = step.shared.get(self.KEY)
        if state is None:                                                # the first block of the step
            state = step.shared[self.KEY] = {"x": None, "hist": None, "n": 0}
            cast = self._rows(t, hidden)
            if self.average is not None:
                state["hist"] = ctx.empty(self.results, t, hidden, dtype=torch.float32)
                k.out_norm_add(state["hist"][0], stream.h, None, None, None, 0.0, 0.0, cast=cast)
                state["n"] = 1
            elif cast is not None:
                k.out_norm_add(stream.h, stream.h, None, None, None, 0.0, 0.0, cast=cast)
            state["x"] = cast if cast is not None else stream.h
        hist, n = state["hist"], state["n"]
        if self.average is not None and (hist is None or n + 1 != self.average or n >= hist.shape[0]):
            raise RuntimeError(f"outnorm: this block averages {self.average} results, the step holds {n} before it")
        mixer, norm = self.mixer, self.mixer_norm
        if hasattr(mixer, "forward_biased"):                             # the last product's bias rides in the norm's kernel
            y, bias = mixer.forward_biased(state["x"], step, cache)
        else:
            y, bias = mixer.forward(state["x"], step, cache), None
        own = hist[n] if self.average is not None else stream.h          # where this block's result is kept
        src = stream.h
        if self.ffn is not None:
            mid = self._rows(t, hidden)
            k.out_norm_add(own, src, y, bias, norm.weight.tensor, norm.eps, norm.offset, cast=mid)
            y, bias, norm, src = self.ffn.forward(mid if mid is not None else own, step), None, self.ffn_norm, own
        cast = self._rows(t, hidden)
        if self.average is not None:
            go = ctx.empty(t, hidden, dtype=torch.float32)
            k.out_norm_add(own, src, y, bias, norm.weight.tensor, norm.eps, norm.offset, hist=hist, n_hist=n + 1,
                           coef=self.coef.tensor, avg=go, cast=cast)
            stream.h, state["n"] = go, n + 1
        else:
            k.out_norm_add(own, src, y, bias, norm.weight.tensor, norm.eps, norm.offset, cast=cast)
        state["x"] = cast if cast is not None else stream.h
        return stream


class Sandwich(Part):
    """Its norms offer `add`, `add_shifted`, `add_then` and `gather` (parts/norm.py: DynamicTanh)."""

    def __init__(self, ctx: BuildContext, *, layer: int, hidden: int, mixer: PartRef, ffn: PartRef | None, norm: PartRef,
                 shift: bool = False) -> None:
        super().__init__()
        self.ctx, self.hidden = ctx, hidden
        self.mixer_norm = self.add_child("mixer_norm", ctx.part(norm, dim=hidden))
        self.mixer = self.add_child("mixer", ctx.part(mixer, layer=layer, hidden=hidden))
        self.mixer_out_norm = self.add_child("mixer_out_norm", ctx.part(norm, dim=hidden))
        self.ffn_norm = self.ffn = self.ffn_out_norm = None
        if ffn is not None:
            self.ffn_norm = self.add_child("ffn_norm", ctx.part(norm, dim=hidden))
            self.ffn = self.add_child("ffn", ctx.part(ffn, layer=layer, hidden=hidden))
            self.ffn_out_norm = self.add_child("ffn_out_norm", ctx.part(norm, dim=hidden))
        self.shift = self.add_param("shift", (hidden,), "coef") if shift else None

    def slot_states(self):
        """What the block itself carries per request and cache entry (the model files it beside the mixer's)."""
        return (SlotState("block.shift", (self.hidden,)),) if self.shift is not None else ()

    def forward(self, stream: Residual, step, cache, after=None) -> Residual:
        stream.normed = stream.normed_by = None
        if self.shift is not None:
            x = self.mixer_norm.add_shifted(stream, self.shift.tensor, cache.slots["block.shift"], step.rows)
        else:
            x = self.mixer_norm.add(stream)
        # for the few rows of a decode step the product that ends the mixer may add its normed output and norm the sum
        # for the feed-forward in its epilogue (base.Link with `post`): it then returns None and leaves the rows behind
        step.link = Link(stream, self.ffn_norm, post=self.mixer_out_norm) \
            if self.ffn is not None and hasattr(self.mixer_out_norm, "triple") and hasattr(self.ffn_norm, "triple") else None
        y = self.mixer.forward(x, step, cache)
        step.link = None
        if self.ffn is None:
            stream.delta, stream.delta_by = y, self.mixer_out_norm
            return stream
        if y is None:
            x, stream.normed, stream.normed_by = stream.normed, None, None
        else:
            x = self.mixer_out_norm.add_then(stream, y, self.ffn_norm)
        stream.delta, stream.delta_by = self.ffn.forward(x, step), self.ffn_out_norm
        return stream
