"""Routed experts: each token runs `top` of `experts` small feed-forwards, chosen by a router.

    z = W_router x (32-bit),  s = softmax(z) over all experts,  chosen = the `top` largest s,
    weight_e = s_e · scale (with `renormalize`: divided by the chosen ones' sum first),
    y = Σ_chosen weight_e · W_down,e act(W_up,e x)  +  sigmoid(w_sg · x) · W_down,s act(W_up,s x)   (the shared expert, if any)

`activation`: "relu2" (the square of relu), "silu" or "gelu_tanh". With `gated` an expert is W_down (act(W_gate x) · W_up x): gate and up
rows are stacked per expert and run as one product, the gate in a kernel of its own (silu only). With `router_bias` a stored
`router.b` is added to the logits before anything else. A softmax over the chosen logits alone is `renormalize` with scale 1
(the shares of the softmax over all experts, divided by their sum, are the same numbers). The tokens are not sorted on the host: the router's kernel
counts the tokens of each expert and lays the (token, choice) pairs out expert by expert (one launch for the few
tokens of a decode step), the two products run over those rows tile by tile (every tile of one expert's weight), and
a last kernel adds each token's `top` rows in the order of its choices, so the sum does not depend on what else is in
the batch. For few tokens the shared expert's first product runs in the experts' kernel too, as one expert that
takes every token, with its activation in the epilogue.

The experts' weights are stacked: up [experts · inter, hidden], down [experts · hidden, inter]; the router's rows
and the shared expert's gate row are one product with 32-bit output.
"""
from __future__ import annotations

import torch

from .base import BuildContext, Part
from .linear import Linear

ACTIVATIONS = {"relu2": 1, "silu": 2, "gelu_tanh": 3}


class Experts(Part):
    def __init__(self, ctx: BuildContext, *, experts: int, top: int, scale: float, inter: int, hidden: int,
                 shared_inter: int | None = None, activation: str = "relu2", renormalize: bool = False,
                 gated: bool = False, router_bias: bool = False, layer: int = 0) -> None:
        super().__init__()
        if activation not in ACTIVATIONS:
            raise ValueError(f"experts: activation {activation!r}; known: {sorted(ACTIVATIONS)}")
        if not 1 <= top <= experts:
            raise ValueError(f"experts: top {top} of {experts} experts")
        self.ctx, self.experts, self.top, self.scale, self.inter, self.hidden = ctx, experts, top, float(scale), inter, hidden
        self.act, self.renormalize, self.shared_inter = ACTIVATIONS[activation], bool(renormalize), shared_inter
        self.gated = bool(gated)
        if self.gated and (activation != "silu" or shared_inter):
            raise ValueError("experts: gated experts have silu gates and no shared expert")
        pieces = {"router": experts}
        if shared_inter:
            pieces["shared.sg"] = 1
        self.router = self.add_child("route", Linear(ctx, "weight", hidden, pieces))
        self.route_bias = self.add_param("router.b", (experts,), "coef") if router_bias else None
        if self.gated:                                                   # per expert: the gate's rows, then up's
            rows = {}
            for e in range(experts):
                rows[f"e{e}.gate"] = (2 * e * inter, (2 * e + 1) * inter)
                rows[f"e{e}.up"] = ((2 * e + 1) * inter, (2 * e + 2) * inter)
            self.up = self.add_param("up", (2 * experts * inter, hidden), "matrix", rows)
        else:
            self.up = self.add_param("up", (experts * inter, hidden), "matrix",
                                     {f"e{e}.up": (e * inter, (e + 1) * inter) for e in range(experts)})
        self.down = self.add_param("down", (experts * hidden, inter), "matrix",
                                   {f"e{e}.down": (e * hidden, (e + 1) * hidden) for e in range(experts)})
        self.shared_up = self.shared_down = None
        if shared_inter:
            self.shared_up = self.add_child("shared_up", Linear(ctx, "weight", hidden, {"shared.up": shared_inter}))
            self.shared_down = self.add_child("shared_down", Linear(ctx, "weight", shared_inter, {"shared.down": hidden}))

    def loadables(self, prefix: str = ""):
        """Stored names: router, e<j>.up, e<j>.down, shared.up, shared.down, shared.sg."""
        for name, p, rows in super().loadables(prefix):
            for child in ("route.", "shared_up.", "shared_down."):
                if name.startswith(prefix + child):
                    name = prefix + name[len(prefix + child):]
            yield name, p, rows

    FEW = 8                  # rows up to which the shared expert's first product runs in the experts' kernel

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        t, k, ctx, e, top = x.shape[0], self.ctx.kernels, self.ctx, self.experts, self.top
        z = self.router.forward(x, out_dtype=torch.float32)             # [t, experts (+ 1)]: router logits, gate
        chosen = ctx.empty(t, top, dtype=torch.int32)
        weight = ctx.empty(t, top, dtype=torch.float32)
        counts = ctx.empty(2 * e + 3, dtype=torch.int32)                 # per expert: tokens, then first row; end; (0, t)
        place = ctx.empty(t * top, dtype=torch.int32)                    # the row of each (token, choice)
        token_of = ctx.empty(t * top, dtype=torch.int32)                 # the token of each row
        if self.route_bias is not None:
            k.route_rows(chosen, weight, counts, place, token_of, z, e, self.scale, self.renormalize, self.route_bias.tensor)
        else:
            k.route_rows(chosen, weight, counts, place, token_of, z, e, self.scale, self.renormalize)
        starts = counts[e:2 * e + 1]
        act = ctx.empty(t * top, self.inter)
        if self.gated:
            both = ctx.empty(t * top, 2 * self.inter)
            k.expert_linear(both, x, token_of, self.up.tensor.view(e, 2 * self.inter, self.hidden), starts, 0)
            k.silu_mul(act, both)
        else:
            k.expert_linear(act, x, token_of, self.up.tensor.view(e, self.inter, self.hidden), starts, self.act)
        y = ctx.empty(t * top, self.hidden)
        k.expert_linear(y, act, None, self.down.tensor.view(e, self.hidden, self.inter), starts, 0)
        shared = None
        if self.shared_up is not None:
            if t <= self.FEW:                                            # few rows: the activation in the product's epilogue
                hs = ctx.empty(t, self.shared_inter)
                k.expert_linear(hs, x, None, self.shared_up.weight.tensor.view(1, self.shared_inter, self.hidden),
                                counts[2 * e + 1:], self.act)
            else:
                hs = self.shared_up.forward(x)
                k.activation(hs, self.act)
            shared = self.shared_down.forward(hs)
        out = ctx.empty(t, self.hidden)
        k.expert_combine(out, y, place, weight, shared, z if shared is not None else None, e)
        return out
