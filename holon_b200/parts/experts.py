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

`identity` more experts stand behind the real ones in the router's rows: they have no tensors, their output is their
input. With `groups` G > 1 the experts (identity ones included) form G equal groups of neighbours; a group's score is its
largest choice score, and only experts of the `keep_groups` best groups can be chosen. With `correction` a stored vector
is added to the scores for the choice alone (the weights use the scores without it; choice scores may be negative). `tiny`
is added to the chosen scores' sum before `renormalize` divides by it. `shared_gated`: the shared expert is a gated unit
like the experts (gate and up rows as one product) and is added without a gate of its own.

The experts' weights are stacked: up [experts · inter, hidden], down [experts · hidden, inter]; the router's rows
and the shared expert's gate row are one product with 32-bit output.
"""
from __future__ import annotations

import torch

from .base import BuildContext, Part
from .linear import Linear

ACTIVATIONS = {"relu2": 1, "silu": 2, "gelu_tanh": 3, "xielu": 4, "tanh": 5}
EXPERT_ACTIVATIONS = ("relu2", "silu", "gelu_tanh")      # what the experts' products know in their epilogues


class Experts(Part):
    def __init__(self, ctx: BuildContext, *, experts: int, top: int, scale: float, inter: int, hidden: int,
                 shared_inter: int | None = None, activation: str = "relu2", renormalize: bool = False,
                 gated: bool = False, router_bias: bool = False, identity: int = 0, groups: int = 1, keep_groups: int = 1,
                 correction: bool = False, shared_gated: bool = False, tiny: float = 0.0, layer: int = 0) -> None:
        super().__init__()
        if activation not in EXPERT_ACTIVATIONS:
            raise ValueError(f"experts: activation {activation!r}; known: {sorted(EXPERT_ACTIVATIONS)}")
        if identity < 0 or not 1 <= top <= experts + identity:
            raise ValueError(f"experts: top {top} of {experts} experts and {identity} identity experts")
        if groups < 1 or (experts + identity) % groups or not 1 <= keep_groups <= groups \
                or keep_groups * ((experts + identity) // groups) < top:
            raise ValueError(f"experts: {groups} groups of which {keep_groups} are kept, for top {top} of {experts + identity}")
        self.ctx, self.experts, self.top, self.scale, self.inter, self.hidden = ctx, experts, top, float(scale), inter, hidden
        self.act, self.renormalize, self.shared_inter = ACTIVATIONS[activation], bool(renormalize), shared_inter
        self.gated, self.shared_gated = bool(gated), bool(shared_gated)
        self.identity, self.routed = int(identity), experts + int(identity)        # routed: the router's rows
        self.groups, self.keep_groups, self.tiny = int(groups), int(keep_groups), float(tiny)
        if self.gated and (activation != "silu" or (shared_inter and not shared_gated)):
            raise ValueError("experts: gated experts have silu gates, and a shared expert beside them is gated too")
        if self.shared_gated and not self.gated:
            raise ValueError("experts: a gated shared expert goes with gated experts")
        pieces = {"router": self.routed}
        if shared_inter and not shared_gated:
            pieces["shared.sg"] = 1
        self.router = self.add_child("route", Linear(ctx, "weight", hidden, pieces))
        self.route_bias = self.add_param("router.b", (self.routed,), "coef") if router_bias else None
        self.correction = self.add_param("correction", (self.routed,), "coef") if correction else None
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
            first = {"shared.gate": shared_inter, "shared.up": shared_inter} if shared_gated else {"shared.up": shared_inter}
            self.shared_up = self.add_child("shared_up", Linear(ctx, "weight", hidden, first))
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
        r = self.routed                                                  # the router's rows: real experts, then identity ones
        z = self.router.forward(x, out_dtype=torch.float32)             # [t, routed (+ 1)]: router logits, gate
        chosen = ctx.empty(t, top, dtype=torch.int32)
        weight = ctx.empty(t, top, dtype=torch.float32)
        counts = ctx.empty(2 * r + 3, dtype=torch.int32)                 # per expert: tokens, then first row; end; (0, t)
        place = ctx.empty(t * top, dtype=torch.int32)                    # the row of each (token, choice)
        token_of = ctx.empty(t * top, dtype=torch.int32)                 # the token of each row
        bias = self.route_bias.tensor if self.route_bias is not None else None
        if self.correction is not None or self.groups > 1 or self.tiny:
            k.route_rows(chosen, weight, counts, place, token_of, z, r, self.scale, self.renormalize, bias,
                         correction=self.correction.tensor if self.correction is not None else None, groups=self.groups,
                         keep=self.keep_groups, tiny=self.tiny)
        elif bias is not None:
            k.route_rows(chosen, weight, counts, place, token_of, z, r, self.scale, self.renormalize, bias)
        else:
            k.route_rows(chosen, weight, counts, place, token_of, z, r, self.scale, self.renormalize)
        starts = counts[r:r + e + 1]                                     # rows are laid out expert by expert: the real ones first
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
        if self.shared_up is not None and self.shared_gated:
            hs = ctx.empty(t, self.shared_inter)
            k.swiglu_gate_up(hs, x, self.shared_up.weight.tensor)
            shared = self.shared_down.forward(hs)
        elif self.shared_up is not None:
            if t <= self.FEW:                                            # few rows: the activation in the product's epilogue
                hs = ctx.empty(t, self.shared_inter)
                k.expert_linear(hs, x, None, self.shared_up.weight.tensor.view(1, self.shared_inter, self.hidden),
                                counts[2 * r + 1:], self.act)
            else:
                hs = self.shared_up.forward(x)
                k.activation(hs, self.act)
            shared = self.shared_down.forward(hs)
        out = ctx.empty(t, self.hidden)
        gate = z if shared is not None and not self.shared_gated else None
        if self.identity:                                                # rows from the first identity expert's on: x itself
            k.expert_combine(out, y, place, weight, shared, gate, r, x=x, identity_from=counts[r + e:r + e + 1])
        else:
            k.expert_combine(out, y, place, weight, shared, gate, r)
        return out
