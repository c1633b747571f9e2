"""SwiGLU: down(silu(gate(x)) · up(x)), gate and up in one product with gate's rows first, silu in 32-bit
(std/holon_std/ffn/units.py:12-50; std/holon_std/ffn/reference.py:7-12).

ClampedGLU: a gated unit whose inputs are clamped, with a bias on every projection: g = min(W_gate x + b, limit),
u = clamp(W_up x + b, −limit, limit), y = g · sigmoid(alpha · g) · (u + 1), output W_down y + b.

MLP: W_down act(W_up x), no gate and no bias; `activation` as the experts name theirs ("gelu_tanh": the tanh form of
gelu, 0.5 z (1 + tanh(√(2/π) (z + 0.044715 z³))); "xielu": with two stored numbers p, q (`act`), softplus(p) z² + z/2 for
z > 0 and (1/2 + softplus(q)) (exp(z) − 1 − z) + z/2 otherwise)."""
from __future__ import annotations

import torch

from .base import BuildContext, Part, take_link
from .linear import Linear


class SwiGLU(Part):
    def __init__(self, ctx: BuildContext, *, inter: int, hidden: int, layer: int = 0) -> None:
        super().__init__()
        self.ctx, self.inter = ctx, inter
        self.gate_up = self.add_child("gate_up", Linear(ctx, "weight", hidden, {
            "gate_proj.weight": inter, "up_proj.weight": inter}))
        self.down = self.add_child("down_proj", Linear(ctx, "weight", inter, {"weight": hidden}))

    def loadables(self, prefix: str = ""):
        for name, p, rows in super().loadables(prefix):
            yield name.replace(prefix + "gate_up.", prefix, 1), p, rows

    takes_scaled = True                      # x may be base.Scaled: the first product applies the row scale

    def forward(self, x: torch.Tensor, step) -> torch.Tensor | None:
        act = self.ctx.empty(x.shape[0], self.inter)
        self.ctx.kernels.swiglu_gate_up(act, x, self.gate_up.weight.tensor)
        return self.down.forward(act, link=take_link(step))


class ClampedGLU(Part):
    def __init__(self, ctx: BuildContext, *, inter: int, hidden: int, limit: float, alpha: float = 1.702,
                 layer: int = 0) -> None:
        super().__init__()
        self.ctx, self.inter, self.limit, self.alpha = ctx, inter, float(limit), float(alpha)
        self.gate_up = self.add_child("gate_up_proj", Linear(ctx, "weight", hidden, {"gate": inter, "up": inter}))
        self.first_bias = self.add_param("first_bias", (2 * inter,), "matrix", {"gate.b": (0, inter), "up.b": (inter, 2 * inter)})
        self.down = self.add_child("down_proj", Linear(ctx, "weight", inter, {"down": hidden}))
        self.down_bias = self.add_param("down.b", (hidden,), "matrix")

    def loadables(self, prefix: str = ""):
        for name, p, rows in super().loadables(prefix):
            for child in ("gate_up_proj.", "down_proj."):
                if name.startswith(prefix + child):
                    name = prefix + name[len(prefix + child):]
            yield name, p, rows

    def forward_biased(self, x: torch.Tensor, step):
        """(W_down y, its bias): a block that sums several parts adds the bias there."""
        k = self.ctx.kernels
        z = self.gate_up.forward(x)
        act = self.ctx.empty(x.shape[0], self.inter)
        k.glu_clamped(act, z, self.first_bias.tensor, self.limit, self.alpha)
        return self.down.forward(act), self.down_bias.tensor

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        y, bias = self.forward_biased(x, step)
        return y + bias


class MLP(Part):
    def __init__(self, ctx: BuildContext, *, inter: int, hidden: int, activation: str = "gelu_tanh", layer: int = 0) -> None:
        super().__init__()
        from .experts import ACTIVATIONS
        if activation not in ACTIVATIONS:
            raise ValueError(f"mlp: activation {activation!r}; known: {sorted(ACTIVATIONS)}")
        self.ctx, self.inter, self.act = ctx, inter, ACTIVATIONS[activation]
        self.numbers = self.add_param("act", (2,), "coef") if activation == "xielu" else None
        self.up = self.add_child("up_proj", Linear(ctx, "weight", hidden, {"up": inter}))
        self.down = self.add_child("down_proj", Linear(ctx, "weight", inter, {"down": hidden}))

    def loadables(self, prefix: str = ""):
        for name, p, rows in super().loadables(prefix):
            for child in ("up_proj.", "down_proj."):
                if name.startswith(prefix + child):
                    name = prefix + name[len(prefix + child):]
            yield name, p, rows

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        z = self.up.forward(x)
        if self.numbers is not None:
            self.ctx.kernels.activation(z, self.act, self.numbers.tensor)
        else:
            self.ctx.kernels.activation(z, self.act)
        return self.down.forward(z)
