"""Mixers whose memory is a matrix per head and request instead of a cache of keys.

Both keep S [key channel, value channel] in 32-bit per request slot and head (`SlotState`, stored column by column:
[heads, vdim, dim]), zero at admission, and update it token by token with the kernel table's `recurrent_scan`:

    S ← diag(g_t) S;   u = β_t (v_t − Sᵀ k_t)  (or u = v_t);   S ← S + k_t uᵀ;   o_t = Sᵀ q_t.

`Retention`: one fixed decay per head, no β (linear attention without softmax or denominator); q and k turned by the
position, k scaled by dim^(−1/2); each head's o divided by its root mean square, times silu(W_g x), then W_o.

`GatedDelta`: the delta rule with a decay per key channel and token. q, k, v pass a short causal convolution over time
(its last taps − 1 inputs are carried per request, a second `SlotState`) and silu; q and k become unit vectors per head,
q times dim^(−1/2); β = sigmoid(W_b x); g = exp(−exp(A_log) · softplus(W_a2 W_a1 x + dt_bias)); each head's o under an
RMS norm with one weight shared by the heads, times sigmoid(W_g2 W_g1 x), then W_o. Query/key heads may be fewer than
value heads (head h reads key head h // (heads / kv_heads)).

`MLSTM`: a matrix memory with exponential gates. Per head and token a log input gate i = c tanh(a / c) and a log forget gate
f = logsigmoid(c tanh(b / c)) (a, b: the gates' projections with biases, c = `gate_cap`), held in range by a running
maximum m that starts at 0: m_t = max(f + m_(t−1), i); S_t = exp(f + m_(t−1) − m_t) S_(t−1) + exp(i − m_t) k vᵀ, and a
normaliser n_t that follows the same rule with k alone; o = Sᵀq / (max(|n · q|, exp(−m)) + 1e-6) with q scaled by
dim^(−1/2); each head's o divided by its root mean square, times a weight over all heads' channels, times sigmoid(W_g x),
then W_o. n rides as one more value column of S (the value row gets a 1 behind it), so the update is the same scan with a
decay per head and token; m is a second `SlotState`. The gates' projections leave their product in 32-bit.

`GeneralDelta`: the generalized delta rule. Per head, with r, k, v of one size `dim`, a decay w per key channel and token
and a removal rate a per key channel and token, and the token's unit key u = k / sqrt(Σk² + unit_eps):

    S ← diag(w) S − (a ∘ u)(uᵀ S) + k vᵀ   (both terms read the old S),   o = Sᵀ r;

w = exp(−decay_scale · sigmoid(W_w2 tanh(W_w1 x) + w0)) through a low-rank pair, a = sigmoid(W_a x + b_a). Since u is k
times one number c per head and token, the removal term is k_i · a_i c² · (kᵀ S)_j: the scan takes the rate a c² per key
channel beside k itself (`recurrent_scan(rate=)`). Each head's o is divided by its root mean square, times a weight over
all heads' channels, times sigmoid(W_g x), then W_o.

Everything that enters the recurrence is 32-bit (the scan's inputs are made in 32-bit from the first product's rows);
the products themselves are the engine's. All first projections of a mixer are one merged product.
"""
from __future__ import annotations

import torch

from ..config.spec import PartRef
from .base import BuildContext, Part, SlotState, take_link
from .linear import Linear

ACT_TANH = 5                          # the kernel table's activation code (parts/experts.py: ACTIVATIONS)


class _MatrixState(Part):
    """What both mixers share: no paged cache, one state matrix per head, loadable names without the children's."""

    def cache(self):
        return None

    def _strip(self, prefix: str, name: str) -> str:
        for child in ("first.", "low.", "high.", "out.", "gates."):
            if name.startswith(prefix + child):
                return prefix + name[len(prefix + child):]
        return name

    def loadables(self, prefix: str = ""):
        for name, p, rows in super().loadables(prefix):
            yield self._strip(prefix, name), p, rows


class Retention(_MatrixState):
    def __init__(self, ctx: BuildContext, *, heads: int, dim: int, vdim: int, decay: tuple[float, ...], eps: float,
                 hidden: int, position: PartRef | None, layer: int = 0) -> None:
        super().__init__()
        if len(decay) != heads:
            raise ValueError(f"retention: {len(decay)} decays for {heads} heads")
        self.ctx, self.heads, self.dim, self.vdim, self.eps = ctx, heads, dim, vdim, float(eps)
        self.decay = tuple(float(d) for d in decay)
        self.first = self.add_child("first", Linear(ctx, "weight", hidden, {
            "q": heads * dim, "k": heads * dim, "v": heads * vdim, "g": heads * vdim}))
        self.out = self.add_child("out", Linear(ctx, "weight", heads * vdim, {"o": hidden}))
        self.position = self.add_child("position", ctx.part(position, head_dim=dim)) if position else None
        self._decay = None

    def finalize(self) -> None:
        super().finalize()
        if self.first.weight.tensor is not None:
            self._decay = torch.tensor(self.decay, dtype=torch.float32, device=self.first.weight.tensor.device)

    def slot_states(self):
        return (SlotState("state", (self.heads, self.vdim, self.dim)),)

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        t, k, ctx, heads, dim, vdim = x.shape[0], self.ctx.kernels, self.ctx, self.heads, self.dim, self.vdim
        first = self.first.forward(x)                                    # [t, q | k | v | g]
        qk = ctx.empty(t, 2, heads, dim, dtype=torch.float32)
        v = ctx.empty(t, heads, vdim, dtype=torch.float32)
        pos = self.position
        k.retention_prepare(qk, v, first, step.positions, pos.table if pos else None, pos.rotary_dim if pos else 0,
                            dim ** -0.5)
        o = ctx.empty(t, heads, vdim, dtype=torch.float32)
        k.recurrent_scan(o, qk, v, None, self._decay, None, cache.slots["state"], step.rows)
        y = ctx.empty(t, heads, vdim)
        at = 2 * heads * dim + heads * vdim
        k.head_norm_gate(y, o, None, None, first[:, at:at + heads * vdim], self.eps)
        return self.out.forward(y.view(t, heads * vdim))


class GatedDelta(_MatrixState):
    UNIT_EPS = 1e-6                       # inside the root of the unit vectors

    def __init__(self, ctx: BuildContext, *, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, decay_rank: int,
                 gate_rank: int, eps: float, hidden: int, layer: int = 0) -> None:
        super().__init__()
        if heads % kv_heads:
            raise ValueError(f"gated delta: {heads} heads are no multiple of {kv_heads} key heads")
        if taps < 1:
            raise ValueError("gated delta: the convolution has at least one tap")
        self.ctx, self.heads, self.kv_heads, self.dim, self.vdim = ctx, heads, kv_heads, dim, vdim
        self.taps, self.eps = int(taps), float(eps)
        nq, nv = kv_heads * dim, heads * vdim
        self.channels = 2 * nq + nv
        self.first = self.add_child("first", Linear(ctx, "weight", hidden, {"q": nq, "k": nq, "v": nv, "b": heads}))
        self.low = self.add_child("low", Linear(ctx, "weight", hidden, {"a1": decay_rank, "g1": gate_rank}))
        self.second = None                 # [heads dim + heads vdim, ranks]: a2 and g2 as one block-diagonal weight (finalize)
        self.conv = self.add_param("conv", (self.channels, taps), "matrix",
                                   {"q.conv": (0, nq), "k.conv": (nq, 2 * nq), "v.conv": (2 * nq, self.channels)})
        self.a2 = self.add_param("a2", (heads * dim, decay_rank), "matrix")
        self.g2 = self.add_param("g2", (nv, gate_rank), "matrix")
        self.dt_bias = self.add_param("dt_bias", (heads * dim,), "coef")
        self.rate_log = self.add_param("A_log", (heads,), "coef")
        self.gain = self.add_param("norm", (vdim,), "coef")
        self.out = self.add_child("out", Linear(ctx, "weight", nv, {"o": hidden}))

    def finalize(self) -> None:
        super().finalize()
        a2, g2 = self.a2.tensor, self.g2.tensor
        if a2 is not None and g2 is not None:                 # one product for both low-rank second projections
            self.second = torch.zeros(a2.shape[0] + g2.shape[0], a2.shape[1] + g2.shape[1], dtype=a2.dtype, device=a2.device)
            self.second[:a2.shape[0], :a2.shape[1]].copy_(a2)
            self.second[a2.shape[0]:, a2.shape[1]:].copy_(g2)

    def slot_states(self):
        states = [SlotState("state", (self.heads, self.vdim, self.dim))]
        if self.taps > 1:
            dtype = str(self.ctx.dtype).replace("torch.", "")
            states.append(SlotState("conv", (self.taps - 1, self.channels), dtype))
        return tuple(states)

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        t, k, ctx = x.shape[0], self.ctx.kernels, self.ctx
        heads, kvh, dim, vdim = self.heads, self.kv_heads, self.dim, self.vdim
        f32 = torch.float32
        first = self.first.forward(x)                                    # [t, q | k | v | b]
        low2 = ctx.empty(t, self.second.shape[0], dtype=f32)             # [t, a | g]: W_a2 (W_a1 x) and W_g2 (W_g1 x)
        k.linear(low2, self.low.forward(x), self.second)
        qk, v = ctx.empty(t, 2, kvh, dim, dtype=f32), ctx.empty(t, heads, vdim, dtype=f32)
        beta, decay = ctx.empty(t, heads, dtype=f32), ctx.empty(t, heads, dim, dtype=f32)
        gate = ctx.empty(t, heads * vdim, dtype=f32)
        carried = cache.slots.get("conv")
        k.delta_prepare(qk, v, beta, decay, gate, first, self.conv.tensor, carried, low2, self.dt_bias.tensor,
                        self.rate_log.tensor, step.rows, dim ** -0.5, self.UNIT_EPS)
        k.conv_carry(carried, first, self.channels, self.taps, step.rows)
        o = ctx.empty(t, heads, vdim, dtype=f32)
        k.recurrent_scan(o, qk, v, decay, None, beta, cache.slots["state"], step.rows)
        y = ctx.empty(t, heads, vdim)
        k.head_norm_gate(y, o, self.gain.tensor, gate, None, self.eps)
        return self.out.forward(y.view(t, heads * vdim))


class MLSTM(_MatrixState):
    TINY = 1e-6                           # added to the denominator of the read-out

    def __init__(self, ctx: BuildContext, *, heads: int, dim: int, vdim: int, gate_cap: float, eps: float, hidden: int,
                 layer: int = 0) -> None:
        super().__init__()
        if not gate_cap > 0:
            raise ValueError("mlstm: gate_cap must be positive")
        self.ctx, self.heads, self.dim, self.vdim = ctx, heads, dim, vdim
        self.cap, self.eps = float(gate_cap), float(eps)
        self.first = self.add_child("first", Linear(ctx, "weight", hidden, {
            "q": heads * dim, "k": heads * dim, "v": heads * vdim, "g": heads * vdim}))
        self.gates = self.add_child("gates", Linear(ctx, "weight", hidden, {"i": heads, "f": heads}))
        self.gate_bias = self.add_param("gate_bias", (2 * heads,), "coef", {"i.b": (0, heads), "f.b": (heads, 2 * heads)})
        self.gain = self.add_param("norm", (heads * vdim,), "coef")
        self.out = self.add_child("out", Linear(ctx, "weight", heads * vdim, {"o": hidden}))

    def slot_states(self):
        return (SlotState("state", (self.heads, self.vdim + 1, self.dim)), SlotState("max", (self.heads,)))

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        t, k, ctx, heads, dim, vdim = x.shape[0], self.ctx.kernels, self.ctx, self.heads, self.dim, self.vdim
        f32 = torch.float32
        first = self.first.forward(x)                                    # [t, q | k | v | g]
        pre = self.gates.forward(x, out_dtype=f32)                       # [t, i | f] before bias, cap and logsigmoid
        gates = ctx.empty(3, t, heads, dtype=f32)                        # keep, take, exp(-m)
        k.mlstm_gates(gates, pre, self.gate_bias.tensor, self.cap, cache.slots["max"], step.rows)
        qk, v1 = ctx.empty(t, 2, heads, dim, dtype=f32), ctx.empty(t, heads, vdim + 1, dtype=f32)
        k.mlstm_prepare(qk, v1, gates[1], first, dim ** -0.5)
        o1 = ctx.empty(t, heads, vdim + 1, dtype=f32)
        k.recurrent_scan(o1, qk, v1, None, None, None, cache.slots["state"], step.rows, token_decay=gates[0])
        y = ctx.empty(t, heads, vdim)
        at = 2 * heads * dim + heads * vdim
        k.mlstm_read_out(y, o1, gates[2], self.gain.tensor, first[:, at:at + heads * vdim], self.eps, self.TINY)
        return self.out.forward(y.view(t, heads * vdim))


class GeneralDelta(_MatrixState):
    def __init__(self, ctx: BuildContext, *, heads: int, dim: int, decay_rank: int, eps: float, hidden: int,
                 decay_scale: float = 0.6065306597126334, unit_eps: float = 1e-6, layer: int = 0) -> None:
        super().__init__()
        if min(heads, dim, decay_rank) < 1:
            raise ValueError("general delta: heads, dim and decay_rank must be positive")
        self.ctx, self.heads, self.dim, self.eps = ctx, heads, dim, float(eps)
        self.decay_scale, self.unit_eps = float(decay_scale), float(unit_eps)
        n = heads * dim
        self.first = self.add_child("first", Linear(ctx, "weight", hidden, {"r": n, "k": n, "v": n, "g": n, "a": n}))
        self.low = self.add_child("low", Linear(ctx, "weight", hidden, {"w1": decay_rank}))
        self.high = self.add_child("high", Linear(ctx, "weight", decay_rank, {"w2": n}))
        self.decay_bias = self.add_param("w0", (n,), "coef")
        self.rate_bias = self.add_param("a.b", (n,), "coef")
        self.gain = self.add_param("norm", (n,), "coef")
        self.out = self.add_child("out", Linear(ctx, "weight", n, {"o": hidden}))

    def slot_states(self):
        return (SlotState("state", (self.heads, self.dim, self.dim)),)

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        t, k, ctx, heads, dim = x.shape[0], self.ctx.kernels, self.ctx, self.heads, self.dim
        f32, n = torch.float32, heads * dim
        first = self.first.forward(x)                                    # [t, r | k | v | g | a]
        low = self.low.forward(x)
        k.activation(low, ACT_TANH)
        pre = self.high.forward(low, out_dtype=f32)                      # [t, heads dim]: the decays before bias and sigmoid
        qk, v = ctx.empty(t, 2, heads, dim, dtype=f32), ctx.empty(t, heads, dim, dtype=f32)
        decay, rate = ctx.empty(t, heads, dim, dtype=f32), ctx.empty(t, heads, dim, dtype=f32)
        k.gdelta_prepare(qk, v, decay, rate, first, pre, self.decay_bias.tensor, self.rate_bias.tensor,
                         self.decay_scale, self.unit_eps)
        o = ctx.empty(t, heads, dim, dtype=f32)
        k.recurrent_scan(o, qk, v, decay, None, None, cache.slots["state"], step.rows, rate=rate)
        y = ctx.empty(t, heads, dim)
        k.head_norm_gate(y, o, self.gain.tensor, None, first[:, 3 * n:4 * n], self.eps, gate="sigmoid")
        return self.out.forward(y.view(t, n), link=take_link(step))
