"""Grouped-query attention over a paged cache.

qkv = x·Wqkvᵀ in one product; per head RMSNorm of q and k (optional), rotation, keys and values written to the
step's pages, attention of the new rows over everything the request holds, output projection
(std/holon_std/mixers/gqa/units.py:108-294; formulas std/holon_std/mixers/gqa/reference.py:26-60, 91-101).
Query head h reads KV head h // (heads / kv_heads); a query at position p sees keys j ≤ p, and with a window W > 0
only those with p − j < W.

Options that other designs use, each a constructor argument: `scale` (the score scale, 1/√head_dim unless given);
`unit_norm_eps` (q and k are divided by their root mean square per head, a norm without a weight, in place of
`qk_norm`); `values_are_keys` (there is no value projection: a token's value is its key as projected, before any norm;
the merged product then has the key's rows twice, so that the cache write stores the normed copy as the key and the
plain copy as the value); `sink` (one learned number per head, stored as `sink`: exp(sink) stands in the softmax's
denominator, without key or value and without the score scale); `names` (the stored names of the q, k, v and output
weights, where they are not `q_proj.weight` and so on); `biases` (q, k and v carry biases, stored under the weights'
names with `.b` behind the stem, added before norm and rotation; the output projection has none).
"""
from __future__ import annotations

import torch

from ..config.spec import PartRef
from .base import BuildContext, PagedKV, PagedRows, Part, take_link
from .linear import Linear


class GQA(Part):
    def __init__(self, ctx: BuildContext, *, heads: int, kv_heads: int, head_dim: int, hidden: int,
                 position: PartRef | None, qk_norm: PartRef | None = None, window: int = 0, layer: int = 0,
                 scale: float | None = None, unit_norm_eps: float | None = None, values_are_keys: bool = False,
                 sink: bool = False, names: tuple[tuple[str, str], ...] = (), biases: bool = False) -> None:
        super().__init__()
        if biases and values_are_keys:
            raise ValueError("gqa: biases do not go with values_are_keys")
        if heads % kv_heads:
            raise ValueError(f"gqa: {heads} heads are no multiple of {kv_heads} kv heads")
        if qk_norm is not None and unit_norm_eps is not None:
            raise ValueError("gqa: give qk_norm or unit_norm_eps, not both")
        self.ctx, self.heads, self.kv_heads, self.head_dim, self.window = ctx, heads, kv_heads, head_dim, int(window)
        self.scale = 1.0 / head_dim ** 0.5 if scale is None else float(scale)
        self.unit_norm_eps, self.values_are_keys = unit_norm_eps, bool(values_are_keys)
        self._names = {"q_proj.weight": "q_proj.weight", "k_proj.weight": "k_proj.weight",
                       "v_proj.weight": "v_proj.weight", "o_proj.weight": "o_proj.weight", **dict(names)}
        pieces = {"q_proj.weight": heads * head_dim, "k_proj.weight": kv_heads * head_dim}
        if not values_are_keys:
            pieces["v_proj.weight"] = kv_heads * head_dim
        self.qkv = self.add_child("qkv", Linear(ctx, "weight", hidden, pieces,
                                                spare=kv_heads * head_dim if values_are_keys else 0))
        self.o_proj = self.add_child("o_proj", Linear(ctx, "weight", heads * head_dim, {"weight": hidden}))
        self.sink = self.add_param("sink", (heads,), "coef") if sink else None
        self.bias = None
        if biases:                           # one vector beside the merged product's rows: q | k | v
            nq, nk = heads * head_dim, kv_heads * head_dim
            def stem(which):                 # `x.weight` goes with `x.bias`, a bare stored name `x` with `x.b`
                name = self._names[which]
                return name[:-len(".weight")] + ".bias" if name.endswith(".weight") else name + ".b"
            self.bias = self.add_param("qkv_bias", (nq + 2 * nk,), "matrix", {
                stem("q_proj.weight"): (0, nq), stem("k_proj.weight"): (nq, nq + nk), stem("v_proj.weight"): (nq + nk, nq + 2 * nk)})
        self._unit = None                    # the gain of a norm without a weight: ones (made in finalize)
        self.q_norm = self.k_norm = None
        if qk_norm is not None:
            self.q_norm = self.add_child("q_norm", ctx.part(qk_norm, dim=head_dim))
            self.k_norm = self.add_child("k_norm", ctx.part(qk_norm, dim=head_dim))
        self.position = self.add_child("position", ctx.part(position, head_dim=head_dim)) if position else None

    # the loadable names of the merged product are the stored ones, without the child's own prefix
    def loadables(self, prefix: str = ""):
        for name, p, rows in super().loadables(prefix):
            name = name.replace(prefix + "qkv.", prefix, 1)
            yield prefix + self._names.get(name[len(prefix):], name[len(prefix):]), p, rows

    def finalize(self) -> None:
        super().finalize()
        w = self.qkv.weight.tensor
        if w is not None:
            if self.values_are_keys:                                 # the value rows: the key's, a second time
                n, at = self.kv_heads * self.head_dim, self.heads * self.head_dim
                w[at + n:at + 2 * n].copy_(w[at:at + n])
            if self.unit_norm_eps is not None:
                self._unit = torch.ones(self.head_dim, dtype=w.dtype, device=w.device)

    takes_scaled = True                      # x may be base.Scaled: both first products apply the row scale

    def cache(self) -> PagedKV:
        return PagedKV(self.kv_heads, self.head_dim, self.window)

    def slot_states(self):
        return ()

    @property
    def plan_group(self):
        """Mixers with equal answers here plan a captured step alike: one of them is asked."""
        return "gqa", self.heads, self.kv_heads, self.head_dim, self.window

    def capture_plan(self, step, max_model_len: int):
        """What the attention kernels pin for a step that is captured as a CUDA graph (see base.Part)."""
        plan = getattr(self.ctx.kernels, "attention_capture_plan", None)
        return plan(step.rows, max_model_len) if plan is not None else None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        t, k = x.shape[0], self.ctx.kernels
        q = self.ctx.empty(t, self.heads, self.head_dim)
        norm, pos = self.q_norm, self.position
        q_gain, k_gain = (norm.weight.tensor, self.k_norm.weight.tensor) if norm else (self._unit, self._unit)
        eps = norm.eps if norm else (self.unit_norm_eps or 0.0)
        after = (step.positions, pos.table if pos else None, pos.rotary_dim if pos else 0,
                 q_gain, k_gain, eps, norm.offset if norm else 0.0,
                 cache.kv if cache.fills else None, cache.group.write_index if cache.fills else None,
                 self.heads, self.kv_heads, self.head_dim)
        fused = getattr(k, "qkv_rope", None)                         # a kernel table may do the product and what follows in one
        if self.bias is not None:                                    # (the fused product knows no bias)
            k.qk_norm_rope_kv_write(q, self.qkv.forward(x), *after, bias=self.bias.tensor)
        elif fused is None or not fused(q, x, self.qkv.weight.tensor, *after):
            k.qk_norm_rope_kv_write(q, self.qkv.forward(x), *after)
        o = self.ctx.empty(t, self.heads, self.head_dim)
        if self.sink is not None:
            k.paged_attention(o, q, cache.kv, cache.group.block_table, step.rows, self.scale, self.window, self.sink.tensor)
        else:
            k.paged_attention(o, q, cache.kv, cache.group.block_table, step.rows, self.scale, self.window)
        return self.o_proj.forward(o.view(t, self.heads * self.head_dim), link=take_link(step))


class TalkingAttention(Part):
    """Grouped-query attention whose heads share their softmax weights, with keys and values of unequal sizes.

        s_g(i, j) = q_g(i) · k_kv(g)(j) · scale · temp[g],    p_g(i, ·) = softmax over the keys i sees,
        out_h(i)  = Σ_j (Σ_g talk[h, g] p_g(i, j)) v_kv(h)(j)

    `talk` [heads, heads] mixes the heads' weights after the softmax (`talking`), `temp` [heads] is a learned factor on each
    head's scores (`head_temperature`); without them the mixer is plain attention. Which keys j ≤ i a query sees: with
    `chunk` C only those of its own block of C positions (blocks counted from the sequence's first token, wherever a
    prompt was cut), with `window` W only the last W. q and k carry biases (`biases`: q.b, k.b, v.b, o.b; "qkv": none on the output) and a per-head
    RMS norm with one plain weight shared by the heads (`qk_eps` not None: q.norm, k.norm), then the position's
    rotation. `blend`: "keep" leaves this layer's values (as projected, 32-bit) on the step under `blend_key` for later
    layers; "mix" replaces this layer's values by (1 − λ) v + λ v_kept with the stored number `vmix`, and that is what the
    cache holds; in both cases the stored `vmix` is loaded (the keeping layer does not use it). Scores, weights and
    sums are 32-bit; q, keys and values are kept in the engine's dtype.

    The cache keeps per token and kv head one row [key | value] (`PagedRows`). `forward_biased` returns the output
    projection's product and its bias apart, for a block that adds the bias in its own sum."""

    def __init__(self, ctx: BuildContext, *, heads: int, kv_heads: int, key_dim: int, value_dim: int, hidden: int,
                 scale: float, position: PartRef | None = None, qk_eps: float | None = None, chunk: int = 0,
                 window: int = 0, talking: bool = True, head_temperature: bool = True, biases: bool | str = True,
                 blend: str | None = None, blend_key: str = "values", layer: int = 0) -> None:
        super().__init__()
        if heads % kv_heads:
            raise ValueError(f"talking attention: {heads} heads are no multiple of {kv_heads} kv heads")
        if blend not in (None, "keep", "mix"):
            raise ValueError(f"talking attention: blend {blend!r}; known: None, 'keep', 'mix'")
        self.ctx, self.heads, self.kv_heads, self.key_dim, self.value_dim = ctx, heads, kv_heads, key_dim, value_dim
        self.scale, self.qk_eps, self.chunk, self.window = float(scale), qk_eps, int(chunk), int(window)
        self.blend, self.blend_key = blend, blend_key
        nq, nk, nv = heads * key_dim, kv_heads * key_dim, kv_heads * value_dim
        self.first = self.add_child("first", Linear(ctx, "weight", hidden, {"q": nq, "k": nk, "v": nv}))
        self.out = self.add_child("out", Linear(ctx, "weight", heads * value_dim, {"o": hidden}))
        self.first_bias = self.out_bias = None
        if biases not in (True, False, "qkv"):
            raise ValueError(f"talking attention: biases {biases!r}; known: True, False, 'qkv' (none on the output)")
        if biases:
            self.first_bias = self.add_param("first_bias", (nq + nk + nv,), "matrix",
                                             {"q.b": (0, nq), "k.b": (nq, nq + nk), "v.b": (nq + nk, nq + nk + nv)})
            if biases is True:
                self.out_bias = self.add_param("o.b", (hidden,), "matrix")
        self.q_gain = self.add_param("q.norm", (key_dim,), "coef") if qk_eps is not None else None
        self.k_gain = self.add_param("k.norm", (key_dim,), "coef") if qk_eps is not None else None
        self.talk = self.add_param("talk", (heads, heads), "coef") if talking else None
        self.temp = self.add_param("temp", (heads,), "coef") if head_temperature else None
        self.lam = self.add_param("vmix", (), "coef", optional=not blend)        # (a layer that does not blend may store it)
        self.position = self.add_child("position", ctx.part(position, head_dim=key_dim)) if position else None

    def loadables(self, prefix: str = ""):
        for name, p, rows in super().loadables(prefix):
            for child in ("first.", "out."):
                if name.startswith(prefix + child):
                    name = prefix + name[len(prefix + child):]
            yield name, p, rows

    @property
    def plan_group(self):
        return "talking", self.heads, self.kv_heads, self.key_dim, self.value_dim, self.chunk, self.window

    def capture_plan(self, step, max_model_len: int):
        """What the attention kernels pin for a step that is captured as a CUDA graph (see base.Part)."""
        plan = getattr(self.ctx.kernels, "attention_capture_plan", None)
        return plan(step.rows, max_model_len) if plan is not None else None

    def cache(self) -> PagedRows:
        return PagedRows(self.kv_heads, self.key_dim, self.value_dim, self.window)

    def slot_states(self):
        return ()

    def forward_biased(self, x: torch.Tensor, step, cache):
        t, k, ctx = x.shape[0], self.ctx.kernels, self.ctx
        heads, kvh, kd, vd = self.heads, self.kv_heads, self.key_dim, self.value_dim
        qkv = self.first.forward(x)
        q = ctx.empty(t, heads, kd)
        keep = first = None
        if self.blend == "keep":
            keep = step.shared[self.blend_key] = ctx.empty(t, kvh, vd, dtype=torch.float32)
        elif self.blend == "mix":
            first = step.shared.get(self.blend_key)
            if first is None:
                raise RuntimeError(f"talking attention: no earlier layer of this step has left its values ({self.blend_key!r})")
        pos = self.position
        k.qkv_talking_prepare(q, cache.kv if cache.fills else None, keep, qkv,
                              self.first_bias.tensor if self.first_bias else None,
                              self.q_gain.tensor if self.q_gain else None, self.k_gain.tensor if self.k_gain else None,
                              self.qk_eps or 0.0, step.positions, pos.table if pos else None, pos.rotary_dim if pos else 0,
                              bool(pos and pos.interleaved), first, self.lam.tensor if first is not None else None,
                              cache.group.write_index if cache.fills else None, heads, kvh, kd, vd)
        o = ctx.empty(t, heads, vd)
        k.attention_talking(o, q, cache.kv, cache.group.block_table, step.rows, self.scale,
                            self.temp.tensor if self.temp else None, self.chunk, self.window,
                            self.talk.tensor if self.talk else None)
        return self.out.forward(o.view(t, heads * vd)), (self.out_bias.tensor if self.out_bias else None)

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        y, bias = self.forward_biased(x, step, cache)
        return y if bias is None else y + bias
