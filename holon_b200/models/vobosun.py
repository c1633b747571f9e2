"""Vobosun: its typed configuration and its recipe.

A decoder whose config.json lists its layers one by one (`layers[i]`: `type`, the mixer's sizes under `mixer`, the
feed-forward under `mlp` or null, and optionally `weights_of: j`). A layer has a norm before and behind each sublayer
(block `sandwich`): x ← x + N1b(mixer(shift(N1(x)))), then x ← x + N2b(ff(N2(x))). The norm is a tanh without mean or
variance, tanh(alpha · x) · w + b (norm `dyt`). What the mixer reads is blended with the token before,
m = h + (h_before − h) · shift, the token before's h being part of a request's state in every layer. Mixer types:
`attention` (grouped-query attention with biases on q, k, v, a half-split rotation whose frequencies are divided by
`rot.scaling.factor`, a score scale from the configuration, key and value sizes free of one another) and
`general_delta` (a matrix state per head under the generalized delta rule: a decay per key channel and token from a
low-rank projection, and a removal rate per key channel along the token's unit key). Feed-forwards are `dense`
(W_down xielu(W_up y) with two stored numbers) or `moe` (gated silu experts without biases, chosen in groups by a
softmax score plus a stored correction, identity experts behind the real ones, a shared expert beside them). A layer
with `weights_of: j` has no tensors: it runs layer j's parts on a cache entry and state of its own. The head has a
weight of its own.

Keys read: `architecture`, `width`, `vocab`, `norm.eps`, `layers[i].{type, weights_of, mixer, mlp}`; attention:
`mixer.{heads, kv_heads, dim, vdim, scale, rot.{base, dims, scaling.factor}}`; general_delta: `mixer.{heads, dim}`;
`mlp.{kind, ff}` or `mlp.{kind, expert.ff, router.{experts, top, identity, groups.{count, keep}}, shared.ff}`. A missing
`rot` is a layer without rotation, a missing `scaling` a factor of 1, a missing `groups` one group, a missing
`identity` none, a missing `shared` no shared expert. One size stands in no key of a stored model's config.json, the
rank of the delta rule's low-rank decay projection: `complete` reads it from the shape of `l<i>.mix.w1` and enters it
as `mixer.decay_rank` (a config dict made by hand, for random weights, gives it itself).
Stored tensors: `embed`, `head`, `final.norm{, .b, .alpha}`, `l<i>.{norm1, norm1b, norm2, norm2b}{, .b, .alpha}`,
`l<i>.shift`, `l<i>.mix.{q, k, v}` with `.b` each and `l<i>.mix.o` (attention), `l<i>.mix.{r, k, v, g, a, a.b, w1, w2,
w0, norm, o}` (general_delta), `l<i>.mlp.{up, down, act}` or `l<i>.mlp.{router, correction, e<j>.{gate, up, down},
shared.{gate, up, down}}`.
"""
from __future__ import annotations

import copy
import dataclasses
import math
from collections.abc import Mapping
from typing import Any

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartRef, Run, WeightRule
from .rulorax import _get

DECAY_SCALE = math.exp(-0.5)          # the decay of a key channel is exp(−DECAY_SCALE · sigmoid(·)): never below 0.545
UNIT_EPS = 1e-6                       # inside the root of the unit key
WEIGHT_TINY = 1e-20                   # added to the sum of the chosen experts' scores


@dataclasses.dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int                 # 0: no rotation
    rot_factor: float


@dataclasses.dataclass(frozen=True)
class DeltaSizes:
    heads: int
    dim: int
    decay_rank: int


@dataclasses.dataclass(frozen=True)
class DenseUnit:
    ff: int


@dataclasses.dataclass(frozen=True)
class ExpertUnits:
    experts: int                  # real experts, with tensors
    identity: int                 # identity experts behind them
    top: int
    groups: int
    keep: int
    ff: int
    shared_ff: int                # 0: no shared expert


@dataclasses.dataclass(frozen=True)
class VobosunLayer:
    kind: str                     # "attention" | "general_delta"
    mixer: AttentionSizes | DeltaSizes
    mlp: DenseUnit | ExpertUnits | None
    weights_of: int | None = None


@dataclasses.dataclass(frozen=True)
class VobosunConfig:
    width: int
    vocab: int
    eps: float
    layers: tuple[VobosunLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs with."""
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "VobosunConfig":
        listed = c.get("layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must list the layers")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _get(entry, "type", str, where)
            m = _get(entry, "mixer", Mapping, where)
            wm = where + ".mixer"
            if kind == "attention":
                rot = m.get("rot")
                scaling = rot.get("scaling") if isinstance(rot, Mapping) else None
                mixer = AttentionSizes(
                    heads=_get(m, "heads", int, wm), kv_heads=_get(m, "kv_heads", int, wm), dim=_get(m, "dim", int, wm),
                    vdim=_get(m, "vdim", int, wm), scale=_get(m, "scale", float, wm),
                    rot_base=_get(rot, "base", float, wm + ".rot") if rot is not None else 0.0,
                    rot_dims=_get(rot, "dims", int, wm + ".rot") if rot is not None else 0,
                    rot_factor=_get(scaling, "factor", float, wm + ".rot.scaling") if scaling is not None else 1.0)
                if min(mixer.heads, mixer.kv_heads, mixer.dim, mixer.vdim) < 1 or mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: {wm}: sizes must be positive and heads a multiple of kv_heads")
                if mixer.rot_dims % 2 or not 0 <= mixer.rot_dims <= mixer.dim:
                    raise ConfigError(f"config.json: {wm}.rot.dims must be even and at most dim")
                if mixer.rot_dims and not (mixer.rot_base > 0 and mixer.rot_factor > 0):
                    raise ConfigError(f"config.json: {wm}.rot: base and scaling.factor must be positive")
            elif kind == "general_delta":
                if "decay_rank" not in m:
                    raise ConfigError(f"config.json: {wm}.decay_rank is given neither by the dict nor by a stored tensor's "
                                      f"shape (l<i>.mix.w1)")
                mixer = DeltaSizes(heads=_get(m, "heads", int, wm), dim=_get(m, "dim", int, wm),
                                   decay_rank=_get(m, "decay_rank", int, wm))
                if min(mixer.heads, mixer.dim, mixer.decay_rank) < 1:
                    raise ConfigError(f"config.json: {wm}: every size must be positive")
            else:
                raise NotImplementedError(f"vobosun: {where} has mixer type {kind!r}; known: attention, general_delta")
            mlp, unit = entry.get("mlp"), None
            if mlp is not None:
                wf = where + ".mlp"
                mkind = _get(mlp, "kind", str, wf)
                if mkind == "dense":
                    unit = DenseUnit(ff=_get(mlp, "ff", int, wf))
                    if unit.ff < 1:
                        raise ConfigError(f"config.json: {wf}.ff must be positive")
                elif mkind == "moe":
                    router = _get(mlp, "router", Mapping, wf)
                    groups, shared = router.get("groups"), mlp.get("shared")
                    listed_all = _get(router, "experts", int, wf + ".router")
                    identity = _get(router, "identity", int, wf + ".router") if router.get("identity") is not None else 0
                    unit = ExpertUnits(
                        experts=listed_all, identity=identity, top=_get(router, "top", int, wf + ".router"),
                        groups=_get(groups, "count", int, wf + ".router.groups") if groups is not None else 1,
                        keep=_get(groups, "keep", int, wf + ".router.groups") if groups is not None else 1,
                        ff=_get(_get(mlp, "expert", Mapping, wf), "ff", int, wf + ".expert"),
                        shared_ff=_get(shared, "ff", int, wf + ".shared") if shared is not None else 0)
                    total = unit.experts + unit.identity
                    if unit.experts < 1 or unit.identity < 0 or unit.ff < 1 or unit.shared_ff < 0 or not 1 <= unit.top <= total:
                        raise ConfigError(f"config.json: {wf}: sizes must be positive and 1 <= top <= experts + identity")
                    if unit.groups < 1 or total % unit.groups or not 1 <= unit.keep <= unit.groups:
                        raise ConfigError(f"config.json: {wf}.router.groups: count must divide experts + identity, "
                                          f"1 <= keep <= count")
                    if unit.keep * (total // unit.groups) < unit.top:
                        raise ConfigError(f"config.json: {wf}.router: the kept groups hold fewer experts than top")
                else:
                    raise NotImplementedError(f"vobosun: {wf}.kind {mkind!r}; known: dense, moe")
            shared_from = entry.get("weights_of")
            if shared_from is not None and (not isinstance(shared_from, int) or isinstance(shared_from, bool)
                                            or not 0 <= shared_from < len(listed) or shared_from == i):
                raise ConfigError(f"config.json: {where}.weights_of must name another layer")
            layers.append(VobosunLayer(kind, mixer, unit, shared_from))
        for i, layer in enumerate(layers):
            j, steps = i, 0
            while layers[j].weights_of is not None:
                j, steps = layers[j].weights_of, steps + 1
                if steps > len(layers):
                    raise ConfigError(f"config.json: layers[{i}].weights_of leads in a circle")
            if (layers[j].kind, layers[j].mixer, layers[j].mlp) != (layer.kind, layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}] runs with layer {j}'s tensors but differs from it")
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        cfg = VobosunConfig(width=_get(c, "width", int, "config"), vocab=_get(c, "vocab", int, "config"),
                            eps=_get(_get(c, "norm", Mapping, "config"), "eps", float, "norm"), layers=tuple(layers),
                            eos_token_ids=eos)
        if cfg.width < 1 or cfg.vocab < 1:
            raise ConfigError("config.json: 'width' and 'vocab' must be positive")
        return cfg


def complete(c: Mapping[str, Any], shapes: Mapping[str, tuple]) -> dict[str, Any]:
    """config.json with `mixer.decay_rank` of the delta-rule layers entered from the stored tensors' shapes."""
    c = copy.deepcopy(dict(c))
    listed = c.get("layers")
    if not isinstance(listed, list):
        return c
    for i, entry in enumerate(listed):
        if not isinstance(entry, dict) or entry.get("type") != "general_delta" or not isinstance(entry.get("mixer"), dict):
            continue
        j, steps = i, 0
        while isinstance(listed[j], dict) and isinstance(listed[j].get("weights_of"), int) \
                and 0 <= listed[j]["weights_of"] < len(listed) and steps <= len(listed):
            j, steps = listed[j]["weights_of"], steps + 1
        stored = f"l{j}.mix.w1"
        if "decay_rank" not in entry["mixer"] and stored in shapes:
            entry["mixer"]["decay_rank"] = int(shapes[stored][0])
    return c


def _norm_rules(stored: str, ours: str) -> tuple[WeightRule, ...]:
    return (WeightRule(stored, ours + ".weight"), WeightRule(stored + ".b", ours + ".bias"),
            WeightRule(stored + ".alpha", ours + ".alpha"))


WEIGHT_RULES = (
    WeightRule("embed", "embed.weight"),
    WeightRule("head", "head.weight"),
    *_norm_rules("final.norm", "norm"),
    *_norm_rules("l{i}.norm1", "layers.{i}.mixer_norm"),
    *_norm_rules("l{i}.norm1b", "layers.{i}.mixer_out_norm"),
    *_norm_rules("l{i}.norm2", "layers.{i}.ffn_norm"),
    *_norm_rules("l{i}.norm2b", "layers.{i}.ffn_out_norm"),
    WeightRule("l{i}.shift", "layers.{i}.shift"),
    WeightRule("l{i}.mix.{rest}", "layers.{i}.mixer.{rest}"),
    WeightRule("l{i}.mlp.{rest}", "layers.{i}.ffn.{rest}"),
)


def recipe(cfg: VobosunConfig) -> ModelSpec:
    norm = PartRef.of("norm", "dyt")
    block = PartRef.of("block", "sandwich", shift=True)
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        order.append(Run(cfg.owner(i), i))
        if layer.weights_of is not None:
            layers.append(None)
            continue
        m = layer.mixer
        if layer.kind == "attention":
            position = PartRef.of("position", "rope", theta=m.rot_base, rotary_dim=m.rot_dims, factor=m.rot_factor) \
                if m.rot_dims else None
            if m.dim == m.vdim:           # keys and values of one size: the cache layout and kernels of plain attention
                mixer = PartRef.of("mixer", "gqa", heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim, position=position,
                                   scale=m.scale, biases=True,
                                   names=(("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"),
                                          ("o_proj.weight", "o")))
            else:                         # sizes that differ: the cache rows [key | value] of the `talking` mixer, unmixed
                mixer = PartRef.of("mixer", "talking", heads=m.heads, kv_heads=m.kv_heads, key_dim=m.dim,
                                   value_dim=m.vdim, scale=m.scale, position=position, talking=False,
                                   head_temperature=False, biases="qkv")
        else:
            mixer = PartRef.of("mixer", "general_delta", heads=m.heads, dim=m.dim, decay_rank=m.decay_rank, eps=cfg.eps,
                               decay_scale=DECAY_SCALE, unit_eps=UNIT_EPS)
        u = layer.mlp
        if u is None:
            ffn = None
        elif isinstance(u, DenseUnit):
            ffn = PartRef.of("ffn", "mlp", inter=u.ff, activation="xielu")
        else:
            ffn = PartRef.of("ffn", "experts", experts=u.experts, identity=u.identity, top=u.top, scale=1.0, inter=u.ff,
                             activation="silu", renormalize=True, gated=True, groups=u.groups, keep_groups=u.keep,
                             correction=True, shared_inter=u.shared_ff or None, shared_gated=True, tiny=WEIGHT_TINY)
        layers.append(LayerSpec(block, mixer, ffn, norm))
    return ModelSpec(hidden=cfg.width, vocab=cfg.vocab, layers=tuple(layers), order=tuple(order),
                     embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=False),
                     weight_rules=WEIGHT_RULES)


register_architecture("Vobosun", VobosunConfig.from_dict, recipe, complete=complete)
