"""Tilarax: its typed configuration and its recipe.

A decoder whose config.json lists its layers one by one (`layers[i]`: `type`, the mixer's sizes under `mixer`, the
feed-forward under `mlp` or null). The norm of a layer stands on each sublayer's output (x ← x + N(mixer(x)), then
x ← x + N(ff(x)), N with a weight stored around zero), and every layer ends with a learned average over the results of
all layers so far and the embedding's rows (block `outnorm`). Mixer types: `attention` (grouped-query attention with
biases, a per-head RMS norm of q and k, a rotation of neighbouring channel pairs, a learned factor per head on the
scores, a mask in blocks of `mask.size` positions, the heads' softmax weights mixed by a learned matrix, and, in layers
that say `v_mix`, values blended with those of the first such layer: mixer `talking`) and `mlstm` (a matrix memory with
exponential gates: mixer `mlstm`). Feed-forwards are `dense` (W_down gelu_tanh(W_up x)) or `moe` (gated silu experts
without biases, chosen by the largest router logits with a bias, weighted by the softmax over the chosen logits). The
head is the embedding table.

Keys read: `architecture`, `width`, `vocab`, `norm.eps`, `layers[i].{type, mixer, mlp}`; attention: `mixer.{heads,
kv_heads, dim, vdim, scale, v_mix, mask.size, rot.{base, dims}}`; mlstm: `mixer.{heads, dim, vdim, gate_cap}`; `mlp.{kind,
ff}` or `mlp.{kind, expert.ff, router.{experts, top}}`. A missing `mask` is an unmasked (causal) layer, a missing `rot`
one without rotation, a missing `v_mix` false. Stored tensors: `embed`, `final.norm`, `l<i>.{norm1, norm2, dwa}`,
`l<i>.mix.{q, k, v, o}` with `.b` each, `l<i>.mix.{q.norm, k.norm, vmix, talk, temp}` (attention),
`l<i>.mix.{q, k, v, g, o, norm, i, i.b, f, f.b}` (mlstm), `l<i>.mlp.{up, down}` or `l<i>.mlp.{router, router.b,
e<j>.{gate, up, down}}`.
"""
from __future__ import annotations

import dataclasses
from collections.abc import Mapping
from typing import Any

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartRef, Run, WeightRule
from .rulorax import _get


@dataclasses.dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int                    # 0: every earlier token is seen
    rot_base: float
    rot_dims: int                 # 0: no rotation
    v_mix: bool


@dataclasses.dataclass(frozen=True)
class MemorySizes:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclasses.dataclass(frozen=True)
class DenseUnit:
    ff: int


@dataclasses.dataclass(frozen=True)
class ExpertUnits:
    experts: int
    top: int
    ff: int


@dataclasses.dataclass(frozen=True)
class TilaraxLayer:
    kind: str                     # "attention" | "mlstm"
    mixer: AttentionSizes | MemorySizes
    mlp: DenseUnit | ExpertUnits | None


@dataclasses.dataclass(frozen=True)
class TilaraxConfig:
    width: int
    vocab: int
    eps: float
    layers: tuple[TilaraxLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "TilaraxConfig":
        listed = c.get("layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must list the layers")
        layers, blended = [], None
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _get(entry, "type", str, where)
            m = _get(entry, "mixer", Mapping, where)
            wm = where + ".mixer"
            if kind == "attention":
                mask, rot = m.get("mask"), m.get("rot")
                v_mix = m.get("v_mix", False)
                if not isinstance(v_mix, bool):
                    raise ConfigError(f"config.json: {wm}.v_mix must be true or false")
                mixer = AttentionSizes(
                    heads=_get(m, "heads", int, wm), kv_heads=_get(m, "kv_heads", int, wm), dim=_get(m, "dim", int, wm),
                    vdim=_get(m, "vdim", int, wm), scale=_get(m, "scale", float, wm),
                    chunk=_get(mask, "size", int, wm + ".mask") if mask is not None else 0,
                    rot_base=_get(rot, "base", float, wm + ".rot") if rot is not None else 0.0,
                    rot_dims=_get(rot, "dims", int, wm + ".rot") if rot is not None else 0, v_mix=v_mix)
                if min(mixer.heads, mixer.kv_heads, mixer.dim, mixer.vdim) < 1 or mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: {wm}: sizes must be positive and heads a multiple of kv_heads")
                if mixer.chunk < 0 or mixer.rot_dims % 2 or not 0 <= mixer.rot_dims <= mixer.dim:
                    raise ConfigError(f"config.json: {wm}: mask.size must not be negative, rot.dims even and at most dim")
                if mixer.rot_dims and not mixer.rot_base > 0:
                    raise ConfigError(f"config.json: {wm}.rot.base must be positive")
                if v_mix:
                    if blended is None:
                        blended = (mixer.kv_heads, mixer.vdim)
                    elif blended != (mixer.kv_heads, mixer.vdim):
                        raise ConfigError(f"config.json: {wm}: layers that blend their values need equal kv_heads and vdim")
            elif kind == "mlstm":
                mixer = MemorySizes(heads=_get(m, "heads", int, wm), dim=_get(m, "dim", int, wm),
                                    vdim=_get(m, "vdim", int, wm), gate_cap=_get(m, "gate_cap", float, wm))
                if min(mixer.heads, mixer.dim, mixer.vdim) < 1 or not mixer.gate_cap > 0:
                    raise ConfigError(f"config.json: {wm}: sizes and gate_cap must be positive")
            else:
                raise NotImplementedError(f"tilarax: {where} has mixer type {kind!r}; known: attention, mlstm")
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
                    unit = ExpertUnits(experts=_get(router, "experts", int, wf + ".router"),
                                       top=_get(router, "top", int, wf + ".router"),
                                       ff=_get(_get(mlp, "expert", Mapping, wf), "ff", int, wf + ".expert"))
                    if unit.ff < 1 or not 1 <= unit.top <= unit.experts:
                        raise ConfigError(f"config.json: {wf}: expert.ff must be positive and 1 <= top <= experts")
                else:
                    raise NotImplementedError(f"tilarax: {wf}.kind {mkind!r}; known: dense, moe")
            layers.append(TilaraxLayer(kind, mixer, unit))
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        cfg = TilaraxConfig(width=_get(c, "width", int, "config"), vocab=_get(c, "vocab", int, "config"),
                            eps=_get(_get(c, "norm", Mapping, "config"), "eps", float, "norm"), layers=tuple(layers),
                            eos_token_ids=eos)
        if cfg.width < 1 or cfg.vocab < 1:
            raise ConfigError("config.json: 'width' and 'vocab' must be positive")
        return cfg


WEIGHT_RULES = (
    WeightRule("embed", "embed.weight"),
    WeightRule("final.norm", "norm.weight"),
    WeightRule("l{i}.norm1", "layers.{i}.mixer_norm.weight"),
    WeightRule("l{i}.norm2", "layers.{i}.ffn_norm.weight"),
    WeightRule("l{i}.dwa", "layers.{i}.depth"),
    WeightRule("l{i}.mix.{rest}", "layers.{i}.mixer.{rest}"),
    WeightRule("l{i}.mlp.{rest}", "layers.{i}.ffn.{rest}"),
)


def recipe(cfg: TilaraxConfig) -> ModelSpec:
    norm = PartRef.of("norm", "rmsnorm", eps=cfg.eps, offset=1.0)
    layers, order, keeper = [], [], None
    for i, layer in enumerate(cfg.layers):
        order.append(Run(i, i))
        m = layer.mixer
        if layer.kind == "attention":
            blend = None
            if m.v_mix:
                blend = "keep" if keeper is None else "mix"
                keeper = i if keeper is None else keeper
            position = PartRef.of("position", "rope", theta=m.rot_base, rotary_dim=m.rot_dims, interleaved=True) \
                if m.rot_dims else None
            mixer = PartRef.of("mixer", "talking", heads=m.heads, kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                               scale=m.scale, position=position, qk_eps=cfg.eps, chunk=m.chunk, blend=blend)
        else:
            mixer = PartRef.of("mixer", "mlstm", heads=m.heads, dim=m.dim, vdim=m.vdim, gate_cap=m.gate_cap, eps=cfg.eps)
        u = layer.mlp
        if u is None:
            ffn = None
        elif isinstance(u, DenseUnit):
            ffn = PartRef.of("ffn", "mlp", inter=u.ff, activation="gelu_tanh")
        else:
            ffn = PartRef.of("ffn", "experts", experts=u.experts, top=u.top, scale=1.0, inter=u.ff, activation="silu",
                             renormalize=True, gated=True, router_bias=True)
        block = PartRef.of("block", "outnorm", average=i + 2, results=len(cfg.layers) + 1)
        layers.append(LayerSpec(block, mixer, ffn, norm))
    return ModelSpec(hidden=cfg.width, vocab=cfg.vocab, layers=tuple(layers), order=tuple(order),
                     embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=True),
                     weight_rules=WEIGHT_RULES)


register_architecture("Tilarax", TilaraxConfig.from_dict, recipe)
