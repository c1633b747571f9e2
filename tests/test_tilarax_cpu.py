"""Tilarax without a GPU: configuration, weight names, and the engine's host side (batch layout, cache entries, the
per-request state of the memory layers, what one layer leaves for later layers of a step) with the CPU twins of the
kernels (tests/ref_kernels.py) against the plain implementation (tests/plain_tilarax.py)."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_tilarax as plain
from helpers import random_prompt
from holon_b200.config.registry import ConfigError, resolve_architecture
from holon_b200.replay import Replayer
from ref_kernels import RefKernels
from replay_tools import portions, run
from tilarax_tools import CONFIGS, compare, exact_logits, make_folder, make_weights, tensor_table


def test_architecture_and_configuration():
    arch = resolve_architecture(CONFIGS["a"])
    cfg = arch.parse(CONFIGS["a"])
    assert arch.name == "Tilarax" and len(cfg.layers) == 5 and cfg.layers[3].mlp is None
    spec = arch.recipe(cfg)
    assert [(r.layer, r.cache, r.fills) for r in spec.order] == [(i, i, True) for i in range(5)]
    assert all(layer.block.name == "outnorm" for layer in spec.layers)
    assert [layer.block.kwargs()["average"] for layer in spec.layers] == [2, 3, 4, 5, 6]
    blends = [layer.mixer.kwargs().get("blend") for layer in spec.layers]
    assert blends == ["keep", None, "mix", None, "mix"]                 # the first blending layer keeps, the later ones mix
    assert spec.layers[0].ffn.name == "mlp" and spec.layers[1].ffn.name == "experts" and spec.layers[3].ffn is None
    b = arch.recipe(arch.parse(CONFIGS["b"]))
    assert [layer.mixer.kwargs().get("blend") for layer in b.layers] == [None, "keep", None]
    assert b.layers[2].mixer.kwargs()["position"] is None and b.layers[2].mixer.kwargs()["chunk"] == 0
    for path, value, error in (
            (("layers", 0, "type"), "retention", NotImplementedError),
            (("layers", 0, "mlp", "kind"), "glu", NotImplementedError),
            (("layers", 0, "mixer", "kv_heads"), 3, ConfigError),
            (("layers", 0, "mixer", "rot", "dims"), 26, ConfigError),
            (("layers", 0, "mixer", "rot", "dims"), 7, ConfigError),
            (("layers", 0, "mixer", "mask", "size"), -1, ConfigError),
            (("layers", 0, "mixer", "v_mix"), 1, ConfigError),
            (("layers", 2, "mixer", "vdim"), 8, ConfigError),               # blending layers: equal value sizes
            (("layers", 1, "mixer", "gate_cap"), 0.0, ConfigError),
            (("layers", 1, "mlp", "router", "top"), 7, ConfigError),
            (("width",), 0, ConfigError)):
        c = copy.deepcopy(CONFIGS["a"])
        at = c
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            arch.parse(c)
    c = copy.deepcopy(CONFIGS["a"])
    del c["layers"][1]["mixer"]["gate_cap"]
    with pytest.raises(ConfigError):
        arch.parse(c)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    from holon_b200.weights import RandomSource
    table = {stored: tuple(shape) for stored, shape, _ in RandomSource(CONFIGS[name], 0).table()}
    assert table == dict(tensor_table(CONFIGS[name]))


def test_a_missing_a_misshapen_and_a_spare_tensor_are_named(tmp_path):
    from safetensors.torch import load_file, save_file
    from holon_b200.weights.loader import WeightError
    folder = make_folder(tmp_path, "b")
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["l1.mix.talk"]
    tensors["l0.mix.i.b"] = torch.zeros(2, dtype=torch.bfloat16)
    tensors["l2.norm2"] = tensors["l1.norm2"].clone()                     # layer 2 has no feed-forward
    tensors["l2.mix.vmix"] = tensors["l1.mix.vmix"].clone()               # a layer that blends nothing may store the number
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels())
    assert e.value.missing == ["l1.mix.talk"] and e.value.unexpected == ["l2.norm2"]
    assert [s[0] for s in e.value.shapes] == ["l0.mix.i.b"]


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param, seed=7)
    config = CONFIGS[request.param]
    prompts = {f"r{i}": random_prompt(config["vocab"], n, 60 + i) for i, n in enumerate((23, 41, 9, 30))}
    return folder, config, prompts, {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}


def test_cache_entries_and_states(model):
    folder, config, _, _ = model
    r = Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels(), page_size=4)
    paged = [i for i, layer in enumerate(config["layers"]) if layer["type"] == "attention"]
    assert sorted(e for g in r.built.cache.groups for e in g.entries) == paged
    states = r.built.cache.slot_states
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        if layer["type"] == "mlstm":                       # the normaliser rides as one more value column
            assert tuple(states[(i, "state")].shape[1:]) == (m["heads"], m["vdim"] + 1, m["dim"])
            assert tuple(states[(i, "max")].shape[1:]) == (m["heads"],) and states[(i, "max")].dtype == torch.float32
        else:
            g = r.built.cache.group_of_entry[i]
            assert tuple(g.kv.shape[2:]) == (m["kv_heads"], 4, m["dim"] + m["vdim"])
    assert r.built.cache.prefix is None or not states


def test_whole_tail_portions_and_mixed(model):
    folder, config, prompts, want = model
    r = Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels(), page_size=4)
    compare(run(r, [([(rid, ids)], [rid]) for rid, ids in prompts.items()]), want, "float32")
    steps = []
    for rid, ids in prompts.items():                                       # a portion, then one by one
        steps.append(([(rid, ids[:5])], []))
        steps += [([(rid, [t])], [rid] if i == len(ids) - 6 else []) for i, t in enumerate(ids[5:])]
    compare(run(r, steps), want, "float32")
    steps = []
    for rid, ids in prompts.items():                                       # from the first token on, one by one
        steps += [([(rid, [t])], [rid] if i == len(ids) - 1 else []) for i, t in enumerate(ids)]
    compare(run(r, steps), want, "float32")
    steps = []
    for rid, ids in prompts.items():                                       # portions down to two tokens, cut inside blocks
        parts = portions(ids, [3, 2, 7, 2, 5])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, "float32")
    # four requests at once in 104 tokens of pool: portions beside single tokens, pages and slots given back and used
    # again (a slot's memory, its running maximum and its pages must not leak into the request that takes it next)
    r = Replayer(str(folder), "float32", 104, device="cpu", kernels=RefKernels(), page_size=4)
    at, steps, sizes = {rid: 0 for rid in prompts}, [], {"r0": [1, 1, 4], "r1": [6, 2, 1], "r2": [2], "r3": [1, 9]}
    live, waiting, turn = ["r0", "r1", "r2"], ["r3"], 0
    while live:
        entries, end = [], []
        for rid in list(live):
            n = min(sizes[rid][turn % len(sizes[rid])], len(prompts[rid]) - at[rid])
            entries.append((rid, prompts[rid][at[rid]:at[rid] + n]))
            at[rid] += n
            if at[rid] == len(prompts[rid]):
                end.append(rid)
                live.remove(rid)
                if waiting:
                    live.append(waiting.pop())
        steps.append((entries, end))
        turn += 1
    got = run(r, steps)
    compare(got, want, "float32")
    assert len(got) == sum(len(ids) for ids in prompts.values())
    again = {"r0": prompts["r1"], "r1": prompts["r0"]}                     # the same slots and pages, other requests
    compare(run(r, [([("r0", again["r0"][:20]), ("r1", again["r1"][:3])], []),
                    ([("r0", again["r0"][20:]), ("r1", again["r1"][3:])], ["r0", "r1"])]),
            {"r0": want["r1"], "r1": want["r0"]}, "float32")


def test_a_request_alone_and_beside_others_agree(model):
    folder, config, prompts, _ = model
    alone = run(Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels(), page_size=4),
                [([("r1", prompts["r1"])], ["r1"])])
    r = Replayer(str(folder), "float32", 128, device="cpu", kernels=RefKernels(), page_size=4)
    both = run(r, [([("r0", prompts["r0"][:7]), ("r1", prompts["r1"][:30])], []),
                   ([("r1", prompts["r1"][30:]), ("r0", prompts["r0"][7:8]), ("r2", prompts["r2"])], ["r0", "r1", "r2"])])
    for pos in range(len(prompts["r1"])):
        assert torch.allclose(alone[("r1", pos)], both[("r1", pos)], atol=2e-5, rtol=0)


def test_planted_keys_at_the_block_s_edges():
    """One attention layer whose query at position p matches the key at position p - 11 and nothing else: with blocks
    of 12 that key is seen from p = 11 + 12 b on only where both lie in one block. The engine's logits follow the
    plain implementation's exactly where the key is inside, and where it is outside; an off-by-one at either edge of a
    block moves a row by most of its spread (the row error is relative to it)."""
    import json
    import pathlib
    import tempfile
    config = copy.deepcopy(CONFIGS["att"])
    m = config["layers"][0]["mixer"]
    m["mask"]["size"], m["scale"] = 12, 12.0 / m["dim"] ** 0.5            # sharp: the best key takes nearly all weight
    weights = make_weights(config, 3)
    ids = random_prompt(config["vocab"], 50, 5)
    with tempfile.TemporaryDirectory() as tmp:
        folder = make_folder(pathlib.Path(tmp), "att", config=config, weights=weights)
        want = {"r": exact_logits(folder, ids)}
        probs = _attention_weights(json.loads((folder / "config.json").read_text()), weights, ids)
        assert float(probs.max(-1).values.median()) > 0.5               # single keys do stand out
        for page in (4, 64):
            r = Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels(), page_size=page)
            compare(run(r, [([("r", ids)], ["r"])]), want, "float32")
            compare(run(r, [([("r", p)], ["r"] if i == 9 else []) for i, p in enumerate(portions(ids, [5]))]), want, "float32")


def _attention_weights(config, weights, ids):
    """The softmax weights of head 0 of the first layer (plain code, for the test above)."""
    m = config["layers"][0]["mixer"]
    x = weights["embed"].double()[torch.tensor(ids)]
    t, dim = len(ids), m["dim"]
    q = (x @ weights["l0.mix.q"].double().T + weights["l0.mix.q.b"].double()).view(t, m["heads"], dim)[:, 0]
    k = (x @ weights["l0.mix.k"].double().T + weights["l0.mix.k.b"].double()).view(t, m["kv_heads"], dim)[:, 0]
    q = plain.rms_unit(q, config["norm"]["eps"]) * weights["l0.mix.q.norm"].double()
    k = plain.rms_unit(k, config["norm"]["eps"]) * weights["l0.mix.k.norm"].double()
    s = (q @ k.T) * m["scale"]
    size = m["mask"]["size"]
    i, j = torch.arange(t)[:, None], torch.arange(t)[None, :]
    s = s.masked_fill((j > i) | (j // size != i // size), -float("inf"))
    return torch.softmax(s, -1)[size:]                                   # (rows that see more than one key)


def test_greedy_generation_through_the_scheduler(model):
    """The engine's own entry point and scheduler: greedy tokens equal the plain implementation's arg max, token by
    token, for requests that arrive together, share three slots and are cut into portions by a small step budget."""
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    from tilarax_tools import read_folder
    folder, config, prompts, _ = model
    stored, weights = read_folder(folder)
    engine = Engine(EngineConfig(model=str(folder), dtype="float32", device="cpu", page_size=4, max_seqs=3, max_model_len=64,
                                 max_step_tokens=16, state_memory=1 << 22, prefix_cache=True, cuda_graphs=False),
                    kernels=RefKernels())
    asked = [prompts["r0"], prompts["r2"], prompts["r0"][:12] + prompts["r1"][:7], prompts["r3"]]
    with torch.inference_mode():
        got = engine.generate(asked, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for prompt, tokens in zip(asked, got):
        ids = list(prompt)
        for token in tokens:
            logits = plain.forward(weights, stored, ids)[-1]
            best = int(logits.argmax())
            second = float(logits.topk(2).values[1])
            assert token == best or float(logits[best]) - second < 1e-3, (len(ids), token, best)
            ids.append(token)
