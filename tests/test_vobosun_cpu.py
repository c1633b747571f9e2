"""Vobosun without a GPU: configuration, weight names, and the engine's host side (batch layout, cache entries, the
per-request state of the delta-rule layers and of every layer's token shift, layers that run with another layer's
tensors) with the CPU twins of the kernels (tests/ref_kernels.py) against the plain implementation
(tests/plain_vobosun.py)."""
from __future__ import annotations

import copy
import json
import pathlib
import tempfile

import pytest
import torch

import plain_vobosun as plain
from helpers import random_prompt
from holon_b200.config.registry import ConfigError, resolve_architecture
from holon_b200.replay import Replayer
from ref_kernels import RefKernels
from replay_tools import portions, run
from vobosun_tools import CONFIGS, compare, exact_logits, make_folder, make_weights, read_folder, stored_config, tensor_table


def test_architecture_and_configuration():
    arch = resolve_architecture(CONFIGS["a"])
    cfg = arch.parse(CONFIGS["a"])
    assert arch.name == "Vobosun" and len(cfg.layers) == 6 and cfg.layers[5].mlp is None
    spec = arch.recipe(cfg)
    assert [(r.layer, r.cache, r.fills) for r in spec.order] == [(0, 0, True), (1, 1, True), (2, 2, True), (0, 3, True),
                                                                 (1, 4, True), (5, 5, True)]
    assert spec.layers[3] is None and spec.layers[4] is None
    assert all(layer.block.name == "sandwich" and layer.norm.name == "dyt" for layer in spec.layers if layer)
    assert [layer.mixer.name for layer in spec.layers if layer] == ["general_delta", "gqa", "talking", "general_delta"]
    rope = spec.layers[1].mixer.kwargs()["position"].kwargs()
    assert rope["factor"] == 4.0 and rope["rotary_dim"] == 8
    assert spec.layers[2].mixer.kwargs()["position"].kwargs()["factor"] == 1.0          # no `scaling`: not stretched
    experts = spec.layers[1].ffn.kwargs()
    assert (experts["experts"], experts["identity"], experts["groups"], experts["keep_groups"], experts["shared_inter"]) == (6, 2, 4, 2, 24)
    plain_moe = arch.recipe(arch.parse(CONFIGS["b"])).layers[0].ffn.kwargs()
    assert (plain_moe["identity"], plain_moe["groups"], plain_moe["keep_groups"], plain_moe["shared_inter"]) == (0, 1, 1, None)
    assert arch.recipe(arch.parse(CONFIGS["b"])).layers[0].mixer.kwargs()["position"] is None
    for path, value, error in (
            (("layers", 0, "type"), "retention", NotImplementedError),
            (("layers", 0, "mlp", "kind"), "glu", NotImplementedError),
            (("layers", 1, "mixer", "kv_heads"), 3, ConfigError),
            (("layers", 1, "mixer", "rot", "dims"), 18, ConfigError),
            (("layers", 1, "mixer", "rot", "dims"), 7, ConfigError),
            (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.0, ConfigError),
            (("layers", 1, "mlp", "router", "top"), 9, ConfigError),
            (("layers", 1, "mlp", "router", "groups", "count"), 3, ConfigError),            # does not divide 8
            (("layers", 1, "mlp", "router", "groups", "keep"), 1, ConfigError),             # one group of two < top 3
            (("layers", 3, "weights_of"), 3, ConfigError),
            (("layers", 3, "weights_of"), 1, ConfigError),                                  # differs from the layer it names
            (("layers", 0, "mixer", "heads"), 0, ConfigError),
            (("width",), 0, ConfigError)):
        c = copy.deepcopy(CONFIGS["a"])
        at = c
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            arch.parse(c)
    with pytest.raises(ConfigError):                                       # the rank comes from a dict or from a shape
        arch.parse(stored_config(CONFIGS["a"]))
    done = arch.complete(stored_config(CONFIGS["a"]), {"l0.mix.w1": (6, 64), "l5.mix.w1": (3, 64)})
    assert arch.parse(done) == cfg


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    from holon_b200.weights import RandomSource
    table = {stored: tuple(shape) for stored, shape, _ in RandomSource(CONFIGS[name], 0).table()}
    assert table == dict(tensor_table(CONFIGS[name]))


def test_a_missing_a_misshapen_and_a_spare_tensor_are_named(tmp_path):
    from safetensors.torch import load_file, save_file
    from holon_b200.weights.loader import WeightError
    folder = make_folder(tmp_path, "a")
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["l1.mlp.correction"]
    tensors["l0.shift"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["l3.norm1"] = tensors["l0.norm1"].clone()                     # layer 3 runs with layer 0's tensors
    tensors["l5.norm2"] = tensors["l0.norm2"].clone()                     # layer 5 has no feed-forward
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        Replayer(str(folder), "float32", 64, device="cpu", kernels=RefKernels())
    assert e.value.missing == ["l1.mlp.correction"] and sorted(e.value.unexpected) == ["l3.norm1", "l5.norm2"]
    assert [s[0] for s in e.value.shapes] == ["l0.shift"]


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
    for i, layer in enumerate(config["layers"]):                         # a state per run, also where tensors are shared
        m = layer["mixer"]
        assert tuple(states[(i, "block.shift")].shape[1:]) == (config["width"],)
        assert states[(i, "block.shift")].dtype == torch.float32
        if layer["type"] == "general_delta":
            assert tuple(states[(i, "state")].shape[1:]) == (m["heads"], m["dim"], m["dim"])
        else:
            g = r.built.cache.group_of_entry[i]
            shape = (2, m["kv_heads"], 4, m["dim"]) if m["dim"] == m["vdim"] else (m["kv_heads"], 4, m["dim"] + m["vdim"])
            assert tuple(g.kv.shape[2:]) == shape
    assert r.built.cache.prefix is None


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
    for rid, ids in prompts.items():                                       # portions down to two tokens
        parts = portions(ids, [3, 2, 7, 2, 5])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, "float32")
    # four requests at once in 104 tokens of pool: portions beside single tokens, pages and slots given back and used
    # again (a slot's matrix state, its previous rows and its pages must not leak into the request that takes it next)
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


def sharp_attention(dim_equal: bool):
    """One attention layer whose scores are so sharp that most queries put most of their weight on one key, which for
    late queries lies anywhere in the 150 tokens before them: (configuration, weights, token ids)."""
    config = copy.deepcopy(CONFIGS["att" if dim_equal else "rows"])
    m = config["layers"][0]["mixer"]
    m["scale"] = 12.0 / m["dim"] ** 0.5
    return config, make_weights(config, 3), random_prompt(config["vocab"], 150, 5)


@pytest.mark.parametrize("dim_equal", [True, False])
def test_far_keys_are_found(dim_equal):
    """Late queries whose best key lies more than a page of 64 back, with most of the weight on it: the logits follow the
    plain implementation's for whole prompts and for tokens decoded one by one, on small and large pages. A lost or
    misplaced far key moves such a row by most of its spread."""
    config, weights, ids = sharp_attention(dim_equal)
    with tempfile.TemporaryDirectory() as tmp:
        folder = make_folder(pathlib.Path(tmp), "far", config=config, weights=weights)
        want = {"r": exact_logits(folder, ids)}
        probs = _attention_weights(config, weights, ids)[100:]
        best = probs.max(-1)
        far = (torch.arange(100, 150) - best.indices) > 64
        assert int(far.sum()) >= 8 and float(best.values[far].median()) > 0.4
        for page in (4, 64):
            r = Replayer(str(folder), "float32", 192, device="cpu", kernels=RefKernels(), page_size=page)
            compare(run(r, [([("r", ids)], ["r"])]), want, "float32")
            steps = [([("r", ids[:60])], [])] + [([("r", [t])], ["r"] if i == 89 else []) for i, t in enumerate(ids[60:])]
            compare(run(r, steps), want, "float32")


def _attention_weights(config, weights, ids):
    """The softmax weights of head 0 of the first layer, [query, key] (plain code, for the test above)."""
    m = config["layers"][0]["mixer"]
    x = weights["embed"].double()[torch.tensor(ids)]
    h = plain.token_shift(plain.tanh_norm(x, weights, "l0.norm1"), weights["l0.shift"].double())
    t = len(ids)
    q = (h @ weights["l0.mix.q"].double().T + weights["l0.mix.q.b"].double()).view(t, m["heads"], m["dim"])
    k = (h @ weights["l0.mix.k"].double().T + weights["l0.mix.k.b"].double()).view(t, m["kv_heads"], m["dim"])
    rot = m["rot"]
    q = plain.turn_halves(q, torch.arange(t), rot["base"], rot["dims"], rot["scaling"]["factor"])
    k = plain.turn_halves(k, torch.arange(t), rot["base"], rot["dims"], rot["scaling"]["factor"])
    s = (q[:, 0] @ k[:, 0].T) * m["scale"]
    s = s.masked_fill(torch.triu(torch.ones(t, t, dtype=torch.bool), 1), -float("inf"))
    return torch.softmax(s, -1)


def test_the_choice_follows_correction_and_groups():
    """The router alone, against the written-out rule: a correction that lifts an expert into the choice without
    touching its weight, a group that is dropped although it holds the second-best expert, a negative choice score that
    still beats what is out of the running."""
    k = RefKernels()
    z = torch.tensor([[2.0, 1.9, 0.0, 0.1, 1.0, 1.5], [0.0, 0.3, 0.1, 0.0, 0.2, 0.4]])
    corr = torch.tensor([0.0, -0.6, 0.0, 0.3, 0.0, -0.9])
    chosen, weight = torch.zeros(2, 2, dtype=torch.int32), torch.zeros(2, 2)
    counts, place, token_of = torch.zeros(15, dtype=torch.int32), torch.zeros(4, dtype=torch.int32), torch.zeros(4, dtype=torch.int32)
    k.route_rows(chosen, weight, counts, place, token_of, z, 6, 1.0, True, None, correction=corr, groups=3, keep=2, tiny=1e-20)
    for t in range(2):
        want = plain.choose(z[t].double(), corr.double(), {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}})
        assert chosen[t].tolist() == [e for e, _ in want]
        assert torch.allclose(weight[t].double(), torch.stack([w for _, w in want]), atol=1e-6)
    assert sorted(chosen[0].tolist()) == [0, 3]          # expert 1 (second by score) loses its place to the corrected 3
    assert sorted(chosen[1].tolist()) == [3, 4]          # the group of experts 0 and 1 is dropped; 1 and 5 are negative


def test_greedy_generation_through_the_scheduler(model):
    """The engine's own entry point and scheduler: greedy tokens equal the plain implementation's arg max, token by
    token, for requests that arrive together, share three slots and are cut into portions by a small step budget."""
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
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


# ---------------------------------------------------------------- faults planted in the kernel table are noticed
class _Planted(RefKernels):
    """The plain kernel table with one fault; `fault` names it."""

    def __init__(self, fault: str) -> None:
        self.fault = fault

    def dyt_shift(self, out, into, h, y, post, pre, mix, carried, rows):
        if self.fault == "the previous row is not carried from step to step":
            kept = carried.clone()
            super().dyt_shift(out, into, h, y, post, pre, mix, carried, rows)
            carried.copy_(kept)
            return
        if self.fault == "a row's first token blends with the row before it in the batch":
            super().dyt_shift(out, into, h, y, post, pre, mix, carried, rows)
            qs = rows.query_start.tolist()
            n = self._dyt(into, pre)
            for b in range(1, rows.n_rows):
                s = qs[b]
                if qs[b + 1] > s:
                    out[s] = (n[s] + (n[s - 1] - n[s]) * mix.float()).to(out.dtype)
            return
        super().dyt_shift(out, into, h, y, post, pre, mix, carried, rows)

    def recurrent_scan(self, out, qk, v, decay, head_decay, beta, state, rows, token_decay=None, rate=None):
        if rate is not None and self.fault == "the removal reads the decayed state":
            qs, slots = rows.query_start.tolist(), rows.row_slot.tolist()
            for b in range(rows.n_rows):
                for h in range(v.shape[1]):
                    s = state[slots[b], h].T.clone()
                    for i in range(qs[b], qs[b + 1]):
                        k = qk[i, 1, h]
                        s = s * decay[i, h][:, None]
                        s = s + torch.outer(k, v[i, h]) - torch.outer(rate[i, h] * k, s.T @ k)
                        out[i, h] = s.T @ qk[i, 0, h]
                    state[slots[b], h] = s.T
            return
        if rate is not None and self.fault == "the state is not written back":
            kept = state.clone()
            super().recurrent_scan(out, qk, v, decay, head_decay, beta, state, rows, token_decay, rate)
            state.copy_(kept)
            return
        super().recurrent_scan(out, qk, v, decay, head_decay, beta, state, rows, token_decay, rate)

    def gdelta_prepare(self, qk, v, decay, rate, first, pre, decay_bias, rate_bias, decay_scale, unit_eps):
        super().gdelta_prepare(qk, v, decay, rate, first, pre, decay_bias, rate_bias, decay_scale, unit_eps)
        if self.fault == "the removal runs along the key, not the unit key":
            k = qk[:, 1]
            rate.mul_((k * k).sum(-1, keepdim=True) + unit_eps)

    def route_rows(self, chosen, weight, counts, place, token_of, z, experts, scale, renormalize, bias=None,
                   correction=None, groups=1, keep=1, tiny=0.0):
        if self.fault == "the choice runs without the correction":
            correction = None
        if self.fault == "the groups are ignored":
            groups, keep = 1, 1
        super().route_rows(chosen, weight, counts, place, token_of, z, experts, scale, renormalize, bias, correction, groups, keep, tiny)

    def expert_combine(self, out, y, place, weight, shared, z, experts, x=None, identity_from=None):
        if self.fault == "identity experts return nothing" and x is not None:
            x = torch.zeros_like(x)
        if self.fault == "the shared expert is left out":
            shared = None
        super().expert_combine(out, y, place, weight, shared, z, experts, x, identity_from)

    def qk_norm_rope_kv_write(self, *args, bias=None):
        if self.fault == "q, k and v lose their biases":
            bias = None
        super().qk_norm_rope_kv_write(*args, bias=bias)

    def activation(self, x, act, numbers=None):
        if self.fault == "xielu's two numbers are swapped" and numbers is not None:
            numbers = numbers.flip(0)
        super().activation(x, act, numbers)

    def head_norm_gate(self, out, o, weight, gate_mul, gate_pre, eps, gate="silu"):
        if self.fault == "the output gate is silu":
            gate = "silu"
        super().head_norm_gate(out, o, weight, gate_mul, gate_pre, eps, gate=gate)


FAULTS = ("the previous row is not carried from step to step", "a row's first token blends with the row before it in the batch",
          "the removal reads the decayed state", "the state is not written back", "the removal runs along the key, not the unit key",
          "the choice runs without the correction", "the groups are ignored", "identity experts return nothing",
          "the shared expert is left out", "q, k and v lose their biases", "xielu's two numbers are swapped",
          "the output gate is silu")


def test_planted_faults_are_noticed(tmp_path):
    """Portions beside single tokens of three requests of configuration `a`, in 32-bit: the comparison accepts the plain
    kernel table and rejects every table with one fault planted (a rotation whose stretch is ignored is planted in the
    configuration)."""
    folder = make_folder(tmp_path, "a", seed=7)
    config = CONFIGS["a"]
    prompts = {f"r{i}": random_prompt(config["vocab"], n, 60 + i) for i, n in enumerate((23, 41, 30))}
    want = {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}
    cut = {rid: portions(ids, sizes) for (rid, ids), sizes in zip(prompts.items(), ([5, 1, 1, 3], [2, 9, 1], [30]))}
    steps = []
    for j in range(max(len(p) for p in cut.values())):
        steps.append(([(rid, p[j]) for rid, p in cut.items() if j < len(p)], [rid for rid, p in cut.items() if j == len(p) - 1]))

    def replay(where, kernels):
        return run(Replayer(str(where), "float32", 128, device="cpu", kernels=kernels, page_size=4), steps)

    compare(replay(folder, RefKernels()), want, "float32")
    missed = []
    for fault in FAULTS:
        try:
            compare(replay(folder, _Planted(fault)), want, "float32")
            missed.append(fault)
        except AssertionError:
            pass
    stored, weights = read_folder(folder)
    for layer in stored["layers"]:
        if layer["type"] == "attention" and "scaling" in layer["mixer"].get("rot", {}):
            layer["mixer"]["rot"]["scaling"]["factor"] = 1.0
    other = make_folder(tmp_path / "unstretched", "a", config=stored, weights=weights)
    try:
        compare(replay(other, RefKernels()), want, "float32")
        missed.append("the rotation's stretch is ignored")
    except AssertionError:
        pass
    assert not missed, f"the comparison accepted: {missed}"
