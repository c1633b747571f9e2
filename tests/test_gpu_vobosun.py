"""Vobosun on the GPU. Each new or extended kernel alone against its plain twin (tests/ref_kernels.py) and, where the
rule is short, against the rule written out here in 64-bit, with inputs made so that a fault shows (a state that must
carry a write over hundreds of tokens, rows in slots that are not their numbers, a first token that must read what the
slot carries, a correction that turns the choice, a dropped group that holds a high score); then the replayer in 32-bit and
bfloat16 against the plain implementation (tests/plain_vobosun.py): whole prompts, prefill against token-by-token
decoding, portions down to two tokens, unequal requests mixed in a pool whose pages and slots are used again, the first
tokens, long decoding, sizes that are multiples of nothing, head sizes the tensor cores take; and greedy generation
through the engine's scheduler and graphs."""
from __future__ import annotations

import math
import types

import pytest
import torch

import plain_vobosun as plain
from helpers import random_prompt
from holon_b200.replay import Replayer
from ref_kernels import RefKernels
from replay_tools import mixed_trace, portions, run
from vobosun_tools import CONFIGS, compare, exact_logits, make_folder, read_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
REF = RefKernels()
F64 = torch.float64


@pytest.fixture(scope="module")
def K():
    from holon_b200.kernels import load_kernels
    return load_kernels(DEV)


def rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, dtype, scale=1.0):
    tol = (3e-5 if dtype == torch.float32 else 1.6e-2) * scale
    diff = (got.float().cpu() - want.float().cpu()).abs().max().item()
    assert diff <= tol, f"difference {diff} > {tol}"


def rows_of(counts, slots, kv_len=None, device=DEV):
    """The rows of a step: `counts` tokens each, in slots `slots`."""
    qs = [0]
    for n in counts:
        qs.append(qs[-1] + n)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=device)      # noqa: E731
    kv = kv_len or counts
    return types.SimpleNamespace(query_start=t(qs), row_slot=t(slots), kv_len=t(kv), n_rows=len(counts), n_tokens=qs[-1],
                                 n_decode=sum(1 for n in counts if n == 1), max_q=max(counts), max_kv=max(kv),
                                 host_query_start=qs, host_kv_len=kv, plan={})


def triple(dim, seed):
    return (torch.tensor(0.6 + 0.1 * seed), 1 + 0.2 * rand(dim, seed=seed), 0.3 * rand(dim, seed=seed + 1))


def gpu(x):
    return tuple(t.to(DEV) for t in x) if isinstance(x, tuple) else (x.to(DEV) if x is not None else None)


# ---------------------------------------------------------------- the norm without statistics, sums, the token before
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,dim", [(7, 64), (3, 72), (5, 1030), (2, 2048), (4, 33)])
def test_tanh_norm_with_sum_and_gather(K, dtype, rows, dim):
    h, y = rand(rows, dim, seed=1, scale=2.0), rand(rows, dim, dtype=dtype, seed=2, scale=1.5)
    post, pre = triple(dim, 1), triple(dim, 3)
    want = torch.tanh(post[0].to(F64) * y.to(F64)) * post[1].to(F64) + post[2].to(F64) + h.to(F64)
    normed = torch.tanh(pre[0].to(F64) * want) * pre[1].to(F64) + pre[2].to(F64)
    hg, out = h.to(DEV), torch.empty(rows, dim, dtype=dtype, device=DEV)
    K.dyt_add_norm(hg, y.to(DEV), gpu(post), out, gpu(pre), None)                     # sum and norm
    close(hg, want, torch.float32, 4.0)
    close(out, normed, dtype, 2.0)
    ht, outt = h.clone(), torch.empty(rows, dim, dtype=dtype)
    REF.dyt_add_norm(ht, y, post, outt, pre, None)
    close(hg, ht, torch.float32, 4.0)
    close(out, outt, dtype, 2.0)
    index = torch.tensor([rows - 1, 0], dtype=torch.int32)                           # gathered rows: the stream stays
    hg2, out2 = h.to(DEV), torch.empty(2, dim, dtype=dtype, device=DEV)
    K.dyt_add_norm(hg2, y.to(DEV), gpu(post), out2, gpu(pre), index.to(DEV))
    assert torch.equal(hg2.cpu(), h)
    close(out2, normed[index.long()], dtype, 2.0)
    out3 = torch.empty(rows, dim, dtype=dtype, device=DEV)                           # the norm alone, of rows of the engine's dtype
    K.dyt_add_norm(None, y.to(DEV), None, out3, gpu(pre), None)
    close(out3, torch.tanh(pre[0].to(F64) * y.to(F64)) * pre[1].to(F64) + pre[2].to(F64), dtype, 2.0)
    hg4 = h.to(DEV)                                                                   # the sum alone
    K.dyt_add_norm(hg4, y.to(DEV), gpu(post), None, None, None)
    close(hg4, want, torch.float32, 4.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim", [64, 72, 1030, 33])
@pytest.mark.parametrize("pending", [False, True])
@pytest.mark.parametrize("counts", [[1, 5, 1, 2], [1, 701, 2, 1, 398]])
def test_rows_blended_with_the_token_before(K, dtype, dim, pending, counts):
    """Rows of 1, 5, 1 and 2 tokens in slots 3, 0, 2, 5 (and rows of hundreds of tokens, where a thread walks several
    tokens and rows begin in the middle of its walk): a row's first token reads what its slot carries, later tokens
    the row before theirs (with what is pending added), and the slot receives the row's last normed row; a second step
    then reads it. Written out in 64-bit."""
    slots = [3, 0, 2, 5, 1][:len(counts)]
    rows, t = rows_of(counts, slots), sum(counts)
    post, pre, mix = triple(dim, 1), triple(dim, 3), torch.rand(dim, generator=torch.Generator().manual_seed(5))
    carried = rand(7, dim, seed=9)
    for step in range(2):
        h = rand(t, dim, seed=10 + step, scale=2.0)
        y = rand(t, dim, dtype=dtype, seed=20 + step) if pending else None
        x = h.to(F64) if y is None else h.to(F64) + torch.tanh(post[0].to(F64) * y.to(F64)) * post[1].to(F64) + post[2].to(F64)
        n = torch.tanh(pre[0].to(F64) * x) * pre[1].to(F64) + pre[2].to(F64)
        want, kept = torch.zeros(t, dim, dtype=F64), carried.to(F64).clone()
        at = 0
        for c, s in zip(counts, slots):
            before = torch.cat((kept[s][None], n[at:at + c - 1]), 0)
            want[at:at + c] = n[at:at + c] + (before - n[at:at + c]) * mix.to(F64)
            kept[s] = n[at + c - 1]
            at += c
        hg, cg = h.to(DEV), carried.to(DEV)
        into = torch.empty_like(hg) if pending else hg
        out = torch.empty(t, dim, dtype=dtype, device=DEV)
        K.dyt_shift(out, into, hg, gpu(y), gpu(post) if pending else None, gpu(pre), mix.to(DEV), cg, rows)
        close(out, want, dtype, 2.0)
        close(into, x, torch.float32, 4.0)
        close(cg, kept, torch.float32, 2.0)
        ht, ct, outt = h.clone(), carried.clone(), torch.empty(t, dim, dtype=dtype)
        REF.dyt_shift(outt, ht, h, y, post if pending else None, pre, mix, ct, rows_of(counts, slots, device="cpu"))
        close(out, outt, dtype, 2.0)
        close(cg, ct, torch.float32, 2.0)
        carried = cg.cpu()


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (8, 256, 128), (16, 72, 200), (5, 2048, 512), (17, 64, 64), (3, 64, 60)])
@pytest.mark.parametrize("with_out", [True, False])
def test_the_sum_and_norm_in_a_product_s_epilogue(K, m, n, k, with_out):
    """For the few rows of a decode step: h += N_post(x · Wᵀ), out = N_pre(h) inside the product, against the product
    followed by the kernel of its own; more than 16 rows and a k that is no multiple of 8 are left to those two."""
    x, w = rand(m, k, dtype=torch.bfloat16, seed=1), rand(n, k, dtype=torch.bfloat16, seed=2, scale=k ** -0.5)
    h, post, pre = rand(m, n, seed=3, scale=2.0), triple(n, 1), triple(n, 3)
    hg = h.to(DEV)
    got = K.linear_dyt(hg, x.to(DEV), w.to(DEV), gpu(post), gpu(pre) if with_out else None)
    if m > 16 or k % 8:
        assert got is None and torch.equal(hg.cpu(), h)
        return
    y = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    K.linear(y, x.to(DEV), w.to(DEV))
    h2, out2 = h.to(DEV), torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    K.dyt_add_norm(h2, y, gpu(post), out2 if with_out else None, gpu(pre) if with_out else None, None)
    close(hg, h2, torch.float32, 4.0)
    if with_out:
        close(got, out2, torch.bfloat16, 2.0)
    else:
        assert got is True
    y64 = (x.to(F64) @ w.to(F64).T).to(torch.bfloat16).to(F64)
    close(hg, h.to(F64) + torch.tanh(post[0].to(F64) * y64) * post[1].to(F64) + post[2].to(F64), torch.bfloat16, 1.0)


# ---------------------------------------------------------------- the generalized delta rule
def _delta_inputs(t, heads, dim, seed, dtype):
    n = heads * dim
    first = rand(t, 5 * n + 3, dtype=dtype, seed=seed)                    # (rows wider than the five parts)
    pre = rand(t, n, seed=seed + 1, scale=1.5)
    return first, pre, rand(n, seed=seed + 2), rand(n, seed=seed + 3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim", [(2, 16), (1, 20), (2, 96), (3, 8), (1, 4), (2, 128), (1, 300), (2, 10), (1, 7)])
def test_delta_rows_in_slots_and_in_portions(K, dtype, heads, dim):
    """The prepare kernel against the written-out rule, and the scan with removal rates against its twin: rows of 1, 37,
    1 and 6 tokens in slots 3, 0, 2, 5 on states that are not zero, then the same tokens again as one-token rows and as
    portions on copies of the states: the same outputs and states whatever the cut."""
    counts, slots = [1, 37, 1, 6], [3, 0, 2, 5]
    t, n = sum(counts), heads * dim
    first, pre, b0, b1 = _delta_inputs(t, heads, dim, 4, dtype)
    scale, eps = math.exp(-0.5), 1e-6
    qk, v = torch.empty(t, 2, heads, dim, device=DEV), torch.empty(t, heads, dim, device=DEV)
    decay, rate = torch.empty_like(v), torch.empty_like(v)
    K.gdelta_prepare(qk, v, decay, rate, first.to(DEV), pre.to(DEV), b0.to(DEV), b1.to(DEV), scale, eps)
    x = first.to(F64)
    k64 = x[:, n:2 * n].view(t, heads, dim)
    close(qk[:, 0], x[:, :n].view(t, heads, dim), torch.float32)
    close(qk[:, 1], k64, torch.float32)
    close(v, x[:, 2 * n:3 * n].view(t, heads, dim), torch.float32)
    close(decay, torch.exp(-scale * torch.sigmoid(pre.to(F64) + b0.to(F64))).view(t, heads, dim), torch.float32)
    want_rate = torch.sigmoid(x[:, 4 * n:5 * n] + b1.to(F64)).view(t, heads, dim) / ((k64 * k64).sum(-1, keepdim=True) + eps)
    assert ((rate.cpu().to(F64) - want_rate).abs() <= 3e-5 * want_rate.abs() + 1e-6).all()
    # the scan: against its twin, and against the rule with the unit key written out
    state0 = rand(7, heads, dim, dim, seed=8, scale=0.3)
    out, state = torch.empty(t, heads, dim, device=DEV), state0.to(DEV)
    K.recurrent_scan(out, qk, v, decay, None, None, state, rows_of(counts, slots), rate=rate)
    out_t, state_t = torch.empty(t, heads, dim), state0.clone()
    REF.recurrent_scan(out_t, qk.cpu(), v.cpu(), decay.cpu(), None, None, state_t, rows_of(counts, slots, device="cpu"), rate=rate.cpu())
    spread = float(out_t.abs().max())
    close(out, out_t, torch.float32, max(1.0, spread))
    close(state, state_t, torch.float32, max(1.0, float(state_t.abs().max())))
    a64 = torch.sigmoid(x[:, 4 * n:5 * n] + b1.to(F64)).view(t, heads, dim)
    u64 = k64 / torch.sqrt((k64 * k64).sum(-1, keepdim=True) + eps)
    w64, r64, v64 = decay.cpu().to(F64), x[:, :n].view(t, heads, dim), x[:, 2 * n:3 * n].view(t, heads, dim)
    at = 0
    for c, s in zip(counts, slots):
        for h in range(heads):
            S = state0[s, h].to(F64).T.clone()                          # (kept column by column)
            for i in range(at, at + c):
                S = w64[i, h][:, None] * S - torch.outer(a64[i, h] * u64[i, h], u64[i, h] @ S) + torch.outer(k64[i, h], v64[i, h])
                assert (out[i, h].cpu().to(F64) - S.T @ r64[i, h]).abs().max() <= 1e-4 * max(1.0, spread)
        at += c
    # one by one, and in portions of 2, 3 and 7: the same numbers
    for sizes in ([1], [2, 3, 7]):
        out2, state2 = torch.empty(t, heads, dim, device=DEV), state0.to(DEV)
        done = [0] * len(counts)
        while any(d < c for d, c in zip(done, counts)):
            take, turn = [], 0
            for r, c in enumerate(counts):
                take.append(min(sizes[(done[r] + r) % len(sizes)], c - done[r]))
            live = [r for r in range(len(counts)) if take[r]]
            starts = [sum(counts[:r]) + done[r] for r in live]
            index = torch.tensor([s + j for r, s in zip(live, starts) for j in range(take[r])], device=DEV)
            step_rows = rows_of([take[r] for r in live], [slots[r] for r in live])
            o = torch.empty(len(index), heads, dim, device=DEV)
            K.recurrent_scan(o, qk[index].contiguous(), v[index].contiguous(), decay[index].contiguous(), None, None, state2,
                             step_rows, rate=rate[index].contiguous())
            out2[index] = o
            for r in live:
                done[r] += take[r]
        close(out2, out, torch.float32, max(1.0, spread))
        close(state2, state, torch.float32, max(1.0, float(state_t.abs().max())))


def test_the_state_keeps_a_far_write(K):
    """Token 0 writes along key channel 0; all later keys lie in the other channels, so no removal touches that write and
    only channel 0's decays shrink it; 600 tokens later a query along channel 0 reads it back: o = v_0 times the product of
    those decays, to 1e-5."""
    t, heads, dim = 601, 1, 16
    qk, v = torch.zeros(t, 2, heads, dim), rand(t, heads, dim, seed=2)
    decay = 0.99 + 0.01 * torch.rand(t, heads, dim, generator=torch.Generator().manual_seed(3))
    qk[0, 1, 0, 0] = 1.0
    qk[1:, 1, 0, 1:] = rand(t - 1, dim - 1, seed=5)
    qk[-1, 0, 0, 0] = 1.0
    rate = torch.rand(t, heads, dim, generator=torch.Generator().manual_seed(4)) / (qk[:, 1] ** 2).sum(-1, keepdim=True)
    out, state = torch.empty(t, heads, dim, device=DEV), torch.zeros(2, heads, dim, dim, device=DEV)
    K.recurrent_scan(out, qk.to(DEV), v.to(DEV), decay.to(DEV), None, None, state, rows_of([t], [1]), rate=rate.to(DEV))
    want = v[0, 0].to(F64) * decay[1:, 0, 0].to(F64).prod()
    assert float(want.abs().max()) > 0.01
    assert (out[-1, 0].cpu().to(F64) - want).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,vdim,per_head,gate", [(2, 16, True, "sigmoid"), (3, 20, True, "silu"), (1, 96, True, "sigmoid"),
                                                      (4, 8, False, "sigmoid")])
def test_head_norm_with_a_weight_per_head_and_a_sigmoid_gate(K, dtype, heads, vdim, per_head, gate):
    t = 9
    o, w = rand(t, heads, vdim, seed=1, scale=3.0), 1 + 0.3 * rand(heads * vdim if per_head else vdim, seed=2)
    wide = rand(t, 3 * heads * vdim, dtype=dtype, seed=3)
    pre = wide[:, heads * vdim:2 * heads * vdim]
    out, out_t = torch.empty(t, heads, vdim, dtype=dtype, device=DEV), torch.empty(t, heads, vdim, dtype=dtype)
    K.head_norm_gate(out, o.to(DEV), w.to(DEV), None, wide.to(DEV)[:, heads * vdim:2 * heads * vdim], 1e-5, gate=gate)
    REF.head_norm_gate(out_t, o, w, None, pre, 1e-5, gate=gate)
    close(out, out_t, dtype, 4.0)
    g = pre.to(F64).reshape(t, heads, vdim)
    want = o.to(F64) / torch.sqrt((o.to(F64) ** 2).mean(-1, keepdim=True) + 1e-5) * (w.to(F64).view(heads, vdim) if per_head else w.to(F64))
    want = want * (torch.sigmoid(g) if gate == "sigmoid" else g * torch.sigmoid(g))
    close(out, want, dtype, 4.0)


# ---------------------------------------------------------------- biases, stretched rotation, the activation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,rot", [(4, 2, 16, 8), (3, 3, 20, 0), (8, 2, 64, 64), (2, 1, 128, 128), (6, 1, 12, 12)])
def test_biases_before_rotation_and_cache_write(K, dtype, heads, kv_heads, dim, rot):
    t, page, pages = 11, 4, 9
    width = (heads + 2 * kv_heads) * dim
    qkv, bias = rand(t, width, dtype=dtype, seed=1), rand(width, dtype=dtype, seed=2, scale=0.5)
    positions = torch.tensor([0, 1, 2, 3, 30, 31, 32, 7, 8, 9, 10], dtype=torch.int32)
    half = rot // 2
    angle = torch.arange(40, dtype=torch.float32)[:, None] * (1.0 / (300.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot)) / 4.0)[None, :]
    table = torch.cat((angle.cos(), angle.sin()), -1).contiguous() if rot else None
    write = torch.tensor([5, 6, 7, 12, 0, 1, 2, 20, 21, 22, -1], dtype=torch.int32)
    q, kv = torch.empty(t, heads, dim, dtype=dtype, device=DEV), torch.zeros(pages, 2, kv_heads, page, dim, dtype=dtype, device=DEV)
    K.qk_norm_rope_kv_write(q, qkv.to(DEV), positions.to(DEV), gpu(table), rot, None, None, 0.0, 0.0, kv, write.to(DEV), heads,
                            kv_heads, dim, bias=bias.to(DEV))
    q_t, kv_t = torch.empty(t, heads, dim, dtype=dtype), torch.zeros(pages, 2, kv_heads, page, dim, dtype=dtype)
    REF.qk_norm_rope_kv_write(q_t, qkv, positions, table, rot, None, None, 0.0, 0.0, kv_t, write, heads, kv_heads, dim, bias=bias)
    close(q, q_t, dtype, 4.0)
    close(kv, kv_t, dtype, 4.0)
    x = (qkv.to(F64) + bias.to(F64))[:, :heads * dim].view(t, heads, dim)              # the rule for q, written out
    if rot:
        cs = table.to(F64)[positions.long()][:, None, :]
        a, b = x[..., :half], x[..., half:rot]
        x = torch.cat((a * cs[..., :half] - b * cs[..., half:], b * cs[..., :half] + a * cs[..., half:], x[..., rot:]), -1)
    close(q, x, dtype, 6.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_xielu_and_tanh(K, dtype):
    z = rand(7, 333, dtype=dtype, seed=1, scale=3.0)
    numbers = torch.tensor([0.7, -0.4])
    got = z.to(DEV)
    K.activation(got, 4, numbers.to(DEV))
    want = plain.xielu(z.to(F64), numbers[0].to(F64), numbers[1].to(F64))
    close(got, want, dtype, float(want.abs().max()))
    got = z.to(DEV)
    K.activation(got, 5)
    close(got, torch.tanh(z.to(F64)), dtype)


# ---------------------------------------------------------------- the choice in groups, identity experts
@pytest.mark.parametrize("tokens", [9, 700])
@pytest.mark.parametrize("experts,top,groups,keep", [(8, 3, 4, 2), (12, 4, 3, 2), (6, 2, 1, 1), (40, 5, 8, 3), (16, 4, 4, 4)])
def test_the_choice_in_groups_with_a_correction(K, tokens, experts, top, groups, keep):
    """Against the written-out rule, token by token (one launch for few tokens, several for many): the chosen sets and
    the weights; the rows are laid out expert by expert."""
    z = rand(tokens, experts + 1, seed=tokens + experts, scale=1.5)
    corr = rand(experts, seed=3, scale=0.3 / experts ** 0.5 * 3)
    chosen = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    weight = torch.empty(tokens, top, device=DEV)
    counts = torch.empty(2 * experts + 3, dtype=torch.int32, device=DEV)
    place = torch.empty(tokens * top, dtype=torch.int32, device=DEV)
    token_of = torch.empty(tokens * top, dtype=torch.int32, device=DEV)
    K.route_rows(chosen, weight, counts, place, token_of, z.to(DEV), experts, 1.0, True, None, correction=corr.to(DEV),
                 groups=groups, keep=keep, tiny=1e-20)
    router = {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}
    close_calls = 0
    for t in range(tokens):
        want = plain.choose(z[t, :experts].to(F64), corr.to(F64), router)
        got = dict(zip(chosen[t].tolist(), weight[t].tolist()))
        if set(got) != {e for e, _ in want}:
            close_calls += 1                              # two choice scores a rounding apart
            continue
        for e, w in want:
            assert abs(got[e] - float(w)) < 1e-5
    assert close_calls <= tokens // 100
    c = counts.cpu()
    assert c[:experts].tolist() == torch.bincount(chosen.cpu().long().reshape(-1), minlength=experts).tolist()
    starts = c[experts:2 * experts + 1].tolist()
    for i in range(tokens * top):
        e, p = int(chosen.reshape(-1)[i]), int(place[i])
        assert starts[e] <= p < starts[e + 1] and int(token_of[p]) == i // top


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [64, 72])
def test_identity_rows_and_a_shared_expert_without_a_gate(K, dtype, hidden):
    t, top, first_identity = 6, 3, 11
    y, x, shared = rand(t * top, hidden, dtype=dtype, seed=1), rand(t, hidden, dtype=dtype, seed=2), rand(t, hidden, dtype=dtype, seed=3)
    place = torch.randperm(t * top, generator=torch.Generator().manual_seed(4)).to(torch.int32)
    weight = torch.rand(t, top, generator=torch.Generator().manual_seed(5))
    ident = torch.tensor([first_identity], dtype=torch.int32)
    out, out_t = torch.empty(t, hidden, dtype=dtype, device=DEV), torch.empty(t, hidden, dtype=dtype)
    K.expert_combine(out, y.to(DEV), place.to(DEV), weight.to(DEV), shared.to(DEV), None, 0, x=x.to(DEV), identity_from=ident.to(DEV))
    REF.expert_combine(out_t, y, place, weight, shared, None, 0, x=x, identity_from=ident)
    close(out, out_t, dtype, 4.0)
    want = shared.to(F64).clone()
    for i in range(t):
        for k in range(top):
            p = int(place[i * top + k])
            want[i] += float(weight[i, k]) * (x[i] if p >= first_identity else y[p]).to(F64)
    close(out, want, dtype, 4.0)


# ---------------------------------------------------------------- the model through the replayer
@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param, seed=11)
    config = CONFIGS[request.param]
    prompts = {f"r{i}": random_prompt(config["vocab"], n, 40 + i) for i, n in enumerate((70, 133, 37, 96))}
    return folder, config, prompts, {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_tail_then_portions(model, dtype):
    folder, config, prompts, want = model
    r = Replayer(str(folder), dtype, 192, device=DEV, page_size=64)
    compare(run(r, [([(rid, ids)], [rid]) for rid, ids in prompts.items()]), want, dtype)
    steps = []
    for rid, ids in prompts.items():                                       # most of it at once, the last 33 one by one
        cut = len(ids) - 33
        steps.append(([(rid, ids[:cut])], []))
        steps += [([(rid, [t])], [rid] if i == 32 else []) for i, t in enumerate(ids[cut:])]
    compare(run(r, steps), want, dtype)
    steps = []
    for rid, ids in prompts.items():                                       # portions down to two tokens, cut inside pages
        parts = portions(ids, [17, 2, 40, 3, 2, 29])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [64, 16])
def test_mixed_requests_in_a_small_pool(model, dtype, page_size):
    """Four requests live at once in a pool that holds no more: portions beside single tokens; pages and slots given back
    and taken again; then the same slots and pages for other requests."""
    folder, config, prompts, want = model
    r = Replayer(str(folder), dtype, 448, device=DEV, page_size=page_size)
    got = run(r, mixed_trace(prompts))
    compare(got, want, dtype)
    assert len(got) == sum(len(ids) for ids in prompts.values())
    swapped = {"r0": prompts["r3"], "r3": prompts["r0"]}
    compare(run(r, [([("r0", swapped["r0"][:50]), ("r3", swapped["r3"][:9])], []),
                    ([("r0", swapped["r0"][50:]), ("r3", swapped["r3"][9:])], ["r0", "r3"])]),
            {"r0": want["r3"], "r3": want["r0"]}, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(model, dtype):
    folder, config, prompts, want = model
    ids = prompts["r1"]
    r = Replayer(str(folder), dtype, 192, device=DEV, page_size=64)
    steps = [([("r1", [t])], ["r1"] if i == len(ids) - 1 else []) for i, t in enumerate(ids)]      # from the first token on
    compare(run(r, steps), want, dtype)
    steps = [([("r1", ids[:2])], [])] + [([("r1", [t])], ["r1"] if i == len(ids) - 3 else []) for i, t in enumerate(ids[2:])]
    compare(run(r, steps), want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_through_the_model(tmp_path, dtype):
    """Sharp attention over 300 tokens with heads of 64 (the tensor-core kernels in bfloat16): whole, and with the last
    120 tokens decoded one by one over keys that lie up to four pages back."""
    import copy
    config = copy.deepcopy(CONFIGS["c"])
    for layer in config["layers"]:
        if layer["type"] == "attention":
            layer["mixer"]["scale"] = 9.0 / layer["mixer"]["dim"] ** 0.5
    folder = make_folder(tmp_path, "sharp", seed=5, config=config)
    ids = random_prompt(config["vocab"], 300, 8)
    want = {"r": exact_logits(folder, ids)}
    r = Replayer(str(folder), dtype, 320, device=DEV, page_size=64)
    compare(run(r, [([("r", ids)], ["r"])]), want, dtype)
    steps = [([("r", ids[:180])], [])] + [([("r", [t])], ["r"] if i == 119 else []) for i, t in enumerate(ids[180:])]
    compare(run(r, steps), want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("vdim", [128, 64])
def test_heads_of_128(tmp_path, dtype, vdim):
    """Attention heads of 128 (the tcgen05 prompt kernel and the cluster decode kernel in bfloat16 where keys and values
    are of one size; rows [key | value] where they are not), a delta head of 64 and one of 128, 300 tokens: whole, the
    last 40 tokens one by one, and portions that end inside pages."""
    from vobosun_tools import _att, _delta, _dense, _layer, _model, _moe
    config = _model(256, 331, 1e-6, [
        _layer("attention", _att(4, 2, 128, vdim, 6.0, 1000000.0, 64, 4.0), _moe(6, 2, 64, identity=2, groups=(4, 2), shared=32)),
        _layer("general_delta", _delta(2, 64, 8), _dense(192)),
        _layer("attention", _att(4, 2, 128, vdim, 6.0, 1000000.0, 64, 4.0), _dense(192), weights_of=None),
        _layer("general_delta", _delta(1, 128, 12), None)])
    folder = make_folder(tmp_path, "wide", seed=9, config=config)
    ids = random_prompt(config["vocab"], 300, 4)
    want = {"r": exact_logits(folder, ids)}
    r = Replayer(str(folder), dtype, 320, device=DEV, page_size=64)
    compare(run(r, [([("r", ids)], ["r"])]), want, dtype)
    steps = [([("r", ids[:260])], [])] + [([("r", [t])], ["r"] if i == 39 else []) for i, t in enumerate(ids[260:])]
    compare(run(r, steps), want, dtype)
    parts = portions(ids, [100, 3, 61, 2, 90])
    compare(run(r, [([("r", p)], ["r"] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]), want, dtype)


def test_a_token_far_back_is_remembered(tmp_path):
    """Delta-rule layers alone, 320 tokens: the last logits change when token 7 changes (only the matrix state can carry
    it there), and the engine follows the plain implementation through that change, in a prompt and in decoding, with
    the two requests side by side in one batch."""
    folder = make_folder(tmp_path, "delta", seed=3)
    vocab = CONFIGS["delta"]["vocab"]
    ids = random_prompt(vocab, 320, 5)
    other = list(ids)
    other[7] = (ids[7] + 1) % vocab
    want = {"x": exact_logits(folder, ids), "y": exact_logits(folder, other)}
    r = Replayer(str(folder), "float32", max_tokens=768)
    steps = [([("x", ids[:200]), ("y", other[:200])], [])] + [([("x", [a]), ("y", [b])], []) for a, b in zip(ids[200:], other[200:])]
    compare(run(r, steps), want, "float32")
    assert float((want["x"][40] - want["y"][40]).abs().max()) > 1e-3          # the changed token matters to later rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(model, dtype, graphs):
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    folder, config, prompts, _ = model
    stored, weights = read_folder(folder)
    engine = Engine(EngineConfig(model=str(folder), dtype=dtype, device=DEV, page_size=16, max_seqs=3, max_model_len=192,
                                 max_step_tokens=64, state_memory=1 << 26, cuda_graphs=graphs))
    asked = [prompts["r0"], prompts["r2"], prompts["r3"][:50], prompts["r1"][:90]]
    with torch.inference_mode():
        got = engine.generate(asked, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    engine.close()
    gap = 1e-3 if dtype == "float32" else 0.25
    for prompt, tokens in zip(asked, got):
        ids = list(prompt)
        for token in tokens:
            logits = plain.forward(weights, stored, ids)[-1]
            best = int(logits.argmax())
            if token != best:                              # a close call: allowed once, then the sequences part
                assert float(logits[best] - logits[token]) < gap * float(logits.std()), (len(ids), token, best)
                break
            ids.append(token)


def test_generate_on_the_command_line(tmp_path, capsys):
    """`holon-b200 generate` with the engine's own sizing of the cache (activation peaks measured on the largest step)."""
    import json

    from holon_b200 import cli
    folder = make_folder(tmp_path, "a", seed=8)
    config, weights = read_folder(folder)
    assert cli.main(["generate", str(folder), "--prompt-ids", "5,17,3,90,12,7", "--prompt-ids", "9 8 7 6", "--max-tokens", "6",
                     "--dtype", "float32", "--max-model-len", "128", "--max-seqs", "4", "--max-step-tokens", "128", "--ignore-eos",
                     "--memory-fraction", "0.05"]) == 0
    captured = capsys.readouterr()
    lines = [json.loads(line) for line in captured.out.splitlines()]
    assert [o["prompt_ids"] for o in lines] == [[5, 17, 3, 90, 12, 7], [9, 8, 7, 6]]
    for o in lines:
        ids = list(o["prompt_ids"])
        assert len(o["token_ids"]) == 6
        for token in o["token_ids"]:
            logits = plain.forward(weights, config, ids)[-1]
            assert float(logits.max() - logits[token]) <= 1e-3 * float(logits.std()), (len(ids), token)
            ids.append(token)
