"""Tilarax on the GPU. Each new kernel alone against a formula written here in 64-bit and against its plain twin
(tests/ref_kernels.py), with inputs made so that a fault shows (one key whose score stands out just inside or just
outside a block of the mask, in a prompt's row and in a row of one token; a mixing matrix far from the identity; a
memory that must carry a write over hundreds of tokens; gates that drive the running maximum both ways); then the
replayer in 32-bit and bfloat16 against the plain implementation (tests/plain_tilarax.py): whole prompts, prefill against
token-by-token decoding, portions down to two tokens, unequal requests mixed in a pool whose pages and slots are used
again, the first tokens, long decoding, sizes that are multiples of nothing, head sizes the tensor cores take; and greedy
generation through the engine's scheduler and graphs."""
from __future__ import annotations

import copy
import math
import types

import pytest
import torch

import plain_tilarax as plain
from helpers import random_prompt
from holon_b200.replay import Replayer
from ref_kernels import RefKernels
from replay_tools import mixed_trace, portions, run
from tilarax_tools import CONFIGS, compare, exact_logits, make_folder, make_weights, read_folder

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
    diff = (got.float().cpu() - want.float()).abs().max().item()
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


# ---------------------------------------------------------------- from the first product to q rows and cache rows
def _angles(positions, base, dims):
    inv = 1.0 / (base ** (torch.arange(0, dims, 2, dtype=torch.float32) / dims))
    a = torch.arange(positions, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat((a.cos(), a.sin()), dim=-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,kd,vd,rot,interleaved,blend", [
    (4, 2, 24, 16, 8, True, "mix"), (3, 3, 20, 28, 20, True, "keep"), (6, 1, 12, 20, 0, True, None),
    (2, 2, 64, 16, 2, True, "mix"), (8, 2, 128, 128, 64, True, "mix"), (2, 1, 40, 72, 16, False, None)])
def test_prepare_norm_rotation_blend_and_cache_rows(K, dtype, heads, kv_heads, kd, vd, rot, interleaved, blend):
    """Against the formula: q and k with bias, each head divided by its root mean square times a weight, channel pairs
    (2c, 2c + 1) turned by position · base^(−2c/dims), the other channels untouched; v with bias, blended with the first
    layer's values; k and v land side by side in the page and place that `write_index` names, nowhere else."""
    t, page, pages, eps, base = 13, 4, 9, 1e-5, 50.0
    width = heads * kd + kv_heads * (kd + vd)
    qkv, bias = rand(t, width, dtype=dtype, seed=1), rand(width, seed=2, scale=0.3).to(torch.bfloat16)
    qw, kw = (1 + 0.2 * rand(kd, seed=3)).to(torch.bfloat16), (1 + 0.2 * rand(kd, seed=4)).to(torch.bfloat16)
    positions = torch.tensor([0, 1, 2, 3, 30, 31, 32, 7, 8, 9, 10, 11, 12], dtype=torch.int32)
    table = _angles(40, base, rot) if rot else None
    first, lam = rand(t, kv_heads, vd, seed=5), torch.tensor(0.37)
    write = torch.tensor([4, 5, 6, 7, 20, 21, 22, 31, 32, 33, 34, -1, 35], dtype=torch.int32)   # (one token is not stored)
    x = qkv.double() + bias.double()
    nq, nk = heads * kd, kv_heads * kd
    q, k, v = x[:, :nq].view(t, heads, kd), x[:, nq:nq + nk].view(t, kv_heads, kd), x[:, nq + nk:].view(t, kv_heads, vd)
    q, k = plain.rms_unit(q, eps) * qw.double(), plain.rms_unit(k, eps) * kw.double()
    if rot:
        turn = plain.turn_pairs if interleaved else _turn_halves
        q, k = turn(q, positions.long(), base, rot), turn(k, positions.long(), base, rot)
    v_kept = v.clone()
    if blend == "mix":
        v = (1 - lam.double()) * v + lam.double() * first.double()
    for kernels, dev in ((K, DEV), (REF, "cpu")):
        q_out = torch.full((t, heads, kd), float("nan"), dtype=dtype, device=dev)
        kv = torch.zeros(pages + 1, kv_heads, page, kd + vd, dtype=dtype, device=dev)
        keep = torch.full((t, kv_heads, vd), float("nan"), device=dev) if blend == "keep" else None
        mv = lambda a: a.to(dev) if a is not None else None      # noqa: E731
        kernels.qkv_talking_prepare(q_out, kv, keep, qkv.to(dev), bias.to(dev), qw.to(dev), kw.to(dev), eps, positions.to(dev),
                                    mv(table), rot, interleaved, first.to(dev) if blend == "mix" else None,
                                    lam.to(dev) if blend == "mix" else None, write.to(dev), heads, kv_heads, kd, vd)
        close(q_out, q, dtype, scale=4.0)
        want = torch.zeros(pages + 1, kv_heads, page, kd + vd, dtype=F64)
        for i, w in enumerate(write.tolist()):
            if w >= 0:
                want[w // page, :, w % page] = torch.cat((k[i], v[i]), dim=-1)
        close(kv, want, dtype, scale=4.0)
        if keep is not None:
            close(keep, v_kept, torch.float32, scale=4.0 if dtype == torch.float32 else 2000.0)


def _turn_halves(x, positions, base, dims):
    """Channel c paired with c + dims / 2 (the other layout that the kernel knows)."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    a = positions.double()[:, None] * f[None, :]
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half], out[..., half:dims] = u * cos - v * sin, v * cos + u * sin
    return out


# ---------------------------------------------------------------- attention whose heads share their weights
def _paged(keys, values, page, dtype, spare=3):
    """A cache [pages + 1, kv_heads, page, kd + vd] whose pages lie in shuffled order, and the table of slot 0."""
    n, kvh = keys.shape[:2]
    count = -(-n // page)
    order = torch.randperm(count + spare, generator=torch.Generator().manual_seed(9))[:count]
    kv = torch.zeros(count + spare + 1, kvh, page, keys.shape[2] + values.shape[2], dtype=dtype)
    table = torch.full((2, count + 2), -1, dtype=torch.int32)
    for i, phys in enumerate(order.tolist()):
        m = min(page, n - i * page)
        kv[phys, :, :m] = torch.cat((keys[i * page:i * page + m], values[i * page:i * page + m]), dim=-1).transpose(0, 1)
        table[0, i] = phys
    return kv, table


def _talk_attend(q, keys, values, scale, temp, talk, chunk, window):
    """64-bit: softmax per head over the keys its block (or window) shows, the heads' weights mixed by `talk`, each head's
    mixed weights on the values of its own kv head. q [queries, heads, kd] are the last queries of the n keys."""
    n, (nq, heads, _) = keys.shape[0], q.shape
    group = heads // keys.shape[1]
    out = torch.zeros(nq, heads, values.shape[2], dtype=F64)
    for i in range(nq):
        pos = n - nq + i
        lo = (pos // chunk) * chunk if chunk else 0
        if window:
            lo = max(lo, pos - window + 1)
        w = torch.stack([torch.softmax((keys[lo:pos + 1, g // group].double() @ q[i, g].double()) * scale * float(temp[g]), 0)
                         for g in range(heads)])
        w = talk.double() @ w
        for h in range(heads):
            out[i, h] = w[h] @ values[lo:pos + 1, h // group].double()
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,kd,vd,chunk,window,n,nq,page", [
    (4, 2, 24, 16, 10, 0, 43, 1, 4), (4, 2, 24, 16, 10, 0, 43, 17, 4), (8, 2, 32, 16, 70, 0, 215, 1, 64),
    (8, 2, 32, 16, 70, 0, 215, 90, 64), (3, 3, 20, 28, 7, 0, 36, 36, 16), (6, 1, 12, 20, 0, 0, 300, 1, 64),
    (6, 1, 12, 20, 0, 0, 300, 2, 16), (2, 2, 64, 16, 33, 0, 100, 1, 64), (4, 1, 128, 128, 96, 0, 400, 1, 64),
    (4, 1, 128, 128, 96, 0, 400, 200, 64), (8, 2, 128, 64, 128, 0, 641, 130, 64), (4, 4, 64, 64, 0, 50, 180, 1, 64),
    (4, 4, 64, 64, 64, 20, 180, 70, 64), (16, 4, 128, 128, 256, 0, 700, 1, 64), (16, 4, 128, 128, 256, 0, 700, 300, 64)])
def test_talking_attention_at_the_block_s_edges(K, dtype, heads, kv_heads, kd, vd, chunk, window, n, nq, page):
    """The first key of the last query's block (or window) and the key just before it both point along that query, the
    outer one twice as far: the inner one must take the weight, the outer one none. Without a mask the fourth key of
    hundreds stands out instead. The mixing matrix has entries of both signs, the heads' factors differ. Rows of one
    token and of many, pages smaller and larger than a block, head sizes the tensor cores take and others."""
    keys, values, q = rand(n, kv_heads, kd, seed=1), rand(n, kv_heads, vd, seed=2), rand(nq, heads, kd, seed=3)
    scale = 2.0 / kd ** 0.5
    pos = n - 1
    inside = (pos // chunk) * chunk if chunk else 0
    if window:
        inside = max(inside, pos - window + 1)
    direction = q[-1, 0] / q[-1, 0].norm()
    if inside > 0:
        keys[inside, 0] = 3.0 * direction * kd ** 0.5 / 2
        keys[inside - 1, 0] = 6.0 * direction * kd ** 0.5 / 2
    else:
        keys[3, 0] = 3.0 * direction * kd ** 0.5 / 2
    keys, values, q = keys.to(dtype), values.to(dtype), q.to(dtype)
    temp = 1.0 + 0.3 * rand(heads, seed=4)
    talk = torch.eye(heads) + 0.4 * rand(heads, heads, seed=5)
    want = _talk_attend(q.float(), keys.float(), values.float(), scale, temp, talk, chunk, window)
    plainly = _talk_attend(q.float(), keys.float(), values.float(), scale, temp, torch.eye(heads), chunk, window)
    assert float((want - plainly).abs().max()) > 0.05                       # the mixing matters here
    kv, table = _paged(keys, values, page, dtype)
    out = torch.full((nq, heads, vd), float("nan"), dtype=dtype, device=DEV)
    K.attention_talking(out, q.to(DEV), kv.to(DEV), table.to(DEV), rows_of([nq], [0], kv_len=[n]), scale, temp.to(DEV),
                        chunk, window, talk.to(DEV))
    close(out, want, dtype, scale=4.0)
    if n * nq <= 20000:
        twin = torch.zeros(nq, heads, vd, dtype=dtype)
        REF.attention_talking(twin, q, kv, table, rows_of([nq], [0], kv_len=[n], device="cpu"), scale, temp, chunk, window, talk)
        close(twin, want, dtype, scale=4.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_talking_attention_rows_of_unequal_requests(K, dtype):
    """Five rows in one call (a long portion, single tokens, a portion of two) against each row alone: what a row gets
    does not depend on its neighbours, and a row with no talk matrix and no factors is plain attention."""
    heads, kv_heads, kd, vd, chunk, page = 4, 2, 32, 48, 40, 16
    lens, counts = [130, 77, 41, 200, 9], [50, 1, 2, 1, 9]
    scale = 1.5 / kd ** 0.5
    temp, talk = 1.0 + 0.3 * rand(heads, seed=4), torch.eye(heads) + 0.4 * rand(heads, heads, seed=5)
    total_pages = sum(-(-n // page) for n in lens)
    kv = torch.zeros(total_pages + 1, kv_heads, page, kd + vd, dtype=dtype)
    table = torch.full((6, max(-(-n // page) for n in lens) + 1), -1, dtype=torch.int32)
    order, at, qs, wants, slots = torch.randperm(total_pages, generator=torch.Generator().manual_seed(2)).tolist(), 0, [], [], [4, 0, 2, 5, 1]
    plain_wants = []
    for r, (n, c) in enumerate(zip(lens, counts)):
        keys, values, q = rand(n, kv_heads, kd, dtype=dtype, seed=10 + r), rand(n, kv_heads, vd, dtype=dtype, seed=20 + r), rand(c, heads, kd, dtype=dtype, seed=30 + r)
        for i in range(-(-n // page)):
            m = min(page, n - i * page)
            kv[order[at], :, :m] = torch.cat((keys[i * page:i * page + m], values[i * page:i * page + m]), dim=-1).transpose(0, 1)
            table[slots[r], i] = order[at]
            at += 1
        qs.append(q)
        wants.append(_talk_attend(q.float(), keys.float(), values.float(), scale, temp, talk, chunk, 0))
        plain_wants.append(_talk_attend(q.float(), keys.float(), values.float(), scale, torch.ones(heads), torch.eye(heads), chunk, 0))
    q = torch.cat(qs)
    for t_, ta, want in ((temp, talk, wants), (None, None, plain_wants)):
        out = torch.full((sum(counts), heads, vd), float("nan"), dtype=dtype, device=DEV)
        K.attention_talking(out, q.to(DEV), kv.to(DEV), table.to(DEV), rows_of(counts, slots, kv_len=lens), scale,
                            t_.to(DEV) if t_ is not None else None, chunk, 0, ta.to(DEV) if ta is not None else None)
        close(out, torch.cat(want), dtype, scale=4.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("part", [8, 32, 64])
@pytest.mark.parametrize("heads,kv_heads,kd,vd", [(6, 2, 40, 24), (8, 2, 64, 64), (16, 4, 128, 128), (32, 8, 128, 128),
                                                  (4, 2, 72, 48), (3, 1, 24, 128), (16, 1, 32, 8)])
def test_one_token_rows_with_their_keys_in_parts(K, dtype, part, heads, kv_heads, kd, vd, monkeypatch):
    """Rows of one token whose keys are cut into parts of unequal fill (the last part short, some parts empty for the
    shorter row), merged by the second kernel: maxima, sums and weighted values of the parts, then the heads' mixing.
    Sizes that the kernel with tiles in shared memory takes (1, 4 and 16 heads a thread, fewer heads than thread
    groups) and sizes it leaves to the plain one."""
    chunk, page = 150, 16
    lens, slots = [431, 309, 7], [2, 0, 1]                   # 132, 10 and 7 keys in sight
    scale = 2.0 / kd ** 0.5
    temp, talk = 1.0 + 0.3 * rand(heads, seed=4), torch.eye(heads) + 0.4 * rand(heads, heads, seed=5)
    total = sum(-(-n // page) for n in lens)
    kv = torch.zeros(total + 1, kv_heads, page, kd + vd, dtype=dtype)
    table = torch.full((3, 30), -1, dtype=torch.int32)
    order, at, qs, wants = torch.randperm(total, generator=torch.Generator().manual_seed(3)).tolist(), 0, [], []
    for r, n in enumerate(lens):
        keys, values, q = rand(n, kv_heads, kd, dtype=dtype, seed=10 + r), rand(n, kv_heads, vd, dtype=dtype, seed=20 + r), rand(1, heads, kd, dtype=dtype, seed=30 + r)
        for i in range(-(-n // page)):
            m = min(page, n - i * page)
            kv[order[at], :, :m] = torch.cat((keys[i * page:i * page + m], values[i * page:i * page + m]), dim=-1).transpose(0, 1)
            table[slots[r], i] = order[at]
            at += 1
        qs.append(q)
        wants.append(_talk_attend(q.float(), keys.float(), values.float(), scale, temp, talk, chunk, 0))
    monkeypatch.setattr(K, "TALKING_SPLIT_KEYS", part)
    out = torch.full((3, heads, vd), float("nan"), dtype=dtype, device=DEV)
    before = K.launches
    K.attention_talking(out, torch.cat(qs).to(DEV), kv.to(DEV), table.to(DEV), rows_of([1, 1, 1], slots, kv_len=lens), scale,
                        temp.to(DEV), chunk, 0, talk.to(DEV))
    assert K.launches == before + 1                          # (one call of the library: it launches both kernels)
    close(out, torch.cat(wants), dtype, scale=4.0)


def test_tensor_core_rows_beside_one_token_rows(K, monkeypatch):
    """bfloat16, keys and values of 128: rows of one token (CUDA cores, keys in parts) come first in a step, rows of
    several tokens (tcgen05, every query head over every kv head's values, then the mixing kernel) after them; each row
    equals the formula for that row alone. Blocks of 96 positions cut across the kernel's tiles of 64 keys, a query tile
    spans several blocks, and one row starts in the middle of a block."""
    dtype, heads, kv_heads, kd, vd, chunk, page = torch.bfloat16, 8, 2, 128, 128, 96, 64
    lens, counts, slots = [250, 97, 300, 131, 420], [1, 1, 270, 2, 150], [4, 0, 2, 5, 1]
    scale = 2.0 / kd ** 0.5
    temp, talk = 1.0 + 0.2 * rand(heads, seed=4), torch.eye(heads) + 0.4 * rand(heads, heads, seed=5)
    temp[3], temp[6] = -0.8, -1.3                            # (factors of either sign: the smallest score then leads)
    total = sum(-(-n // page) for n in lens)
    kv = torch.zeros(total + 1, kv_heads, page, kd + vd, dtype=dtype)
    table = torch.full((6, 8), -1, dtype=torch.int32)
    order, at, qs, wants = torch.randperm(total, generator=torch.Generator().manual_seed(2)).tolist(), 0, [], []
    for r, (n, c) in enumerate(zip(lens, counts)):
        keys, values, q = rand(n, kv_heads, kd, dtype=dtype, seed=10 + r), rand(n, kv_heads, vd, dtype=dtype, seed=20 + r), rand(c, heads, kd, dtype=dtype, seed=30 + r)
        pos = n - 1                                          # the last query's block: its first key stands out, the key before
        inside = (pos // chunk) * chunk                      # it would stand out twice as far if it were seen
        direction = (q[-1, 0] / q[-1, 0].float().norm()).float()
        if inside > 0:
            keys[inside, 0] = (3.0 * direction * kd ** 0.5 / 2).to(dtype)
            keys[inside - 1, 0] = (6.0 * direction * kd ** 0.5 / 2).to(dtype)
        for i in range(-(-n // page)):
            m = min(page, n - i * page)
            kv[order[at], :, :m] = torch.cat((keys[i * page:i * page + m], values[i * page:i * page + m]), dim=-1).transpose(0, 1)
            table[slots[r], i] = order[at]
            at += 1
        qs.append(q)
        wants.append(_talk_attend(q.float(), keys.float(), values.float(), scale, temp, talk, chunk, 0))
    for ta, want in ((talk, torch.cat(wants)), ):
        out = torch.full((sum(counts), heads, vd), float("nan"), dtype=dtype, device=DEV)
        K.attention_talking(out, torch.cat(qs).to(DEV), kv.to(DEV), table.to(DEV), rows_of(counts, slots, kv_len=lens), scale,
                            temp.to(DEV), chunk, 0, ta.to(DEV))
        close(out, want, dtype, scale=4.0)
        monkeypatch.setattr(K, "prefill_attention", "mma")   # the same on CUDA cores
        slow = torch.full((sum(counts), heads, vd), float("nan"), dtype=dtype, device=DEV)
        K.attention_talking(slow, torch.cat(qs).to(DEV), kv.to(DEV), table.to(DEV), rows_of(counts, slots, kv_len=lens), scale,
                            temp.to(DEV), chunk, 0, ta.to(DEV))
        close(slow, want, dtype, scale=4.0)
    assert K.tcgen05_status() == 0                           # no bounded wait of the tensor-core kernel ran out


# ---------------------------------------------------------------- the matrix memory with exponential gates
def _memory(first, pre, bias, cap, heads, dim, vdim, state):
    """64-bit, one sequence: first [t, q | k | v | g], pre [t, i | f]; state (S [heads, dim, vdim], n [heads, dim],
    m [heads]) is carried and returned. Returns the quotient S^T q / (max(|n . q|, exp(-m)) + 1e-6) per head."""
    t = first.shape[0]
    f = first.double()
    q = f[:, :heads * dim].view(t, heads, dim) * dim ** -0.5
    k = f[:, heads * dim:2 * heads * dim].view(t, heads, dim)
    v = f[:, 2 * heads * dim:2 * heads * dim + heads * vdim].view(t, heads, vdim)
    a = pre.double() + bias.double()
    gi = cap * torch.tanh(a[:, :heads] / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh(a[:, heads:] / cap))
    S, n, m = (x.clone() for x in state)
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for s in range(t):
        for h in range(heads):
            new = max(float(gf[s, h] + m[h]), float(gi[s, h]))
            keep, take = math.exp(float(gf[s, h] + m[h]) - new), math.exp(float(gi[s, h]) - new)
            S[h] = keep * S[h] + take * torch.outer(k[s, h], v[s, h])
            n[h] = keep * n[h] + take * k[s, h]
            m[h] = new
            out[s, h] = (S[h].T @ q[s, h]) / (max(abs(float(n[h] @ q[s, h])), math.exp(-new)) + 1e-6)
    return out, (S, n, m)


def _memory_step(kernels, dev, first, pre, bias, gain, cap, eps, heads, dim, vdim, state, maxes, rows):
    """The mixer's kernels in the order the part calls them; returns the normed, gated rows."""
    t = first.shape[0]
    gates = torch.empty(3, t, heads, device=dev)
    kernels.mlstm_gates(gates, pre, bias, cap, maxes, rows)
    qk, v1 = torch.empty(t, 2, heads, dim, device=dev), torch.empty(t, heads, vdim + 1, device=dev)
    kernels.mlstm_prepare(qk, v1, gates[1], first, dim ** -0.5)
    o1 = torch.empty(t, heads, vdim + 1, device=dev)
    kernels.recurrent_scan(o1, qk, v1, None, None, None, state, rows, token_decay=gates[0])
    y = torch.empty(t, heads, vdim, dtype=first.dtype, device=dev)
    at = 2 * heads * dim + heads * vdim
    kernels.mlstm_read_out(y, o1, gates[2], gain, first[:, at:at + heads * vdim], eps, 1e-6)
    return y


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim,cap", [(2, 8, 12, 12.0), (1, 12, 20, 3.0), (2, 96, 40, 8.0), (3, 16, 8, 5.0),
                                               (2, 128, 256, 15.0), (1, 4, 4, 5.0), (4, 32, 48, 11.0)])
def test_memory_rows_in_slots_and_in_portions(K, dtype, heads, dim, vdim, cap):
    """Rows of 1, 1, 2, 11 and 37 tokens in slots of their own, twice: the second call goes on from the state, the
    normaliser and the running maximum that the first left. The gates' pre-activations spread over ± 3 caps, so the cap
    bites, the maximum rises with an input gate and sinks with the forget gates, and exp(-m) decides some denominators."""
    counts, slots, eps = [1, 1, 2, 11, 37], [3, 0, 5, 1, 4], 1e-5
    t = sum(counts)
    width = 2 * heads * dim + 2 * heads * vdim
    bias = torch.cat((rand(heads, seed=1), 2.0 + rand(heads, seed=2)))
    gain = 1 + 0.1 * rand(heads * vdim, seed=3)
    states = {s: (torch.zeros(heads, dim, vdim, dtype=F64), torch.zeros(heads, dim, dtype=F64), torch.zeros(heads, dtype=F64))
              for s in slots}
    packs = {}
    for name, kernels, dev in (("gpu", K, DEV), ("twin", REF, "cpu")):
        packs[name] = (kernels, dev, torch.zeros(7, heads, vdim + 1, dim, device=dev), torch.zeros(7, heads, device=dev))
    for call in range(2):
        first = rand(t, width, seed=10 + call).to(dtype)
        pre = rand(t, 2 * heads, seed=20 + call, scale=cap)
        want, at = [], 0
        for n, s in zip(counts, slots):
            o, states[s] = _memory(first[at:at + n].float(), pre[at:at + n], bias, cap, heads, dim, vdim, states[s])
            o = plain.rms_unit(o, eps) * gain.double().view(1, heads, vdim)
            g = first[at:at + n, 2 * heads * dim + heads * vdim:].double().view(n, heads, vdim)
            want.append(o * torch.sigmoid(g))
            at += n
        want = torch.cat(want)
        for name, (kernels, dev, state, maxes) in packs.items():
            y = _memory_step(kernels, dev, first.to(dev), pre.to(dev), bias.to(dev), gain.to(dev), cap, eps, heads, dim, vdim,
                             state, maxes, rows_of(counts, slots, device=dev))
            close(y, want, dtype, scale=8.0)
    for name, (kernels, dev, state, maxes) in packs.items():             # what the slots hold afterwards
        for s in slots:
            S, n, m = states[s]
            close(state[s, :, :vdim].transpose(1, 2), S, torch.float32, scale=30.0 * max(1.0, float(S.abs().max())))
            close(state[s, :, vdim], n, torch.float32, scale=30.0 * max(1.0, float(n.abs().max())))
            close(maxes[s], m, torch.float32, scale=10.0)


def test_the_memory_keeps_a_far_write(K):
    """Forget gates near one (log f about -0.001) and one strong write 400 tokens back: a query along that key reads its
    value long after, in a prompt's row and token by token; with the write left out the read-out differs visibly."""
    heads, dim, vdim, cap, t = 2, 32, 16, 12.0, 420
    width = 2 * heads * dim + 2 * heads * vdim
    first = rand(t, width, seed=1) * 0.3
    key = rand(dim, seed=2)
    key = key / key.norm()
    first[5, heads * dim:heads * dim + dim] = 4.0 * key                    # head 0's key at token 5
    first[5, 2 * heads * dim:2 * heads * dim + vdim] = 5.0                  # its value
    first[-1, :dim] = 6.0 * key                                            # the last query of head 0
    pre = torch.cat((torch.full((t, heads), -2.0), torch.full((t, heads), 7.0)), dim=1)
    pre[5, 0] = 3.0                                                        # the input gate opens for the write
    bias, gain = torch.zeros(2 * heads), torch.ones(heads * vdim)
    zero = lambda: (torch.zeros(heads, dim, vdim, dtype=F64), torch.zeros(heads, dim, dtype=F64), torch.zeros(heads, dtype=F64))   # noqa: E731
    want, _ = _memory(first, pre, bias, cap, heads, dim, vdim, zero())
    other = first.clone()
    other[5, 2 * heads * dim:2 * heads * dim + vdim] = 0.0
    without, _ = _memory(other, pre, bias, cap, heads, dim, vdim, zero())
    assert float((want[-1, 0] - without[-1, 0]).abs().max()) > 0.5
    want = plain.rms_unit(want, 1e-5) * torch.sigmoid(first[:, 2 * heads * dim + heads * vdim:].double().view(t, heads, vdim))
    for cut in (t, 300, 0):                                                # whole; a prompt and single tokens; all single
        state, maxes = torch.zeros(3, heads, vdim + 1, dim, device=DEV), torch.zeros(3, heads, device=DEV)
        pieces = ([(0, cut)] if cut else []) + [(i, i + 1) for i in range(cut, t)]
        got = torch.cat([_memory_step(K, DEV, first[a:b].to(DEV), pre[a:b].to(DEV), bias.to(DEV), gain.to(DEV), cap, 1e-5, heads,
                                      dim, vdim, state, maxes, rows_of([b - a], [1])) for a, b in pieces])
        close(got, want, torch.float32, scale=10.0)


# ---------------------------------------------------------------- the norm on a sublayer's output, the depth average
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,dim,kept", [(5, 64, 3), (3, 72, 1), (9, 2048, 6), (2, 1000, 2)])
def test_output_norm_and_depth_average(K, dtype, rows, dim, kept):
    """dst = src + (y + bias) / rms(y + bias) · (1 + w); then Σ_j c[j] X_j over the kept results, the last being dst."""
    eps = 1e-5
    y, bias, w = rand(rows, dim, seed=1).to(dtype), rand(dim, seed=2, scale=0.3).to(torch.bfloat16), rand(dim, seed=3, scale=0.2).to(torch.bfloat16)
    src, coef = rand(rows, dim, seed=4), 1.0 / kept + 0.3 * rand(kept, seed=5)
    hist = rand(kept, rows, dim, seed=6)
    z = y.double() + bias.double()
    own = src.double() + plain.out_norm(z, w.double(), eps)
    avg = sum(coef[j].double() * hist[j].double() for j in range(kept - 1)) + coef[kept - 1].double() * own
    for kernels, dev in ((K, DEV), (REF, "cpu")):
        h = hist.clone().to(dev)
        go, cast = torch.empty(rows, dim, device=dev), torch.empty(rows, dim, dtype=dtype, device=dev)
        kernels.out_norm_add(h[kept - 1], src.to(dev), y.to(dev), bias.to(dev), w.to(dev), eps, 1.0, hist=h, n_hist=kept,
                             coef=coef.to(dev), avg=go, cast=cast)
        close(h[kept - 1], own, torch.float32, scale=4.0)
        close(go, avg, torch.float32, scale=8.0)
        close(cast, avg, dtype, scale=8.0)
        assert torch.equal(h[:kept - 1].cpu(), hist[:kept - 1])
        dst = torch.empty(rows, dim, device=dev)                          # without the average: the stream goes on
        kernels.out_norm_add(dst, src.to(dev), y.to(dev), None, w.to(dev), eps, 1.0, cast=cast)
        close(dst, src.double() + plain.out_norm(y.double(), w.double(), eps), torch.float32, scale=4.0)


# ---------------------------------------------------------------- a router whose bias decides
@pytest.mark.parametrize("tokens", [9, 700])
def test_router_bias_decides_the_choice(K, tokens):
    """Logits whose two largest lie 0.1 apart and a bias that turns their order: the chosen experts follow logits + bias,
    and the weights are the softmax over the chosen (biased) logits alone."""
    experts, top = 7, 3
    z = rand(tokens, experts, seed=1)
    bias = rand(experts, seed=2)
    for i in range(tokens):
        a, b = i % experts, (i + 3) % experts
        z[i, a], z[i, b] = 5.0 - bias[a], 4.9 - bias[b] + 0.3            # biased: b leads by 0.2; unbiased the order may differ
    zb = z.double() + bias.double()
    best = torch.topk(zb, top, dim=-1)
    share = torch.softmax(best.values, -1)
    chosen = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    weight = torch.empty(tokens, top, device=DEV)
    counts = torch.zeros(2 * experts + 3, dtype=torch.int32, device=DEV)
    place = torch.empty(tokens * top, dtype=torch.int32, device=DEV)
    token_of = torch.empty(tokens * top, dtype=torch.int32, device=DEV)
    K.route_rows(chosen, weight, counts, place, token_of, z.to(DEV), experts, 1.0, True, bias=bias.to(DEV))
    for i in range(tokens):
        got = dict(zip(chosen[i].tolist(), weight[i].tolist()))
        assert set(got) == set(best.indices[i].tolist())
        for e, w in zip(best.indices[i].tolist(), share[i].tolist()):
            assert abs(got[e] - w) < 1e-5


# ---------------------------------------------------------------- the model through the replayer and the engine
# D: head sizes and blocks that the tensor-core kernels take (keys of 128 and 64, values of 128 and 64, blocks of 128 and
# 96 positions), a memory whose threads hold sixteen key channels, kv groups of four and of one.
def _big():
    from tilarax_tools import _att, _dense, _layer, _mem, _model, _moe
    return _model(256, 311, 1e-6, [
        _layer("attention", _att(4, 1, 128, 128, 128, 6.0, 1e4, 64), _dense(128)),
        _layer("mlstm", _mem(2, 128, 64, 10.0), _moe(8, 2, 64)),
        _layer("attention", _att(4, 1, 128, 128, 128, 6.0, 1e4, 64), _moe(8, 2, 64)),
        _layer("attention", _att(4, 4, 64, 64, 96, 5.0, 1e5, 64, v_mix=False), None)])


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param, seed=7)
    config = CONFIGS[request.param]
    prompts = {f"r{i}": random_prompt(config["vocab"], n, 40 + i) for i, n in enumerate((70, 133, 37, 96))}
    return folder, config, prompts, {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_tail_then_portions(model, dtype):
    folder, config, prompts, want = model
    r = Replayer(str(folder), dtype, max_tokens=192)
    compare(run(r, [([(rid, ids)], [rid]) for rid, ids in prompts.items()]), want, dtype)
    steps = []
    for rid, ids in prompts.items():                     # most of it in one step, the last 32 tokens one by one
        cut = len(ids) - 32
        steps.append(([(rid, ids[:cut])], []))
        steps += [([(rid, [t])], [rid] if i == 31 else []) for i, t in enumerate(ids[cut:])]
    compare(run(r, steps), want, dtype)
    steps = []
    for rid, ids in prompts.items():                     # portions of changing size, down to two tokens
        parts = portions(ids, [7, 2, 19, 3, 2, 64, 5])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [64, 16])
def test_mixed_requests_in_a_small_pool(model, dtype, page_size):
    """Four unequal requests live at once in 448 tokens of pool: three arrive in portions while one decodes; when it
    ends, the last one grows into pages it gave back. Every row must equal the request run alone."""
    folder, config, prompts, want = model
    r = Replayer(str(folder), dtype, max_tokens=448, page_size=page_size)
    got = run(r, mixed_trace(prompts))
    assert len(got) == sum(map(len, prompts.values())) and not r.built.cache.live
    compare(got, want, dtype)
    got = run(r, mixed_trace(prompts))                   # once more in the same engine: every page and slot used again
    compare(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(model, dtype):
    folder, config, _, _ = model
    ids = random_prompt(config["vocab"], 330, 77)
    want = {"x": exact_logits(folder, ids)}
    r = Replayer(str(folder), dtype, max_tokens=384)
    got = run(r, [([("x", [t])], ["x"] if i == len(ids) - 1 else []) for i, t in enumerate(ids)])   # all one by one
    compare(got, want, dtype)
    compare({k: v for k, v in got.items() if k[1] < 4}, want, dtype)
    # a prompt of 260 tokens (past four page borders and many blocks), then single tokens
    got = run(r, [([("x", ids[:260])], [])] + [([("x", [t])], []) for t in ids[260:]])
    compare(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_of_128_and_blocks_of_128(tmp_path, dtype):
    """Whole prompts of 300 and 133 tokens, their last 32 tokens one by one (over a block's edge at 256), and portions
    that start and end inside blocks."""
    config = _big()
    folder = make_folder(tmp_path, "d", seed=3, config=config)
    prompts = {f"r{i}": random_prompt(config["vocab"], n, 50 + i) for i, n in enumerate((300, 133))}
    want = {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}
    r = Replayer(str(folder), dtype, max_tokens=512)
    compare(run(r, [([(rid, ids)], [rid]) for rid, ids in prompts.items()]), want, dtype)
    steps = []
    for rid, ids in prompts.items():
        cut = len(ids) - 48
        steps.append(([(rid, ids[:cut])], []))
        steps += [([(rid, [t])], [rid] if i == 47 else []) for i, t in enumerate(ids[cut:])]
    compare(run(r, steps), want, dtype)
    steps = []
    for rid, ids in prompts.items():
        parts = portions(ids, [7, 2, 130, 3, 64])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, dtype)
    both = [([("r0", prompts["r0"][:200]), ("r1", prompts["r1"][:131])], []),
            ([("r0", prompts["r0"][200:]), ("r1", prompts["r1"][131:])], ["r0", "r1"])]
    compare(run(r, both), want, dtype)


def test_a_token_far_back_is_remembered(tmp_path):
    """The memory must carry a token from 300 places back (the attention's blocks have long forgotten it): the logits of
    the last rows change when token 7 changes, and the engine follows the plain implementation through that change, in
    a prompt and in decoding, with the two requests side by side in one batch."""
    config = copy.deepcopy(CONFIGS["b"])
    folder = make_folder(tmp_path, "b", seed=11, config=config)
    vocab = config["vocab"]
    ids = random_prompt(vocab, 320, 5)
    other = list(ids)
    other[7] = (ids[7] + 1) % vocab
    want = {"x": exact_logits(folder, ids), "y": exact_logits(folder, other)}
    assert float((want["x"][-1] - want["y"][-1]).abs().max()) > 1e-3         # the far token matters to the last row
    r = Replayer(str(folder), "float32", max_tokens=768)
    steps = [([("x", ids[:300]), ("y", other[:300])], [])] + [([("x", [a]), ("y", [b])], []) for a, b in zip(ids[300:], other[300:])]
    compare(run(r, steps), want, "float32")


def test_planted_keys_at_the_block_s_edges_through_the_model(tmp_path):
    """One attention layer with scores so sharp that the best key takes nearly all weight, blocks of 12: an off-by-one at
    either edge of a block moves a row by most of its spread. Whole, in portions of five, and token by token."""
    config = copy.deepcopy(CONFIGS["att"])
    m = config["layers"][0]["mixer"]
    m["mask"]["size"], m["scale"] = 12, 12.0 / m["dim"] ** 0.5
    folder = make_folder(tmp_path, "att", config=config, weights=make_weights(config, 3))
    ids = random_prompt(config["vocab"], 50, 5)
    want = {"r": exact_logits(folder, ids)}
    for page in (16, 64):
        r = Replayer(str(folder), "float32", 64, page_size=page)
        compare(run(r, [([("r", ids)], ["r"])]), want, "float32")
        compare(run(r, [([("r", p)], ["r"] if i == 9 else []) for i, p in enumerate(portions(ids, [5]))]), want, "float32")
        compare(run(r, [([("r", [t])], ["r"] if i == 49 else []) for i, t in enumerate(ids)]), want, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(model, dtype, graphs):
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    folder, config, prompts, _ = model
    stored, weights = read_folder(folder)
    engine = Engine(EngineConfig(model=str(folder), dtype=dtype, page_size=64, max_seqs=4, max_model_len=256,
                                 max_step_tokens=96, state_memory=1 << 26, cuda_graphs=graphs, chunk_with_decode=32))
    asked = [prompts["r0"], prompts["r2"], prompts["r1"], prompts["r3"], prompts["r0"][:40] + prompts["r2"]]
    with torch.inference_mode():
        got = engine.generate(asked, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    engine.close()
    margin, off = (1e-3 if dtype == "float32" else 0.25), []
    for prompt, tokens in zip(asked, got):
        ids = list(prompt)
        assert len(tokens) == 12
        for token in tokens:                             # (each token judged after the engine's own earlier ones)
            logits = plain.forward(weights, stored, ids)[-1]
            if float(logits.max() - logits[token]) > margin * float(logits.std()):
                off.append((len(ids), token, int(logits.argmax())))
            ids.append(token)
    assert len(off) <= (0 if dtype == "float32" else 2), off


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
