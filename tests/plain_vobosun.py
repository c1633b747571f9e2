"""Vobosun written out plainly: one function per mechanism, 64-bit, whole sequences, no cache, no batch.

The yardstick of the Vobosun tests. It shares no code with the engine: it reads a configuration dict and a dict of
stored tensors and walks a sequence's tokens with loops and small matrix products. Notation: x a token's row of the
stream, W y a stored weight [out, in] applied to y, N a norm.

    norm:       N(y) = tanh(alpha · y) · w + b  (no mean, no variance; alpha one stored number)
    layer:      h = N1(x);  m = h + (h_prev − h) · shift  (h_prev: the token before, zeros for the first);
                x ← x + N1b(mixer(m));  x ← x + N2b(ff(N2(x)))
    delta:      per head a matrix S [key channel, value channel]; with the unit key u = k / sqrt(Σk² + 1e-6),
                S ← diag(w) S − (a ∘ u)(uᵀ S) + k vᵀ (both terms read the old S), o = Sᵀ r;
                w = exp(−e^(−1/2) sigmoid(W_w2 tanh(W_w1 m) + w0)), a = sigmoid(W_a m + b_a);
                o / rms(o) per head · weight · sigmoid(W_g m), then W_o
    attention:  q, k, v with biases; the first `rot.dims` channels of q and k turned in pairs (c, c + dims/2) by
                position · base^(−2c/dims) / factor; scores · scale; token i sees j ≤ i; softmax; W_o
    ff:         W_down xielu(W_up y), or experts W_down (silu(W_gate y) · W_up y) chosen in groups (below)
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def _w(weights, name):
    return weights[name].to(F)


def tanh_norm(y, weights, name):
    return torch.tanh(_w(weights, name + ".alpha") * y) * _w(weights, name) + _w(weights, name + ".b")


def token_shift(h, mu):
    """m_t = h_t + (h_(t−1) − h_t) · mu, h_(−1) = 0."""
    before = torch.cat((torch.zeros_like(h[:1]), h[:-1]), 0)
    return h + (before - h) * mu


def turn_halves(x, positions, base, dims, factor):
    """x [t, heads, dim]: channels (c, c + dims/2), c < dims/2, turned by position · base^(−2c/dims) / factor."""
    if not dims:
        return x
    half = dims // 2
    c = torch.arange(half, dtype=F)
    angle = positions.to(F)[:, None] * (base ** (-2.0 * c / dims) / factor)[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., dims:]), -1)


def attention(m_in, weights, p, m):
    t = m_in.shape[0]
    heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (m_in @ _w(weights, p + "q").T + _w(weights, p + "q.b")).view(t, heads, dim)
    k = (m_in @ _w(weights, p + "k").T + _w(weights, p + "k.b")).view(t, kvh, dim)
    v = (m_in @ _w(weights, p + "v").T + _w(weights, p + "v.b")).view(t, kvh, vdim)
    rot = m.get("rot")
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        pos = torch.arange(t)
        q = turn_halves(q, pos, float(rot["base"]), rot["dims"], factor)
        k = turn_halves(k, pos, float(rot["base"]), rot["dims"], factor)
    group = heads // kvh
    out = torch.zeros(t, heads, vdim, dtype=F)
    hidden = torch.triu(torch.ones(t, t, dtype=torch.bool), 1)
    for h in range(heads):
        s = (q[:, h] @ k[:, h // group].T) * float(m["scale"])
        out[:, h] = torch.softmax(s.masked_fill(hidden, -math.inf), -1) @ v[:, h // group]
    return out.reshape(t, heads * vdim) @ _w(weights, p + "o").T


def general_delta(m_in, weights, p, m, eps):
    t = m_in.shape[0]
    heads, dim = m["heads"], m["dim"]
    r = (m_in @ _w(weights, p + "r").T).view(t, heads, dim)
    k = (m_in @ _w(weights, p + "k").T).view(t, heads, dim)
    v = (m_in @ _w(weights, p + "v").T).view(t, heads, dim)
    low = torch.tanh(m_in @ _w(weights, p + "w1").T) @ _w(weights, p + "w2").T + _w(weights, p + "w0")
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(low)).view(t, heads, dim)
    a = torch.sigmoid(m_in @ _w(weights, p + "a").T + _w(weights, p + "a.b")).view(t, heads, dim)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    out = torch.zeros(t, heads, dim, dtype=F)
    for h in range(heads):
        S = torch.zeros(dim, dim, dtype=F)
        for s in range(t):
            S = w[s, h][:, None] * S - torch.outer(a[s, h] * u[s, h], u[s, h] @ S) + torch.outer(k[s, h], v[s, h])
            out[s, h] = S.T @ r[s, h]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps)
    y = out.reshape(t, heads * dim) * _w(weights, p + "norm") * torch.sigmoid(m_in @ _w(weights, p + "g").T)
    return y @ _w(weights, p + "o").T


def xielu(z, p, q):
    sp = torch.nn.functional.softplus
    return torch.where(z > 0, sp(p) * z * z + z / 2, (0.5 + sp(q)) * (torch.expm1(z) - z) + z / 2)


def dense_ff(y, weights, p):
    act = _w(weights, p + "act")
    return xielu(y @ _w(weights, p + "up").T, act[0], act[1]) @ _w(weights, p + "down").T


def gated_unit(y, weights, p):
    return (torch.nn.functional.silu(y @ _w(weights, p + "gate").T) * (y @ _w(weights, p + "up").T)) @ _w(weights, p + "down").T


def choose(z, correction, router):
    """For one token's router logits z: [(expert, weight)], identity experts numbered behind the real ones."""
    n, ident, top = router["experts"], router.get("identity", 0), router["top"]
    s = torch.softmax(z, -1)
    choice = s + correction
    groups = router.get("groups")
    if groups:
        per = (n + ident) // groups["count"]
        best = choice.view(groups["count"], per).max(-1).values
        kept = torch.topk(best, groups["keep"]).indices.tolist()
        masked = torch.full_like(choice, -math.inf)
        for g in kept:
            masked[g * per:(g + 1) * per] = choice[g * per:(g + 1) * per]
        choice = masked
    picked = torch.topk(choice, top).indices.tolist()
    total = sum(s[e] for e in picked) + 1e-20
    return [(e, s[e] / total) for e in picked]


def experts_ff(y, weights, p, mlp):
    router = mlp["router"]
    z = y @ _w(weights, p + "router").T
    correction = _w(weights, p + "correction")
    out = torch.zeros_like(y)
    for s in range(y.shape[0]):
        for e, share in choose(z[s], correction, router):
            if e >= router["experts"]:
                out[s] += share * y[s]
            else:
                out[s] += share * gated_unit(y[s], weights, f"{p}e{e}.")
    if mlp.get("shared"):
        out = out + gated_unit(y, weights, p + "shared.")
    return out


def forward(weights, config, ids, streams=None):
    """Logits [tokens, vocab] of one sequence; `streams`, a list, receives the stream after every layer."""
    eps = float(config["norm"]["eps"])
    x = _w(weights, "embed")[torch.tensor(list(ids))]
    for i, layer in enumerate(config["layers"]):
        j = i
        while config["layers"][j].get("weights_of") is not None:
            j = config["layers"][j]["weights_of"]
        p = f"l{j}."
        m = layer["mixer"]
        h = token_shift(tanh_norm(x, weights, p + "norm1"), _w(weights, p + "shift"))
        if layer["type"] == "attention":
            y = attention(h, weights, p + "mix.", m)
        elif layer["type"] == "general_delta":
            y = general_delta(h, weights, p + "mix.", m, eps)
        else:
            raise NotImplementedError(layer["type"])
        x = x + tanh_norm(y, weights, p + "norm1b")
        mlp = layer.get("mlp")
        if mlp is not None:
            h = tanh_norm(x, weights, p + "norm2")
            y = dense_ff(h, weights, p + "mlp.") if mlp["kind"] == "dense" else experts_ff(h, weights, p + "mlp.", mlp)
            x = x + tanh_norm(y, weights, p + "norm2b")
        if streams is not None:
            streams.append(x)
    return tanh_norm(x, weights, "final.norm") @ _w(weights, "head").T
