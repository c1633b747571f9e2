"""Tilarax written out plainly: one function per mechanism, 64-bit, whole sequences, no cache, no batch.

The yardstick of the Tilarax tests. It shares no code with the engine: it reads a configuration dict and a dict of
stored tensors and walks a sequence's tokens with loops and small matrix products. Notation: x a token's row of the
stream, W y a stored weight [out, in] applied to y.

    layer:      x ← x + N1(mixer(x));  x ← x + N2(ff(x));  N(y) = y / sqrt(mean(y²) + eps) · (1 + w)
    depth mix:  with X_0 the embedding's rows and X_(i+1) what layer i leaves, layer i hands on Σ_j c_i[j] · X_j
    attention:  q, k, v with biases; q and k under a per-head RMS norm with a plain weight; the first `rot.dims`
                channels turned in neighbouring pairs (2c, 2c+1) by position · base^(−2c/dims); scores · scale · temp_h;
                token i sees j ≤ i of its own block of `mask.size` positions; softmax; the heads' weights mixed by a
                matrix T (after the softmax); values of the head's own key/value head; v blended with the first
                blending layer's v of the same token
    mlstm:      a matrix state per head with exponential gates held in range by a running maximum m
    ff:         W_down gelu_tanh(W_up x), or experts W_down (silu(W_gate x) · W_up x) chosen by the largest router
                logits, weighted by the softmax over the chosen logits
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def _w(weights, name):
    return weights[name].to(F)


def rms_unit(y, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def out_norm(y, w, eps):
    """The norm on a sublayer's output and the model's last norm: weight stored around zero."""
    return rms_unit(y, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def turn_pairs(x, positions, base, dims):
    """x [t, heads, dim]: channels (2c, 2c + 1), c < dims / 2, turned by position · base^(−2c/dims)."""
    if not dims:
        return x
    c = torch.arange(dims // 2, dtype=F)
    angle = positions.to(F)[:, None] * base ** (-2.0 * c / dims)[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def block_attention(x, weights, p, m, eps, v_first):
    """One attention mixer over a whole sequence. Returns (output [t, width], the values it used [t, kv_heads, vdim])."""
    t = x.shape[0]
    heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (x @ _w(weights, p + "q").T + _w(weights, p + "q.b")).view(t, heads, dim)
    k = (x @ _w(weights, p + "k").T + _w(weights, p + "k.b")).view(t, kvh, dim)
    v = (x @ _w(weights, p + "v").T + _w(weights, p + "v.b")).view(t, kvh, vdim)
    q = rms_unit(q, eps) * _w(weights, p + "q.norm")
    k = rms_unit(k, eps) * _w(weights, p + "k.norm")
    pos = torch.arange(t)
    rot = m.get("rot")
    if rot:
        q, k = turn_pairs(q, pos, rot["base"], rot["dims"]), turn_pairs(k, pos, rot["base"], rot["dims"])
    if v_first is not None:
        lam = _w(weights, p + "vmix")
        v = (1.0 - lam) * v + lam * v_first
    temp, talk = _w(weights, p + "temp"), _w(weights, p + "talk")
    size = m.get("mask", {}).get("size", 0) if m.get("mask") else 0
    group = heads // kvh
    prob = torch.zeros(heads, t, t, dtype=F)
    for h in range(heads):
        s = (q[:, h] @ k[:, h // group].T) * m["scale"] * temp[h]
        for i in range(t):
            lo = (i // size) * size if size else 0
            row = torch.full((t,), -math.inf, dtype=F)
            row[lo:i + 1] = s[i, lo:i + 1]
            prob[h, i] = torch.softmax(row, -1)
    mixed = torch.einsum("hg,gij->hij", talk, prob)
    out = torch.stack([mixed[h] @ v[:, h // group] for h in range(heads)], dim=1)        # [t, heads, vdim]
    y = out.reshape(t, heads * vdim) @ _w(weights, p + "o").T + _w(weights, p + "o.b")
    return y, v


def mlstm(x, weights, p, m, eps):
    t = x.shape[0]
    heads, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (x @ _w(weights, p + "q").T).view(t, heads, dim) * dim ** -0.5
    k = (x @ _w(weights, p + "k").T).view(t, heads, dim)
    v = (x @ _w(weights, p + "v").T).view(t, heads, vdim)
    gi = cap * torch.tanh((x @ _w(weights, p + "i").T + _w(weights, p + "i.b")) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((x @ _w(weights, p + "f").T + _w(weights, p + "f.b")) / cap))
    out = torch.zeros(t, heads, vdim, dtype=F)
    for h in range(heads):
        S, n, mx = torch.zeros(dim, vdim, dtype=F), torch.zeros(dim, dtype=F), 0.0
        for s in range(t):
            new = max(float(gf[s, h]) + mx, float(gi[s, h]))
            keep, take = math.exp(float(gf[s, h]) + mx - new), math.exp(float(gi[s, h]) - new)
            S = keep * S + take * torch.outer(k[s, h], v[s, h])
            n = keep * n + take * k[s, h]
            mx = new
            out[s, h] = (S.T @ q[s, h]) / (max(abs(float(n @ q[s, h])), math.exp(-mx)) + 1e-6)
    y = rms_unit(out, eps).reshape(t, heads * vdim) * _w(weights, p + "norm")
    y = y * torch.sigmoid(x @ _w(weights, p + "g").T)
    return y @ _w(weights, p + "o").T


def dense_ff(x, weights, p):
    return gelu_tanh(x @ _w(weights, p + "up").T) @ _w(weights, p + "down").T


def experts_ff(x, weights, p, mlp):
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = x @ _w(weights, p + "router").T + _w(weights, p + "router.b")
    out = torch.zeros_like(x)
    for s in range(x.shape[0]):
        best = torch.topk(z[s], top)
        share = torch.softmax(best.values, -1)
        for w, e in zip(share.tolist(), best.indices.tolist()):
            pe = f"{p}e{e}."
            hid = torch.nn.functional.silu(x[s] @ _w(weights, pe + "gate").T) * (x[s] @ _w(weights, pe + "up").T)
            out[s] += w * (hid @ _w(weights, pe + "down").T)
    return out


def forward(weights, config, ids, streams=None):
    """Logits [tokens, vocab] of one sequence; `streams`, a list, receives what every layer hands on."""
    eps = float(config["norm"]["eps"])
    table = _w(weights, "embed")
    x = table[torch.tensor(list(ids))]
    history = [x]
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            y, v = block_attention(x, weights, p + "mix.", m, eps, v_first if m.get("v_mix") else None)
            if m.get("v_mix") and v_first is None:
                v_first = v
        elif layer["type"] == "mlstm":
            y = mlstm(x, weights, p + "mix.", m, eps)
        else:
            raise NotImplementedError(layer["type"])
        x = x + out_norm(y, _w(weights, p + "norm1"), eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, weights, p + "mlp.") if mlp["kind"] == "dense" else experts_ff(x, weights, p + "mlp.", mlp)
            x = x + out_norm(y, _w(weights, p + "norm2"), eps)
        history.append(x)
        c = _w(weights, p + "dwa")
        x = sum(c[j] * history[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x)
    return out_norm(x, _w(weights, "final.norm"), eps) @ table.T
