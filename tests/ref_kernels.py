"""Every kernel of the engine as plain torch code on the CPU, one function per kernel, same arguments.

Two uses. The `-m gpu` tests compare each CUDA kernel with its function here, at sizes of their own. And the
`-m "not gpu"` tests hand this table to the engine in place of the CUDA one, so that the host side (batch layout,
cache, scheduler) runs on a machine without a GPU. The product never loads this file; mxinO/holon keeps its CPU
oracle kernels test-only in the same way (testing/holon_testing/ref_kernels/plugin.py:24-35).
Formulas: std/holon_std/ops/reference.py:7-30, std/holon_std/mixers/gqa/reference.py:26-60 and 91-101,
std/holon_std/ffn/reference.py:7-12, std/holon_std/sampling/sampler.py:24-61.
"""
from __future__ import annotations

import torch

_M32 = 0xFFFFFFFF


def _mix32(x):
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & _M32
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & _M32
    return x ^ (x >> 16)


class RefKernels:
    name = "reference (torch, CPU)"

    def embed(self, out, table, ids):
        out.copy_(table[ids.long()].float())

    def rmsnorm(self, out, x, weight, eps, offset):
        x = x.float()
        out.copy_((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * (weight.float() + offset)).to(out.dtype))

    def add_rmsnorm(self, out, h, delta, weight, eps, offset, index):
        rows = slice(None) if index is None else index.long()
        v = h[rows] if delta is None else h[rows] + delta[rows].float()
        if index is None and delta is not None:
            h.copy_(v)
        self.rmsnorm(out, v, weight, eps, offset)

    def qk_norm_rope_kv_write(self, q_out, qkv, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                              write_index, heads, kv_heads, head_dim, bias=None):
        t, dt = qkv.shape[0], qkv.dtype
        if bias is not None:
            qkv = (qkv.float() + bias.float()).to(dt)
        q, k, v = qkv.split([heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], dim=-1)
        q, k, v = q.reshape(t, heads, head_dim), k.reshape(t, kv_heads, head_dim), v.reshape(t, kv_heads, head_dim)

        def prepare(x, weight):
            x = x.float()
            if weight is not None:
                x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * (weight.float() + offset)
                x = x.to(dt).float()
            if rotary_dim:
                half = rotary_dim // 2
                cs = table[positions.long()]
                cos, sin = cs[:, None, :half], cs[:, None, half:]
                a, b, rest = x[..., :half], x[..., half:rotary_dim], x[..., rotary_dim:]
                x = torch.cat((a * cos - b * sin, b * cos + a * sin, rest), dim=-1)
            return x.to(dt)

        q_out.copy_(prepare(q, q_weight))
        if kv is not None:
            k = prepare(k, k_weight)
            page_size = kv.shape[3]
            w = write_index.long()
            ok = w >= 0
            page, off = w[ok] // page_size, w[ok] % page_size
            kv[page, 0, :, off] = k[ok]
            kv[page, 1, :, off] = v[ok]

    def paged_attention(self, out, q, kv, block_table, rows, scale, window, sinks=None):
        page_size, hq, hkv = kv.shape[3], q.shape[1], kv.shape[2]
        out.zero_()
        qs, slots, lens = rows.query_start.tolist(), rows.row_slot.tolist(), rows.kv_len.tolist()
        for b in range(rows.n_rows):
            s, e, n = qs[b], qs[b + 1], lens[b]
            if n == 0 or s == e:
                continue
            pages = block_table[slots[b], : -(-n // page_size)].long()
            k, v = (kv[pages, i].transpose(1, 2).reshape(-1, hkv, kv.shape[4])[:n].float()
                    .repeat_interleave(hq // hkv, dim=1) for i in (0, 1))
            scores = torch.einsum("qhd,khd->hqk", q[s:e].float(), k) * scale
            pos = torch.arange(n - (e - s), n)[:, None]
            key = torch.arange(n)[None, :]
            hidden = key > pos
            if window > 0:
                hidden = hidden | (pos - key >= window)
            scores = scores.masked_fill(hidden, float("-inf"))
            if sinks is not None:                          # a weight in the denominator without key or value
                scores = torch.cat((scores, sinks.float()[:, None, None].expand(-1, e - s, 1)), -1)
            probs = scores.softmax(-1)[..., :n]
            out[s:e] = torch.einsum("hqk,khd->qhd", probs, v).to(out.dtype)

    def silu_mul(self, out, gate_up):
        gate, up = gate_up.float().chunk(2, dim=-1)
        out.copy_((torch.nn.functional.silu(gate) * up).to(out.dtype))

    def swiglu_gate_up(self, out, x, weight):
        gate_up = torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype)
        self.linear(gate_up, x, weight)
        self.silu_mul(out, gate_up)

    def linear(self, out, x, weight):
        out.copy_((x.float() @ weight.float().T).to(out.dtype))

    # ---- a block whose parts run side by side, an embedding with a pair table, mixers with a matrix state per head
    def embed_pair(self, out, table, scale, pair, ids, positions, rows, prev, mul_prev, mul_cur, buckets):
        ids_, pos = ids.tolist(), positions.tolist()
        qs, slots = rows.query_start.tolist(), rows.row_slot.tolist()
        x = table[ids.long()].float() * scale
        for b in range(rows.n_rows):
            for t in range(qs[b], qs[b + 1]):
                before = ids_[t - 1] if t > qs[b] else int(prev[slots[b]])
                if pair is not None:
                    r = buckets if pos[t] == 0 else (before * mul_prev + ids_[t] * mul_cur) % buckets
                    x[t] += pair[r].float()
            if prev is not None and qs[b + 1] > qs[b]:
                prev[slots[b]] = ids_[qs[b + 1] - 1]
        out.copy_(x)

    def sum_into(self, h, terms, bias=None):
        for x, scale in terms:
            h += scale * x.float()
        if bias is not None:
            h += bias.float()

    def sum_norm(self, h, terms, bias, out, weight, eps, offset):
        self.sum_into(h, terms, bias)
        self.rmsnorm(out, h, weight, eps, offset)

    def glu_clamped(self, out, gate_up, bias, limit, alpha):
        z = gate_up.float() + (bias.float() if bias is not None else 0.0)
        g, u = z.chunk(2, dim=-1)
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        out.copy_((g * torch.sigmoid(alpha * g) * (u + 1)).to(out.dtype))

    def recurrent_scan(self, out, qk, v, decay, head_decay, beta, state, rows, token_decay=None, rate=None):
        t, heads, vdim = v.shape
        group = heads // qk.shape[2]
        qs, slots = rows.query_start.tolist(), rows.row_slot.tolist()
        for b in range(rows.n_rows):
            for h in range(heads):
                s = state[slots[b], h].T.clone()               # (kept column by column: [vdim, dim])
                for i in range(qs[b], qs[b + 1]):
                    q, k = qk[i, 0, h // group], qk[i, 1, h // group]
                    if rate is not None:                       # the generalized rule: the removal reads the old state
                        s = s * decay[i, h][:, None] + torch.outer(k, v[i, h]) - torch.outer(rate[i, h] * k, s.T @ k)
                        out[i, h] = s.T @ q
                        continue
                    s = s * (decay[i, h][:, None] if decay is not None else
                             token_decay[i, h] if token_decay is not None else head_decay[h])
                    u = v[i, h] if beta is None else beta[i, h] * (v[i, h] - s.T @ k)
                    s = s + torch.outer(k, u)
                    out[i, h] = s.T @ q
                state[slots[b], h] = s.T

    def delta_prepare(self, qk, v, beta, decay, gate, first, conv, conv_state, low2, dt_bias, rate_log, rows, q_scale,
                      unit_eps):
        t, heads, vdim = v.shape
        kv_heads, dim = qk.shape[2], qk.shape[3]
        taps = conv.shape[1]
        nq, nv = kv_heads * dim, heads * vdim
        c = 2 * nq + nv
        x = first.float()
        y = torch.zeros(t, c)
        qs, slots = rows.query_start.tolist(), rows.row_slot.tolist()
        for b in range(rows.n_rows):
            s, e = qs[b], qs[b + 1]
            carried = conv_state[slots[b]].float() if taps > 1 else torch.zeros(0, c)
            seq = torch.cat((carried, x[s:e, :c]), 0)
            y[s:e] = sum(seq[j:j + e - s] * conv.float()[:, j] for j in range(taps))
        y = y * torch.sigmoid(y)
        unit = lambda z: z / torch.sqrt((z * z).sum(-1, keepdim=True) + unit_eps)      # noqa: E731
        qk[:, 0] = unit(y[:, :nq].view(t, kv_heads, dim)) * q_scale
        qk[:, 1] = unit(y[:, nq:2 * nq].view(t, kv_heads, dim))
        v.copy_(y[:, 2 * nq:].view(t, heads, vdim))
        beta.copy_(torch.sigmoid(x[:, c:c + heads]))
        a = low2[:, :heads * dim] + dt_bias
        decay.copy_(torch.exp(-torch.exp(rate_log)[None, :, None] * torch.nn.functional.softplus(a).view(t, heads, dim)))
        gate.copy_(torch.sigmoid(low2[:, heads * dim:]).view(gate.shape))

    def conv_carry(self, conv_state, first, channels, taps, rows):
        if taps <= 1:
            return
        qs, slots = rows.query_start.tolist(), rows.row_slot.tolist()
        for b in range(rows.n_rows):
            seq = torch.cat((conv_state[slots[b]], first[qs[b]:qs[b + 1], :channels]), 0)
            conv_state[slots[b]] = seq[-(taps - 1):]

    def retention_prepare(self, qk, v, first, positions, table, rot_dims, k_scale):
        t, heads, vdim = v.shape
        dim = qk.shape[3]
        x = first.float()
        for which in (0, 1):
            z = x[:, which * heads * dim:(which + 1) * heads * dim].view(t, heads, dim)
            if rot_dims:
                z = self._turn(z, table[positions.long()][:, None, :], rot_dims)
            qk[:, which] = z * (k_scale if which else 1.0)
        v.copy_(x[:, 2 * heads * dim:2 * heads * dim + heads * vdim].view(t, heads, vdim))

    def head_norm_gate(self, out, o, weight, gate_mul, gate_pre, eps, gate="silu"):
        y = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps)
        if weight is not None:                                 # one weight for all heads, or one per head and channel
            y = y * (weight.view(o.shape[1:]) if weight.numel() == o.shape[1] * o.shape[2] else weight)
        if gate_mul is not None:
            y = y * gate_mul.view(o.shape)
        elif gate_pre is not None:
            g = gate_pre.float().reshape(o.shape)
            y = y * (g * torch.sigmoid(g) if gate == "silu" else torch.sigmoid(g))
        out.copy_(y.to(out.dtype))

    def feed_tokens(self, token_ids, last_tokens, rows, from_last):
        for r in range(rows.n_rows):
            if int(from_last[r]):
                token_ids[int(rows.query_start[r])] = last_tokens[int(rows.row_slot[r])]

    def scatter_rows(self, table, slots, rows):
        table[slots.long()] = rows.view(slots.shape[0], table.shape[1])

    def store_tokens(self, last_tokens, slots, tokens, n):
        last_tokens[slots[:n].long()] = tokens[:n]

    def logprobs(self, chosen, top_ids, top, logits, tokens):
        """log softmax of the raw logits: the given token's, and the k most likely ranked (equal ones by ascending id)."""
        k = top.shape[1]
        for r in range(logits.shape[0]):
            lp = logits[r].double().log_softmax(-1)
            chosen[r] = lp[int(tokens[r])]
            order = torch.tensor(sorted(range(lp.numel()), key=lambda i: (-float(lp[i]), i))[:k], dtype=torch.long)
            top_ids[r] = order.to(torch.int32)
            top[r] = lp[order].float()

    def sample(self, tokens, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, position, filtered):
        """temperature 0: arg max. Else softmax(logits / T) filtered by top-k, top-p, min-p, drawn by inverse CDF in
        vocabulary order with the uniform of (seed, position)."""
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t == 0:
                tokens[r] = int(logits[r].argmax())
                continue
            x = logits[r].double() / t
            keep = torch.ones_like(x, dtype=torch.bool)
            if filtered:
                order = x.argsort(descending=True, stable=True)
                if int(top_k[r]) > 0:
                    keep[order[int(top_k[r]):]] = False
                q = torch.where(keep, x, float("-inf")).softmax(-1)
                if float(top_p[r]) < 1:
                    sq = q[order]
                    keep[order[sq.cumsum(-1) - sq > float(top_p[r])]] = False
                if float(min_p[r]) > 0:
                    keep &= q >= float(min_p[r]) * q.max()
            q = torch.where(keep, x, float("-inf")).softmax(-1)
            lo, hi, pos = int(seed_lo[r]) & _M32, int(seed_hi[r]) & _M32, int(position[r]) & _M32
            h = _mix32(_mix32(lo) ^ hi ^ _mix32(pos))
            u = min(float((torch.tensor(float(h >> 8), dtype=torch.float32) + 0.5) * 2.0 ** -24), 1 - 2.0 ** -24)
            c = q.cumsum(-1)
            i = int(torch.searchsorted(c, torch.tensor([u * float(c[-1])], dtype=c.dtype), right=True)[0])
            tokens[r] = min(i, q.numel() - 1)

    # ---- hyper-connections, latent attention, routed experts

    def hyper_mix_norm(self, out, xs, src, y, mix, outc, inc, weight, eps, offset, index):
        """Old streams: xs [T, S, H], or src [T, H] standing for every stream. New ones: Σ_s mix[s, t] old_s +
        outc[t] y (y None: the old ones). Without index they are written to xs. out = norm(Σ_t inc[t] new_t)."""
        rows = slice(None) if index is None else index.long()
        s = xs.shape[1]
        old = xs[rows] if src is None else src[rows][:, None, :].expand(-1, s, -1)
        new = old
        if y is not None:
            new = torch.einsum("st,nsh->nth", mix.float(), old) + outc.float()[None, :, None] * y[rows].float()[:, None, :]
        if index is None:
            xs.copy_(new)
        u = new.sum(1) if inc is None else torch.einsum("t,nth->nh", inc.float(), new)
        self.rmsnorm(out, u, weight, eps, offset)

    @staticmethod
    def _turn(x, cs, dims):
        half = dims // 2
        cos, sin = cs[..., :half], cs[..., half:]
        a, b, rest = x[..., :half], x[..., half:dims], x[..., dims:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin, rest), dim=-1)

    def latent_prepare(self, qa, first, heads, dim, rot, rank, dkv_at, positions, table, rot_dims, norm_weight, eps,
                       cache, write_index):
        t, dt = first.shape[0], first.dtype
        cs = table[positions.long()] if rot_dims else None
        q_r = first[:, :heads * (dim + rot)].view(t, heads, dim + rot)[:, :, dim:].float()
        if rot_dims:
            q_r = self._turn(q_r, cs[:, None, :], rot_dims)
        qa[:, :, rank:] = q_r.to(dt)
        if dkv_at >= 0:
            d = first[:, dkv_at:dkv_at + rank + rot].float()
            c = d[:, :rank]
            c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * norm_weight.float()
            k_r = d[:, rank:]
            if rot_dims:
                k_r = self._turn(k_r, cs, rot_dims)
            w = write_index.long()
            ok = w >= 0
            cache.view(-1, rank + rot)[w[ok]] = torch.cat((c, k_r), dim=-1).to(dt)[ok]

    def linear_heads(self, out, x, w):
        out.copy_(torch.einsum("tbk,bnk->tbn", x.float(), w.float()).to(out.dtype))

    def latent_attention(self, out, qa, cache, block_table, rows, scale, rank, window):
        page_size = cache.shape[1]
        out.zero_()
        qs, slots, lens = rows.query_start.tolist(), rows.row_slot.tolist(), rows.kv_len.tolist()
        for b in range(rows.n_rows):
            s, e, n = qs[b], qs[b + 1], lens[b]
            if n == 0 or s == e:
                continue
            pages = block_table[slots[b], : -(-n // page_size)].long()
            kc = cache[pages].reshape(-1, cache.shape[2])[:n].float()
            scores = torch.einsum("qhd,kd->hqk", qa[s:e].float(), kc) * scale
            pos = torch.arange(n - (e - s), n)[:, None]
            key = torch.arange(n)[None, :]
            hidden = key > pos
            if window > 0:
                hidden = hidden | (pos - key >= window)
            probs = scores.masked_fill(hidden, float("-inf")).softmax(-1)
            out[s:e] = torch.einsum("hqk,kd->qhd", probs, kc[:, :rank]).to(out.dtype)

    def sigmoid_gate(self, o, g):
        o.copy_((o.float() * torch.sigmoid(g.float())).to(o.dtype))

    def route_top(self, chosen, weight, counts, z, experts, scale, renormalize, bias=None, correction=None, groups=1,
                  keep=1, tiny=0.0):
        z = z[:, :experts].float() + (bias.float() if bias is not None else 0.0)
        s = torch.softmax(z, dim=-1)
        top = chosen.shape[1]
        choice = s + correction.float() if correction is not None else s.clone()
        if groups > 1:                                         # only experts of the best groups stay in the running
            best = choice.view(-1, groups, experts // groups).max(-1).values
            kept = torch.argsort(-best, dim=-1, stable=True)[:, :keep]
            allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
            choice = choice.masked_fill(~allowed.repeat_interleave(experts // groups, dim=1), float("-inf"))
        order = torch.argsort(-choice, dim=-1, stable=True)[:, :top]      # equal scores: the lower expert first
        w = torch.gather(s, 1, order)
        if renormalize:
            w = w / (w.sum(-1, keepdim=True) + tiny)
        chosen.copy_(order.to(torch.int32))
        weight.copy_(w * scale)
        counts[:experts] += torch.bincount(order.reshape(-1), minlength=experts).to(torch.int32)

    def route_rows(self, chosen, weight, counts, place, token_of, z, experts, scale, renormalize, bias=None,
                   correction=None, groups=1, keep=1, tiny=0.0):
        counts.zero_()
        self.route_top(chosen, weight, counts, z, experts, scale, renormalize, bias, correction, groups, keep, tiny)
        self.expert_rows(place, token_of, counts, chosen, experts)
        counts[2 * experts + 1], counts[2 * experts + 2] = 0, chosen.shape[0]

    def expert_rows(self, place, token_of, counts, chosen, experts):
        """counts[experts:] = first row of each expert and the end; pairs laid out expert by expert."""
        t, top = chosen.shape
        starts = torch.zeros(experts + 1, dtype=torch.int64)
        starts[1:] = torch.cumsum(counts[:experts].long(), 0)
        counts[experts:2 * experts + 1] = starts.to(torch.int32)
        order = torch.argsort(chosen.reshape(-1).long(), stable=True)
        place[order] = torch.arange(t * top, dtype=torch.int32)
        token_of.copy_((order // top).to(torch.int32))

    @staticmethod
    def _act(x, act, numbers=None):
        if act == 4:                                           # xielu with its two stored numbers
            sp = torch.nn.functional.softplus
            p, q = numbers.float()
            return torch.where(x > 0, sp(p) * x * x + 0.5 * x, (0.5 + sp(q)) * (torch.expm1(x) - x) + 0.5 * x)
        if act == 5:
            return torch.tanh(x)
        if act == 1:
            return torch.relu(x) ** 2
        if act == 2:
            return torch.nn.functional.silu(x)
        if act == 3:
            return torch.nn.functional.gelu(x, approximate="tanh")
        return x

    def expert_linear(self, out, x, token_of, w, starts, act):
        st = starts.tolist()
        for e in range(w.shape[0]):
            a, b = st[e], st[e + 1]
            if b > a:
                rows = x[token_of[a:b].long()] if token_of is not None else x[a:b]
                out[a:b] = self._act(rows.float() @ w[e].float().T, act).to(out.dtype)

    def activation(self, x, act, numbers=None):
        x.copy_(self._act(x.float(), act, numbers).to(x.dtype))

    def expert_combine(self, out, y, place, weight, shared, z, experts, x=None, identity_from=None):
        t, top = weight.shape
        acc = torch.zeros(out.shape, dtype=torch.float32)
        for k in range(top):
            rows = place.view(t, top)[:, k].long()
            term = y[rows].float()
            if x is not None:                                  # rows of identity experts: the token's input itself
                term = torch.where((rows >= int(identity_from[0]))[:, None], x.float(), term)
            acc += weight[:, k:k + 1] * term
        if shared is not None:
            acc += (torch.sigmoid(z[:, experts:experts + 1].float()) if z is not None else 1.0) * shared.float()
        out.copy_(acc.to(out.dtype))

    # ---- the matrix memory with exponential gates
    def mlstm_gates(self, out, pre, bias, cap, m_state, rows):
        heads = out.shape[2]
        a = pre[:, :2 * heads].float() + (bias.float() if bias is not None else 0.0)
        gi = cap * torch.tanh(a[:, :heads] / cap)
        gf = torch.nn.functional.logsigmoid(cap * torch.tanh(a[:, heads:] / cap))
        qs, slots = rows.query_start.tolist(), rows.row_slot.tolist()
        for b in range(rows.n_rows):
            m = m_state[slots[b]].clone()
            for i in range(qs[b], qs[b + 1]):
                new = torch.maximum(gf[i] + m, gi[i])
                out[0, i], out[1, i], out[2, i] = torch.exp(gf[i] + m - new), torch.exp(gi[i] - new), torch.exp(-new)
                m = new
            m_state[slots[b]] = m

    def mlstm_prepare(self, qk, v1, take, first, q_scale):
        t, _, heads, dim = qk.shape
        vdim = v1.shape[2] - 1
        f, nq = first.float(), heads * dim
        qk[:, 0] = f[:, :nq].view(t, heads, dim) * q_scale
        qk[:, 1] = f[:, nq:2 * nq].view(t, heads, dim) * take[:, :, None]
        v1[:, :, :vdim] = f[:, 2 * nq:2 * nq + heads * vdim].view(t, heads, vdim)
        v1[:, :, vdim] = 1.0

    def mlstm_read_out(self, out, o1, floor, weight, gate_pre, eps, tiny):
        t, heads, vdim = out.shape
        y = o1[:, :, :vdim] / (torch.maximum(o1[:, :, vdim].abs(), floor) + tiny)[:, :, None]
        y = y * torch.rsqrt((y * y).mean(-1, keepdim=True) + eps)
        y = y * weight.float().view(1, heads, vdim) * torch.sigmoid(gate_pre.float()).view(t, heads, vdim)
        out.copy_(y.to(out.dtype))

    # ---- a norm on a sublayer's output and the average over the layers' results
    def out_norm_add(self, dst, src, y, bias, weight, eps, offset, hist=None, n_hist=0, coef=None, avg=None, cast=None):
        x = src.float()
        if y is not None:
            z = y.float() + (bias.float() if bias is not None else 0.0)
            x = x + z * torch.rsqrt((z * z).mean(-1, keepdim=True) + eps) * (weight.float() + offset)
        if y is not None or dst.data_ptr() != src.data_ptr():
            dst.copy_(x)
        go = x
        if hist is not None:
            assert hist[n_hist - 1].data_ptr() == dst.data_ptr()
            go = torch.zeros_like(x)
            for j in range(n_hist - 1):
                go = go + coef[j] * hist[j]
            go = go + coef[n_hist - 1] * x
            avg.copy_(go)
        if cast is not None:
            cast.copy_(go.to(cast.dtype))

    # ---- attention whose heads share their weights after the softmax
    def qkv_talking_prepare(self, q_out, kv, keep, qkv, bias, q_weight, k_weight, eps, positions, table, rot_dims, interleaved,
                            first, blend, write_index, heads, kv_heads, key_dim, value_dim):
        t = qkv.shape[0]
        x = qkv.float() + (bias.float() if bias is not None else 0.0)
        nq, nk = heads * key_dim, kv_heads * key_dim
        q, k = x[:, :nq].view(t, heads, key_dim), x[:, nq:nq + nk].view(t, kv_heads, key_dim)
        v = x[:, nq + nk:].view(t, kv_heads, value_dim)

        def prepare(u, weight):
            if weight is not None:
                u = u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * weight.float()
            if rot_dims:
                cs = table[positions.long()]
                half = rot_dims // 2
                cos, sin = cs[:, None, :half], cs[:, None, half:]
                u = u.clone()
                if interleaved:
                    a, b = u[..., 0:rot_dims:2].clone(), u[..., 1:rot_dims:2].clone()
                    u[..., 0:rot_dims:2], u[..., 1:rot_dims:2] = a * cos - b * sin, b * cos + a * sin
                else:
                    a, b = u[..., :half].clone(), u[..., half:rot_dims].clone()
                    u[..., :half], u[..., half:rot_dims] = a * cos - b * sin, b * cos + a * sin
            return u

        q_out.copy_(prepare(q, q_weight).to(q_out.dtype))
        k = prepare(k, k_weight)
        if keep is not None:
            keep.copy_(v)
        if blend is not None:
            lam = float(blend)
            v = (1.0 - lam) * v + lam * first
        if kv is not None:
            page = kv.shape[2]
            w = write_index.long()
            ok = (w >= 0) & (w < (kv.shape[0] - 1) * page)
            rows = torch.cat((k, v), dim=-1).to(kv.dtype)
            for i in torch.nonzero(ok).flatten().tolist():
                kv[int(w[i]) // page, :, int(w[i]) % page] = rows[i]

    def attention_talking(self, out, q, kv, block_table, rows, scale, head_scale, chunk, window, talk):
        t, heads, kd = q.shape
        vd, kvh, page = out.shape[2], kv.shape[1], kv.shape[2]
        group = heads // kvh
        qs, slots, lens = rows.query_start.tolist(), rows.row_slot.tolist(), rows.kv_len.tolist()
        for b in range(rows.n_rows):
            n, s, e = lens[b], qs[b], qs[b + 1]
            pages = block_table[slots[b], :-(-n // page)].long()
            held = kv[pages].float().permute(1, 0, 2, 3).reshape(kvh, -1, kd + vd)[:, :n]      # [kvh, n, kd + vd]
            keys, values = held[..., :kd], held[..., kd:]
            for i in range(s, e):
                pos = n - e + i
                lo = (pos // chunk) * chunk if chunk else 0
                if window:
                    lo = max(lo, pos - window + 1)
                probs = torch.zeros(heads, pos + 1 - lo)
                for g in range(heads):
                    sc = (keys[g // group, lo:pos + 1] @ q[i, g].float()) * scale * (float(head_scale[g]) if head_scale is not None else 1.0)
                    probs[g] = torch.softmax(sc, -1)
                if talk is not None:
                    probs = talk.float() @ probs
                for h in range(heads):
                    out[i, h] = (probs[h] @ values[h // group, lo:pos + 1]).to(out.dtype)

    # ---- a norm without statistics, a token's rows blended with the token before's, the generalized delta rule
    @staticmethod
    def _dyt(x, triple):
        alpha, w, b = triple
        return torch.tanh(alpha.float() * x.float()) * w.float() + b.float()

    def dyt_add_norm(self, h, y, post, out, pre, index):
        """h += N_post(y) (y None: nothing is added; `h` None: `y` itself is the input of N_pre); out = N_pre(rows)."""
        if h is None:
            out.copy_(self._dyt(y, pre).to(out.dtype))
            return
        rows = slice(None) if index is None else index.long()
        v = h[rows] if y is None else h[rows] + self._dyt(y[rows], post)
        if index is None and y is not None:
            h.copy_(v)
        if out is not None:
            out.copy_(self._dyt(v, pre).to(out.dtype))

    def dyt_shift(self, out, into, h, y, post, pre, mix, carried, rows):
        v = h if y is None else h + self._dyt(y, post)
        n = self._dyt(v, pre)
        qs, slots = rows.query_start.tolist(), rows.row_slot.tolist()
        for b in range(rows.n_rows):
            s, e = qs[b], qs[b + 1]
            if e == s:
                continue
            before = torch.cat((carried[slots[b]][None].float(), n[s:e - 1]), 0)
            out[s:e] = (n[s:e] + (before - n[s:e]) * mix.float()).to(out.dtype)
            carried[slots[b]] = n[e - 1]
        into.copy_(v)

    def gdelta_prepare(self, qk, v, decay, rate, first, pre, decay_bias, rate_bias, decay_scale, unit_eps):
        t, heads, dim = v.shape
        n = heads * dim
        x = first.float()
        r, k = x[:, :n].view(t, heads, dim), x[:, n:2 * n].view(t, heads, dim)
        qk[:, 0], qk[:, 1] = r, k
        v.copy_(x[:, 2 * n:3 * n].view(t, heads, dim))
        decay.copy_(torch.exp(-decay_scale * torch.sigmoid(pre.float() + decay_bias)).view(t, heads, dim))
        a = torch.sigmoid(x[:, 4 * n:5 * n] + rate_bias).view(t, heads, dim)
        rate.copy_(a / ((k * k).sum(-1, keepdim=True) + unit_eps))
