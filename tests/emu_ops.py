"""Slow torch stand-ins for the CUDA kernels, for tests that run without a GPU.

They have the signatures of ``rust_inference_b200.ops`` and exist only so that
the host logic of the engine (packing, cache, slots, generation loop, trace
replay) can be exercised on the CPU.  They are no part of the product: the
package never imports this file, and on a GPU the tests use the real kernels.
"""
from __future__ import annotations

import math

import numpy as np
import torch

__all__ = ["embed", "rmsnorm", "add_rows", "silu_mul", "linear_swiglu", "linear", "qk_norm_rope_append", "attention", "argmax",
           "sample", "mark_seen", "stream_norm", "activation", "gate_heads", "linear_heads", "latent_prep", "gla_recurrent",
           "head_norm_gate", "linear_act", "scale_", "embed_pair_hash", "short_conv", "delta_rule_recurrent", "gated_act",
           "linear_gated", "moe_route", "moe_plan", "moe_grouped_linear", "moe_combine", "rms_gains", "qkv_prep", "softcap_",
           "embed_same", "mlstm_gates", "scalar_decay_recurrent", "mlstm_head_norm_gate"]


def embed(ids, table, scale=1.0, copies=1):
    x = table[ids.long()].float() * scale
    return x if copies == 1 else x[:, None, :].repeat(1, copies, 1)


def stream_norm(resid, gain, eps, out_dtype, kind="layernorm", delta=None, mix=None, out_w=None, read=None, rows=None,
                bias=None, more=()):
    n, S, dim = resid.shape
    x = resid if rows is None else resid[rows.long()]
    if delta is not None:
        m = torch.eye(S) if mix is None else mix
        x = torch.einsum("st,nsd->ntd", m, x)
        for y, w in [(delta, out_w)] + list(more):
            y = (y if rows is None else y[rows.long()]).float()
            o = torch.ones(S) if w is None else w
            x = x + o[None, :, None] * y[:, None, :]
        if rows is None:
            resid.copy_(x)
    r = torch.ones(S) if read is None else read
    u = torch.einsum("s,nsd->nd", r, x)
    b = 0.0 if bias is None else bias
    if kind == "layernorm":
        mu = u.mean(-1, keepdim=True)
        var = ((u - mu) ** 2).mean(-1, keepdim=True)
        return ((u - mu) / torch.sqrt(var + eps) * gain + b).to(out_dtype)
    return (u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * gain + b).to(out_dtype)


def activation(x, kind):
    f = x.float()
    if kind == "relu2":
        return (torch.clamp(f, min=0.0) ** 2).to(x.dtype)
    if kind == "gelu":
        return (0.5 * f * (1.0 + torch.erf(f / math.sqrt(2.0)))).to(x.dtype)
    return (0.5 * f * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (f + 0.044715 * f ** 3)))).to(x.dtype)


def linear_act(x, w, act):
    return activation(linear(x, w), act)


def _gate(z, fn):
    s = 1.0 / (1.0 + torch.exp(-z))
    return z * s if fn == "silu" else s


def gate_heads(x, g, fn="sigmoid"):
    tokens, heads, width = x.shape
    gz = _gate(g.float(), fn)
    gz = gz[:, :, None] if g.shape[1] == heads else gz.view(tokens, heads, width)
    x.copy_((x.float() * gz).to(x.dtype))
    return x


def linear_heads(x, w):
    return torch.einsum("thk,hnk->thn", x.double(), w.double()).to(x.dtype).contiguous()


def latent_prep(proj, q_col, dkv_col, qa, heads, dim, rot, rank, gain, eps, rope_table, pool, page_table, tok_seq, tok_pos,
                seq_slot, write=True):
    T = proj.shape[0]
    p = proj.float()

    def turn(v):                                   # [T, ..., rot]
        cs = rope_table[tok_pos.long()]
        shape = (T,) + (1,) * (v.dim() - 2) + (rot // 2,)
        c, s = cs[..., 0].view(shape), cs[..., 1].view(shape)
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)

    down = p[:, dkv_col:dkv_col + rank + rot]
    c = down[:, :rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * gain
    row = torch.cat([c, turn(down[:, rank:]) if rot else down[:, rank:]], dim=-1)
    if write:
        P = pool.shape[2]
        for t in range(T):
            pos = int(tok_pos[t])
            page = int(page_table[int(seq_slot[int(tok_seq[t])]), pos // P])
            assert page >= 0, "write to an unmapped page"
            pool[page, 0, pos % P, :] = row[t].to(pool.dtype)
    q = p[:, q_col:q_col + heads * (dim + rot)].view(T, heads, dim + rot)
    qr = turn(q[..., dim:]) if rot else q[..., dim:]
    return torch.cat([qa.float(), qr], dim=-1).to(proj.dtype).contiguous()


def gla_recurrent(proj, q_col, k_col, v_col, z, bias, tau, qscale, state, seq_slot, seq_start, heads, dim, vdim, single=False):
    T = proj.shape[0]
    p = proj.float()
    q = p[:, q_col:q_col + heads * dim].view(T, heads, dim) * qscale
    k = p[:, k_col:k_col + heads * dim].view(T, heads, dim)
    v = p[:, v_col:v_col + heads * vdim].view(T, heads, vdim)
    a = torch.exp(torch.nn.functional.logsigmoid(z.float() + bias) / tau).view(T, heads, dim)
    o = torch.zeros(T, heads, vdim)
    for b in range(seq_slot.numel()):
        S = state[int(seq_slot[b])]
        for t in range(int(seq_start[b]), int(seq_start[b + 1])):
            S.copy_(a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :])
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def head_norm_gate(o, gain, eps, g, out_dtype, fn="silu"):
    tokens, H, width = o.shape
    y = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * gain
    return (y * _gate(g.float(), fn).view(tokens, H, width)).view(tokens, H * width).to(out_dtype)


def rmsnorm(resid, gain, eps, out_dtype, delta=None, rows=None, then=None):
    if rows is not None:
        x = resid[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    else:
        if delta is not None:
            resid += delta.float()
        x = resid
    inv = 1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return (x * inv * gain).to(out_dtype)


def add_rows(resid, delta):
    resid += delta.float()


def silu_mul(gate_up, block=None):
    rows, two = gate_up.shape
    inter = two // 2
    block = block or inter
    v = gate_up.float().view(rows, inter // block, 2, block)
    g, u = v[:, :, 0, :].reshape(rows, inter), v[:, :, 1, :].reshape(rows, inter)
    return ((g / (1.0 + torch.exp(-g))) * u).to(gate_up.dtype)


def linear_swiglu(x, w_gate_up, block):
    return silu_mul(linear(x, w_gate_up), block)


def linear(x, w, out_dtype=None):
    y = x.double() @ w.double().t()
    return y.to(out_dtype or x.dtype)


def qk_norm_rope_append(qkv, num_heads, num_kv_heads, head_dim, q_gain, k_gain, eps, rope_table, rotary_dim, k_pool,
                        v_pool, page_table, tok_seq, tok_pos, seq_slot, write_kv=True, pairs=False):
    T = qkv.shape[0]
    H, KV, Dh = num_heads, num_kv_heads, head_dim
    x = qkv.float().view(T, H + 2 * KV, Dh)
    q, k, v = x[:, :H], x[:, H:H + KV], x[:, H + KV:]

    def norm(t, gain):
        if gain is None:
            return t
        return t * (1.0 / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)) * gain

    def rope(t):
        if rope_table is None:
            return t
        half = rotary_dim // 2
        cs = rope_table[tok_pos.long()]            # [T, half, 2]
        c, s = cs[:, None, :, 0], cs[:, None, :, 1]
        if pairs:
            a, b2 = t[..., 0:rotary_dim:2], t[..., 1:rotary_dim:2]
            turned = torch.stack([a * c - b2 * s, b2 * c + a * s], dim=-1).flatten(-2)
            return torch.cat([turned, t[..., rotary_dim:]], dim=-1)
        lo, hi, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
        return torch.cat([lo * c - hi * s, hi * c + lo * s, rest], dim=-1)

    q, k = rope(norm(q, q_gain)), rope(norm(k, k_gain))
    if write_kv:
        P = k_pool.shape[2]
        for t in range(T):
            pos = int(tok_pos[t])
            page = int(page_table[int(seq_slot[int(tok_seq[t])]), pos // P])
            assert page >= 0, "write to an unmapped page"
            k_pool[page, :, pos % P, :] = k[t].to(k_pool.dtype)
            v_pool[page, :, pos % P, :] = v[t].to(v_pool.dtype)
    return q.to(qkv.dtype).contiguous()


def attention(q, k_pool, v_pool, page_table, seq_slot, seq_start, seq_len, max_new, scale, window=0, sink=None, chunk=0,
              softcap=0.0):
    T, H, Dh = q.shape
    KV, P = k_pool.shape[1], k_pool.shape[2]
    G = H // KV
    out = torch.zeros_like(q, dtype=torch.float32)
    for b in range(seq_slot.numel()):
        t0, t1, n = int(seq_start[b]), int(seq_start[b + 1]), int(seq_len[b])
        slot = int(seq_slot[b])
        for t in range(t0, t1):
            pos = n - (t1 - t0) + (t - t0)
            first = max(0, pos - window + 1) if window > 0 else (pos - pos % chunk if chunk > 0 else 0)
            idx = torch.arange(first, pos + 1)
            pages = page_table[slot, (idx // P).long()].long()
            assert (pages >= 0).all(), "read from an unmapped page"
            kk = k_pool[pages, :, (idx % P).long(), :].float()      # [n, KV, Dh]
            vv = v_pool[pages, :, (idx % P).long(), :].float()
            for h in range(H):
                s = (kk[:, h // G, :] @ q[t, h].float()) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                if sink is None:
                    p = torch.softmax(s, dim=0)
                else:
                    p = torch.softmax(torch.cat([s, sink[h].view(1)]), dim=0)[:-1]
                out[t, h] = p @ vv[:, h // G, :]
    return out.to(q.dtype)


def argmax(logits):
    return torch.argmax(logits, dim=-1).to(torch.int32)      # torch returns the first maximum on the CPU


def sample(logits, temperature, uniform, top_k=None, top_p=None, penalty=None, seen=None, seen_rows=None,
           uses_top_k=True, uses_top_p=True):
    from plain_qwen3 import plain_sample

    class _Fixed:
        def __init__(self, u):
            self.u = u

        def next_f32(self):
            return np.float32(self.u)

    out = []
    for r in range(logits.shape[0]):
        hist = []
        pen = float(penalty[r]) if penalty is not None else 1.0
        if seen is not None and pen != 1.0:
            row = int(seen_rows[r]) if seen_rows is not None else r
            hist = torch.nonzero(seen[row]).flatten().tolist()
        out.append(plain_sample(logits[r].numpy(), hist, _Fixed(float(uniform[r])), temperature=float(temperature[r]),
                                top_k=int(top_k[r]) if top_k is not None else 0,
                                top_p=float(top_p[r]) if top_p is not None else 1.0, repetition_penalty=pen))
    return torch.tensor(out, dtype=torch.int32)


def mark_seen(seen, rows, tokens):
    seen[rows.long(), tokens.long()] = 1


# ---- the parts of the third architecture ------------------------------------------------------------------------------
def scale_(x, factor):
    x *= factor
    return x


def embed_pair_hash(ids, table, pairs, last_token, tok_seq, tok_pos, seq_slot, seq_start, mul_prev, mul_cur, single=False):
    T = ids.numel()
    buckets = pairs.shape[0] - 1
    out = torch.zeros(T, table.shape[1])
    for t in range(T):
        b = int(tok_seq[t])
        row = buckets
        if int(tok_pos[t]) > 0:
            prev = int(ids[t - 1]) if t > int(seq_start[b]) else int(last_token[int(seq_slot[b])])
            row = (prev * mul_prev + int(ids[t]) * mul_cur) % buckets
        out[t] = table[int(ids[t])].float() + pairs[row].float()
    for b in range(seq_slot.numel()):
        if int(seq_start[b + 1]) > int(seq_start[b]):
            last_token[int(seq_slot[b])] = ids[int(seq_start[b + 1]) - 1]
    return out


def short_conv(x, col0, weight, state, tok_seq, seq_slot, seq_start, single=False, weight_t=None):
    C, taps = weight.shape
    xin = x[:, col0:col0 + C].float()
    y = torch.zeros(x.shape[0], C)
    for b in range(seq_slot.numel()):
        t0, t1 = int(seq_start[b]), int(seq_start[b + 1])
        hist = torch.cat([state[int(seq_slot[b])], xin[t0:t1]], dim=0)          # [taps-1 + n, C]
        for i in range(t1 - t0):
            y[t0 + i] = (hist[i:i + taps] * weight.t()).sum(0)
        if taps > 1:
            state[int(seq_slot[b])] = hist[hist.shape[0] - (taps - 1):]
    return y / (1.0 + torch.exp(-y))


def delta_rule_recurrent(qkv, q_col, k_col, v_col, proj, beta_col, z, dt_bias, a_log, qscale, state, seq_slot, seq_start,
                         heads, qk_heads, dim, vdim, single=False):
    T = qkv.shape[0]
    rep = heads // qk_heads
    q = qkv[:, q_col:q_col + qk_heads * dim].view(T, qk_heads, dim)
    k = qkv[:, k_col:k_col + qk_heads * dim].view(T, qk_heads, dim)
    q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * qscale).repeat_interleave(rep, dim=1)
    k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(rep, dim=1)
    v = qkv[:, v_col:v_col + heads * vdim].view(T, heads, vdim)
    beta = torch.sigmoid(proj[:, beta_col:beta_col + heads].float())
    g = torch.exp(-torch.exp(a_log)[None, :, None] * torch.nn.functional.softplus((z.float() + dt_bias).view(T, heads, dim)))
    o = torch.zeros(T, heads, vdim)
    for b in range(seq_slot.numel()):
        S = state[int(seq_slot[b])]
        for t in range(int(seq_start[b]), int(seq_start[b + 1])):
            S.mul_(g[t][:, :, None])
            u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
            S.add_(k[t][:, :, None] * u[:, None, :])
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def gated_act(gate_up, kind, block=None, limit=0.0, alpha=1.0):
    rows, two = gate_up.shape
    inter = two // 2
    block = block or inter
    v = gate_up.float().view(rows, inter // block, 2, block)
    g, u = v[:, :, 0, :].reshape(rows, inter), v[:, :, 1, :].reshape(rows, inter)
    if kind == "silu":
        r = g * torch.sigmoid(g) * u
    elif kind == "gelu_tanh":
        r = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3))) * u
    else:
        g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
        r = g * torch.sigmoid(alpha * g) * (u + 1.0)
    return r.to(gate_up.dtype)


def linear_gated(x, w_gate_up, block, kind="silu", limit=0.0, alpha=1.0):
    return gated_act(linear(x, w_gate_up), kind, block, limit, alpha)


def moe_route(x, router, correction, top, score="softmax", groups=1, keep=1, group_top=2, scale=1.0, renormalize=True):
    z = x.float() @ router.t()
    s = torch.softmax(z, dim=-1) if score == "softmax" else torch.sigmoid(z)
    c = s + correction
    if groups > 1:
        T, N = c.shape
        size = N // groups
        gs = torch.topk(c.view(T, groups, size), min(group_top, size), dim=-1).values.sum(-1)
        kept = torch.zeros(T, groups, dtype=torch.bool)
        for _ in range(keep):
            at = torch.argmax(gs, dim=-1)
            kept[torch.arange(T), at] = True
            gs[torch.arange(T), at] = -math.inf
        c = torch.where(kept[:, :, None].expand(T, groups, size).reshape(T, N), c, torch.full_like(c, -math.inf))
    idx = torch.zeros(x.shape[0], top, dtype=torch.int32)
    for j in range(top):
        at = torch.argmax(c, dim=-1)                    # the first of equals
        idx[:, j] = at.to(torch.int32)
        c[torch.arange(x.shape[0]), at] = -math.inf
    w = torch.gather(s, 1, idx.long())
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx, w * scale


def moe_plan(idx, experts, wide=False):
    flat = idx.flatten()
    perm = torch.tensor([p for e in range(experts) for p in torch.nonzero(flat == e).flatten().tolist()], dtype=torch.int32)
    tiles = torch.tensor([[e, 0, 0] for e in range(experts)], dtype=torch.int32)
    off = 0
    for e in range(experts):
        n = int((flat == e).sum())
        tiles[e, 1], tiles[e, 2] = off, n
        off += n
    return perm, tiles, torch.tensor([experts, off], dtype=torch.int32), 0


def moe_grouped_linear(a, w, plan, rows_out, gather_div=0, scatter=False, out_dtype=None):
    perm, tiles, meta, _ = plan
    y = torch.zeros(rows_out, w.shape[1], dtype=out_dtype or a.dtype)
    for e, r0, n in tiles[:int(meta[0])].tolist():
        for r in range(r0, r0 + n):
            src = int(perm[r]) // gather_div if gather_div > 0 else r
            dst = int(perm[r]) if scatter else r
            y[dst] = (w[e].double() @ a[src].double()).to(y.dtype)
    return y


def moe_combine(pair_out, idx, weight, x, experts, extra=None):
    T, D = x.shape
    top = idx.shape[1]
    y = torch.zeros(T, D)
    for j in range(top):
        ident = (idx[:, j] >= experts)[:, None]
        v = torch.where(ident, x.float(), pair_out.view(T, top, D)[:, j])
        y += weight[:, j:j + 1] * v
    if extra is not None:
        y += extra.float()
    return y.to(x.dtype)


def rms_gains(resid, gains, eps, out_dtype, terms=(), entry=None, rows=None, then=None, post=None, out=None):
    x = resid if rows is None else resid[rows.long()]
    terms = list(terms)
    if terms:
        ys = [(y if rows is None else y[rows.long()]).float() * (1.0 if w is None else w[0]) for y, w in terms]
        total = ys[0] if len(ys) == 1 else ys[0] + ys[1]
        if post is not None and post[0] is not None:
            total = total / torch.sqrt((total * total).mean(-1, keepdim=True) + post[1]) * post[0]
        x = x + total
    if entry is not None:
        if entry.ids is not None:
            x = x + entry.table[entry.ids.long()].float() * entry.scale
        if entry.vec is not None:
            x = x + entry.vec
    if rows is None and (terms or entry is not None):
        resid.copy_(x)
    if not gains:
        if out is not None:
            out.copy_(x.to(out_dtype))
        return ()
    r = 1.0 / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return tuple((x * r * g).to(out_dtype) for g in gains)


def embed_same(ids, table, out):
    out.copy_(table[ids.long()])


def mlstm_gates(proj, i_col, f_col, i_bias, f_bias, cap, m_state, seq_slot, seq_start, heads, single=False):
    p = proj.float()
    li = cap * torch.tanh((p[:, i_col:i_col + heads] + i_bias) / cap)
    lf = torch.nn.functional.logsigmoid(cap * torch.tanh((p[:, f_col:f_col + heads] + f_bias) / cap))
    gates = torch.zeros(proj.shape[0], heads, 3)
    for b in range(seq_slot.numel()):
        m = m_state[int(seq_slot[b])]
        for t in range(int(seq_start[b]), int(seq_start[b + 1])):
            m_new = torch.maximum(lf[t] + m, li[t])
            gates[t, :, 0] = torch.exp(lf[t] + m - m_new)
            gates[t, :, 1] = torch.exp(li[t] - m_new)
            gates[t, :, 2] = torch.exp(-m_new)
            m.copy_(m_new)
    return gates


def scalar_decay_recurrent(proj, q_col, k_col, v_col, gates, qscale, state, seq_slot, seq_start, heads, dim, vdim, ones=True,
                           single=False):
    T = proj.shape[0]
    p = proj.float()
    q = p[:, q_col:q_col + heads * dim].view(T, heads, dim) * qscale
    k = p[:, k_col:k_col + heads * dim].view(T, heads, dim)
    v = p[:, v_col:v_col + heads * vdim].view(T, heads, vdim)
    if ones:
        v = torch.cat([v, torch.ones(T, heads, 1)], dim=-1)
    o = torch.zeros(T, heads, v.shape[-1])
    for b in range(seq_slot.numel()):
        S = state[int(seq_slot[b])]
        for t in range(int(seq_start[b]), int(seq_start[b + 1])):
            S.copy_(gates[t, :, 0, None, None] * S + (gates[t, :, 1, None] * k[t])[:, :, None] * v[t][:, None, :])
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def mlstm_head_norm_gate(o, gates, gain, eps, g, out_dtype):
    tokens, H, wide = o.shape
    vdim = wide - 1
    den = torch.maximum(o[..., vdim].abs(), gates[..., 2]) + 1e-6
    h = o[..., :vdim] / den[..., None]
    y = h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps)
    return (y.reshape(tokens, H * vdim) * gain * torch.sigmoid(g.float())).to(out_dtype)


def qkv_prep(proj, q_col, k_col, v_col, heads, kv_heads, Dp, Dk, bias, rope_table, rot, pairs, unit, eps, k_pool, v_pool,
             page_table, tok_seq, tok_pos, seq_slot, write_kv=True, norm="", q_gain=None, k_gain=None, norm_eps=0.0):
    T = proj.shape[0]
    x = proj.float()
    if bias is not None:
        x = x.clone()
        x[:, :bias.numel()] += bias
    q = x[:, q_col:q_col + heads * Dp].reshape(T, heads, Dp)
    k = x[:, k_col:k_col + kv_heads * Dp].reshape(T, kv_heads, Dp)
    v = None if v_col < 0 else x[:, v_col:v_col + kv_heads * Dp].reshape(T, kv_heads, Dp)

    def turn(t):
        if rope_table is None or not rot:
            return t
        cs = rope_table[tok_pos.long()]
        c, s = cs[:, None, :, 0], cs[:, None, :, 1]
        if pairs:
            a, b = t[..., 0:rot:2], t[..., 1:rot:2]
            return torch.cat([torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2), t[..., rot:]], dim=-1)
        half = rot // 2
        lo, hi = t[..., :half], t[..., half:rot]
        return torch.cat([lo * c - hi * s, hi * c + lo * s, t[..., rot:]], dim=-1)

    def unit_rms(t):
        return t / torch.sqrt((t * t).sum(-1, keepdim=True) / Dk + eps) if unit else t

    def normed(t, gain):
        if norm == "head":
            return t / torch.sqrt((t * t).sum(-1, keepdim=True) / Dk + norm_eps) * gain
        if norm == "all":
            return t / torch.sqrt((t * t).sum((-1, -2), keepdim=True) / (Dk * t.shape[1]) + norm_eps) * gain
        return t

    q, k = unit_rms(turn(normed(q, q_gain))), unit_rms(turn(normed(k, k_gain)))
    if write_kv:
        P = k_pool.shape[2]
        for t in range(T):
            pos = int(tok_pos[t])
            page = int(page_table[int(seq_slot[int(tok_seq[t])]), pos // P])
            assert page >= 0, "write to an unmapped page"
            k_pool[page, :, pos % P, :] = k[t].to(k_pool.dtype)
            if v is not None:
                v_pool[page, :, pos % P, :] = v[t].to(v_pool.dtype)
    return q.to(proj.dtype).contiguous()


def softcap_(x, cap):
    if cap:
        x.copy_(cap * torch.tanh(x / cap))
    return x
