"""Puratar, plainly: numpy float64, one function per mechanism, token by token where that is the clearest form.

This is the yardstick of the tests and shares no code with the package.  Weights are a dict name -> float64 array
(linear weights [out, in]); ``config`` is the dict of config.json.

    x_0 = embed[token]
    a layer:     x <- x + ls1 * n1b(mixer(n1(x)));  x <- x + ls2 * n2b(ff(n2(x)))     n(x) = rms(x) * (1 + w)
    the loop:    layers start .. stop-1 run `times` times; before pass t: x <- W_in [x; x_0], then x += loop.step[t]
    the output:  logit_scale * embed n_final(x)
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces --------------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose tensor w holds the gain minus one."""
    return rms_unit(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return np.minimum(z, 0.0) - np.log1p(np.exp(-np.abs(z)))


def gelu_erf(z):
    return np.array([0.5 * v * (1.0 + math.erf(v / math.sqrt(2.0))) for v in np.ravel(z)]).reshape(np.shape(z))


def silu(z):
    return z * sigmoid(z)


# ---- rotation ---------------------------------------------------------------------------------------------------------
def rotate_halves(x, pos, base, dims):
    """x [..., dim] at position pos: element i < dims/2 and element i + dims/2 are turned by pos * base^(-2i/dims)."""
    y = np.array(x, dtype=np.float64, copy=True)
    half = dims // 2
    for i in range(half):
        a = pos * base ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        u, v = x[..., i], x[..., i + half]
        y[..., i] = u * c - v * s
        y[..., i + half] = v * c + u * s
    return y


def rotate_all(m, x, positions):
    rot = m.get("rot")
    if not rot or not rot.get("dims"):
        return x
    return np.stack([rotate_halves(x[t], positions[t], rot["base"], rot["dims"]) for t in range(x.shape[0])])


# ---- attention over explicit keys ---------------------------------------------------------------------------------------
def attend(q, k, v, scale):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; head h reads key/value head h // (H / G); position i sees
    every j <= i."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        for h in range(H):
            g = h // (H // G)
            s = (k[:i + 1, g] @ q[i, h]) * scale
            w = np.exp(s - s.max())
            out[i, h] = (w / w.sum()) @ v[:i + 1, g]
    return out


def mixer_attention(W, p, m, h, eps, positions=None):
    """Per-head RMS norm of queries and keys (one plain weight of the head's size for all heads), rotation, softmax
    attention, one sigmoid gate per head."""
    T = h.shape[0]
    positions = range(T) if positions is None else positions
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    k = (h @ W[p + "k"].T).reshape(T, G, d)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    q = rms_unit(q, eps) * W[p + "q.norm"]
    k = rms_unit(k, eps) * W[p + "k.norm"]
    q, k = rotate_all(m, q, positions), rotate_all(m, k, positions)
    y = attend(q, k, v, m["scale"])
    y = y * sigmoid(h @ W[p + "g"].T)[:, :, None]
    return y.reshape(T, H * dv) @ W[p + "o"].T


def mixer_left(W, p, m, h, eps, positions=None):
    """Biases on q, k, v; RMS norm over the whole projection (all heads at once) with a plain weight of that size."""
    T = h.shape[0]
    positions = range(T) if positions is None else positions
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ W[p + "q"].T + W[p + "q.b"]
    k = h @ W[p + "k"].T + W[p + "k.b"]
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv)
    q = (rms_unit(q, eps) * W[p + "q.norm"]).reshape(T, H, d)
    k = (rms_unit(k, eps) * W[p + "k.norm"]).reshape(T, G, d)
    q, k = rotate_all(m, q, positions), rotate_all(m, k, positions)
    return attend(q, k, v, m["scale"]).reshape(T, H * dv) @ W[p + "o"].T


def matrix_memory(q, k, v, li, lf, state=None):
    """One head of the matrix memory, token by token.  q, k [T, d], v [T, dv], li, lf [T] the log input and log forget
    gates.  ``state`` (S [d, dv], n [d], m) or None for a fresh one (zeros, m = 0).  Returns (o [T, dv], state)."""
    T, d = q.shape
    S, n, m = (np.zeros((d, v.shape[1])), np.zeros(d), 0.0) if state is None else state
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        m_new = max(lf[t] + m, li[t])
        a, b = math.exp(lf[t] + m - m_new), math.exp(li[t] - m_new)
        S = a * S + b * np.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        out[t] = (S.T @ q[t]) / (max(abs(n @ q[t]), math.exp(-m)) + 1e-6)
    return out, (S, n, m)


def mixer_right(W, p, m, h, eps):
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ W[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, d)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    li = cap * np.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    lf = log_sigmoid(cap * np.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    o = np.stack([matrix_memory(q[:, j], k[:, j], v[:, j], li[:, j], lf[:, j])[0] for j in range(H)], axis=1)
    o = rms_unit(o, eps).reshape(T, H * dv) * W[p + "norm"] * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def mixer_parallel(W, p, m, h, eps):
    return m["left_scale"] * mixer_left(W, p + "left.", m["left"], h, eps) + \
        m["right_scale"] * mixer_right(W, p + "right.", m["right"], h, eps)


# ---- feed-forwards ------------------------------------------------------------------------------------------------------
def ff_dense(W, p, h):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


def expert(W, p, h):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(z, correction, top, groups, keep, scale):
    """For one token's router logits z: (chosen experts, their weights)."""
    s = sigmoid(z)
    c = s + correction
    E = len(z)
    size = E // groups
    gscore = [np.sort(c[g * size:(g + 1) * size])[-2:].sum() for g in range(groups)]
    best = sorted(range(groups), key=lambda g: (-gscore[g], g))[:keep]
    masked = np.full(E, -np.inf)
    for g in best:
        masked[g * size:(g + 1) * size] = c[g * size:(g + 1) * size]
    chosen = sorted(range(E), key=lambda e: (-masked[e], e))[:top]
    return chosen, [s[e] * scale for e in chosen]


def ff_moe(W, p, mlp, h):
    r = mlp["router"]
    out = np.zeros_like(h)
    z = h @ W[p + "router"].T
    for t in range(h.shape[0]):
        groups = r.get("groups") or {"count": 1, "keep": 1}
        chosen, weights = route(z[t], W[p + "correction"], r["top"], groups["count"], groups["keep"], r["scale"])
        for e, w in zip(chosen, weights):
            out[t] += w * expert(W, f"{p}e{e}.", h[t:t + 1])[0]
    if mlp.get("shared") is not None:
        out = out + expert(W, p + "shared.", h)
    return out


# ---- the model -----------------------------------------------------------------------------------------------------------
def layer(config, W, i, x):
    rec, eps = config["layers"][i], config["norm"]["eps"]
    p = f"l{i}."
    h = norm_one_plus(x, W[p + "norm1"], eps)
    if rec["type"] == "attention":
        a = mixer_attention(W, p + "mix.", rec["mixer"], h, eps)
    elif rec["type"] == "parallel":
        a = mixer_parallel(W, p + "mix.", rec["mixer"], h, eps)
    else:
        raise ValueError(rec["type"])
    x = x + W[p + "ls1"] * norm_one_plus(a, W[p + "norm1b"], eps)
    mlp = rec.get("mlp")
    if mlp is None:
        return x
    h = norm_one_plus(x, W[p + "norm2"], eps)
    f = ff_dense(W, p + "mlp.", h) if mlp["kind"] == "dense" else ff_moe(W, p + "mlp.", mlp, h)
    return x + W[p + "ls2"] * norm_one_plus(f, W[p + "norm2b"], eps)


def forward(config, W, tokens):
    """(logits [T, vocab], residual after every layer run [runs, T, width])."""
    x0 = W["embed"][np.asarray(tokens)]
    x = x0.copy()
    n = len(config["layers"])
    loop = config.get("loop")
    start, stop, times = (loop["start"], loop["stop"], loop["times"]) if loop else (0, 0, 0)
    after = []
    for i in range(start):
        x = layer(config, W, i, x)
        after.append(x)
    for t in range(times if stop > start else 0):
        x = np.concatenate([x, x0], axis=1) @ W["loop.in"].T + W["loop.step"][t]
        for i in range(start, stop):
            x = layer(config, W, i, x)
            after.append(x)
    for i in range(stop, n):
        x = layer(config, W, i, x)
        after.append(x)
    z = norm_one_plus(x, W["final.norm"], config["norm"]["eps"]) @ W["embed"].T * config.get("logit_scale", 1.0)
    return z, np.stack(after)
