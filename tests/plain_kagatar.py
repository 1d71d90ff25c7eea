"""Kagatar, plainly: numpy float64, one function per mechanism, token by token where that is the clearest form.

This is the yardstick of the tests and shares no code with the package.  Weights are a dict name -> float64 array
(linear weights [out, in]); ``config`` is the dict of config.json.

    x_0 = embed[token] * embedding.scale
    a layer:     x <- x + mixer(rms(x) * norm1) + ff(rms(x) * norm2)
    the loop:    layers start .. stop-1 run `times` times; before pass t: x += x_0 (t > 0), then x += loop.step[t]
    the output:  cap * tanh(embed (rms(x) * final.norm) / cap)
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces --------------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, gain, eps):
    return rms_unit(x, eps) * gain


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def soft_cap(z, cap):
    return cap * np.tanh(z / cap)


# ---- rotation ---------------------------------------------------------------------------------------------------------
def plain_frequencies(base, dims):
    return np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)


def yarn_frequencies(base, dims, factor, original, fast, slow):
    """(frequencies, factor on cos and sin): a blend of f and f / factor along a ramp between two pair indices."""
    f = plain_frequencies(base, dims)

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = np.empty_like(f)
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def wavelength_frequencies(base, dims, factor, low, high, original):
    """Short waves keep their frequency, long ones are slowed by `factor`, those between are blended."""
    f = plain_frequencies(base, dims)
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            out[i] = fi
        elif wave > original / low:
            out[i] = fi / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_pairs(x, pos, freqs, mult=1.0):
    """x [..., dim] at position pos: elements (2i, 2i+1), i < len(freqs), are turned by pos * freqs[i]."""
    y = np.array(x, dtype=np.float64, copy=True)
    for i, f in enumerate(freqs):
        c, s = math.cos(pos * f) * mult, math.sin(pos * f) * mult
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        y[..., 2 * i] = u * c - v * s
        y[..., 2 * i + 1] = v * c + u * s
    return y


# ---- attention over explicit keys ---------------------------------------------------------------------------------------
def visible(i, window):
    """The keys that position i sees: itself and the window - 1 before it (window 0: all of 0 .. i)."""
    lo = 0 if not window else max(0, i - window + 1)
    return range(lo, i + 1)


def attend(q, k, v, scale, window=0, cap=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H * dv]; head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for i in range(T):
        js = visible(i, window)
        lo, hi = js[0], js[-1] + 1
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:hi, g] @ q[i, h]) * scale
            if cap:
                s = soft_cap(s, cap)
            w = np.exp(s - s.max())
            out[i, h] = (w / w.sum()) @ v[lo:hi, g]
    return out.reshape(T, -1)


def project(W, p, name, h, heads, size, bias=True):
    y = h @ W[p + name].T
    if bias:
        y = y + W[p + name + ".b"]
    return y.reshape(h.shape[0], heads, size)


def mixer_keys_as_values(W, p, m, h):
    """'attention': no rotation, the values are the keys, a window."""
    q = project(W, p, "q", h, m["heads"], m["dim"])
    k = project(W, p, "k", h, m["kv_heads"], m["dim"])
    y = attend(q, k, k, m["scale"], window=(m.get("mask") or {}).get("size", 0))
    return y @ W[p + "o"].T


def _rotated(m, q, k):
    rot = m.get("rot")
    if not rot or not rot.get("dims"):
        return q, k
    sc, dims, base = rot.get("scaling"), rot["dims"], rot["base"]
    mult = 1.0
    if sc is None:
        f = plain_frequencies(base, dims)
    elif "fast" in sc:
        f, mult = yarn_frequencies(base, dims, sc["factor"], sc["original"], sc["fast"], sc["slow"])
    else:
        f = wavelength_frequencies(base, dims, sc["factor"], sc["low"], sc["high"], sc["original"])
    q = np.stack([rotate_pairs(q[t], t, f, mult) for t in range(q.shape[0])])
    k = np.stack([rotate_pairs(k[t], t, f, mult) for t in range(k.shape[0])])
    return q, k


def mixer_gated(W, p, m, h):
    """'attention_2': rotation (YaRN), every earlier key (or a window, if the record has one), a sigmoid gate per output
    element."""
    q = project(W, p, "q", h, m["heads"], m["dim"])
    k = project(W, p, "k", h, m["kv_heads"], m["dim"])
    v = project(W, p, "v", h, m["kv_heads"], m["vdim"])
    q, k = _rotated(m, q, k)
    y = attend(q, k, v, m["scale"], window=(m.get("mask") or {}).get("size", 0))
    return (y * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def mixer_unit_capped(W, p, m, h, eps):
    """'attention_3': rotation, then unit-RMS queries and keys, capped scores, a window."""
    q = project(W, p, "q", h, m["heads"], m["dim"])
    k = project(W, p, "k", h, m["kv_heads"], m["dim"])
    v = project(W, p, "v", h, m["kv_heads"], m["vdim"])
    q, k = _rotated(m, q, k)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    y = attend(q, k, v, m["scale"], window=(m.get("mask") or {}).get("size", 0), cap=m.get("softcap"))
    return y @ W[p + "o"].T


def feed_forward(W, p, mlp, h):
    g = np.minimum(h @ W[p + "gate"].T, mlp["limit"])
    u = np.clip(h @ W[p + "up"].T, -mlp["limit"], mlp["limit"])
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def layer(config, W, i, x):
    rec, eps = config["layers"][i], config["norm"]["eps"]
    p = f"l{i}."
    h = rms_norm(x, W[p + "norm1"], eps)
    kind, m = rec["type"], rec["mixer"]
    if kind == "attention":
        a = mixer_keys_as_values(W, p + "mix.", m, h)
    elif kind == "attention_2":
        a = mixer_gated(W, p + "mix.", m, h)
    elif kind == "attention_3":
        a = mixer_unit_capped(W, p + "mix.", m, h, eps)
    else:
        raise ValueError(kind)
    if rec.get("mlp") is None:
        return x + a
    return x + (a + feed_forward(W, p + "mlp.", rec["mlp"], rms_norm(x, W[p + "norm2"], eps)))


def forward(config, W, tokens):
    """(logits [T, vocab], residual after every layer run [runs, T, width])."""
    x0 = W["embed"][np.asarray(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    x = x0.copy()
    n = len(config["layers"])
    loop = config.get("loop")
    start, stop, times = (loop["start"], loop["stop"], loop["times"]) if loop else (0, 0, 0)
    after = []
    for i in range(start):
        x = layer(config, W, i, x)
        after.append(x)
    for t in range(times if stop > start else 0):
        if t > 0:
            x = x + x0
        x = x + W["loop.step"][t]
        for i in range(start, stop):
            x = layer(config, W, i, x)
            after.append(x)
    for i in range(stop, n):
        x = layer(config, W, i, x)
        after.append(x)
    z = rms_norm(x, W["final.norm"], config["norm"]["eps"]) @ W["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        z = soft_cap(z, cap)
    return z, np.stack(after)
