"""Small Kagatar configurations and weights for the tests, and the comparison with the plain model.

The configurations differ from each other in every size and option.  A: the first two layers repeated three times, all
three mixers, keys larger than values and values larger than keys, head sizes that are padded, a layer without
feed-forward, frequencies slowed by wavelength on a part of a head, short windows.  B: no repeated run, no cap on the
logits, no factor on the embedding but 1, a width that is no multiple of 8, a window of one key, rotation of a whole
head with plain frequencies, one head, a gated layer with a window.  C: head sizes of 64 and 128 (the tensor-core
kernels), windows of exactly a page and of several, a run of one layer repeated twice at the end, YaRN.

Weights are made here, with activations of order one (so that attention is far from uniform and a window's edge, a
missing bias or a lost entry term shows), rounded to bfloat16 and stored as bfloat16.
"""
from __future__ import annotations

import json
import os

import numpy as np

import plain_kagatar
import plain_qwen3


def _mixer(heads, kv, dim, vdim, scale=None, window=None, rot=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = rot
    if softcap:
        m["softcap"] = softcap
    return m


def _layer(kind, mixer, ff, limit=2.0):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


CFG_A = {
    "architecture": "Kagatar", "vocab": 101, "width": 40, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "logit_softcap": 12.0, "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        _layer("attention_3", _mixer(6, 2, 24, 40, scale=0.9, window=9, softcap=5.0,
                                     rot={"base": 200.0, "dims": 10,
                                          "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 16}}), 56),
        _layer("attention", _mixer(4, 4, 12, 12, window=33), None),
        _layer("attention_2", _mixer(2, 1, 16, 8, rot={"base": 5000.0, "dims": 16,
                                                      "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 2.0}}),
               72, limit=0.75),
    ],
}
CFG_B = {
    "architecture": "Kagatar", "vocab": 131, "width": 52, "embedding": {"scale": 1.0}, "norm": {"eps": 2e-6},
    "layers": [
        _layer("attention", _mixer(3, 1, 20, 20, window=1), 44),
        _layer("attention_2", _mixer(1, 1, 10, 30, window=20, rot={"base": 50.0, "dims": 10}), 100, limit=1.0),
        _layer("attention_3", _mixer(4, 4, 6, 6, scale=1.5, softcap=50.0, rot={"base": 1000.0, "dims": 6}), None),
        _layer("attention", _mixer(2, 2, 34, 34), 36),
    ],
}
CFG_C = {
    "architecture": "Kagatar", "vocab": 300, "width": 128, "embedding": {"scale": 7.0}, "norm": {"eps": 1e-6},
    "logit_softcap": 25.0, "loop": {"start": 2, "stop": 3, "times": 2},
    "layers": [
        _layer("attention_2", _mixer(4, 2, 128, 128, rot={"base": 100000.0, "dims": 32,
                                                         "scaling": {"factor": 16.0, "original": 64, "fast": 16.0, "slow": 1.0}}), 96),
        _layer("attention", _mixer(4, 1, 64, 64, window=32), 160),
        _layer("attention_3", _mixer(2, 2, 64, 64, scale=0.7, window=70, softcap=8.0,
                                     rot={"base": 1000.0, "dims": 64,
                                          "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 48}}), 64),
    ],
}
ALL = {"A": CFG_A, "B": CFG_B, "C": CFG_C}


def _bf16(a):
    return plain_qwen3.bf16_round(np.asarray(a, dtype=np.float32)).astype(np.float32)


def make_weights(config, seed):
    """name -> float32 array (every value a bfloat16 number)."""
    rng = np.random.default_rng(seed)
    D = config["width"]
    W = {}

    def mat(name, n_out, n_in, gain=1.0):
        W[name] = _bf16(rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in))

    def vec(name, n, lo, hi):
        W[name] = _bf16(rng.uniform(lo, hi, size=n))

    W["embed"] = _bf16(rng.standard_normal((config["vocab"], D)) * 0.5)
    vec("final.norm", D, 0.7, 1.3)
    loop = config.get("loop")
    if loop and loop["stop"] > loop["start"]:
        W["loop.step"] = _bf16(rng.standard_normal((loop["times"], D)) * 0.7)
    for i, layer in enumerate(config["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        vec(p + "norm1", D, 0.7, 1.3)
        H, G, d = m["heads"], m["kv_heads"], m["dim"]
        dv = d if kind == "attention" else m["vdim"]
        # sharp scores: attention far from uniform, unless the heads are made unit vectors anyway
        mat(p + "mix.q", H * d, D, 3.0)
        mat(p + "mix.k", G * d, D, 2.0)
        vec(p + "mix.q.b", H * d, -0.5, 0.5)
        vec(p + "mix.k.b", G * d, -0.5, 0.5)
        if kind != "attention":
            mat(p + "mix.v", G * dv, D)
            vec(p + "mix.v.b", G * dv, -0.5, 0.5)
        if kind == "attention_2":
            mat(p + "mix.g", H * dv, D, 2.0)
        mat(p + "mix.o", D, H * dv)
        if layer["mlp"]:
            vec(p + "norm2", D, 0.7, 1.3)
            mat(p + "mlp.gate", layer["mlp"]["ff"], D, 2.0)
            mat(p + "mlp.up", layer["mlp"]["ff"], D, 2.0)
            mat(p + "mlp.down", D, layer["mlp"]["ff"])
    return W


def write_model(folder, config, weights):
    """config.json and model.safetensors (bfloat16) in ``folder``."""
    import torch
    from rust_inference_b200.weights.safetensors_io import save_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    save_safetensors(os.path.join(folder, "model.safetensors"),
                     {k: torch.from_numpy(np.ascontiguousarray(v)).to(torch.bfloat16) for k, v in weights.items()})
    return folder


def make_model_dir(base, name, seed=1):
    config = ALL[name]
    weights = make_weights(config, seed)
    return write_model(os.path.join(str(base), f"kagatar_{name}"), config, weights), config, weights


def plain_logits(config, weights, requests):
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    return {rid: plain_kagatar.forward(config, W, toks)[0] for rid, toks in requests.items()}


def row_error(got, want):
    """The difference of two rows of logits with the mean taken off, relative to the spread of the wanted row."""
    d = got.astype(np.float64) - want
    d = d - d.mean()
    w = want - want.mean()
    return float(np.sqrt((d * d).mean()) / max(np.sqrt((w * w).mean()), 1e-30))


# float32: rounding alone.  bfloat16: activations are rounded to 8 bits between the parts of every sublayer and the
# scores are sharp, so single rows are a few tenths off where a rounding tips a softmax; the mean over all rows is held
# much tighter (a wrong mechanism moves every row by about one).
BOUND = {"float32": (3e-5, 1e-5), "bfloat16": (6e-1, 6e-2)}


def assert_rows_close(rows, want_by_request, dtype, what=""):
    worst, total = 0.0, 0.0
    for (rid, p), got in sorted(rows.items()):
        err = row_error(got, want_by_request[rid][p])
        worst, total = max(worst, err), total + err
        assert err <= BOUND[dtype][0], f"{what}: request {rid} position {p}: error {err:.3e} exceeds {BOUND[dtype][0]:.1e}"
    mean = total / max(len(rows), 1)
    assert mean <= BOUND[dtype][1], f"{what}: mean error {mean:.3e} exceeds {BOUND[dtype][1]:.1e}"
    return round(worst, 7), round(mean, 7)
