"""Small Puratar configurations and weights for the tests, and the comparison with the plain model.

The configurations differ from each other in every size and option.  A: a run of two layers in the middle repeated three
times; values larger than keys and smaller than keys (head sizes that are padded, a per-head norm over a padded head); a
rotation of a part of a head, of a whole head and none; a layer without feed-forward; experts in three groups of which two
are kept, and a router without groups that takes one expert and has no shared expert; a memory of one head.  B: no
repeated run, no factor on the logits, a width that is no multiple of 8, one key/value head for all query heads, a memory
whose heads have more key channels than the register kernel takes, experts in two groups of which one is kept.  C: head
sizes of 64 and 128 (the tensor-core kernels and the vectorised preparation kernel), one layer at the start repeated
twice, a memory with 96 key channels.  D: sizes that are multiples of nothing.

Weights are made here, with activations of order one (so that attention is far from uniform and a missing norm, bias,
gate or entry term shows), rounded to bfloat16 and stored as bfloat16.
"""
from __future__ import annotations

import json
import os

import numpy as np

import plain_puratar
import plain_qwen3


def attn(heads, kv, dim, vdim, scale=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def memory(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, scale, ff, groups=None, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "router": r, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def single(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def double(left, right, ls, rs, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


CFG_A = {
    "architecture": "Puratar", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "logit_scale": 0.8,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        single(attn(4, 2, 24, 40, scale=0.9, rot=(300.0, 10)), moe(6, 3, 2.0, 24, groups=(3, 2), shared=40)),
        double(attn(2, 1, 12, 20, rot=(50.0, 12)), memory(3, 12, 20, 8.0), 0.7, 1.3, dense(56)),
        single(attn(3, 3, 16, 8), None),
        double(attn(4, 4, 8, 8, scale=0.5, rot=(1000.0, 4)), memory(1, 20, 12, 15.0), 1.2, 0.4, moe(4, 1, 0.75, 16)),
    ],
}
CFG_B = {
    "architecture": "Puratar", "vocab": 131, "width": 52, "norm": {"eps": 2e-6},
    "layers": [
        double(attn(3, 1, 20, 12, rot=(20.0, 20)), memory(2, 136, 24, 5.0), 1.0, 1.0, moe(8, 2, 1.0, 20, groups=(2, 1), shared=12)),
        single(attn(5, 1, 10, 30, rot=(7000.0, 6)), dense(100)),
        double(attn(2, 2, 34, 34), memory(4, 6, 6, 30.0), 0.3, 2.0, None),
    ],
}
CFG_C = {
    "architecture": "Puratar", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 1.5,
    "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        double(attn(2, 2, 128, 64, rot=(100000.0, 32)), memory(2, 96, 128, 10.0), 0.8, 0.6, moe(16, 4, 2.5, 32, groups=(4, 2), shared=64)),
        single(attn(4, 2, 64, 64, rot=(10000.0, 64)), dense(160)),
        single(attn(8, 1, 64, 128, scale=0.2, rot=(500.0, 16)), moe(4, 2, 1.0, 48, groups=(2, 2))),
    ],
}
# D: nothing is a multiple of 4: a width of 50, heads of 10 and 6 elements, seven heads, five experts; one layer in the
# middle repeated twice
CFG_D = {
    "architecture": "Puratar", "vocab": 83, "width": 50, "norm": {"eps": 3e-6}, "logit_scale": 0.6,
    "loop": {"start": 1, "stop": 2, "times": 2},
    "layers": [
        single(attn(7, 7, 10, 6, rot=(40.0, 6)), dense(30)),
        double(attn(3, 1, 14, 18, scale=0.3, rot=(900.0, 14)), memory(5, 10, 6, 3.0), 0.5, 0.5, moe(5, 2, 1.25, 14, shared=10)),
        single(attn(1, 1, 22, 22, rot=(10.0, 2)), moe(9, 3, 0.5, 10, groups=(3, 1))),
    ],
}
ALL = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}


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

    def attention(p, m, left):
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        mat(p + "q", H * d, D, 3.0)                      # sharp scores: attention far from uniform
        mat(p + "k", G * d, D, 2.0)
        mat(p + "v", G * dv, D)
        mat(p + "o", D, H * dv)
        if left:
            for name, n in (("q", H * d), ("k", G * d), ("v", G * dv)):
                vec(p + name + ".b", n, -0.5, 0.5)
            vec(p + "q.norm", H * d, 0.5, 2.0)
            vec(p + "k.norm", G * d, 0.5, 2.0)
        else:
            vec(p + "q.norm", d, 0.5, 2.0)
            vec(p + "k.norm", d, 0.5, 2.0)
            mat(p + "g", H, D, 3.0)

    def gated(p, ff):
        mat(p + "gate", ff, D, 2.0)
        mat(p + "up", ff, D, 2.0)
        mat(p + "down", D, ff)

    W["embed"] = _bf16(rng.standard_normal((config["vocab"], D)) * 0.5)
    vec("final.norm", D, -0.3, 0.3)
    loop = config.get("loop")
    if loop and loop["stop"] > loop["start"]:
        mat("loop.in", D, 2 * D, 1.5)
        W["loop.step"] = _bf16(rng.standard_normal((loop["times"], D)) * 0.7)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for name in ("norm1", "norm1b"):
            vec(p + name, D, -0.3, 0.3)
        vec(p + "ls1", D, 0.5, 1.5)
        if layer["type"] == "attention":
            attention(p + "mix.", m, left=False)
        else:
            attention(p + "mix.left.", m["left"], left=True)
            r, q = m["right"], p + "mix.right."
            H, d, dv = r["heads"], r["dim"], r["vdim"]
            mat(q + "q", H * d, D, 2.0)
            mat(q + "k", H * d, D, 2.0)
            mat(q + "v", H * dv, D)
            mat(q + "g", H * dv, D, 2.0)
            mat(q + "o", D, H * dv)
            vec(q + "norm", H * dv, 0.5, 1.5)
            mat(q + "i", H, D, 3.0)
            mat(q + "f", H, D, 3.0)
            vec(q + "i.b", H, -1.0, 1.0)
            vec(q + "f.b", H, 0.0, 4.0)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        for name in ("norm2", "norm2b"):
            vec(p + name, D, -0.3, 0.3)
        vec(p + "ls2", D, 0.5, 1.5)
        if mlp["kind"] == "dense":
            mat(p + "mlp.up", mlp["ff"], D, 2.0)
            mat(p + "mlp.down", D, mlp["ff"])
        else:
            E = mlp["router"]["experts"]
            W[p + "mlp.router"] = _bf16(rng.standard_normal((E, D)) * 2.0 / np.sqrt(D))
            vec(p + "mlp.correction", E, -0.4, 0.4)
            for e in range(E):
                gated(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            if mlp.get("shared"):
                gated(p + "mlp.shared.", mlp["shared"]["ff"])
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
    return write_model(os.path.join(str(base), f"puratar_{name}"), config, weights), config, weights


def plain_logits(config, weights, requests):
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    return {rid: plain_puratar.forward(config, W, toks)[0] for rid, toks in requests.items()}


def row_error(got, want):
    """The difference of two rows of logits with the mean taken off, relative to the spread of the wanted row."""
    d = got.astype(np.float64) - want
    d = d - d.mean()
    w = want - want.mean()
    return float(np.sqrt((d * d).mean()) / max(np.sqrt((w * w).mean()), 1e-30))


# float32: rounding alone.  bfloat16: activations are rounded to 8 bits between the parts of every sublayer, the scores
# are sharp and a router's choice can tip, so single rows are a few tenths off; the mean over all rows is held much
# tighter (a wrong mechanism moves every row by about one).
BOUND = {"float32": (1e-4, 2e-5), "bfloat16": (8e-1, 8e-2)}


def assert_rows_close(rows, want_by_request, dtype, what=""):
    worst, total = 0.0, 0.0
    for (rid, p), got in sorted(rows.items()):
        err = row_error(got, want_by_request[rid][p])
        worst, total = max(worst, err), total + err
        assert err <= BOUND[dtype][0], f"{what}: request {rid} position {p}: error {err:.3e} exceeds {BOUND[dtype][0]:.1e}"
    mean = total / max(len(rows), 1)
    assert mean <= BOUND[dtype][1], f"{what}: mean error {mean:.3e} exceeds {BOUND[dtype][1]:.1e}"
    return round(worst, 7), round(mean, 7)
