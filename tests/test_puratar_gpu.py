"""Puratar on the GPU: each kernel against the plain formulas of tests/plain_puratar.py, then whole models through trace
replay in several cuttings (whole prompts; prompts then single tokens; prompts in portions down to two tokens; batches of
unequal requests that follow each other on the same slots and pages), in float32 and bfloat16, against the plain model."""
import math

import numpy as np
import pytest
import torch

import helpers as H
import plain_puratar as P
import puratar_models as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV, dtype)


def _i(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


def _np(t):
    return t.double().cpu().numpy()


def _close(got, want, dtype, what, tol32=2e-5, tol16=1.2e-2):
    got, want = _np(got), np.asarray(want, dtype=np.float64)
    tol = tol32 if dtype == torch.float32 else tol16
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, f"{what}: error {err:.3e} of the largest value exceeds {tol:.1e}"


# ---- a norm behind the sublayer, a layer scale, and the norm in front of the next one, in one pass ------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, n", [(52, 5), (48, 70), (3001, 9), (1, 3), (320, 33)])
def test_norm_behind_a_sublayer_joins_in_the_next_norm(dim, n, dtype):
    from rust_inference_b200 import ops
    from rust_inference_b200.parts.base import Injection
    rng = np.random.default_rng(dim)
    x = (rng.standard_normal((n, dim)) * 3 + 1.5).astype(np.float32)
    ya, yb = _t(rng.standard_normal((n, dim)) * 4, dtype), _t(rng.standard_normal((n, dim)), dtype)
    g1, pg, eps, peps = rng.uniform(0.7, 1.3, dim), rng.uniform(0.3, 1.9, dim), 1e-5, 3e-4
    fa, fb = 0.6, 0.9
    vec = rng.standard_normal(dim).astype(np.float32)
    x64 = x.astype(np.float64)
    one = lambda f: torch.full((1,), f, dtype=torch.float32, device=DEV)
    # one output
    resid = _t(x)
    (got,) = ops.rms_gains(resid, (_t(g1),), eps, dtype, terms=[(ya, None)], post=(_t(pg), peps))
    new = x64 + P.rms_unit(_np(ya), peps) * pg
    _close(resid, new, torch.float32, "residual after a normed output", tol32=1e-6)
    _close(got, P.rms_unit(new, eps) * g1, dtype, "norm in front")
    # a weighted sum of two outputs, normed as one, then a vector
    resid = _t(x)
    (got,) = ops.rms_gains(resid, (_t(g1),), eps, dtype, terms=[(ya, one(fa)), (yb, one(fb))], post=(_t(pg), peps),
                           entry=Injection(None, None, 1.0, _t(vec)))
    new = x64 + P.rms_unit(fa * _np(ya) + fb * _np(yb), peps) * pg + vec
    _close(resid, new, torch.float32, "residual after a normed sum", tol32=1e-6)
    _close(got, P.rms_unit(new, eps) * g1, dtype, "norm in front after a normed sum")
    # selected rows: nothing written back, the same bits as in the whole call
    resid = _t(x)
    rows = _i([n - 1, 0])
    (some,) = ops.rms_gains(resid, (_t(g1),), eps, dtype, terms=[(ya, one(fa)), (yb, one(fb))], post=(_t(pg), peps), rows=rows)
    assert torch.equal(resid, _t(x))
    (whole,) = ops.rms_gains(resid, (_t(g1),), eps, dtype, terms=[(ya, one(fa)), (yb, one(fb))], post=(_t(pg), peps))
    assert torch.equal(some, whole[[n - 1, 0]])
    # no norm in front: the new residual's rows into the left half of a wider matrix, the table's rows into the right one
    resid = _t(x)
    both = torch.full((n, 2 * dim + 3), 7.0, dtype=dtype, device=DEV)
    assert ops.rms_gains(resid, (), 0.0, dtype, terms=[(ya, None)], post=(_t(pg), peps), out=both[:, :dim]) == ()
    new = x64 + P.rms_unit(_np(ya), peps) * pg
    _close(resid, new, torch.float32, "residual without a norm in front", tol32=1e-6)
    _close(both[:, :dim], new, dtype, "the residual's rows in the compute dtype", tol16=5e-3)
    table, ids = _t(rng.standard_normal((11, dim)), dtype), rng.integers(0, 11, n)
    ops.embed_same(_i(ids), table, both[:, dim:2 * dim])
    assert torch.equal(both[:, dim:2 * dim], table[torch.from_numpy(ids).to(DEV)]) and torch.all(both[:, 2 * dim:] == 7.0)


# ---- bias, norm over a head or over the whole projection, rotation of half-apart partners, append ---------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Dk, Dp, rot, span, bias", [(24, 48, 10, "head", False), (12, 16, 12, "all", True), (96, 96, 96, "head", False),
                                                     (128, 128, 64, "all", True), (64, 128, 32, "head", True), (6, 16, 0, "all", False),
                                                     (20, 20, 4, "head", True), (64, 64, 16, "all", True)])
def test_qkv_prep_norms_before_the_rotation(Dk, Dp, rot, span, bias, dtype):
    from rust_inference_b200 import ops
    from rust_inference_b200.config.specs import RopeSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    rng = np.random.default_rng(Dk + rot)
    T, Hq, KV, eps, base = 9, 3, 2, 1e-5, 300.0
    table = None
    if rot:
        part = build_part("position", RopeSpec(head_dim=Dk, theta=base, rotary_dim=rot, freq64=True),
                          BuildEnv(torch.float32, torch.device(DEV)))
        part.prepare(128)
        table = part.fused_table()
    heads = Hq + 2 * KV
    x = np.zeros((T, heads, Dp))
    x[:, :, :Dk] = rng.standard_normal((T, heads, Dk)) * 2
    proj = _t(np.concatenate([x.reshape(T, -1), rng.standard_normal((T, 8))], axis=1), dtype)
    b = np.zeros((heads, Dp))
    if bias:
        b[:, :Dk] = rng.uniform(-0.5, 0.5, (heads, Dk))
    gq = rng.uniform(0.5, 2.0, (Hq, Dk) if span == "all" else (Dk,))
    gk = rng.uniform(0.5, 2.0, (KV, Dk) if span == "all" else (Dk,))

    def padded(g):
        out = np.zeros(g.shape[:-1] + (Dp,))
        out[..., :Dk] = g
        return _t(out)

    pos = [40 + t for t in range(T)]
    order = [2, 0, 1, 3]
    kp = torch.zeros((4, KV, 32, Dp), dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    q = ops.qkv_prep(proj, 0, Hq * Dp, (Hq + KV) * Dp, Hq, KV, Dp, Dk, _t(b.reshape(-1)) if bias else None, table, rot, False,
                     False, 0.0, kp, vp, _i(order).view(1, 4), _i([0] * T), _i(pos), _i([0]), norm=span, q_gain=padded(gq),
                     k_gain=padded(gk), norm_eps=eps)
    y = _np(proj)[:, :heads * Dp].reshape(T, heads, Dp)[:, :, :Dk] + b[None, :, :Dk]
    yq, yk = y[:, :Hq], y[:, Hq:Hq + KV]
    if span == "all":
        yq = (P.rms_unit(yq.reshape(T, -1), eps) * gq.reshape(-1)).reshape(T, Hq, Dk)
        yk = (P.rms_unit(yk.reshape(T, -1), eps) * gk.reshape(-1)).reshape(T, KV, Dk)
    else:
        yq, yk = P.rms_unit(yq, eps) * gq, P.rms_unit(yk, eps) * gk
    if rot:
        yq = np.stack([P.rotate_halves(yq[t], pos[t], base, rot) for t in range(T)])
        yk = np.stack([P.rotate_halves(yk[t], pos[t], base, rot) for t in range(T)])
    tol = dict(tol32=1e-5, tol16=6e-3)
    _close(q[:, :, :Dk], yq, dtype, "queries", **tol)
    assert torch.all(q[:, :, Dk:] == 0)
    for t, p in enumerate(pos):
        page = order[p // 32]
        _close(kp[page, :, p % 32, :Dk], yk[t], dtype, "keys", **tol)
        _close(vp[page, :, p % 32, :Dk], y[t, Hq + KV:], dtype, "values", **tol)
    assert torch.all(kp[order[0]] == 0) and torch.all(kp[order[3]] == 0)


# ---- the router: sigmoid scores, groups, weights without the correction ------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E, top, groups, keep, D", [(8, 3, 4, 2, 40), (6, 1, 1, 1, 52), (64, 6, 8, 3, 128), (12, 4, 3, 2, 37),
                                                    (300, 5, 5, 1, 2000)])
def test_router_with_groups_matches_plain(E, top, groups, keep, D, dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(E + D)
    T = 23
    x = _t(rng.standard_normal((T, D)), dtype)
    router = rng.standard_normal((E, D)) * 2 / math.sqrt(D)
    corr = rng.uniform(-0.4, 0.4, E)
    # ties between choice scores: copies of a row with equal corrections; the lower index wins
    router[E - 1], corr[E - 1] = router[0], corr[0]
    idx, w = ops.moe_route(x, _t(router), _t(corr), top, "sigmoid", groups, keep, 2, 1.75, False)
    z = _np(x) @ np.asarray(_np(_t(router))).T
    for t in range(T):
        chosen, weights = P.route(z[t], _np(_t(corr)), top, groups, keep, 1.75)
        got = idx[t].tolist()
        if got != chosen:                  # a close call between two scores may tip in float32: the sets' scores must agree
            c = P.sigmoid(z[t]) + _np(_t(corr))
            assert np.allclose(sorted(c[got]), sorted(c[chosen]), atol=2e-6), f"token {t}: chose {got}, plain {chosen}"
        else:
            assert np.allclose(_np(w[t]), weights, rtol=2e-5)
    # softmax scores with weights divided by their sum stay what they were
    idx2, w2 = ops.moe_route(x, _t(router), _t(corr), top)
    s = np.exp(z - z.max(-1, keepdims=True))
    s = s / s.sum(-1, keepdims=True)
    assert np.allclose(_np(w2).sum(-1), 1.0, atol=1e-5)
    first = np.argmax(s + _np(_t(corr)), axis=-1)
    close_call = np.sort(s + _np(_t(corr)), axis=-1)
    sure = close_call[:, -1] - close_call[:, -2] > 1e-5
    assert np.array_equal(idx2[:, 0].cpu().numpy()[sure], first[sure])


# ---- the matrix memory: gates, recurrence with the normaliser's column, division, norm and gate -----------------------------
def _memory_plain(p, H, d, dv, ib, fb, cap, gain, eps, g, state=None):
    """p [T, 2 H d + H dv + ..] float64 rows (q, k, v, then the gates' pre-activations at the given columns)."""
    T = p.shape[0]
    q = p[:, :H * d].reshape(T, H, d) * d ** -0.5
    k = p[:, H * d:2 * H * d].reshape(T, H, d)
    v = p[:, 2 * H * d:2 * H * d + H * dv].reshape(T, H, dv)
    zi, zf = p[:, 2 * H * d + H * dv:][:, :H], p[:, 2 * H * d + H * dv + H:][:, :H]
    li = cap * np.tanh((zi + ib) / cap)
    lf = P.log_sigmoid(cap * np.tanh((zf + fb) / cap))
    outs, states = [], []
    for j in range(H):
        o, st = P.matrix_memory(q[:, j], k[:, j], v[:, j], li[:, j], lf[:, j], None if state is None else state[j])
        outs.append(o)
        states.append(st)
    o = np.stack(outs, axis=1)
    return P.rms_unit(o, eps).reshape(T, H * dv) * gain * P.sigmoid(g), states


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, d, dv", [(3, 12, 20), (2, 64, 64), (1, 96, 33), (2, 136, 24), (4, 6, 6), (2, 128, 128)])
def test_matrix_memory_whole_in_pieces_and_token_by_token(H, d, dv, dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(H * d + dv)
    T, cap, eps = 75, 8.0, 1e-5
    N = 2 * H * d + H * dv + 2 * H
    proj = rng.standard_normal((T, N))
    proj[:, -2 * H:-H] *= 3.0                                  # input gates that move the running maximum
    proj[:, -H:] = proj[:, -H:] * 2.0 + 2.0
    proj[0, -2 * H:-H] = -6.0                                  # a first token below the maximum's start of zero
    proj_t = _t(proj, dtype)
    g = _t(rng.standard_normal((T, H * dv)), dtype)
    ib, fb, gain = rng.uniform(-1, 1, H), rng.uniform(0, 3, H), rng.uniform(0.5, 1.5, H * dv)
    want, _ = _memory_plain(_np(proj_t), H, d, dv, ib, fb, cap, gain, eps, _np(g))
    i_col, f_col = N - 2 * H, N - H

    def run(cuts, slot, S, m):
        ys, at = [], 0
        for c in cuts:
            part, gp = proj_t[at:at + c].contiguous(), g[at:at + c].contiguous()
            gates = ops.mlstm_gates(part, i_col, f_col, _t(ib), _t(fb), cap, m, _i([slot]), _i([0, c]), H, single=(c == 1))
            o = ops.scalar_decay_recurrent(part, 0, H * d, 2 * H * d, gates, d ** -0.5, S, _i([slot]), _i([0, c]), H, d, dv,
                                           ones=True, single=(c == 1))
            ys.append(ops.mlstm_head_norm_gate(o, gates, _t(gain), eps, gp, dtype))
            at += c
        return torch.cat(ys)

    S = torch.zeros((3, H, d, dv + 1), dtype=torch.float32, device=DEV)
    m = torch.zeros((3, H), dtype=torch.float32, device=DEV)
    whole = run([T], 1, S, m)
    _close(whole, want, dtype, "whole", tol32=3e-5, tol16=1.5e-2)
    S_whole, m_whole = S[1].clone(), m[1].clone()
    assert torch.all(S[0] == 0) and torch.all(S[2] == 0) and torch.all(m[0] == 0)
    pieces = run([2, 1, 7, 33, 30, 2], 2, S, m)
    single = run([1] * T, 0, S, m)
    assert torch.equal(pieces, whole) and torch.equal(single, whole), "the cutting must not change a bit"
    assert torch.equal(S[2], S_whole) and torch.equal(S[0], S_whole) and torch.equal(m[0], m_whole)
    # a slot that is given out again starts from zeros
    S[1].zero_()
    m[1].zero_()
    assert torch.equal(run([T], 1, S, m), whole)


def test_memory_gates_of_two_sequences_in_one_step():
    from rust_inference_b200 import ops
    rng = np.random.default_rng(5)
    H, cap = 3, 4.0
    proj = _t(rng.standard_normal((50, 2 * H)) * 3)
    ib, fb = _t(rng.uniform(-1, 1, H)), _t(rng.uniform(0, 3, H))
    m = torch.zeros((4, H), dtype=torch.float32, device=DEV)
    both = ops.mlstm_gates(proj, 0, H, ib, fb, cap, m, _i([3, 1]), _i([0, 37, 50]), H)
    m2 = torch.zeros_like(m)
    a = ops.mlstm_gates(proj[:37].contiguous(), 0, H, ib, fb, cap, m2, _i([0]), _i([0, 37]), H)
    b = ops.mlstm_gates(proj[37:].contiguous(), 0, H, ib, fb, cap, m2, _i([2]), _i([0, 13]), H)
    assert torch.equal(both, torch.cat([a, b])) and torch.equal(m[3], m2[0]) and torch.equal(m[1], m2[2])


# ---- the exact gelu behind a product ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_exact_gelu_behind_a_product(dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(2)
    w = _t(rng.standard_normal((72, 48)) * 0.5, dtype)
    for n in (1, 3, 12, 70):
        x = _t(rng.standard_normal((n, 48)), dtype)
        z = _np(x) @ _np(w).T
        _close(ops.linear_act(x, w, "gelu"), P.gelu_erf(z), dtype, f"{n} tokens", tol32=1e-5, tol16=1.2e-2)
    z = _t(np.linspace(-6, 6, 801), dtype)
    _close(ops.activation(z, "gelu"), P.gelu_erf(_np(z)), dtype, "the function alone", tol32=1e-6, tol16=5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, width", [(6, 96), (3, 12), (16, 128), (1, 8)])
def test_one_gate_per_head(heads, width, dtype):
    """A sigmoid gate per head from columns of a wider matrix: eight elements per thread where a head is whole 16-byte
    pieces, one otherwise."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(heads + width)
    T = 37
    x = _t(rng.standard_normal((T, heads, width)), dtype)
    wide = _t(rng.standard_normal((T, 24 + heads)) * 3, dtype)
    want = _np(x) * P.sigmoid(_np(wide)[:, 8:8 + heads])[:, :, None]
    ops.gate_heads(x, wide[:, 8:8 + heads], "sigmoid")
    _close(x, want, dtype, "gated heads", tol32=1e-6, tol16=5e-3)


# ---- whole models ------------------------------------------------------------------------------------------------------------
def _portions(reqs, sizes):
    """Each request alone, its prompt brought in portions of ``sizes`` tokens (repeated), every position wanted."""
    steps, n = [], 0
    for rid, toks in reqs.items():
        at, j = 0, 0
        while at < len(toks):
            c = min(sizes[j % len(sizes)], len(toks) - at)
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + c], "want": list(range(c))}],
                          "end": [rid] if at + c == len(toks) else []})
            at, j, n = at + c, j + 1, n + 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_in_five_cuttings_matches_plain(tmp_path, name, dtype):
    d, config, weights = K.make_model_dir(tmp_path, name, seed=3)
    rng = np.random.default_rng(4)
    reqs = H.random_requests(rng, config["vocab"], [5, 1, 23, 150, 2, 70, 37])
    want = K.plain_logits(config, weights, reqs)
    by_cutting = {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=40)),
                         ("portions", _portions(reqs, [2, 7, 1, 33, 2])), ("pairs", _portions(reqs, [2])),
                         ("batches", H.trace_batches(reqs, 3, [6, 0, 9, 3, 70, 1, 36]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, dtype, steps, out, device="cuda:0")
        rows = H.collect(steps, out, config["vocab"])
        assert len(rows) == sum(len(t) for t in reqs.values())
        K.assert_rows_close(rows, want, dtype, f"{name} {label} {dtype}")
        by_cutting[label] = rows
    if dtype == "float32":
        H.assert_rows_identical(by_cutting, f"{name} float32")


@pytest.mark.parametrize("kind", ["attention", "parallel_left", "parallel_right"])
def test_one_layer_of_each_mixer_alone(tmp_path, kind):
    """A model of one layer without feed-forward or repeated run: the mixer alone decides the logits (for the parallel
    layer one side at a time: the other side's factor is zero)."""
    if kind == "attention":
        layer = K.single(K.attn(6, 3, 20, 36, rot=(700.0, 12)), None)
    else:
        left = kind == "parallel_left"
        layer = K.double(K.attn(4, 2, 28, 12, scale=0.4, rot=(90.0, 28)), K.memory(2, 40, 12, 6.0), 1.0 if left else 0.0,
                         0.0 if left else 1.0, None)
    config = {"architecture": "Puratar", "vocab": 77, "width": 44, "norm": {"eps": 1e-5}, "logit_scale": 2.0, "layers": [layer]}
    weights = K.make_weights(config, 11)
    d = K.write_model(str(tmp_path / kind), config, weights)
    reqs = H.random_requests(np.random.default_rng(12), config["vocab"], [90, 3, 41])
    want = K.plain_logits(config, weights, reqs)
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=60)), ("pairs", _portions(reqs, [2]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, "float32", steps, out, device="cuda:0")
        K.assert_rows_close(H.collect(steps, out, config["vocab"]), want, "float32", f"{kind} {label}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 31, 32, 95, 96, 255])
def test_a_far_key_among_hundreds_is_found(tmp_path, far, dtype):
    """One attention layer whose queries and keys copy the normed input: the last token repeats the token at position
    ``far`` (a page's first or last place among them), and nothing else in 300 tokens looks like it, so its output is that
    token's value (and its own).  As the last token of a prompt and as a token decoded alone."""
    D, d = 32, 16
    config = {"architecture": "Puratar", "vocab": 400, "width": D, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
              "layers": [K.single(K.attn(2, 1, d, d, scale=1.0), None)]}
    W = K.make_weights(config, 21)
    eye = np.concatenate([np.eye(d), np.zeros((d, D - d))], axis=1)
    W["l0.mix.q"] = K._bf16(np.concatenate([eye, eye]))
    W["l0.mix.k"] = K._bf16(eye)
    W["l0.mix.q.norm"] = K._bf16(np.full(d, 6.0))               # sharp scores: 36 times a cosine
    W["l0.mix.k.norm"] = K._bf16(np.ones(d))
    W["l0.norm1"] = K._bf16(np.zeros(D))
    W["l0.mix.g"] = K._bf16(np.zeros((2, D)))
    folder = K.write_model(str(tmp_path / "far"), config, W)
    rng = np.random.default_rng(far)
    toks = [int(t) for t in rng.permutation(399)[:300] + 1]
    toks[far] = 0
    toks.append(0)
    reqs = {"r": toks}
    W64 = {k: v.astype(np.float64) for k, v in W.items()}
    want = {"r": P.forward(config, W64, toks)[0]}
    h = P.norm_one_plus(W64["embed"][toks], W64["l0.norm1"], 1e-6)
    qn = P.rms_unit(h[-1, :d], 1e-6) * 6.0
    kn = P.rms_unit(h[:, :d], 1e-6)
    s = kn @ qn
    w = np.exp(s - s.max())
    assert (w / w.sum())[far] > 0.3, "the far key does not stand out: the test would not see it missing"
    for label, steps in (("prompt", H.trace_whole(reqs)), ("decoded", H.trace_tail(reqs, tail=3))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(folder, dtype, steps, out, device="cuda:0")
        rows = H.collect(steps, out, config["vocab"])
        err = K.row_error(rows[("r", 300)], want["r"][300])
        assert err < (1e-4 if dtype == "float32" else 8e-2), f"{label}: error {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_through_page_edges(tmp_path, name, dtype):
    """A short prompt, then 260 tokens one by one (graph replays) against the plain model; two sequences of unequal
    length whose states and pages live side by side."""
    d, config, weights = K.make_model_dir(tmp_path, name, seed=6)
    rng = np.random.default_rng(7)
    reqs = H.random_requests(rng, config["vocab"], [270, 200])
    want = K.plain_logits(config, weights, reqs)
    steps = H.trace_batches(reqs, 2, [260, 195])
    out = str(tmp_path / "out")
    H.replay_inprocess(d, dtype, steps, out, device="cuda:0", max_tokens=640)
    K.assert_rows_close(H.collect(steps, out, config["vocab"]), want, dtype, f"long decoding {name} {dtype}")


def test_greedy_generation_with_more_requests_than_slots(tmp_path):
    import rust_inference_b200 as ri
    d, config, weights = K.make_model_dir(tmp_path, "A", seed=8)
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    rng = np.random.default_rng(9)
    prompts = [[int(t) for t in rng.integers(0, config["vocab"], n)] for n in (3, 1, 9, 40, 2)]
    llm = ri.LLM(d, dtype="float32", max_pages=32, pages_per_seq=4, max_seqs=2)
    got = llm.generate(prompts, max_new_tokens=12)
    assert llm.engine.graph_replays > 0
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(12):
            seq.append(int(np.argmax(P.forward(config, W, seq)[0][-1])))
        assert g == seq[len(p):]
