"""Kagatar on the GPU: each kernel against the plain formulas of tests/plain_kagatar.py, then whole models through trace
replay in several cuttings (whole prompts; prompts then single tokens; prompts in portions down to two tokens; batches of
unequal requests that follow each other on the same slots and pages), in float32 and bfloat16, against the plain model."""
import numpy as np
import pytest
import torch

import helpers as H
import kagatar_models as K
import plain_kagatar as P

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


# ---- one RMS statistic, two gains, and everything that joins the residual in front of it --------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, n", [(52, 5), (48, 70), (3001, 9), (1, 3)])
def test_rms_gains_with_pending_outputs_and_entry_terms(dim, n, dtype):
    from rust_inference_b200 import ops
    from rust_inference_b200.parts.base import Injection
    rng = np.random.default_rng(dim)
    x = (rng.standard_normal((n, dim)) * 3 + 1.5).astype(np.float32)
    ya, yb = _t(rng.standard_normal((n, dim)), dtype), _t(rng.standard_normal((n, dim)), dtype)
    g1, g2, eps = rng.uniform(0.7, 1.3, dim), rng.uniform(0.7, 1.3, dim), 1e-5
    vocab = 11
    table, ids = _t(rng.standard_normal((vocab, dim)), dtype), rng.integers(0, vocab, n)
    vec = rng.standard_normal(dim).astype(np.float32)
    x64 = x.astype(np.float64)
    # nothing pending, one gain: the plain norm, the residual untouched
    resid = _t(x)
    (got,) = ops.rms_gains(resid, (_t(g1),), eps, dtype)
    _close(got, P.rms_norm(x64, g1, eps), dtype, "one gain")
    assert torch.equal(resid, _t(x))
    # two outputs (their sum first), two gains
    resid = _t(x)
    o1, o2 = ops.rms_gains(resid, (_t(g1), _t(g2)), eps, dtype, terms=[(ya, None), (yb, None)])
    new = x64 + (_np(ya) + _np(yb))
    _close(resid, new, torch.float32, "residual after two outputs", tol32=1e-6)
    _close(o1, P.rms_norm(new, g1, eps), dtype, "first gain")
    _close(o2, P.rms_norm(new, g2, eps), dtype, "second gain")
    # an output, then the embedding's rows again and the pass's vector
    resid = _t(x)
    entry = Injection(_i(ids), table, 2.5, _t(vec))
    o1, o2 = ops.rms_gains(resid, (_t(g1), _t(g2)), eps, dtype, terms=[(ya, None)], entry=entry)
    new = x64 + _np(ya) + _np(table)[ids] * 2.5 + vec
    _close(resid, new, torch.float32, "residual after an entry", tol32=1e-6)
    _close(o2, P.rms_norm(new, g2, eps), dtype, "second gain after an entry")
    # the first pass: nothing pending, no rows of the table, the vector alone
    resid = _t(x)
    (got,) = ops.rms_gains(resid, (_t(g1),), eps, dtype, entry=Injection(None, None, 1.0, _t(vec)))
    _close(resid, x64 + vec, torch.float32, "residual after the vector", tol32=1e-6)
    _close(got, P.rms_norm(x64 + vec, g1, eps), dtype, "gain after the vector")
    # selected rows: read, not written back; a row's bits do not depend on the other rows of the call
    resid = _t(x)
    rows = _i([n - 1, 0])
    (some,) = ops.rms_gains(resid, (_t(g1),), eps, dtype, terms=[(ya, None), (yb, None)], rows=rows)
    assert torch.equal(resid, _t(x))
    resid = _t(x)
    (whole,) = ops.rms_gains(resid, (_t(g1),), eps, dtype, terms=[(ya, None), (yb, None)])
    assert torch.equal(some, whole[[n - 1, 0]])
    resid = _t(x[:1])
    (alone,) = ops.rms_gains(resid, (_t(g1),), eps, dtype, terms=[(ya[:1].contiguous(), None), (yb[:1].contiguous(), None)])
    assert torch.equal(alone[0], whole[0])


# ---- between the q/k/v product and attention: bias, rotation, unit norm, append ------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Dk, Dp, rot, unit, own_v", [(24, 32, 10, True, True), (12, 16, 0, False, False), (20, 20, 20, True, True),
                                                      (64, 64, 64, True, False), (96, 96, 24, False, True), (6, 16, 6, True, True)])
def test_qkv_prep_bias_rotation_unit_norm_append(Dk, Dp, rot, unit, own_v, dtype):
    from rust_inference_b200 import ops
    from rust_inference_b200.config.specs import RopePairsSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    rng = np.random.default_rng(Dk + rot)
    T, Hq, KV, eps = 9, 3, 2, 1e-5
    wave = (4.0, 1.0, 4.0, 16.0)
    table = None
    if rot:
        part = build_part("position", RopePairsSpec(rotary_dim=rot, theta=300.0, by_wavelength=wave),
                          BuildEnv(torch.float32, torch.device(DEV)))
        part.prepare(128)
        table = part.fused_table()
    heads = Hq + KV + (KV if own_v else 0)
    extra = 8                                                   # columns of something else behind the heads (a gate)
    x = np.zeros((T, heads, Dp))
    x[:, :, :Dk] = rng.standard_normal((T, heads, Dk))
    proj = _t(np.concatenate([x.reshape(T, -1), rng.standard_normal((T, extra))], axis=1), dtype)
    bias = np.zeros((heads, Dp))
    bias[:, :Dk] = rng.uniform(-0.5, 0.5, (heads, Dk))
    pos = [40 + t for t in range(T)]                            # pages 1 and 2 of the sequence
    order = [2, 0, 1, 3]
    kp = torch.zeros((4, KV, 32, Dp), dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp) if own_v else kp
    pt = _i(order).view(1, 4)
    q = ops.qkv_prep(proj, 0, Hq * Dp, (Hq + KV) * Dp if own_v else -1, Hq, KV, Dp, Dk, _t(bias.reshape(-1)), table, rot, True,
                     unit, eps, kp, vp, pt, _i([0] * T), _i(pos), _i([0]))
    y = _np(proj)[:, :heads * Dp].reshape(T, heads, Dp)[:, :, :Dk] + bias[None, :, :Dk]
    f = P.wavelength_frequencies(300.0, rot, *wave) if rot else []
    want = np.stack([P.rotate_pairs(y[t, :Hq + KV], pos[t], f) for t in range(T)])
    if unit:
        want = P.rms_unit(want, eps)
    tol = dict(tol32=1e-5, tol16=6e-3)
    _close(q[:, :, :Dk], want[:, :Hq], dtype, "queries", **tol)
    assert torch.all(q[:, :, Dk:] == 0)
    for t, p in enumerate(pos):
        page = order[p // 32]
        _close(kp[page, :, p % 32, :Dk], want[t, Hq:], dtype, "keys", **tol)
        if own_v:
            _close(vp[page, :, p % 32, :Dk], y[t, Hq + KV:], dtype, "values", **tol)
    assert torch.all(kp[order[0]] == 0) and torch.all(kp[order[3]] == 0)


# ---- windows, capped scores, values that are the keys -------------------------------------------------------------------
def _paged(rng, k, v, page_size=32, spare=3):
    """Keys and values [n, KV, D] of one sequence in pools whose pages are in no order; slot 1 of 2.  ``v`` None: one pool."""
    n, KV, D = k.shape
    pages = -(-n // page_size)
    order = rng.permutation(pages + spare)[:pages]
    kp = torch.zeros((pages + spare, KV, page_size, D), dtype=k.dtype, device=DEV)
    vp = kp if v is None else torch.zeros_like(kp)
    for p in range(n):
        kp[order[p // page_size], :, p % page_size] = k[p]
        if v is not None:
            vp[order[p // page_size], :, p % page_size] = v[p]
    table = torch.full((2, pages + 2), -1, dtype=torch.int32, device=DEV)
    table[1, :pages] = _i(order)
    return kp, vp, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D, window, cap, own_v", [(32, 7, 0.0, True), (80, 33, 3.0, True), (64, 90, 2.5, False), (128, 32, 0.0, False),
                                                   (64, 1, 4.0, True), (48, 0, 1.5, True), (128, 100, 6.0, True)])
def test_window_attention_with_a_loud_key_at_the_edge(D, window, cap, own_v, dtype):
    """One key is made loud (its score stands out among hundreds).  The last query that has it in its window must follow its
    value, the next one must not see it; in a prompt, in a portion of a prompt, and token by token; with capped scores the cap
    decides how far the loud key stands out."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(D + window)
    n, Hq, KV, scale = 300, 4, 2, 0.25
    k = rng.standard_normal((n, KV, D)) * 0.3
    v = rng.standard_normal((n, KV, D)) if own_v else None
    q = rng.standard_normal((n, Hq, D)) * 0.3
    direction = rng.standard_normal(D)
    direction /= np.linalg.norm(direction)
    loud = [5, 150, 223]                                   # a far key, one whose window ends in the prompt, one near a page's edge
    for j in loud:
        k[j] += 6.0 * direction
    q += 4.0 * direction                                 # every query looks for the loud keys
    kt, qt = _t(k, dtype), _t(q, dtype)
    vt = None if v is None else _t(v, dtype)
    kp, vp, table = _paged(rng, kt, vt)
    kn = _np(kt)
    want = P.attend(_np(qt), kn, kn if v is None else _np(vt), scale, window=window, cap=cap or None).reshape(n, Hq, D)
    slot = _i([1])
    tol = dict(tol32=3e-5, tol16=2e-2)
    for first in (0, n - 100):
        new = n - first
        start, length = _i([0, new]), _i([n])
        got = ops.attention(qt[first:].contiguous(), kp, vp, table, slot, start, length, new, scale, window, softcap=cap)
        _close(got, want[first:], dtype, f"rows kernel from {first}", **tol)
        if dtype == torch.bfloat16:
            got = ops.attention_prefill(qt[first:].contiguous(), kp, vp, table, slot, start, length, new, scale, window, softcap=cap)
            _close(got, want[first:], dtype, f"prefill kernel from {first}", **tol)
    edge = 150 + window - 1 if window else n - 1           # the last query that sees key 150
    for p in sorted({max(edge - 1, 0), edge, min(edge + 1, n - 1), 223, min(223 + window, n - 1), n - 1}):
        length = _i([p + 1])
        got = ops.attention(qt[p:p + 1].contiguous(), kp, vp, table, slot, _i([0, 1]), length, 1, scale, window, softcap=cap)
        _close(got, want[p:p + 1], dtype, f"rows kernel, token {p}", **tol)
        if dtype == torch.bfloat16:
            got = ops.attention_decode(qt[p:p + 1].contiguous(), kp, vp, table, slot, length, scale, window, 1024, softcap=cap)
            _close(got, want[p:p + 1], dtype, f"decode kernel, token {p}", **tol)
    # the loud key decides what the queries that see it return: a window that is one token off, or a cap left out, cannot
    # hide in the tolerance
    if window and edge + 1 < n:
        moved = P.attend(_np(qt)[:edge + 2], kn[:edge + 2], (kn if v is None else _np(vt))[:edge + 2], scale, window=window + 1,
                         cap=cap or None).reshape(-1, Hq, D)
        assert np.abs(moved[edge + 1] - want[edge + 1]).max() > 0.2 * np.abs(want[edge + 1]).max()
    if cap and window != 1:
        bare = P.attend(_np(qt)[:225], kn[:225], (kn if v is None else _np(vt))[:225], scale, window=window).reshape(225, Hq, D)
        assert np.abs(bare[224] - want[224]).max() > 0.05 * np.abs(want[224]).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_swish_feed_forward_gate_behind_a_product(dtype):
    """g sigmoid(1.702 g) (u + 1) with g = min(gate x, limit), u = clamp(up x, -limit, limit): for a handful of bfloat16 tokens in
    the weight-streaming product's epilogue, otherwise after the product; limits that cut many values and that cut none."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(2)
    inter, Kd = 40, 64
    wg, wu = _t(rng.standard_normal((inter, Kd)) * 0.3, dtype), _t(rng.standard_normal((inter, Kd)) * 0.3, dtype)
    stacked = torch.stack([wg.view(inter // 8, 8, Kd), wu.view(inter // 8, 8, Kd)], dim=1).reshape(2 * inter, Kd).contiguous()
    for m in (1, 3, 12, 20, 32, 70):                     # (13 to 32 bfloat16 tokens: the tcgen05 weight-streaming product)
        for limit in (0.8, 30.0):
            xin = _t(rng.standard_normal((m, Kd)), dtype)
            g = np.minimum(_np(xin) @ _np(wg).T, limit)
            u = np.clip(_np(xin) @ _np(wu).T, -limit, limit)
            got = ops.linear_gated(xin, stacked, 8, "clamped_swish", limit, 1.702)
            _close(got, g * P.sigmoid(1.702 * g) * (u + 1.0), dtype, f"{m} tokens, limit {limit}")
    if dtype == torch.bfloat16:
        # a matrix large enough for the tcgen05 product at a handful of tokens (K split over a cluster), both other gates
        inter, Kd, m = 11008, 4096, 8
        wg, wu = _t(rng.standard_normal((inter, Kd)) * 0.02, dtype), _t(rng.standard_normal((inter, Kd)) * 0.02, dtype)
        stacked = torch.stack([wg.view(inter // 8, 8, Kd), wu.view(inter // 8, 8, Kd)], dim=1).reshape(2 * inter, Kd).contiguous()
        xin = _t(rng.standard_normal((m, Kd)), dtype)
        gz, uz = _np(xin) @ _np(wg).T, _np(xin) @ _np(wu).T
        g, u = np.minimum(gz, 1.0), np.clip(uz, -1.0, 1.0)
        _close(ops.linear_gated(xin, stacked, 8, "clamped_swish", 1.0, 1.702), g * P.sigmoid(1.702 * g) * (u + 1.0), dtype, "large")
        gelu = 0.5 * gz * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (gz + 0.044715 * gz ** 3)))
        _close(ops.linear_gated(xin, stacked, 8, "gelu_tanh"), gelu * uz, dtype, "large, gelu")


def test_soft_cap_on_logits():
    from rust_inference_b200 import ops
    rng = np.random.default_rng(1)
    z = rng.standard_normal((7, 333)) * 40
    got = ops.softcap_(_t(z), 18.0)
    _close(got, P.soft_cap(z.astype(np.float32).astype(np.float64), 18.0), torch.float32, "capped logits", tol32=1e-6)
    same = _t(z)
    assert ops.softcap_(same, 0.0) is same and torch.equal(same, _t(z))


# ---- whole models ----------------------------------------------------------------------------------------------------------
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
@pytest.mark.parametrize("name", ["A", "B", "C"])
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


@pytest.mark.parametrize("kind", ["attention", "attention_2", "attention_3"])
def test_one_layer_of_each_mixer_alone(tmp_path, kind):
    """A model of one layer without feed-forward, repeated run or caps on the logits: the mixer alone decides the logits."""
    rot = {"base": 700.0, "dims": 12, "scaling": {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 24}}
    mixer = {"attention": K._mixer(4, 2, 28, 28, window=19),
             "attention_2": K._mixer(6, 3, 20, 36, rot=dict(rot, scaling={"factor": 3.0, "original": 24, "fast": 6.0, "slow": 1.0})),
             "attention_3": K._mixer(2, 1, 40, 12, scale=0.8, window=50, softcap=4.0, rot=rot)}[kind]
    config = {"architecture": "Kagatar", "vocab": 77, "width": 44, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
              "layers": [K._layer(kind, mixer, None)]}
    weights = K.make_weights(config, 11)
    d = K.write_model(str(tmp_path / kind), config, weights)
    reqs = H.random_requests(np.random.default_rng(12), config["vocab"], [90, 3, 41])
    want = K.plain_logits(config, weights, reqs)
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=60)), ("pairs", _portions(reqs, [2]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, "float32", steps, out, device="cuda:0")
        K.assert_rows_close(H.collect(steps, out, config["vocab"]), want, "float32", f"{kind} {label}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_through_window_and_page_edges(tmp_path, name, dtype):
    """A short prompt, then 260 tokens one by one (graph replays), against the plain model: windows of 9, 32, 33 and 70 keys
    pass over decoded tokens, pages behind a window go back to the free list and are used again."""
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
