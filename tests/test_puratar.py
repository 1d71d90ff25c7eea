"""Puratar without a GPU: the configuration class, the tensor list, the schedule with its pass entries, the plain model's
mechanisms against each other, and the engine's host logic (a repeated run with caches and states of their own per pass,
pages beside three kinds of state, slots used again) with the kernels replaced by the stand-ins of tests/emu_ops.py,
against the plain model of tests/plain_puratar.py."""
import copy

import numpy as np
import pytest

import helpers as H
import plain_puratar as P
import puratar_models as K


def test_spec_lists_parts_and_schedule():
    from rust_inference_b200.config import config_from_dict
    from rust_inference_b200.engine.model import expected_tensors
    cfg = config_from_dict(copy.deepcopy(K.CFG_A))
    assert type(cfg).__name__ == "PuratarConfig" and cfg.to_dict()["layers"] == K.CFG_A["layers"]
    spec = cfg.to_spec()
    assert [(e.layer, e.cache, e.enters) for e in spec.schedule] == \
        [(0, 0, -1), (1, 1, 0), (2, 2, -1), (1, 3, 1), (2, 4, -1), (1, 5, 2), (2, 6, -1), (3, 7, -1)]
    assert spec.tie_embeddings and spec.head.scale == 0.8 and spec.final_norm.one_plus
    assert spec.pass_entry.kind == "pass_mix" and spec.pass_entry.passes == 3
    first = spec.layers[0]
    assert first.arrangement == "sandwich" and first.mixer_link.gain_name == "norm1b" and first.ffn_link.scale_name == "ls2"
    m = first.mixer
    assert (m.gate, m.qk_norm_span, m.bias, m.v_head_dim, m.position.rotary_dim, m.position.freq64) == ("head", "head", (), 40, 10, True)
    f = first.ffn
    assert (f.score, f.groups, f.group_keep, f.group_top, f.renormalize, f.route_scale, f.expert.gate) == \
        ("sigmoid", 3, 2, 2, False, 2.0, "silu")
    second = spec.layers[1].mixer
    assert second.kind == "parallel" and (second.left_scale, second.right_scale) == (0.7, 1.3)
    assert (second.left.qk_norm_span, second.left.bias, second.left.gate) == ("all", ("q", "k", "v"), "")
    assert (second.right.kind, second.right.gate_cap, second.right.num_heads) == ("mlstm", 8.0, 3)
    assert spec.layers[1].ffn.activation == "gelu" and spec.layers[2].ffn is None
    assert spec.layers[3].ffn.shared is None and spec.layers[3].ffn.groups == 1
    assert set(expected_tensors(spec)) == set(K.make_weights(K.CFG_A, 0))
    plain = config_from_dict(copy.deepcopy(K.CFG_B)).to_spec()
    assert plain.pass_entry is None and all(e.enters < 0 for e in plain.schedule) and plain.head.scale == 1.0
    assert set(expected_tensors(plain)) == set(K.make_weights(K.CFG_B, 0))
    first_twice = config_from_dict(copy.deepcopy(K.CFG_C)).to_spec()
    assert [(e.layer, e.cache, e.enters) for e in first_twice.schedule] == [(0, 0, 0), (0, 1, 1), (1, 2, -1), (2, 3, -1)]
    assert set(expected_tensors(first_twice)) == set(K.make_weights(K.CFG_C, 0))


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "not built"),
    (lambda c: c["layers"][1]["mlp"].update(kind="experts"), "not built"),
    (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(gate_cap=0.0), "gate_cap"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
])
def test_bad_configurations_are_refused(change, text):
    from rust_inference_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(K.CFG_A)
    change(c)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(c)


def test_rotary_table_matches_the_plain_rotation():
    import torch
    from rust_inference_b200.config.specs import RopeSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    env = BuildEnv(torch.float32, torch.device("cpu"))
    for dims, base in ((10, 300.0), (64, 1e6), (4, 7.0)):
        part = build_part("position", RopeSpec(head_dim=dims + 2, theta=base, rotary_dim=dims, freq64=True), env)
        part.prepare(200)
        table = part.fused_table().numpy()
        x = np.zeros(dims + 2)
        x[0] = 1.0                                            # element 0 turns into (cos, sin) at elements 0 and dims/2
        for pos in (0, 1, 57, 199):
            y = P.rotate_halves(x, pos, base, dims)
            assert abs(table[pos, 0, 0] - y[0]) < 1e-6 and abs(table[pos, 0, 1] - y[dims // 2]) < 1e-6
        f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
        assert np.abs(table[:, :, 0] - np.cos(np.arange(200)[:, None] * f)).max() < 3e-5


def test_plain_matrix_memory_carries_its_state():
    """The plain recurrence in one go equals the same in two pieces with the state handed over; the running maximum starts
    at zero (a first token with a very negative input gate keeps exp(-m) = 1 in the denominator)."""
    rng = np.random.default_rng(0)
    T, d, dv = 9, 5, 3
    q, k, v = rng.standard_normal((T, d)), rng.standard_normal((T, d)), rng.standard_normal((T, dv))
    li, lf = rng.uniform(-3, 3, T), -rng.uniform(0.01, 2, T)
    whole, _ = P.matrix_memory(q, k, v, li, lf)
    a, st = P.matrix_memory(q[:4], k[:4], v[:4], li[:4], lf[:4])
    b, _ = P.matrix_memory(q[4:], k[4:], v[4:], li[4:], lf[4:], st)
    assert np.allclose(np.concatenate([a, b]), whole, rtol=1e-12, atol=1e-12)
    li[0] = -9.0
    first, (S, n, m) = P.matrix_memory(q[:1], k[:1], v[:1], li[:1], lf[:1])
    assert m == max(lf[0], -9.0) and np.allclose(first[0], (S.T @ q[0]) / (np.exp(-m) + 1e-6))


def test_plain_route_takes_groups_and_leaves_the_correction_out_of_the_weights():
    z = np.array([2.0, -1.0, 0.5, 0.4, 3.0, -3.0])
    corr = np.array([0.0, 0.0, 0.3, 0.3, -2.5, 0.0])
    # groups of two: choice scores (0.88, 0.27 | 0.92, 0.90 | -1.55, 0.05): the first two groups are kept
    chosen, w = P.route(z, corr, top=3, groups=3, keep=2, scale=2.0)
    assert chosen == [2, 3, 0]
    assert np.allclose(w, [2.0 * P.sigmoid(0.5), 2.0 * P.sigmoid(0.4), 2.0 * P.sigmoid(2.0)])
    chosen, _ = P.route(z, corr, top=2, groups=1, keep=1, scale=1.0)
    assert chosen == [2, 3]


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_three_ways_matches_plain(tmp_path, emulated_ops, name):
    d, config, weights = K.make_model_dir(tmp_path, name, seed=3)
    rng = np.random.default_rng(4)
    reqs = H.random_requests(rng, config["vocab"], [5, 1, 23, 40, 2, 35])
    want = K.plain_logits(config, weights, reqs)
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=12)),
                         ("batches", H.trace_batches(reqs, 3, [6, 0, 9, 3]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, "float32", steps, out)
        rows = H.collect(steps, out, config["vocab"])
        assert len(rows) == sum(len(t) for t in reqs.values())
        K.assert_rows_close(rows, want, "float32", f"{name} {label}")


def test_greedy_generation_matches_plain(tmp_path, emulated_ops):
    """Greedy tokens through the generation loop (two batches on the same slots) against the plain model."""
    import rust_inference_b200 as ri
    d, config, weights = K.make_model_dir(tmp_path, "A", seed=8)
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    prompts = [[5, 9, 2], [7], [90, 3, 3, 8, 1, 60]]
    llm = ri.LLM(d, dtype="float32", device="cpu", max_pages=16, pages_per_seq=2, max_seqs=2, use_graphs=False)
    got = llm.generate(prompts, max_new_tokens=5)
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(5):
            seq.append(int(np.argmax(P.forward(config, W, seq)[0][-1])))
        assert g == seq[len(p):]
