"""Kagatar without a GPU: the configuration class, the tensor list, the schedule with its pass entries, and the engine's
host logic (a repeated run with a cache of its own per pass, cache groups whose values are the keys, slots used again)
with the kernels replaced by the stand-ins of tests/emu_ops.py, against the plain model of tests/plain_kagatar.py."""
import copy

import numpy as np
import pytest

import helpers as H
import kagatar_models as K


def test_spec_lists_parts_and_schedule():
    from rust_inference_b200.config import config_from_dict
    from rust_inference_b200.engine.model import expected_tensors
    cfg = config_from_dict(copy.deepcopy(K.CFG_A))
    assert type(cfg).__name__ == "KagatarConfig" and cfg.to_dict()["layers"] == K.CFG_A["layers"]
    spec = cfg.to_spec()
    assert [(e.layer, e.cache, e.enters) for e in spec.schedule] == \
        [(0, 0, 0), (1, 1, -1), (0, 2, 1), (1, 3, -1), (0, 4, 2), (1, 5, -1), (2, 6, -1)]
    assert spec.tie_embeddings and spec.embedding.scale == 3.0 and spec.head.softcap == 12.0
    assert spec.pass_entry.passes == 3 and spec.pass_entry.name == "loop.step"
    first, second, third = (l.mixer for l in spec.layers)
    assert (first.unit_rms, first.softcap, first.window, first.values, first.gate, first.bias) == \
        (True, 5.0, 9, "own", "", ("q", "k", "v"))
    assert first.position.by_wavelength == (8.0, 1.0, 4.0, 16.0) and first.position.yarn is None
    assert (second.values, second.bias, second.window, second.position.kind, second.unit_rms) == \
        ("keys", ("q", "k"), 33, "none", False)
    assert (third.gate, third.window, third.softcap, third.v_head_dim) == ("element", 0, 0.0, 8)
    assert third.position.yarn == (4.0, 32.0, 8.0, 2.0)
    assert spec.layers[1].ffn is None and spec.layers[1].norms.names == ("norm1",)
    assert spec.layers[2].ffn.gate == "clamped_swish" and spec.layers[2].ffn.limit == 0.75
    assert set(expected_tensors(spec)) == set(K.make_weights(K.CFG_A, 0))
    # no repeated run: no entry part and none of its tensors; a run at the end
    plain = config_from_dict(copy.deepcopy(K.CFG_B)).to_spec()
    assert plain.pass_entry is None and all(e.enters < 0 for e in plain.schedule) and plain.head.softcap == 0.0
    assert set(expected_tensors(plain)) == set(K.make_weights(K.CFG_B, 0))
    last = config_from_dict(copy.deepcopy(K.CFG_C)).to_spec()
    assert [(e.layer, e.cache, e.enters) for e in last.schedule] == [(0, 0, -1), (1, 1, -1), (2, 2, 0), (2, 3, 1)]


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "not built"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "not built"),
    (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=16), "values that are the keys"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][2]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=-1.0), "softcap"),
])
def test_bad_configurations_are_refused(change, text):
    from rust_inference_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(K.CFG_A)
    change(c)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(c)


def test_rotary_tables_match_the_plain_frequencies():
    """The angles of the pairwise rotation with the frequencies slowed by wavelength, blended (YaRN) and plain."""
    import torch
    import plain_kagatar as P
    from rust_inference_b200.config.specs import RopePairsSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    env = BuildEnv(torch.float32, torch.device("cpu"))
    cases = [(16, 5000.0, None, (8.0, 1.0, 4.0, 64.0)), (10, 200.0, None, (8.0, 1.0, 4.0, 16.0)),
             (64, 1e6, None, (4.0, 1.0, 4.0, 1024.0)), (32, 1e4, None, (32.0, 2.0, 2.5, 300.0)),
             (12, 300.0, (4.0, 32.0, 8.0, 2.0), None), (6, 50.0, None, None)]
    for dims, base, yarn, wave in cases:
        part = build_part("position", RopePairsSpec(rotary_dim=dims, theta=base, yarn=yarn, by_wavelength=wave), env)
        part.prepare(300)
        mult = 1.0
        if yarn is not None:
            f, mult = P.yarn_frequencies(base, dims, *yarn)
        elif wave is not None:
            f = P.wavelength_frequencies(base, dims, *wave)
            assert not np.allclose(f, P.plain_frequencies(base, dims))          # the case does slow something
        else:
            f = P.plain_frequencies(base, dims)
        ang = np.arange(300)[:, None] * f[None, :]
        want = np.stack([np.cos(ang) * mult, np.sin(ang) * mult], axis=-1)
        assert np.abs(part.fused_table().numpy() - want).max() < 3e-5
    with pytest.raises(ValueError, match="not both"):
        build_part("position", RopePairsSpec(rotary_dim=8, theta=10.0, yarn=(2.0, 8.0, 4.0, 1.0),
                                             by_wavelength=(2.0, 1.0, 4.0, 8.0)), env)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_three_ways_matches_plain(tmp_path, emulated_ops, name):
    d, config, weights = K.make_model_dir(tmp_path, name, seed=3)
    rng = np.random.default_rng(4)
    reqs = H.random_requests(rng, config["vocab"], [5, 1, 23, 44, 2, 37])
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
    import plain_kagatar as P
    import rust_inference_b200 as ri
    d, config, weights = K.make_model_dir(tmp_path, "A", seed=8)
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    prompts = [[5, 9, 2], [7], [100, 3, 3, 8, 1, 60]]
    llm = ri.LLM(d, dtype="float32", device="cpu", max_pages=16, pages_per_seq=2, max_seqs=2, use_graphs=False)
    got = llm.generate(prompts, max_new_tokens=5)
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(5):
            seq.append(int(np.argmax(P.forward(config, W, seq)[0][-1])))
        assert g == seq[len(p):]
