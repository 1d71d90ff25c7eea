"""Kagatar: a decoder whose layers run a mixer and a feed-forward side by side, each behind an RMS norm of its own
over the same residual, x <- x + (mixer(n1(x)) + ff(n2(x))).  The mixers are three kinds of grouped-query attention
with biases on their projections; a run of layers may repeat with shared weights, and every pass over it adds the
embedding's output again (all passes but the first) and a learned vector of its own; the output matrix is the
embedding table without its factor, and the logits are soft-capped.

config.json keys (every size and every constant that may differ between models comes from here)::

    architecture        "Kagatar"
    vocab, width        sizes of the embedding table
    embedding.scale     factor on the embedding's rows
    norm.eps            eps of every norm (the layers', the final one, and the unit norm of "attention_3")
    logit_softcap       optional: logits <- cap * tanh(logits / cap)
    loop                optional: {start, stop, times}: layers start .. stop-1 run ``times`` times in a row with the
                        same weights and a cache of their own per pass; tensor ``loop.step`` [times, width]
    layers[i]           {type, mixer, mlp}: type "attention", "attention_2" or "attention_3"; mlp: {kind "dense", ff,
                        limit} or null for a layer without feed-forward

Mixer records have heads, kv_heads, dim (queries and keys), vdim (values), scale, and optionally mask {size} (a
window of that many keys; absent: every earlier key), rot {base, dims, scaling} (rotation of neighbouring pairs on
the first ``dims`` elements of a head; ``scaling`` absent: plain frequencies, {factor, original, fast, slow}: YaRN's
blend, {factor, low, high, original}: slowed by wavelength) and softcap (on the scores).  What the types fix:

    attention      the values are the keys as projected (no v tensor), biases on q and k
    attention_2    biases on q, k, v; a sigmoid gate per output element from a projection ``g`` of the mixer's input
    attention_3    biases on q, k, v; after the rotation q and k are divided by their root mean square over the head

The feed-forward is down(g sigmoid(1.702 g) (u + 1)) with g = min(gate x, limit), u = clamp(up x, -limit, limit).

Tensor names: ``embed``, ``final.norm``, ``loop.step``, and per layer i ``l<i>.norm1|norm2``,
``l<i>.mix.q|k|v|g|o`` (+ ``.b`` for the biases), ``l<i>.mlp.gate|up|down``.  The model itself is not written here:
``to_spec`` names the parts and the order in which the generic model runs them (``engine/model.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, EmbeddingSpec, GatedFFSpec, HeadSpec, HyperConnectionSpec, ModelSpec,
                            NoPositionSpec, ParallelNormsLayerSpec, PassEntrySpec, RMSGainsSpec, RopePairsSpec,
                            ScheduleEntry)
from .ranudra import MAX_POSITIONS, _freeze, _get, _pos_int, _thaw

SWISH_ALPHA = 1.702          # the feed-forward's gate: g sigmoid(1.702 g)
MIXER_TYPES = ("attention", "attention_2", "attention_3")
STEP_NAME = "loop.step"


@register_architecture("Kagatar", "kagatar")
@dataclass(frozen=True)
class KagatarConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: Tuple[tuple, ...]                    # frozen layer records of config.json
    logit_softcap: float = 0.0
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    eos_token_ids: Tuple[int, ...] = ()

    # ---- config.json <-> object -------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "KagatarConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = (_get(lp, "start", "loop", int), _get(lp, "stop", "loop", int), _get(lp, "times", "loop", int))
        cap = d.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float))):
            raise ConfigError(f"config.json: logit_softcap must be a number, got {cap!r}")
        emb = d.get("embedding")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]))
        return cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"),
                   embedding_scale=float(_get(emb, "scale", "embedding")) if emb is not None else 1.0,
                   eps=float(_get(d.get("norm"), "eps", "norm")), layers=tuple(_freeze(l) for l in layers),
                   logit_softcap=float(cap or 0.0), loop=loop, eos_token_ids=eos_ids)

    def layer_records(self):
        return [_thaw(l) for l in self.layers]

    def to_dict(self) -> dict:
        d = {"architecture": "Kagatar", "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": self.layer_records()}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- checks ------------------------------------------------------------------
    def validate(self) -> None:
        if not (self.eps > 0):
            raise ConfigError("norm.eps must be positive")
        if self.logit_softcap < 0:
            raise ConfigError("logit_softcap must be positive")
        n = len(self.layers)
        if self.loop is not None:
            start, stop, times = self.loop
            if not (0 <= start <= stop <= n) or times < 1:
                raise ConfigError(f"loop {self.loop} does not fit {n} layers")
        for i, layer in enumerate(self.layer_records()):
            what = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {what}.type {kind!r} is not built (known: {', '.join(MIXER_TYPES)})")
            m = layer.get("mixer")
            for key in ("heads", "kv_heads", "dim"):
                _pos_int(m, key, what + ".mixer")
            if kind != "attention" or "vdim" in m:
                _pos_int(m, "vdim", what + ".mixer")
            if kind == "attention" and m.get("vdim", m["dim"]) != m["dim"]:
                raise ConfigError(f"config.json: {what}.mixer: values that are the keys have their size {m['dim']}, "
                                  f"not vdim {m['vdim']}")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: {what}.mixer: {m['heads']} heads over {m['kv_heads']} kv_heads")
            _get(m, "scale", what + ".mixer")
            if m.get("softcap") is not None and not float(_get(m, "softcap", what + ".mixer")) > 0:
                raise ConfigError(f"config.json: {what}.mixer.softcap must be positive")
            if m.get("mask") is not None:
                _pos_int(m["mask"], "size", what + ".mixer.mask")
            rot = m.get("rot")
            if rot is not None and rot.get("dims", 0):
                dims = _pos_int(rot, "dims", what + ".mixer.rot")
                if dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"config.json: {what}.mixer.rot.dims {dims} must be even and at most dim {m['dim']}")
                if not float(_get(rot, "base", what + ".mixer.rot")) > 0:
                    raise ConfigError(f"config.json: {what}.mixer.rot.base must be positive")
                sc = rot.get("scaling")
                if sc is not None:
                    keys = ("factor", "original", "fast", "slow") if "fast" in sc else ("factor", "low", "high", "original")
                    for key in keys:
                        if not float(_get(sc, key, what + ".mixer.rot.scaling")) > 0:
                            raise ConfigError(f"config.json: {what}.mixer.rot.scaling.{key} must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {what}.mlp.kind {mlp.get('kind')!r} is not built (known: dense)")
                _pos_int(mlp, "ff", what + ".mlp")
                if not float(_get(mlp, "limit", what + ".mlp")) > 0:
                    raise ConfigError(f"config.json: {what}.mlp.limit must be positive")

    # ---- the model as parts --------------------------------------------------------
    def _mixer(self, kind, m):
        position = NoPositionSpec()
        rot = m.get("rot") or {}
        if kind != "attention" and rot.get("dims", 0):
            sc = rot.get("scaling")
            yarn = wave = None
            if sc is not None and "fast" in sc:
                yarn = (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
            elif sc is not None:
                wave = (float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"]))
            position = RopePairsSpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]), yarn=yarn, by_wavelength=wave)
        keys_serve = kind == "attention"
        third = kind == "attention_3"
        return AttentionSpec(
            hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], position=position,
            scale=float(m["scale"]), window=int((m.get("mask") or {}).get("size", 0)),
            v_head_dim=0 if keys_serve else int(m["vdim"]), names=("q", "k", "v", "o", "sink"),
            bias=("q", "k") if keys_serve else ("q", "k", "v"), bias_suffix=".b", values="keys" if keys_serve else "own",
            unit_rms=third, unit_eps=self.eps if third else 0.0, softcap=float(m.get("softcap") or 0.0) if third else 0.0,
            gate="element" if kind == "attention_2" else "", gate_name="g")

    def to_spec(self) -> ModelSpec:
        D = self.width
        link = HyperConnectionSpec(streams=1, learned=False)
        layers = []
        for i, layer in enumerate(self.layer_records()):
            mlp = layer.get("mlp")
            ffn = None
            if mlp is not None:
                ffn = GatedFFSpec(hidden_size=D, intermediate_size=mlp["ff"], gate="clamped_swish", limit=float(mlp["limit"]),
                                  alpha=SWISH_ALPHA)
            norms = RMSGainsSpec(size=D, eps=self.eps, names=("norm1",) if ffn is None else ("norm1", "norm2"))
            names = (("norms", f"l{i}."), ("mixer", f"l{i}.mix."), ("ffn", f"l{i}.mlp."), ("link", f"l{i}."))
            layers.append(ParallelNormsLayerSpec(mixer=self._mixer(layer["type"], layer["mixer"]), norms=norms, link=link,
                                                 ffn=ffn, names=names))
        n = len(layers)
        start, stop, times = self.loop if self.loop is not None else (0, 0, 0)
        if stop <= start:
            times = 0
        # every run of a layer has a cache entry of its own: a repeated layer shares weights, not keys
        order = [(i, -1) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else -1) for i in range(start, stop)]
        order += [(i, -1) for i in range(stop, n)]
        schedule = tuple(ScheduleEntry(layer=i, cache=run, enters=t) for run, (i, t) in enumerate(order))
        entry = PassEntrySpec(passes=times, hidden_size=D, readd_embedding=True, name=STEP_NAME) if times else None
        return ModelSpec(
            architecture="Kagatar", vocab_size=self.vocab, hidden_size=D, layers=tuple(layers), schedule=schedule,
            final_norm=RMSGainsSpec(size=D, eps=self.eps, names=("",)), tie_embeddings=True, max_positions=MAX_POSITIONS,
            embedding_name="embed", head_name="embed", final_norm_prefix="final.norm", stop_ids=self.eos_token_ids,
            head_optional=False, embedding=EmbeddingSpec(self.vocab, D, scale=self.embedding_scale),
            head=HeadSpec(self.vocab, D, softcap=self.logit_softcap), pass_entry=entry)
