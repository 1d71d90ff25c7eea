"""Puratar: a decoder whose layers have a norm in front of and behind each sublayer and a layer scale,
x <- x + ls1 * n1b(mixer(n1(x))), x <- x + ls2 * n2b(ff(n2(x))), all norms RMS norms whose tensors hold the gain
minus one (gain 1 + w).  The mixers are grouped-query attention with a per-head RMS norm of queries and keys, rotation of
half-apart partners on a part of a head and one sigmoid gate per head ("attention"), or two mixers side by side
("parallel"): attention with biases and an RMS norm over the whole query (key) projection, beside the matrix memory of
xLSTM.  Feed-forwards are dense (exact gelu) or routed (sigmoid scores, a correction on the choice only, a choice
limited to the best groups of experts, weights that are not renormalised, silu-gated experts, a shared expert).  A run
of layers may repeat with shared weights and a cache of its own per pass; every pass starts by projecting the residual
and the embedding's output, side by side, back to the width, and adds a learned vector of its own.  The output matrix
is the embedding table and the logits are multiplied by a constant.

config.json keys (every size and every constant that may differ between models comes from here)::

    architecture        "Puratar"
    vocab, width        sizes of the embedding table
    norm.eps            eps of every norm (the layers', the final one, the norms of queries and keys, the memory's heads)
    logit_scale         factor on the logits (absent: 1)
    loop                optional: {start, stop, times}: layers start .. stop-1 run ``times`` times in a row with the
                        same weights and a cache or state of their own per pass; tensors ``loop.in`` [width, 2 width]
                        and ``loop.step`` [times, width]
    layers[i]           {type "attention" | "parallel", mixer, mlp}
      mixer (attention)   heads, kv_heads, dim (queries and keys), vdim (values), scale, rot {base, dims} (optional)
      mixer (parallel)    left {the same keys}, right {heads, dim, vdim, gate_cap}, left_scale, right_scale
      mlp                 null, {kind "dense", ff} or {kind "moe", router {experts, top, scale, groups {count, keep}},
                          expert {ff}, shared {ff} (optional)}

Fixed by the design (constants in this file or in the parts): a group of experts is scored by its two largest choice
scores; the memory's denominator floor 1e-6; which projections have biases.

Tensor names: ``embed``, ``final.norm``, ``loop.in``, ``loop.step``, and per layer i ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.ls1|ls2``, ``l<i>.mix.q|k|v|o|g|q.norm|k.norm`` or ``l<i>.mix.left.q|k|v`` (+ ``.b``) ``|o|q.norm|k.norm`` and
``l<i>.mix.right.q|k|v|g|o|norm|i|f`` (+ ``i.b``, ``f.b``), ``l<i>.mlp.up|down`` or
``l<i>.mlp.router|correction|e<j>.gate|up|down|shared.gate|up|down``.  The model itself is not written here:
``to_spec`` names the parts and the order in which the generic model runs them (``engine/model.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, DenseFFSpec, EmbeddingSpec, GatedFFSpec, HeadSpec, MLSTMSpec, ModelSpec, MoESpec,
                            NoPositionSpec, ParallelMixerSpec, PassMixSpec, PostNormSpec, RMSGainsSpec, RMSNormSpec,
                            RopeSpec, SandwichLayerSpec, ScheduleEntry)
from .ranudra import MAX_POSITIONS, _freeze, _get, _pos_int, _thaw

LAYER_TYPES = ("attention", "parallel")
GROUP_TOP = 2                # a group of experts is scored by the sum of this many of its largest choice scores
IN_NAME, STEP_NAME = "loop.in", "loop.step"


@register_architecture("Puratar", "puratar")
@dataclass(frozen=True)
class PuratarConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[tuple, ...]                    # frozen layer records of config.json
    logit_scale: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    eos_token_ids: Tuple[int, ...] = ()

    # ---- config.json <-> object -------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "PuratarConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = (_get(lp, "start", "loop", int), _get(lp, "stop", "loop", int), _get(lp, "times", "loop", int))
        scale = d.get("logit_scale", 1.0)
        if isinstance(scale, bool) or not isinstance(scale, (int, float)):
            raise ConfigError(f"config.json: logit_scale must be a number, got {scale!r}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]))
        return cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"),
                   eps=float(_get(d.get("norm"), "eps", "norm")), layers=tuple(_freeze(l) for l in layers),
                   logit_scale=float(scale), loop=loop, eos_token_ids=eos_ids)

    def layer_records(self):
        return [_thaw(l) for l in self.layers]

    def to_dict(self) -> dict:
        d = {"architecture": "Puratar", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "logit_scale": self.logit_scale, "layers": self.layer_records()}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- checks ------------------------------------------------------------------
    @staticmethod
    def _check_attention(m, what):
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _pos_int(m, key, what)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"config.json: {what}: {m['heads']} heads over {m['kv_heads']} kv_heads")
        _get(m, "scale", what)
        rot = m.get("rot")
        if rot is not None and rot.get("dims", 0):
            dims = _pos_int(rot, "dims", what + ".rot")
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"config.json: {what}.rot.dims {dims} must be even and at most dim {m['dim']}")
            if not float(_get(rot, "base", what + ".rot")) > 0:
                raise ConfigError(f"config.json: {what}.rot.base must be positive")

    def validate(self) -> None:
        if not (self.eps > 0):
            raise ConfigError("norm.eps must be positive")
        n = len(self.layers)
        if self.loop is not None:
            start, stop, times = self.loop
            if not (0 <= start <= stop <= n) or times < 1:
                raise ConfigError(f"loop {self.loop} does not fit {n} layers")
        for i, layer in enumerate(self.layer_records()):
            what = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {what}.type {kind!r} is not built (known: {', '.join(LAYER_TYPES)})")
            m = layer.get("mixer")
            if kind == "attention":
                self._check_attention(m, what + ".mixer")
            else:
                self._check_attention((m or {}).get("left"), what + ".mixer.left")
                right = (m or {}).get("right")
                for key in ("heads", "dim", "vdim"):
                    _pos_int(right, key, what + ".mixer.right")
                if not float(_get(right, "gate_cap", what + ".mixer.right")) > 0:
                    raise ConfigError(f"config.json: {what}.mixer.right.gate_cap must be positive")
                for key in ("left_scale", "right_scale"):
                    _get(m, key, what + ".mixer")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                _pos_int(mlp, "ff", what + ".mlp")
            elif mlp.get("kind") == "moe":
                r = mlp.get("router")
                E, top = _pos_int(r, "experts", what + ".mlp.router"), _pos_int(r, "top", what + ".mlp.router")
                _get(r, "scale", what + ".mlp.router")
                count, keep = 1, 1
                if r.get("groups") is not None:
                    count = _pos_int(r["groups"], "count", what + ".mlp.router.groups")
                    keep = _pos_int(r["groups"], "keep", what + ".mlp.router.groups")
                if E % count or keep > count or top > keep * (E // count):
                    raise ConfigError(f"config.json: {what}.mlp.router: top {top} of {E} experts in {count} groups of "
                                      f"which {keep} are kept")
                _pos_int(mlp.get("expert"), "ff", what + ".mlp.expert")
                if mlp.get("shared") is not None:
                    _pos_int(mlp["shared"], "ff", what + ".mlp.shared")
            else:
                raise ConfigError(f"config.json: {what}.mlp.kind {mlp.get('kind')!r} is not built (known: dense, moe)")

    # ---- the model as parts --------------------------------------------------------
    def _attention(self, m, left: bool):
        rot = m.get("rot") or {}
        position = NoPositionSpec()
        if rot.get("dims", 0):
            position = RopeSpec(head_dim=m["dim"], theta=float(rot["base"]), rotary_dim=int(rot["dims"]), freq64=True)
        return AttentionSpec(
            hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], position=position,
            qk_norm=RMSNormSpec(size=m["dim"], eps=self.eps), scale=float(m["scale"]), v_head_dim=int(m["vdim"]),
            names=("q", "k", "v", "o", "sink"), bias=("q", "k", "v") if left else (), bias_suffix=".b",
            gate="" if left else "head", gate_name="g", qk_norm_span="all" if left else "head",
            qk_norm_names=("q.norm", "k.norm"))

    def _mixer(self, kind, m):
        if kind == "attention":
            return self._attention(m, left=False)
        r = m["right"]
        memory = MLSTMSpec(hidden_size=self.width, num_heads=r["heads"], dim=r["dim"], vdim=r["vdim"],
                           gate_cap=float(r["gate_cap"]), eps=self.eps)
        return ParallelMixerSpec(left=self._attention(m["left"], left=True), right=memory,
                                 left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))

    def _ffn(self, mlp):
        D = self.width
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return DenseFFSpec(hidden_size=D, intermediate_size=mlp["ff"], activation="gelu")
        r = mlp["router"]
        groups = r.get("groups") or {}
        shared = mlp.get("shared")
        return MoESpec(hidden_size=D, experts=r["experts"], top=r["top"],
                       expert=GatedFFSpec(hidden_size=D, intermediate_size=mlp["expert"]["ff"], gate="silu"),
                       shared=None if shared is None else GatedFFSpec(hidden_size=D, intermediate_size=shared["ff"], gate="silu"),
                       score="sigmoid", groups=int(groups.get("count", 1)), group_keep=int(groups.get("keep", 1)),
                       group_top=GROUP_TOP, renormalize=False, route_scale=float(r["scale"]))

    def to_spec(self) -> ModelSpec:
        D = self.width

        def front():
            return RMSGainsSpec(size=D, eps=self.eps, names=("",), one_plus=True)

        def behind(gain, scale):
            return PostNormSpec(size=D, eps=self.eps, gain_name=gain, scale_name=scale, one_plus=True)

        layers = []
        for i, layer in enumerate(self.layer_records()):
            ffn = self._ffn(layer.get("mlp"))
            names = (("mixer_norm", f"l{i}.norm1"), ("mixer_link", f"l{i}."), ("mixer", f"l{i}.mix."),
                     ("ffn_norm", f"l{i}.norm2"), ("ffn_link", f"l{i}."), ("ffn", f"l{i}.mlp."))
            layers.append(SandwichLayerSpec(
                mixer=self._mixer(layer["type"], layer["mixer"]), mixer_norm=front(), mixer_link=behind("norm1b", "ls1"),
                ffn=ffn, ffn_norm=None if ffn is None else front(), ffn_link=None if ffn is None else behind("norm2b", "ls2"),
                names=names))
        n = len(layers)
        start, stop, times = self.loop if self.loop is not None else (0, 0, 0)
        if stop <= start:
            times = 0
        # every run of a layer has a cache entry of its own: a repeated layer shares weights, not keys or state
        order = [(i, -1) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else -1) for i in range(start, stop)]
        order += [(i, -1) for i in range(stop, n)]
        schedule = tuple(ScheduleEntry(layer=i, cache=run, enters=t) for run, (i, t) in enumerate(order))
        entry = PassMixSpec(passes=times, hidden_size=D, in_name=IN_NAME, step_name=STEP_NAME) if times else None
        return ModelSpec(
            architecture="Puratar", vocab_size=self.vocab, hidden_size=D, layers=tuple(layers), schedule=schedule,
            final_norm=front(), tie_embeddings=True, max_positions=MAX_POSITIONS, embedding_name="embed", head_name="embed",
            final_norm_prefix="final.norm", stop_ids=self.eos_token_ids, head_optional=False,
            embedding=EmbeddingSpec(self.vocab, D), head=HeadSpec(self.vocab, D, scale=self.logit_scale), pass_entry=entry)
