"""How a sublayer meets the residual.

``hyper``: hyper-connections.  The residual is kept as S streams x_1 .. x_S (all equal to the embedding's output at
the start; the model's final norm reads their sum).  A sublayer reads u = sum_s in[s] x_s, and its output y turns
the streams, all at once from the old ones, into x_t <- sum_s mix[s, t] x_s + out[t] y (``mix`` is indexed
[from, to]).  The three tensors ``in`` [S], ``out`` [S] and ``mix`` [S, S] stay float32.  A record with
``learned`` False has no tensors and one stream: u = x and x <- x + scale * y, the ordinary residual sum (with the
record's constant ``scale``, 1 by default).

Several outputs may join at once (``pending(a, b)``: a layer whose mixer and feed-forward read the same norm), and an
output may itself be a weighted sum that has not been taken (:class:`~.base.WeightedSum`): every term is then added
with out[t] times its factor, in float32, in the order given.

The part computes nothing itself: the norm in front of the next sublayer does the update while it reads the streams
(``ops.stream_norm``); this part holds the weights and wraps an output as :class:`~.base.Pending`.
"""
from __future__ import annotations

import torch

from .base import Injection, Part, Pending, WeightedSum
from .registry import ParamInfo, register_link


@register_link("hyper")
class HyperConnection(Part):
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.streams < 1:
            raise ValueError(f"a residual needs at least one stream, got {spec.streams}")
        if not spec.learned and spec.streams != 1:
            raise ValueError("a connection without weights is the plain residual sum and has one stream")
        self.read = self.mix = self.out = None
        self._scaled = {}

    @classmethod
    def param_infos(cls, spec):
        if not spec.learned:
            return {}
        S = spec.streams
        return {"in": ParamInfo((S,), "gain"), "out": ParamInfo((S,), "gain"), "mix": ParamInfo((S, S), "gain")}

    def load(self, tensors):
        if self.spec.learned:
            self.read, self.out, self.mix = tensors["in"], tensors["out"], tensors["mix"].contiguous()
            self._scaled = {}

    def weight_bytes(self):
        return 0 if self.read is None else 4 * (self.read.numel() + self.out.numel() + self.mix.numel())

    def _out_times(self, factor: float):
        """The weights out[t] * factor (float32 [streams]); None stands for ones."""
        factor = float(factor) * float(getattr(self.spec, "scale", 1.0))
        if factor == 1.0:
            return self.out
        w = self._scaled.get(factor)
        if w is None:
            if self.out is None:
                w = torch.full((self.spec.streams,), factor, dtype=torch.float32, device=self.env.device)
            else:
                w = (self.out.double() * factor).float().contiguous()
            self._scaled[factor] = w
        return w

    def pending(self, *outputs) -> Pending:
        terms = []
        for y in outputs:
            if y is None:
                continue
            if isinstance(y, WeightedSum):
                terms += [(t, self._out_times(f)) for t, f in y.terms]
            else:
                terms.append((y, self._out_times(1.0)))
        if not terms:
            raise ValueError("a sublayer without output")
        return Pending(terms[0][0], self.mix, terms[0][1], tuple(terms[1:]))


@register_link("pass_entry")
class PassEntry(Part):
    """What a pass over a repeated run of layers adds to the residual on entry: for every pass but the first the
    embedding's output once more, and for every pass row t of a learned table [passes, hidden], in this order and in
    float32.  Like the connection above it computes nothing itself: it wraps whatever is pending together with these
    terms, and the norm in front of the pass's first layer adds them in the pass in which it reads the residual.
    The embedding's rows are taken from its table again (the token ids are at hand), not from a kept copy."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.passes < 1:
            raise ValueError(f"a repeated run has at least one pass, got {spec.passes}")
        self.steps = None
        self.embedding = None

    @classmethod
    def param_infos(cls, spec):
        return {spec.name: ParamInfo((spec.passes, spec.hidden_size), "vector")}

    def load(self, tensors):
        self.steps = tensors[self.spec.name].contiguous()

    def weight_bytes(self):
        return 0 if self.steps is None else 4 * self.steps.numel()

    def bind(self, embedding) -> None:
        """The model's embedding part: its ``table`` and the factor of its record are what is added again."""
        if self.spec.readd_embedding and getattr(embedding.spec, "kind", "") != "embedding":
            raise ValueError("a pass that adds the embedding's output again needs the plain (scaled) embedding")
        self.embedding = embedding

    def __call__(self, delta, t: int, ids) -> Pending:
        if not 0 <= t < self.spec.passes:
            raise ValueError(f"pass {t} of {self.spec.passes}")
        again = self.spec.readd_embedding and t > 0
        entry = Injection(ids if again else None, self.embedding.table if again else None,
                          float(getattr(self.embedding.spec, "scale", 1.0)) if again else 1.0, self.steps[t])
        if delta is None:
            return Pending(None, entry=entry)
        if isinstance(delta, Pending):
            if delta.entry is not None:
                raise ValueError("two entries of a pass in front of one layer")
            return Pending(delta.y, delta.mix, delta.out, delta.more, entry)
        return Pending(delta, entry=entry)
