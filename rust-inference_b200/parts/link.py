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

from .. import ops
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


@register_link("post_norm")
class PostNormLink(Part):
    """A norm BEHIND the sublayer and a layer scale: x <- x + scale * (y / sqrt(mean(y^2) + eps) * gain) on a residual of
    one stream.  Like the connections above it computes nothing itself: it wraps the output (or the terms of a weighted
    sum, whose sum is taken first, in float32) together with gain * scale and eps, and the norm in front of the next
    sublayer norms and adds it in the pass in which it reads the residual."""
    graph_safe = True
    read = None

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.gain = None
        self._factors = {}

    @classmethod
    def param_infos(cls, spec):
        infos = {spec.gain_name: ParamInfo((spec.size,), "vector" if spec.one_plus else "gain")}
        if spec.scale_name:
            infos[spec.scale_name] = ParamInfo((spec.size,), "gain")
        return infos

    def load(self, tensors):
        g = tensors[self.spec.gain_name]
        if self.spec.one_plus:
            g = g + 1.0
        if self.spec.scale_name:
            g = g * tensors[self.spec.scale_name]
        self.gain = g.contiguous()

    def weight_bytes(self):
        return 0 if self.gain is None else 4 * self.gain.numel()

    def _factor(self, f: float):
        if f == 1.0:
            return None
        w = self._factors.get(f)
        if w is None:
            w = self._factors[f] = torch.full((1,), f, dtype=torch.float32, device=self.env.device)
        return w

    def pending(self, *outputs) -> Pending:
        terms = []
        for y in outputs:
            if y is None:
                continue
            if isinstance(y, WeightedSum):
                terms += [(t, self._factor(float(f))) for t, f in y.terms]
            else:
                terms.append((y, None))
        if not terms:
            raise ValueError("a sublayer without output")
        return Pending(terms[0][0], None, terms[0][1], tuple(terms[1:]), post=(self.gain, float(self.spec.eps)))


@register_link("pass_mix")
class PassMix(Part):
    """What a pass over a repeated run of layers does to the residual on entry: x <- W [x; x0] with x0 the embedding's
    output (the token's row of the table, read again), then + row t of a learned table [passes, hidden] for pass t.
    Order of work: whatever is still pending joins the residual, and the new residual's rows go, in the compute dtype,
    into the left half of a matrix [tokens, 2 hidden] (one launch of the norm kernel without a norm); the embedding's rows
    go into the right half; one product gives the new float32 residual; the pass's vector is left pending as an
    :class:`~.base.Injection`, which the norm in front of the pass's first layer adds in float32."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.passes < 1:
            raise ValueError(f"a repeated run has at least one pass, got {spec.passes}")
        self.w_in = self.steps = self.embedding = None

    @classmethod
    def param_infos(cls, spec):
        D = spec.hidden_size
        return {spec.in_name: ParamInfo((D, 2 * D)), spec.step_name: ParamInfo((spec.passes, D), "vector")}

    def load(self, tensors):
        self.w_in = tensors[self.spec.in_name].contiguous()
        self.steps = tensors[self.spec.step_name].contiguous()

    def weight_bytes(self):
        if self.w_in is None:
            return 0
        return self.spec.passes * self.w_in.numel() * self.w_in.element_size() + 4 * self.steps.numel()

    def bind(self, embedding) -> None:
        """The model's embedding part: rows of its ``table`` are the second half of the product's input."""
        if getattr(embedding.spec, "kind", "") != "embedding" or float(getattr(embedding.spec, "scale", 1.0)) != 1.0 \
                or getattr(embedding.spec, "copies", 1) != 1:
            raise ValueError("a pass that mixes the embedding's output in needs the plain embedding (no factor, one stream)")
        self.embedding = embedding

    def enter(self, resid, delta, t: int, ids):
        if not 0 <= t < self.spec.passes:
            raise ValueError(f"pass {t} of {self.spec.passes}")
        if resid.dim() != 2:
            raise ValueError("a pass that projects the residual needs a residual of one stream")
        terms, entry, post = [], None, None
        if isinstance(delta, Pending):
            if delta.mix is not None:
                raise ValueError("pass_mix reads a residual of one stream without mixing weights")
            if delta.y is not None:
                terms = [(delta.y, delta.out)] + list(delta.more)
            entry, post = delta.entry, delta.post
        elif delta is not None:
            terms = [(delta, None)]
        n, D = resid.shape
        both = torch.empty((n, 2 * D), dtype=self.env.dtype, device=resid.device)
        ops.rms_gains(resid, (), 0.0, self.env.dtype, terms=terms, entry=entry, post=post, out=both[:, :D])
        ops.embed_same(ids, self.embedding.table, both[:, D:])
        new = ops.linear(both, self.w_in, out_dtype=torch.float32)
        return new, Pending(None, entry=Injection(None, None, 1.0, self.steps[t]))


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

    def enter(self, resid, delta, t: int, ids):
        """(residual, what is pending) in front of the first layer of pass ``t``: the model calls this for every kind
        of pass entry."""
        return resid, self(delta, t, ids)

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
