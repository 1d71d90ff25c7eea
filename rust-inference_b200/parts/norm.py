"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * gain, all in float32
(thanhauco/rust-inference src/ops/norm.rs:7-62).  Reads the float32 residual
stream, adds the pending output of the previous part on the way if there is
one, and writes the normed rows in the compute dtype.

LayerNorm: y = (x - mean) / sqrt(var + eps) * gain (+ bias, where the record names one) with var
the mean squared deviation, float32.  It reads a residual of one or several streams ([tokens, dim] or
[tokens, streams, dim]): the pending output joins the streams by its connection's weights
(:class:`~.base.Pending`) and the row that is normed is the streams' weighted sum (``read``;
absent: their plain sum), all in the same kernel."""
from __future__ import annotations

from .. import ops
from ..profiler import section
from .base import Norm, Pending
from .registry import ParamInfo, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    takes_hint = True

    @classmethod
    def param_infos(cls, spec):
        return {"weight": ParamInfo((spec.size,), "gain")}

    def load(self, tensors):
        self.gain = tensors["weight"]

    def weight_bytes(self):
        return self.gain.numel() * 4

    def __call__(self, resid, delta=None, rows=None, then=None):
        with section("rmsnorm"):
            return ops.rmsnorm(resid, self.gain, self.spec.eps, self.env.dtype, delta=delta, rows=rows, then=then)


@register_norm("layernorm")
class LayerNorm(Norm):
    graph_safe = True
    takes_hint = True

    @classmethod
    def param_infos(cls, spec):
        infos = {spec.weight_name: ParamInfo((spec.size,), "gain")}
        if getattr(spec, "bias_name", ""):
            infos[spec.bias_name] = ParamInfo((spec.size,), "vector")
        return infos

    def load(self, tensors):
        self.gain = tensors[self.spec.weight_name]
        self.bias = tensors[self.spec.bias_name] if getattr(self.spec, "bias_name", "") else None

    def weight_bytes(self):
        return self.gain.numel() * 4 * (1 if getattr(self, "bias", None) is None else 2)

    def __call__(self, resid, delta=None, rows=None, then=None, read=None):
        streams = resid if resid.dim() == 3 else resid.view(resid.shape[0], 1, resid.shape[1])
        y = mix = out = None
        more = ()
        if isinstance(delta, Pending):
            y, mix, out, more = delta.y, delta.mix, delta.out, delta.more
        elif delta is not None:
            y = delta
        with section("layernorm"):
            return ops.stream_norm(streams, self.gain, self.spec.eps, self.env.dtype, "layernorm", delta=y, mix=mix,
                                   out_w=out, read=read, rows=rows, bias=self.bias, more=more)


@register_norm("rms_gains")
class RMSGains(Norm):
    """RMS norm of the (single-stream) residual with one gain per name of the record: one pass computes
    1 / sqrt(mean(x^2) + eps) once and writes x times it times every gain.  The pending outputs (up to two, the sum of
    the two taken first: x + (a + b)) and the terms of a pass's entry (:class:`~.base.Injection`) join in the same
    pass, in float32; outputs that come with a norm behind their sublayer (``Pending.post``) are normed on the way.
    ``one_plus``: the tensors hold the gains minus one, the gains are 1 + tensor.  Returns one tensor for one name, a tuple
    for several."""
    graph_safe = True
    takes_hint = True

    @classmethod
    def param_infos(cls, spec):
        # tensors that hold a gain minus one (``one_plus``) are drawn near 0 in the random-weights mode as well
        role = "vector" if getattr(spec, "one_plus", False) else "gain"
        return {name: ParamInfo((spec.size,), role) for name in spec.names}

    def load(self, tensors):
        self.gains = tuple(tensors[name] for name in self.spec.names)
        if getattr(self.spec, "one_plus", False):
            self.gains = tuple((g + 1.0).contiguous() for g in self.gains)
        if not 1 <= len(self.gains) <= 2:
            raise ValueError(f"rms_gains: {len(self.gains)} gains (one or two are built)")

    def weight_bytes(self):
        return sum(g.numel() * 4 for g in self.gains)

    def __call__(self, resid, delta=None, rows=None, then=None):
        terms, entry, post = [], None, None
        if isinstance(delta, Pending):
            post = delta.post
            if delta.mix is not None:
                raise ValueError("rms_gains reads a residual of one stream without mixing weights")
            if delta.y is not None:
                terms = [(delta.y, delta.out)] + list(delta.more)
            entry = delta.entry
        elif delta is not None:
            terms = [(delta, None)]
        if resid.dim() == 3:
            if resid.shape[1] != 1:
                raise ValueError("rms_gains reads a residual of one stream")
            resid = resid.view(resid.shape[0], resid.shape[2])
        with section("rmsnorm"):
            outs = ops.rms_gains(resid, self.gains, self.spec.eps, self.env.dtype, terms=terms, entry=entry, rows=rows,
                                 then=then, post=post)
        return outs[0] if len(outs) == 1 else outs
