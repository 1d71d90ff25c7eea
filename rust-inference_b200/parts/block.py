"""A layer: the arrangement of a mixer, a feed-forward and their norms.

"prenorm": each sub-layer reads the normed residual stream and its output is
added to the stream (thanhauco/rust-inference src/models/qwen3.rs:120-146).
The addition is left pending and done by the next norm while it reads the
stream, wherever that norm is: in this block or the next, or the model's final
norm.

An arrangement is a class registered with ``@register_block(kind)`` for the
``arrangement`` of its layer record.  It says which parts the layer has
(``slots``), builds them, and runs them::

    slots(spec) -> ((slot name, family, record), ...)        a class method; the slot name is what
                                                             ``spec.prefix(slot)`` maps to tensor names
    parts()     -> ((slot name, part, family, record), ...)  the built parts, same order
    mixer                                                    the part whose cache request sizes the layer's cache entry
    __call__(resid, delta, ctx, cache) -> (resid, delta)     the float32 stream and the output not yet added
"""
from __future__ import annotations

from .registry import build_part, part_class, register_block


class BlockBase:
    def __init__(self, spec, env):
        self.spec = spec
        self.env = env
        self._parts = tuple((name, build_part(family, record, env), family, record)
                            for name, family, record in self.slots(spec))
        for name, part, _, _ in self._parts:
            setattr(self, name, part)

    @classmethod
    def slots(cls, spec):
        raise NotImplementedError

    def parts(self):
        return self._parts

    def __call__(self, resid, delta, ctx, cache):
        raise NotImplementedError


@register_block("prenorm")
class PreNormBlock(BlockBase):
    @classmethod
    def slots(cls, spec):
        return (("mixer_norm", "norm", spec.mixer_norm), ("mixer", "mixer", spec.mixer),
                ("ffn_norm", "norm", spec.ffn_norm), ("ffn", "ffn", spec.ffn))

    def __call__(self, resid, delta, ctx, cache):
        x = norm_before(self.mixer_norm, resid, delta, self.mixer)
        a = self.mixer(x, ctx, cache)
        x = norm_before(self.ffn_norm, resid, a, self.ffn)
        return resid, self.ffn(x, ctx)


@register_block("streams")
class StreamBlock(BlockBase):
    """A pre-norm layer over a residual of one or several streams [tokens, streams, width]: each sublayer reads the
    norm of the streams' weighted sum and its output joins the streams by its connection's weights (``parts/link.py``).
    The feed-forward half is optional.  The update is left pending, as in "prenorm": the next norm does it."""

    @classmethod
    def slots(cls, spec):
        out = [("mixer_norm", "norm", spec.mixer_norm), ("mixer_link", "link", spec.mixer_link),
               ("mixer", "mixer", spec.mixer)]
        if spec.ffn is not None:
            out += [("ffn_norm", "norm", spec.ffn_norm), ("ffn_link", "link", spec.ffn_link), ("ffn", "ffn", spec.ffn)]
        return tuple(out)

    def __call__(self, resid, delta, ctx, cache):
        x = self.mixer_norm(resid, delta, read=self.mixer_link.read)
        delta = self.mixer_link.pending(self.mixer(x, ctx, cache))
        if self.spec.ffn is None:
            return resid, delta
        x = self.ffn_norm(resid, delta, read=self.ffn_link.read)
        return resid, self.ffn_link.pending(self.ffn(x, ctx))


@register_block("parallel")
class ParallelBlock(BlockBase):
    """One norm whose output the mixer and the feed-forward (optional) both read; their outputs join the residual
    together, through the layer's connection (``parts/link.py``): x <- x + scale * (mixer(h) + ffn(h)) for a
    connection without weights.  The sum is taken in float32 by the next norm, term by term."""

    @classmethod
    def slots(cls, spec):
        out = [("norm", "norm", spec.norm), ("link", "link", spec.link), ("mixer", "mixer", spec.mixer)]
        if spec.ffn is not None:
            out.append(("ffn", "ffn", spec.ffn))
        return tuple(out)

    def __call__(self, resid, delta, ctx, cache):
        x = self.norm(resid, delta, read=self.link.read)
        a = self.mixer(x, ctx, cache)
        f = self.ffn(x, ctx) if self.spec.ffn is not None else None
        return resid, self.link.pending(a, f)


@register_block("parallel_norms")
class ParallelNormsBlock(BlockBase):
    """A mixer and a feed-forward (optional) side by side, each behind a gain of its own over the one RMS statistic of
    the same residual: x <- x + (mixer(x r g1) + ffn(x r g2)).  One norm part (``rms_gains``) gives both inputs from one
    pass; the outputs join the residual together through the layer's connection, in float32, in the next norm."""

    @classmethod
    def slots(cls, spec):
        out = [("norms", "norm", spec.norms), ("link", "link", spec.link), ("mixer", "mixer", spec.mixer)]
        if spec.ffn is not None:
            out.append(("ffn", "ffn", spec.ffn))
        return tuple(out)

    def __call__(self, resid, delta, ctx, cache):
        xs = self.norms(resid, delta, None, self.mixer.reads_first())
        if self.spec.ffn is None:
            return resid, self.link.pending(self.mixer(xs, ctx, cache))
        a = self.mixer(xs[0], ctx, cache)
        return resid, self.link.pending(a, self.ffn(xs[1], ctx))


@register_block("sandwich")
class SandwichBlock(BlockBase):
    """A norm in front of and behind each sublayer: x <- x + link1(mixer(norm1(x))), x <- x + link2(ffn(norm2(x))), the
    links being norms with a layer scale (``post_norm`` in ``parts/link.py``).  The feed-forward half is optional.  As in
    the other arrangements an output is left pending: the norm in front of the next sublayer norms it, scales it, adds
    it and norms the new residual in one pass."""

    @classmethod
    def slots(cls, spec):
        out = [("mixer_norm", "norm", spec.mixer_norm), ("mixer_link", "link", spec.mixer_link),
               ("mixer", "mixer", spec.mixer)]
        if spec.ffn is not None:
            out += [("ffn_norm", "norm", spec.ffn_norm), ("ffn_link", "link", spec.ffn_link), ("ffn", "ffn", spec.ffn)]
        return tuple(out)

    def __call__(self, resid, delta, ctx, cache):
        x = norm_before(self.mixer_norm, resid, delta, self.mixer)
        delta = self.mixer_link.pending(self.mixer(x, ctx, cache))
        if self.spec.ffn is None:
            return resid, delta
        x = norm_before(self.ffn_norm, resid, delta, self.ffn)
        return resid, self.ffn_link.pending(self.ffn(x, ctx))


def norm_before(norm, resid, delta, reader):
    """``norm(resid + delta)`` for the part ``reader``; a norm that takes hints is told which matrix is read next."""
    if norm.takes_hint:
        return norm(resid, delta, None, reader.reads_first())
    return norm(resid, delta)


def build_block(spec, env):
    """The block of a layer record: the class registered for its ``arrangement``."""
    return part_class("block", spec)(spec, env)
