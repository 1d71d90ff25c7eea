"""Descriptions of a model as data: which parts, with which sizes, in which order.

An architecture (see ``models/``) turns its ``config.json`` into a
:class:`ModelSpec`.  Everything below the architecture works from these
records only: the part factories in ``parts/`` build one object per record,
the cache reads the mixers' storage needs from them, and the engine runs the
``schedule``.  No record knows which model it belongs to, and no size lives
anywhere but here.

A record names its part by ``kind``; ``parts.registry`` maps kinds to classes,
so a new mixer, feed-forward, norm or position encoding is a new record class
plus a registered part class, with no change to existing files.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class RMSNormSpec:
    """y = x / sqrt(mean(x^2) + eps) * gain over ``size`` elements."""
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RMSGainsSpec:
    """One RMS statistic, several gains: y_k = x / sqrt(mean(x^2) + eps) * gain_k for every name in ``names`` (the
    gains' local tensor names; an empty name is the norm's prefix alone).  The sublayers of a layer that all read
    the same residual through norms of their own get their inputs from one pass over it.  ``one_plus``: the tensors
    hold the gains minus one: the gain is 1 + tensor."""
    size: int
    eps: float
    names: Tuple[str, ...] = ("",)
    kind: str = "rms_gains"
    one_plus: bool = False


@dataclass(frozen=True)
class LayerNormSpec:
    """y = (x - mean) / sqrt(var + eps) * gain (+ bias) over ``size`` elements, var the mean squared deviation.

    ``weight_name`` is the local name of the gain tensor; empty where the checkpoint names that tensor by the
    norm's prefix alone.  ``bias_name``: the local name of the bias tensor; empty for a norm without bias."""
    size: int
    eps: float
    weight_name: str = "weight"
    kind: str = "layernorm"
    bias_name: str = ""


@dataclass(frozen=True)
class RopePairsSpec:
    """Rotary encoding of neighbouring pairs: elements 2i and 2i+1 of the first ``rotary_dim`` of a vector are turned
    by position * f_i with f_i = theta^(-2i/rotary_dim).

    ``yarn`` (None for none) holds (factor, original, fast, slow): with
    d(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is
    f_i / factor * ramp_i + f_i * (1 - ramp_i), and cos and sin are both multiplied by 0.1 ln(factor) + 1.

    ``by_wavelength`` (None for none) holds (factor, low, high, original): with the wavelength w_i = 2 pi / f_i a
    frequency stays as it is where w_i < original / high, becomes f_i / factor where w_i > original / low, and between
    the two is (1 - s) f_i / factor + s f_i with s = (original / w_i - low) / (high - low).  At most one of the two."""
    rotary_dim: int
    theta: float
    yarn: Optional[Tuple[float, float, float, float]] = None
    kind: str = "rope_pairs"
    by_wavelength: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary encoding of the first ``rotary_dim`` elements of a head.

    ``theta`` is the base; angles are float32(position) * float32(inv_freq) and
    ``scaling`` multiplies cos and sin (1.0 for the "default" rope type).  ``freq64``: the frequencies
    theta^(-2i/rotary_dim) are evaluated in float64 and rounded to float32 once (default: float32 power).
    """
    head_dim: int
    theta: float
    rotary_dim: int = 0          # 0 means the whole head
    scaling: float = 1.0
    kind: str = "rope"
    freq64: bool = False

    @property
    def rot(self) -> int:
        return self.rotary_dim or self.head_dim


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding inside the mixer."""
    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a key/value cache.

    ``qk_norm`` is the per-head norm applied to queries and keys before the
    position encoding (None for none); ``window`` > 0 limits a query to the last
    ``window`` keys; ``scale`` 0 means 1/sqrt(head_dim).  ``chunk`` > 0 (instead of a window): a query sees the
    keys of its own chunk of that many positions, chunks counted from the sequence's start.  ``sink``: a learned
    term per head in the softmax's denominator, with no key and no value.  ``v_head_dim`` > 0: values (and the
    heads' outputs) have that size instead of ``head_dim``.  ``names``: the tensors' local names as
    (q, k, v, o, sink) where they are not the default ones.

    ``bias``: which of the projections "q", "k", "v" have a bias (tensor: the matrix's name plus ``bias_suffix``).
    ``values``: "own" (a projection of their own) or "keys" (the values are the keys as cached: no v tensor, one pool).
    ``unit_rms``: queries and keys are divided by their root mean square over the head (eps ``unit_eps``, no gain)
    AFTER the position encoding.  ``softcap`` > 0: score <- softcap * tanh(score / softcap) after the scale.
    ``gate``: "element" multiplies the heads' outputs element by element with the sigmoid of a projection of the
    mixer's input (tensor ``gate_name``) before the output projection; "head": one such gate per head (a projection
    of ``num_heads`` rows); "" for none.
    ``qk_norm_span``: "head" (the norm runs over each head's elements, one gain of the head's size for all heads) or
    "all" (over the whole q projection, and the whole k projection, of a token at once, gains of those sizes);
    ``qk_norm_names``: the two gains' local tensor names.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: object = NoPositionSpec()
    qk_norm: Optional[RMSNormSpec] = None
    window: int = 0
    scale: float = 0.0
    kind: str = "attention"
    chunk: int = 0
    sink: bool = False
    v_head_dim: int = 0
    names: Tuple[str, ...] = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "sink")
    bias: Tuple[str, ...] = ()
    bias_suffix: str = ".b"
    values: str = "own"
    unit_rms: bool = False
    unit_eps: float = 0.0
    softcap: float = 0.0
    gate: str = ""
    gate_name: str = "g"
    qk_norm_span: str = "head"
    qk_norm_names: Tuple[str, str] = ("q_norm.weight", "k_norm.weight")


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are expanded from a cached latent.

    Per head ``dim`` query/key elements without position and ``rot_dim`` with (``position`` turns them), values of
    ``vdim``; the token's cache row is the RMS-normed latent (``kv_rank``, gain and ``eps``) and one rotated key part
    that all heads share.  ``scale`` multiplies the whole score; ``window`` > 0 limits a query to the last
    ``window`` keys; ``sink``: a learned term per head in the softmax's denominator; ``gate``: "head" (one sigmoid
    gate per head), "element" (one per output element) or "" (none), from a projection of the mixer's input."""
    hidden_size: int
    num_heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    eps: float
    position: object = NoPositionSpec()
    window: int = 0
    sink: bool = False
    gate: str = ""
    kind: str = "latent_attention"


@dataclass(frozen=True)
class GLASpec:
    """Gated linear attention: per head a state [dim, vdim] that each token decays per key channel
    (sigmoid(low-rank projection + bias)^(1/tau)), feeds with k v^T and reads with q / sqrt(dim); the heads'
    outputs are RMS-normed over ``vdim`` (one gain for all heads, ``eps``), gated with silu of a projection and
    projected back.  ``decay_rank`` is the inner size of the decay's two projections."""
    hidden_size: int
    num_heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int
    eps: float
    kind: str = "gla"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule: per head a state [dim, vdim] that each token decays per key channel, corrects towards
    its value along its key (with strength beta) and reads with its query.  ``num_heads`` value heads share
    ``num_qk_heads`` query/key heads; q, k and v pass a causal convolution of ``conv`` taps per channel and silu, q and
    k are made unit vectors; the decay comes from a low-rank projection (inner size ``decay_rank``), a bias and a rate
    per head; the heads' outputs are RMS-normed over ``vdim`` (one gain for all heads, ``eps``) and gated with the
    sigmoid of another low-rank projection (``gate_rank``)."""
    hidden_size: int
    num_heads: int
    num_qk_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int
    gate_rank: int
    eps: float
    kind: str = "gated_delta"


@dataclass(frozen=True)
class MLSTMSpec:
    """The matrix memory of xLSTM: per head a state S [dim, vdim], a vector n [dim] and a running maximum m, all
    float32.  With log input and forget gates li = cap tanh((Wi h + bi) / cap), lf = log_sigmoid(cap tanh((Wf h + bf) /
    cap)) (``gate_cap``): m_t = max(lf + m_(t-1), li), S_t = exp(lf + m_(t-1) - m_t) S_(t-1) + exp(li - m_t) k v^T, n_t
    likewise with k alone, o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6) with q scaled by dim^(-1/2).  Each head's o is
    divided by its root mean square (``eps``), the heads' concatenation multiplied by a gain of that size and by the
    sigmoid of a projection, and projected back."""
    hidden_size: int
    num_heads: int
    dim: int
    vdim: int
    gate_cap: float
    eps: float
    kind: str = "mlstm"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side on the same input: ``left_scale`` * left + ``right_scale`` * right.  Their tensors
    carry the prefixes "left." and "right."."""
    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0
    kind: str = "parallel"


@dataclass(frozen=True)
class GatedFFSpec:
    """down(f(gate x) * up x), no biases; ``gate``: "silu", "gelu_tanh", or "clamped_swish"
    (g sigmoid(alpha g) (u + 1) with g = min(gate x, limit) and u = clamp(up x, -limit, limit))."""
    hidden_size: int
    intermediate_size: int
    gate: str = "gelu_tanh"
    limit: float = 0.0
    alpha: float = 1.702
    kind: str = "gated"


@dataclass(frozen=True)
class MoESpec:
    """A routed feed-forward: ``experts`` gated feed-forwards (record ``expert``, tensors "e<i>.") of which a token
    uses ``top``; the router also has ``identity`` outputs after the experts' whose "expert" returns its input.
    Scores are the softmax over all router outputs; the choice adds a learned correction to them, the weights are the
    chosen scores divided by their sum.  ``shared`` (or None): a feed-forward that every token takes, added.

    ``score`` "sigmoid": a score is the sigmoid of its router output alone.  ``groups`` > 1: the router's outputs form
    that many equal groups of neighbours; a group's score is the sum of its ``group_top`` largest choice scores (score
    plus correction), and only experts of the ``group_keep`` best groups can be chosen.  ``renormalize`` False: the
    weights are the chosen scores as they are; ``route_scale`` multiplies them."""
    hidden_size: int
    experts: int
    top: int
    expert: object
    identity: int = 0
    shared: object = None
    kind: str = "moe"
    score: str = "softmax"
    groups: int = 1
    group_keep: int = 1
    group_top: int = 2
    renormalize: bool = True
    route_scale: float = 1.0


@dataclass(frozen=True)
class DenseFFSpec:
    """down(act(up x)), no biases; ``activation``: "relu2" (the square of relu), "gelu_tanh" or "gelu" (the exact
    form with erf)."""
    hidden_size: int
    intermediate_size: int
    activation: str = "relu2"
    kind: str = "dense"


@dataclass(frozen=True)
class HyperConnectionSpec:
    """How a sublayer meets a residual kept as ``streams`` copies: it reads sum_s in[s] x_s, and its output y
    turns the streams into x_t <- sum_s mix[s, t] x_s + out[t] y.  ``learned`` False: no tensors, in = out = [1]
    and mix = [[1]] on one stream, which is the ordinary residual sum."""
    streams: int
    learned: bool = True
    kind: str = "hyper"
    scale: float = 1.0          # without weights: x <- x + scale * y


@dataclass(frozen=True)
class PostNormSpec:
    """How a sublayer's output joins a single-stream residual when a norm stands BEHIND the sublayer:
    x <- x + scale * (y / sqrt(mean(y^2) + eps) * gain), y the sublayer's output (a weighted sum of several outputs is
    taken first).  ``gain_name``: the gain's tensor; ``one_plus``: it holds the gain minus one (gain = 1 + tensor);
    ``scale_name``: a vector of the residual's size that multiplies the normed output element by element (a layer
    scale), "" for none."""
    size: int
    eps: float
    gain_name: str
    scale_name: str = ""
    one_plus: bool = False
    kind: str = "post_norm"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(silu(gate x) * up x), no biases."""
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class EmbeddingSpec:
    """h[t] = table[ids[t]] * scale; ``copies`` > 1: [tokens, copies, hidden] with every row that many times
    (a residual kept as several streams starts with all of them equal)."""
    vocab_size: int
    hidden_size: int
    kind: str = "embedding"
    scale: float = 1.0
    copies: int = 1


@dataclass(frozen=True)
class PairHashEmbeddingSpec:
    """h[t] = table[ids[t]] + pairs[(ids[t-1] * mul_prev + ids[t] * mul_cur) mod buckets]; a sequence's first token
    takes row ``buckets`` of ``pairs`` [buckets + 1, hidden].  The previous token is per-sequence state.
    ``pairs_name``: the pair table's tensor name."""
    vocab_size: int
    hidden_size: int
    buckets: int
    mul_prev: int
    mul_cur: int
    pairs_name: str = "bigram"
    kind: str = "pair_hash"


@dataclass(frozen=True)
class HeadSpec:
    """logits = x W^T * scale in float32, no bias; W may be the embedding table (tied).  ``softcap`` > 0:
    logits <- softcap * tanh(logits / softcap) afterwards."""
    vocab_size: int
    hidden_size: int
    kind: str = "linear"
    scale: float = 1.0
    softcap: float = 0.0


@dataclass(frozen=True)
class LayerSpec:
    """One block: two sub-layers, each a norm followed by a part, each added to
    the residual stream (``arrangement`` "prenorm").

    ``names`` maps the block's four parts to the prefixes their tensors carry in
    the checkpoint, e.g. {"mixer": "model.layers.0.self_attn."}.

    A layer with another arrangement is another record class: it needs
    ``arrangement`` (the kind its block class is registered for) and
    ``prefix(part)``; which parts it has is for its block class to say.
    """
    mixer: object
    ffn: object
    mixer_norm: object
    ffn_norm: object
    names: Tuple[Tuple[str, str], ...] = ()
    arrangement: str = "prenorm"

    def prefix(self, part: str) -> str:
        return dict(self.names)[part]


@dataclass(frozen=True)
class StreamLayerSpec:
    """One block over a residual of one or several streams (``arrangement`` "streams"): a norm and a mixer, then
    (``ffn`` not None) a norm and a feed-forward, each met through its connection record (``mixer_link``,
    ``ffn_link``: :class:`HyperConnectionSpec`).  ``names`` maps the parts to the prefixes of their tensors."""
    mixer: object
    mixer_norm: object
    mixer_link: object
    ffn: object = None
    ffn_norm: object = None
    ffn_link: object = None
    names: Tuple[Tuple[str, str], ...] = ()
    arrangement: str = "streams"

    def prefix(self, part: str) -> str:
        return dict(self.names)[part]


@dataclass(frozen=True)
class ParallelLayerSpec:
    """One block whose mixer and feed-forward (``ffn`` None: none) both read the one norm's output, and whose outputs
    join the residual together through ``link`` (``arrangement`` "parallel").  ``names`` maps the parts ("norm",
    "mixer", "ffn", "link") to the prefixes of their tensors."""
    mixer: object
    norm: object
    link: object
    ffn: object = None
    names: Tuple[Tuple[str, str], ...] = ()
    arrangement: str = "parallel"

    def prefix(self, part: str) -> str:
        return dict(self.names).get(part, "")


@dataclass(frozen=True)
class ParallelNormsLayerSpec:
    """One block whose mixer and feed-forward (``ffn`` None: none) read the SAME residual, each through a gain of its
    own over the one RMS statistic (``norms``: an :class:`RMSGainsSpec` with one name per sublayer), and whose outputs
    join the residual together through ``link``: x <- x + (mixer(n1(x)) + ffn(n2(x))) (``arrangement``
    "parallel_norms").  ``names`` maps the parts ("norms", "mixer", "ffn", "link") to the prefixes of their tensors."""
    mixer: object
    norms: object
    link: object
    ffn: object = None
    names: Tuple[Tuple[str, str], ...] = ()
    arrangement: str = "parallel_norms"

    def prefix(self, part: str) -> str:
        return dict(self.names).get(part, "")


@dataclass(frozen=True)
class SandwichLayerSpec:
    """One block with a norm in front of and behind each sublayer (``arrangement`` "sandwich"):
    x <- x + link1(mixer(norm1(x))), then (``ffn`` not None) x <- x + link2(ffn(norm2(x))).  ``mixer_norm`` and
    ``ffn_norm`` are norms in front (:class:`RMSGainsSpec` with one name), ``mixer_link`` and ``ffn_link`` the norms
    behind with their layer scales (:class:`PostNormSpec`).  ``names`` maps the parts to the prefixes of their tensors."""
    mixer: object
    mixer_norm: object
    mixer_link: object
    ffn: object = None
    ffn_norm: object = None
    ffn_link: object = None
    names: Tuple[Tuple[str, str], ...] = ()
    arrangement: str = "sandwich"

    def prefix(self, part: str) -> str:
        return dict(self.names).get(part, "")


@dataclass(frozen=True)
class PassMixSpec:
    """What happens to the residual right before the first layer of a pass over a repeated run of layers: it is
    replaced by a projection of itself and the embedding's output side by side, x <- W [x; x0] (tensor ``in_name``
    [hidden, 2 hidden], x first), and then row t of the tensor ``step_name`` [passes, hidden] is added for pass t."""
    passes: int
    hidden_size: int
    in_name: str = "loop.in"
    step_name: str = "loop.step"
    kind: str = "pass_mix"


@dataclass(frozen=True)
class PassEntrySpec:
    """What joins the residual right before the first layer of a pass over a repeated run of layers: the embedding's
    output once more (``readd_embedding``, for every pass but the first) and then row t of the tensor ``name``
    [passes, hidden] for pass t (every pass)."""
    passes: int
    hidden_size: int
    readd_embedding: bool = True
    name: str = "loop.step"
    kind: str = "pass_entry"


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  ``layer`` indexes ``ModelSpec.layers``;
    ``cache`` names the cache entry (an index into the list of cache entries)
    that this execution reads, and ``writes`` says whether it also appends to
    it.  Two entries may name the same layer (weights shared) or the same cache
    (a layer that reads what another layer wrote).  ``enters`` >= 0: this execution is the first of pass
    ``enters`` over a repeated run, and the model's ``pass_entry`` part adds its terms to the residual right before it."""
    layer: int
    cache: int
    writes: bool = True
    enters: int = -1


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    tie_embeddings: bool
    max_positions: int
    embedding_name: str = "model.embed_tokens.weight"
    head_name: str = "lm_head.weight"
    final_norm_prefix: str = "model.norm."
    stop_ids: Tuple[int, ...] = ()
    # a head tensor that is absent from the checkpoint means tied embeddings
    head_optional: bool = True
    # records of the embedding and of the output head (None: the plain table and the plain linear head);
    # the tensor "weight" of each carries ``embedding_name`` / ``head_name``, further tensors the same
    # name with "weight" replaced by theirs
    embedding: object = None
    head: object = None
    # tensors of the embedding or the head whose names do not derive from ``embedding_name`` / ``head_name``:
    # (local name, full name) pairs
    end_names: Tuple[Tuple[str, str], ...] = ()
    # what a pass over a repeated run of layers does on entry (a :class:`PassEntrySpec`: terms that are added; a
    # :class:`PassMixSpec`: a projection of the residual beside the embedding's output; None: nothing); the
    # schedule entries with ``enters`` >= 0 say where
    pass_entry: object = None

    def embedding_record(self):
        return self.embedding or EmbeddingSpec(self.vocab_size, self.hidden_size)

    def head_record(self):
        return self.head or HeadSpec(self.vocab_size, self.hidden_size)

    def cache_entries(self):
        """For every cache entry, the layer whose mixer decides its storage: the
        (first) scheduled execution that writes it."""
        owners = {}
        for e in self.schedule:
            if e.writes and e.cache not in owners:
                owners[e.cache] = e.layer
        for e in self.schedule:
            if e.cache not in owners:
                raise ValueError(f"schedule reads cache {e.cache} that no layer writes")
        n = max(owners) + 1 if owners else 0
        if sorted(owners) != list(range(n)):
            raise ValueError("cache indices of the schedule must be 0..n-1 without gaps")
        return [owners[i] for i in range(n)]
