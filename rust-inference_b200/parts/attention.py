"""Causal grouped-query attention over the paged cache.

Order of work, as in thanhauco/rust-inference src/models/qwen3.rs:71-100:
q/k/v projections (one product with the stacked matrix), per-head RMSNorm of q
and k, position encoding, append k and v to the cache, attention over the
cache, output projection.  Norm, rotation and append are one kernel.

Sizes, the window (or the chunked mask), the scale, the per-head norm, the sink term and the
position encoding all come from the spec; the part does not know which model it is in.

Values of another size than the keys (``v_head_dim``): the kernels work with one head size, so the
part runs them at Dp = the larger of the two rounded up to 16 and pads at load: the query, key and
value matrices get zero rows (a zero query element times a zero key element adds exactly 0 to a
score), the output matrix zero columns.  Nothing of the padding reaches a result.

Further options of the record, each a field with its constants: biases on the q/k/v projections
(added in float32 by the kernel that rotates and appends), values that are the keys as cached
(no v tensor, one pool), queries and keys divided by their root mean square AFTER the rotation
(no gain), a soft-cap on the scores, and a sigmoid gate per output element from a projection of
the mixer's input (or one gate per head), stacked into the q/k/v product; a norm of queries and keys
before the rotation that runs over the whole projection of a token instead of over each head.  A record
that uses any of them (or a per-head norm together with values of another size) runs the
"extended" order of work: one product for q, k, (v), (gate); ``ops.qkv_prep`` (bias, rotation,
unit norm, append); attention; gate; output projection.  Heads are then always padded to a
multiple of 16 elements, so that the tensor-core kernels take every size.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..profiler import section
from .base import CacheRequest, Mixer, PositionEncoding
from .registry import ParamInfo, build_part, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are not a multiple of {spec.num_kv_heads} kv heads")
        if spec.qk_norm is not None and getattr(spec.qk_norm, "kind", None) != "rmsnorm":
            raise ValueError(f"the attention part norms its heads with RMSNorm inside its kernel; a per-head norm of kind "
                             f"{getattr(spec.qk_norm, 'kind', None)!r} is not built")
        self.position = build_part("position", spec.position, env)
        self.scale = spec.scale or 1.0 / math.sqrt(spec.head_dim)
        self.q_gain = self.k_gain = self.sink = None
        self.Dk, self.Dv = spec.head_dim, (spec.v_head_dim or spec.head_dim)
        self.Dp = self.Dk if self.Dk == self.Dv else -(-max(self.Dk, self.Dv) // 16) * 16
        self.norm_span = getattr(spec, "qk_norm_span", "head") if spec.qk_norm is not None else ""
        if self.norm_span not in ("", "head", "all"):
            raise ValueError(f"qk_norm_span {self.norm_span!r}: 'head' or 'all'")
        if spec.window and spec.chunk:
            raise ValueError("an attention layer has a window or a chunked mask, not both")
        self.rot = getattr(spec.position, "rot", None) or getattr(spec.position, "rotary_dim", 0)
        if self.rot > self.Dk:
            raise ValueError(f"{self.rot} rotated elements in heads of {self.Dk}")
        self.bias_of = tuple(getattr(spec, "bias", ()) or ())
        self.keys_are_values = getattr(spec, "values", "own") == "keys"
        self.unit_rms = bool(getattr(spec, "unit_rms", False))
        self.softcap = float(getattr(spec, "softcap", 0.0) or 0.0)
        self.gated = getattr(spec, "gate", "") or ""
        if getattr(spec, "values", "own") not in ("own", "keys"):
            raise ValueError(f"values {spec.values!r}: 'own' or 'keys'")
        if self.gated not in ("", "element", "head"):
            raise ValueError(f"gate {self.gated!r} is not built (known: element, head)")
        if set(self.bias_of) - {"q", "k", "v"}:
            raise ValueError(f"biases {self.bias_of}: of q, k, v")
        self.extended = bool(self.bias_of or self.keys_are_values or self.unit_rms or self.softcap or self.gated
                             or self.norm_span == "all" or (self.norm_span and self.Dp != self.Dk))
        if self.extended:
            if spec.sink or spec.chunk:
                raise ValueError("the extended attention options do not combine with a sink or a chunked mask")
            if self.keys_are_values and self.Dv != self.Dk:
                raise ValueError(f"values that are the keys have the keys' size {self.Dk}, not {self.Dv}")
            self.Dp = -(-max(self.Dk, self.Dv) // 16) * 16
            self.bias = None

    @classmethod
    def param_infos(cls, spec):
        D, H, KV, Dh = spec.hidden_size, spec.num_heads, spec.num_kv_heads, spec.head_dim
        Dv = spec.v_head_dim or Dh
        q, k, v, o, sink = spec.names
        infos = {q: ParamInfo((H * Dh, D)), k: ParamInfo((KV * Dh, D)), v: ParamInfo((KV * Dv, D)), o: ParamInfo((D, H * Dv))}
        if getattr(spec, "values", "own") == "keys":
            del infos[v]
        suffix = getattr(spec, "bias_suffix", ".b")
        for which, name in (("q", q), ("k", k), ("v", v)):
            if which in (getattr(spec, "bias", ()) or ()) and name in infos:
                infos[name + suffix] = ParamInfo(infos[name].shape[:1], "vector")
        if getattr(spec, "gate", ""):
            infos[spec.gate_name] = ParamInfo((H if spec.gate == "head" else H * Dv, D))
        if spec.qk_norm is not None:
            qn, kn = getattr(spec, "qk_norm_names", ("q_norm.weight", "k_norm.weight"))
            whole = getattr(spec, "qk_norm_span", "head") == "all"
            infos[qn] = ParamInfo((H * Dh if whole else Dh,), "gain")
            infos[kn] = ParamInfo((KV * Dh if whole else Dh,), "gain")
        if spec.sink:
            infos[sink] = ParamInfo((H,), "vector")
        return infos

    def load(self, tensors):
        s = self.spec
        q, k, v, o, sink = s.names
        D, Dp = s.hidden_size, self.Dp

        def rows(t, heads, size):          # [heads * size, D] -> [heads * Dp, D] with zero rows after each head's own
            if size == Dp:
                return t
            out = t.new_zeros((heads, Dp, D))
            out[:, :size] = t.view(heads, size, D)
            return out.view(heads * Dp, D)

        blocks = [rows(tensors[q], s.num_heads, self.Dk), rows(tensors[k], s.num_kv_heads, self.Dk)]
        if not self.keys_are_values:
            blocks.append(rows(tensors[v], s.num_kv_heads, self.Dv))
        if self.gated == "element":
            blocks.append(rows(tensors[s.gate_name], s.num_heads, self.Dv))
        elif self.gated == "head":
            # one row per head, then zero rows up to a multiple of 8: the product's rows stay whole 16-byte pieces
            g = tensors[s.gate_name]
            blocks.append(g)
            if g.shape[0] % 8:
                blocks.append(g.new_zeros((8 - g.shape[0] % 8, D)))
        self.qkv = torch.cat(blocks, dim=0).contiguous()
        if self.extended:
            # the columns of the product: q heads, k heads, v heads (unless the keys serve), gate; the biases as one
            # float32 vector over the q/k/v columns, zero where a projection has none and in the padding
            H, KV = s.num_heads, s.num_kv_heads
            self.k_col = H * Dp
            self.v_col = -1 if self.keys_are_values else (H + KV) * Dp
            self.g_col = (H + KV + (0 if self.keys_are_values else KV)) * Dp
            self.bias = None
            if self.bias_of:
                bias = torch.zeros(self.g_col, dtype=torch.float32, device=self.qkv.device)
                for which, name, col, heads, size in (("q", q, 0, H, self.Dk), ("k", k, self.k_col, KV, self.Dk),
                                                      ("v", v, self.v_col, KV, self.Dv)):
                    if which in self.bias_of and col >= 0:
                        bias[col:col + heads * Dp].view(heads, Dp)[:, :size] = tensors[name + s.bias_suffix].float().view(heads, size)
                self.bias = bias
        wo = tensors[o]
        if self.Dv != Dp:
            padded = wo.new_zeros((D, s.num_heads, Dp))
            padded[:, :, :self.Dv] = wo.view(D, s.num_heads, self.Dv)
            wo = padded.view(D, s.num_heads * Dp)
        self.o = wo.contiguous()
        if s.qk_norm is not None:
            qn, kn = getattr(s, "qk_norm_names", ("q_norm.weight", "k_norm.weight"))
            self.q_gain, self.k_gain = tensors[qn], tensors[kn]
            if self.extended:
                # the kernel indexes the gains by the padded head's column: zeros in the padding
                def padded(g, heads):
                    if self.norm_span == "head":
                        out = g.new_zeros((Dp,))
                        out[:self.Dk] = g
                    else:
                        out = g.new_zeros((heads, Dp))
                        out[:, :self.Dk] = g.view(heads, self.Dk)
                    return out.contiguous()
                self.q_gain, self.k_gain = padded(self.q_gain, s.num_heads), padded(self.k_gain, s.num_kv_heads)
        if s.sink:
            self.sink = tensors[sink]

    def weight_bytes(self):
        return (self.qkv.numel() + self.o.numel()) * self.qkv.element_size()

    def reads_first(self):
        return self.qkv

    def cache_request(self):
        s = self.spec
        return CacheRequest(kv_heads=s.num_kv_heads, head_dim=self.Dp, window=s.window, chunk=s.chunk,
                            shared_kv=self.keys_are_values)

    def prepare(self, max_positions):
        self.position.prepare(max_positions)

    def _extended(self, x, ctx, cache):
        s = self.spec
        T, H, KV, Dp = x.shape[0], s.num_heads, s.num_kv_heads, self.Dp
        with section("attn q/k/v proj"):
            proj = ops.linear(x, self.qkv)
        table = self.position.fused_table()
        if table is None and type(self.position).apply is not PositionEncoding.apply:
            raise ValueError("the extended attention options need a position part whose table the kernel applies")
        with section("attn norm/rope/append"):
            q = ops.qkv_prep(proj, 0, self.k_col, self.v_col, H, KV, Dp, self.Dk, self.bias, table,
                             self.rot if table is not None else 0, getattr(self.position, "pairs", False),
                             self.unit_rms, s.unit_eps, cache.k_pool, cache.v_pool, cache.page_table, ctx.tok_seq,
                             ctx.tok_pos, ctx.seq_slot, write_kv=cache.writes, norm=self.norm_span, q_gain=self.q_gain,
                             k_gain=self.k_gain, norm_eps=s.qk_norm.eps if s.qk_norm is not None else 0.0)
        fast = ops.fast_attention_supported(q.dtype, Dp, cache.page_size)
        with section("attention"):
            if fast and ctx.decode_only:
                out = ops.attention_decode(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot, ctx.seq_len,
                                           self.scale, s.window, ctx.len_bucket, softcap=self.softcap)
            elif fast:
                out = ops.attention_prefill(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot,
                                            ctx.seq_start, ctx.seq_len, ctx.max_new, self.scale, s.window,
                                            softcap=self.softcap)
            else:
                out = ops.attention(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot, ctx.seq_start,
                                    ctx.seq_len, ctx.max_new, self.scale, s.window, softcap=self.softcap)
        if self.gated:
            with section("attn gate"):
                ops.gate_heads(out, proj[:, self.g_col:self.g_col + (H if self.gated == "head" else H * Dp)], "sigmoid")
        with section("attn o proj"):
            return ops.linear(out.view(T, H * Dp), self.o)

    def __call__(self, x, ctx, cache):
        if self.extended:
            return self._extended(x, ctx, cache)
        s = self.spec
        with section("attn q/k/v proj"):
            qkv = ops.linear(x, self.qkv)
        table = self.position.fused_table()
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        meta = (ctx.tok_seq, ctx.tok_pos, ctx.seq_slot)
        with section("attn norm/rope/append"):
            if table is not None or type(self.position).apply is PositionEncoding.apply:
                # norm, rotation (by table, or none) and append in one kernel
                rot = self.rot if table is not None else 0
                q = ops.qk_norm_rope_append(qkv, s.num_heads, s.num_kv_heads, self.Dp, self.q_gain, self.k_gain, eps,
                                            table, rot, cache.k_pool, cache.v_pool, cache.page_table, *meta,
                                            write_kv=cache.writes, pairs=getattr(self.position, "pairs", False))
            else:
                # a position encoding with a rule of its own: norm q and k, let it work on them, append
                T, H, KV, Dh = x.shape[0], s.num_heads, s.num_kv_heads, self.Dp
                qw, kw = H * Dh, KV * Dh
                q = ops.qk_norm_rope_append(qkv[:, :qw].contiguous(), H, 0, Dh, self.q_gain, None, eps, None, 0,
                                            None, None, None, *meta, write_kv=False)
                k = ops.qk_norm_rope_append(qkv[:, qw:qw + kw].contiguous(), KV, 0, Dh, self.k_gain, None, eps, None, 0,
                                            None, None, None, *meta, write_kv=False)
                q, k = self.position.apply(q, k, ctx)
                if cache.writes:
                    kv = torch.cat([k.reshape(T, kw), qkv[:, qw + kw:]], dim=1).contiguous()
                    ops.qk_norm_rope_append(kv, 0, KV, Dh, None, None, eps, None, 0, cache.k_pool, cache.v_pool,
                                            cache.page_table, *meta, write_kv=True)
                q = q.contiguous()
        fast = ops.fast_attention_supported(q.dtype, self.Dp, cache.page_size)
        with section("attention"):
            if fast and ctx.decode_only:
                out = ops.attention_decode(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot, ctx.seq_len,
                                           self.scale, s.window, ctx.len_bucket, sink=self.sink, chunk=s.chunk)
            elif fast:
                out = ops.attention_prefill(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot,
                                            ctx.seq_start, ctx.seq_len, ctx.max_new, self.scale, s.window, sink=self.sink,
                                            chunk=s.chunk)
            else:
                out = ops.attention(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot, ctx.seq_start,
                                    ctx.seq_len, ctx.max_new, self.scale, s.window, sink=self.sink, chunk=s.chunk)
        with section("attn o proj"):
            return ops.linear(out.view(x.shape[0], s.num_heads * self.Dp), self.o)
