"""The matrix memory of xLSTM (mLSTM): a recurrent mixer with a matrix-valued state, a normaliser vector and a running
maximum per head.

With h the mixer's input, per token t and head (all of the recurrence in float32):
    q = Wq h / sqrt(dim),  k = Wk h  (dim each),  v = Wv h  (vdim)
    li = cap tanh((Wi h + bi) / cap)                     log input gate
    lf = log_sigmoid(cap tanh((Wf h + bf) / cap))        log forget gate
    m_t = max(lf + m_(t-1), li)                          m = 0 at a sequence's start
    S_t = exp(lf + m_(t-1) - m_t) S_(t-1) + exp(li - m_t) k v^T          n_t likewise with k alone
    o   = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    out = Wo ( concat_heads(o / rms(o)) * gain * sigmoid(Wg h) )          the gain over all heads' elements
The state lives in the cache's per-sequence state: S and n together as [slots, H, dim, vdim + 1] (n is the column that
a value of 1 feeds), m as [slots, H]; a step walks its new tokens in order from what the steps before left, so a
prompt, its pieces and single tokens give the same result.

Order of work: q, k, v, the output gate and both gates' pre-activations are one product with the stacked matrix, kept
in float32 whatever the compute dtype (the gates' pre-activations enter exponentials); the gates and the chain of
maxima (``ops.mlstm_gates``); the recurrence (``ops.scalar_decay_recurrent``: the kernel of gated linear attention with
one decay per token and the column of ones); division, norm, gain and gate in one kernel; the output projection.
"""
from __future__ import annotations

import torch

from .. import ops
from ..profiler import section
from .base import CacheRequest, Mixer
from .registry import ParamInfo, register_mixer

DENOMINATOR_FLOOR = 1e-6          # fixed by the design; the kernel carries the same constant


@register_mixer("mlstm")
class MatrixMemory(Mixer):
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if not spec.gate_cap > 0:
            raise ValueError(f"gate_cap {spec.gate_cap} must be positive")

    @classmethod
    def param_infos(cls, spec):
        D, H = spec.hidden_size, spec.num_heads
        return {"q": ParamInfo((H * spec.dim, D)), "k": ParamInfo((H * spec.dim, D)), "v": ParamInfo((H * spec.vdim, D)),
                "g": ParamInfo((H * spec.vdim, D)), "o": ParamInfo((D, H * spec.vdim)),
                "norm": ParamInfo((H * spec.vdim,), "gain"), "i": ParamInfo((H, D)), "i.b": ParamInfo((H,), "vector"),
                "f": ParamInfo((H, D)), "f.b": ParamInfo((H,), "vector")}

    def load(self, tensors):
        s = self.spec
        H = s.num_heads
        blocks = [tensors["q"], tensors["k"], tensors["v"], tensors["g"], tensors["i"], tensors["f"]]
        rows = sum(b.shape[0] for b in blocks)
        if rows % 8:                                  # rows of the product that are whole 16-byte pieces in both dtypes
            blocks.append(blocks[0].new_zeros((8 - rows % 8, s.hidden_size)))
        self.proj = torch.cat(blocks, dim=0).contiguous()
        self.q_col, self.k_col = 0, H * s.dim
        self.v_col = 2 * H * s.dim
        self.g_col = self.v_col + H * s.vdim
        self.i_col = self.g_col + H * s.vdim
        self.f_col = self.i_col + H
        self.i_bias, self.f_bias = tensors["i.b"], tensors["f.b"]
        self.gain, self.o = tensors["norm"], tensors["o"].contiguous()

    def weight_bytes(self):
        return (self.proj.numel() + self.o.numel()) * self.proj.element_size()

    def reads_first(self):
        return self.proj

    def cache_request(self):
        s = self.spec
        return CacheRequest(state_shape=(s.num_heads, s.dim, s.vdim + 1), state_dtype=torch.float32,
                            more_state=(((s.num_heads,), torch.float32),))

    def __call__(self, x, ctx, cache):
        s = self.spec
        H = s.num_heads
        with section("mlstm q/k/v/gate proj"):
            proj = ops.linear(x, self.proj, out_dtype=torch.float32)
        with section("mlstm gates"):
            gates = ops.mlstm_gates(proj, self.i_col, self.f_col, self.i_bias, self.f_bias, s.gate_cap, cache.more_state[0],
                                    ctx.seq_slot, ctx.seq_start, H, single=ctx.decode_only)
        with section("mlstm recurrence"):
            o = ops.scalar_decay_recurrent(proj, self.q_col, self.k_col, self.v_col, gates, s.dim ** -0.5, cache.state,
                                           ctx.seq_slot, ctx.seq_start, H, s.dim, s.vdim, ones=True, single=ctx.decode_only)
        with section("mlstm norm/gate"):
            y = ops.mlstm_head_norm_gate(o, gates, self.gain, s.eps, proj[:, self.g_col:self.g_col + H * s.vdim], self.env.dtype)
        with section("mlstm o proj"):
            return ops.linear(y, self.o)
