"""A routed feed-forward (mixture of experts).

    z = R h (float32),  s = softmax(z) over all router outputs,  choice = the ``top`` largest of s + correction
    w_j = s[choice_j] / (sum_j s[choice_j] + 1e-20)
Options of the record: s = sigmoid(z) element by element; a choice only among the experts of the best groups of
neighbouring experts (a group's score: the sum of its largest choice scores); weights that are not divided by their
sum; a constant factor on the weights.
    y = sum_j w_j expert_{choice_j}(h)  (+ shared(h))
The router's last ``identity`` outputs stand for experts that return h itself and have no tensors.  The experts are
gated feed-forwards of one record (``parts/mlp.py``'s "gated" kind gives the formula); their matrices are stacked
[experts, ...] at load.  ``shared`` is a feed-forward part of its own that every token takes.

Order of work: router and choice (``ops.moe_route``); the step's (token, choice) pairs grouped by expert, on the device
(``ops.moe_plan``); gate and up of every pair as one grouped product over the experts' tiles, the gate function, the down
product scattered back to the pairs' places (``ops.moe_grouped_linear``, ``ops.gated_act``); the weighted sum over a
token's choices with the identity experts and the shared output (``ops.moe_combine``).  Nothing comes back to the host,
so one-token steps replay from a graph.
"""
from __future__ import annotations

import torch

from .. import ops
from ..profiler import section
from .base import FeedForward
from .registry import ParamInfo, build_part, part_class, register_ffn


@register_ffn("moe")
class MixtureOfExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if getattr(spec.expert, "kind", None) != "gated":
            raise ValueError(f"experts of kind {getattr(spec.expert, 'kind', None)!r} are not built (known: gated)")
        if not 1 <= spec.top <= spec.experts + spec.identity:
            raise ValueError(f"top {spec.top} of {spec.experts} + {spec.identity} experts")
        if getattr(spec, "score", "softmax") not in ops.MOE_SCORES:
            raise ValueError(f"score {spec.score!r} is not built (known: {', '.join(sorted(ops.MOE_SCORES))})")
        groups, keep = getattr(spec, "groups", 1), getattr(spec, "group_keep", 1)
        outputs = spec.experts + spec.identity
        if groups < 1 or outputs % groups or not 1 <= keep <= groups or getattr(spec, "group_top", 2) < 1:
            raise ValueError(f"{outputs} router outputs in {groups} groups of which {keep} are kept")
        if groups > 1 and spec.top > keep * (outputs // groups):
            raise ValueError(f"top {spec.top} of the {keep * (outputs // groups)} outputs of the kept groups")
        self.shared = build_part("ffn", spec.shared, env) if spec.shared is not None else None

    @classmethod
    def param_infos(cls, spec):
        D, I, N = spec.hidden_size, spec.expert.intermediate_size, spec.experts + spec.identity
        infos = {"router": ParamInfo((N, D), "vector"), "correction": ParamInfo((N,), "vector")}
        for e in range(spec.experts):
            infos[f"e{e}.gate"], infos[f"e{e}.up"] = ParamInfo((I, D)), ParamInfo((I, D))
            infos[f"e{e}.down"] = ParamInfo((D, I))
        if spec.shared is not None:
            for local, info in part_class("ffn", spec.shared).param_infos(spec.shared).items():
                infos["shared." + local] = info
        return infos

    def load(self, tensors):
        E = self.spec.experts
        self.router, self.correction = tensors["router"], tensors["correction"]
        # per expert [gate rows; up rows], all experts stacked
        self.gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0) for e in range(E)]).contiguous()
        self.down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()
        if self.shared is not None:
            self.shared.load({k[len("shared."):]: v for k, v in tensors.items() if k.startswith("shared.")})

    def weight_bytes(self):
        n = (self.gate_up.numel() + self.down.numel()) * self.gate_up.element_size() + self.router.numel() * 4
        return n + (self.shared.weight_bytes() if self.shared is not None else 0)

    def __call__(self, x, ctx):
        s, ex = self.spec, self.spec.expert
        T = x.shape[0]
        with section("moe router"):
            idx, weight = ops.moe_route(x, self.router, self.correction, s.top, getattr(s, "score", "softmax"),
                                        getattr(s, "groups", 1), getattr(s, "group_keep", 1), getattr(s, "group_top", 2),
                                        getattr(s, "route_scale", 1.0), getattr(s, "renormalize", True))
            # many pairs per expert (a prompt): tiles of 64 rows, where the bfloat16 kernel for them takes the sizes
            wide = (x.dtype == torch.bfloat16 and T * s.top >= 48 * s.experts and s.hidden_size % 8 == 0
                    and ex.intermediate_size % 8 == 0)
            plan = ops.moe_plan(idx, s.experts, wide)
        with section("moe experts"):
            gu = ops.moe_grouped_linear(x, self.gate_up, plan, T * s.top, gather_div=s.top)
            act = ops.gated_act(gu, ex.gate, None, ex.limit, ex.alpha)
            pair_out = ops.moe_grouped_linear(act, self.down, plan, T * s.top, scatter=True, out_dtype=torch.float32)
        extra = self.shared(x, ctx) if self.shared is not None else None
        with section("moe combine"):
            return ops.moe_combine(pair_out, idx, weight, x, s.experts, extra)
