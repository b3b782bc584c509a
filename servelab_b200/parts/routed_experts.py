"""Routed experts with a softmax router, group-limited choice and an optional shared expert
(spec: ``RoutedExpertsSpec``).

Per step: the router's logits in float32 (a float32 matrix against the step's rows), one kernel
for softmax + choice + weights, a plan that sorts the (token, choice) pairs by expert on the
device, the experts' gate|up product with the activation and their down product over the sorted
rows, and one kernel that adds a token's weighted results (and the shared expert's) in the order
of its choice.  Nothing of the routing is read on the host, so a step replays as a graph.
"""

from __future__ import annotations

import torch

from ..ops import kernels as K
from ..weights.source import BIAS, MATRIX, TensorDecl
from .base import FeedForward
from .registry import FEED_FORWARDS, build_part, part_class, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec, prefix, env):
        super().__init__(spec, prefix, env)
        if spec.num_experts % spec.num_groups or not 0 < spec.keep_groups <= spec.num_groups:
            raise ValueError("routed_experts: experts must split into equal groups, 0 < keep <= groups")
        if not 0 < spec.top <= spec.num_experts // spec.num_groups * spec.keep_groups:
            raise ValueError("routed_experts: top experts must fit into the kept groups")
        if spec.score_fn not in ("softmax", "sigmoid") or spec.group_best < 1:
            raise ValueError("routed_experts: score_fn is 'softmax' or 'sigmoid'; group_best at least 1")
        self.shared = (build_part(FEED_FORWARDS, spec.shared, f"{prefix}.{spec.shared_name}", env)
                       if spec.shared is not None else None)

    @classmethod
    def _expert(cls, spec, prefix, j):
        base = f"{prefix}.{spec.expert_prefix.format(j)}"
        return tuple(f"{base}.{n}{spec.weight_suffix}" for n in (spec.gate_name, spec.up_name, spec.down_name))

    @classmethod
    def declare(cls, spec, prefix):
        h, i = spec.hidden_size, spec.expert_size
        out = [TensorDecl(f"{prefix}.{spec.router_name}{spec.weight_suffix}", (spec.num_experts, h), BIAS)]
        if spec.correction_name:
            out.append(TensorDecl(f"{prefix}.{spec.correction_name}", (spec.num_experts,), BIAS))
        for j in range(spec.num_experts):
            g, u, d = cls._expert(spec, prefix, j)
            out += [TensorDecl(g, (i, h), MATRIX), TensorDecl(u, (i, h), MATRIX), TensorDecl(d, (h, i), MATRIX)]
        if spec.shared is not None:
            out += part_class(FEED_FORWARDS, spec.shared).declare(spec.shared, f"{prefix}.{spec.shared_name}")
        return out

    def load(self, store):
        s = self.spec
        self.router = store.get(f"{self.prefix}.{s.router_name}{s.weight_suffix}")      # float32
        self.correction = store.get(f"{self.prefix}.{s.correction_name}") if s.correction_name else None
        names = [self._expert(s, self.prefix, j) for j in range(s.num_experts)]
        # [E, 2 I, h]: an expert's gate rows, then its up rows; [E, h, I]
        self.w_gate_up = torch.stack([torch.cat([store.get(g), store.get(u)]) for g, u, _ in names]).contiguous()
        self.w_down = torch.stack([store.get(d) for _, _, d in names]).contiguous()
        if self.shared is not None:
            self.shared.load(store)

    def forward(self, ctx, x):
        s = self.spec
        x = K.plain_unless(None, x)
        logits = K.router_logits(x, self.router)
        if s.score_fn == "softmax" and self.correction is None and s.group_best == 1 and s.norm_eps == 0.0:
            ids, weights = K.moe_route(logits, s.num_groups, s.keep_groups, s.top, s.route_scale, s.renormalize)
        else:
            ids, weights = K.moe_route_scored(logits, s.num_groups, s.keep_groups, s.top, s.route_scale,
                                              s.renormalize, s.score_fn, self.correction, s.group_best,
                                              s.norm_eps)
        shared = K.plain_unless(None, self.shared.forward(ctx, x)) if self.shared is not None else None
        return K.moe_experts(x, ids, weights, self.w_gate_up, self.w_down, shared)
