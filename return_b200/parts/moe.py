"""Feed-forwards with a capped gated unit, dense or as a mixture of experts.

``clamped_glu``: y = down( g * sigmoid(alpha g) * (u + 1) ), g = min(gate(x), limit), u = clamp(up(x), -limit, limit).
``moe``: a router (float32 logits, optionally with a bias per expert, softmax over all experts, optionally only the
experts of the best groups, the top few chosen, their scores renormalised) picks experts per token; the experts'
outputs are summed with those weights, in the order of falling score, and a shared feed-forward may run for every token
beside them.  The experts are capped gated units or plain ones (silu(gate) * up), which are the same kernel with no
cap, alpha = 1 and nothing added to the up part.

The experts' weights are stacked: ``experts.gate_up`` [E * 2F, hidden] (per expert its gate rows, then its up rows)
and ``experts.down`` [E * hidden, F].  Everything from the router's choice on happens on the device with grids that
depend on the token count alone, so a step of decoded tokens is captured in a graph like any other.
"""
from __future__ import annotations

import torch

from ..ext import ops
from .base import FEED_FORWARDS, FeedForward, ParamSpec, work_buffer


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    def params(self):
        s = self.spec
        return {"gate_up": ParamSpec((2 * s.intermediate_size, s.hidden_size)),
                "down": ParamSpec((s.hidden_size, s.intermediate_size))}

    def forward(self, x, ctx):
        s = self.spec
        T = x.shape[0]
        gu = work_buffer(ctx, "clamped_glu.gate_up", (T, 2 * s.intermediate_size), x.dtype, x.device)
        ops.linear(x, self.p_gate_up, gu)
        act = work_buffer(ctx, "clamped_glu.act", (T, s.intermediate_size), x.dtype, x.device)
        ops.clamped_glu(gu, act, s.limit, s.alpha)
        y = work_buffer(ctx, "clamped_glu.y", (T, s.hidden_size), x.dtype, x.device)
        ops.linear(act, self.p_down, y)
        return y


@FEED_FORWARDS.register("moe")
class MixtureOfExperts(FeedForward):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        kind = getattr(s.expert, "kind", None)
        if kind == "clamped_glu":
            self.unit = (float(s.expert.limit), float(s.expert.alpha), 1.0)       # cap, alpha, what is added to the up part
        elif kind == "swiglu" and not s.expert.interleave:
            self.unit = (float("inf"), 1.0, 0.0)
        else:
            raise ValueError("the experts of a mixture are gated units: kind 'clamped_glu', or 'swiglu' with rows not woven")
        if s.expert.hidden_size != s.hidden_size:
            raise ValueError("an expert maps the model's width to itself")
        if s.groups < 1 or s.num_experts % s.groups or not (1 <= s.keep_groups <= s.groups):
            raise ValueError(f"{s.num_experts} experts do not form {s.groups} equal groups of which {s.keep_groups} are kept")
        if not (1 <= s.top <= s.keep_groups * (s.num_experts // s.groups)):
            raise ValueError(f"top={s.top} experts cannot be chosen from {s.keep_groups} groups of {s.num_experts // s.groups}")
        if s.score not in ("softmax", "sigmoid") or s.group_top not in (1, 2):
            raise ValueError("score is 'softmax' or 'sigmoid'; a group is ranked by its best score or its two best")
        self.shared = FEED_FORWARDS.build(s.shared, env) if s.shared is not None else None

    @property
    def graph_safe(self):
        return self.shared is None or self.shared.graph_safe

    def params(self):
        s, e = self.spec, self.spec.expert
        p = {"router": ParamSpec((s.num_experts, s.hidden_size)),
             **({"router_bias": ParamSpec((s.num_experts,), role="vector", init="normal:0.5")} if s.router_bias else {}),
             "experts.gate_up": ParamSpec((s.num_experts * 2 * e.intermediate_size, s.hidden_size)),
             "experts.down": ParamSpec((s.num_experts * s.hidden_size, e.intermediate_size))}
        if self.shared is not None:
            for name, ps in self.shared.params().items():
                p["shared." + name] = ps
        return p

    def bind(self, tensors):
        s, e = self.spec, self.spec.expert
        self.p_router = tensors["router"]
        self.router_bias = tensors["router_bias"].float().contiguous() if s.router_bias else None
        self.gate_up = tensors["experts.gate_up"].view(s.num_experts, 2 * e.intermediate_size, s.hidden_size)
        self.down = tensors["experts.down"].view(s.num_experts, s.hidden_size, e.intermediate_size)
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in tensors.items() if k.startswith("shared.")})

    def forward(self, x, ctx):
        s, e = self.spec, self.spec.expert
        T, dt, dev = x.shape[0], x.dtype, x.device
        logits = work_buffer(ctx, "moe.logits", (T, s.num_experts), torch.float32, dev)
        ops.linear(x, self.p_router, logits)
        expert_of = work_buffer(ctx, "moe.expert_of", (T, s.top), torch.int32, dev)
        weight = work_buffer(ctx, "moe.weight", (T, s.top), torch.float32, dev)
        ops.moe_route(logits, expert_of, weight, s.top, s.groups, s.keep_groups, s.renorm_tiny, bias=self.router_bias,
                      score=s.score, group_top=s.group_top, scale=s.weight_scale)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        y = work_buffer(ctx, "moe.y", (T, s.hidden_size), dt, dev)
        limit, alpha, shift = self.unit
        ops.moe_experts(x, self.gate_up, self.down, expert_of, weight, shared, y, limit, alpha, ctx, shift=shift)
        return y
