"""A mixer that is the weighted sum of several mixers on the same input.

Each child keeps a cache or state of its own kind (``CompositeNeed``): one may page keys and values while
another holds a matrix state in the request's slot.  Parameters of a child are named ``<child>.<param>``.
"""
from __future__ import annotations

import torch

from ..ext import ops
from .base import MIXERS, CompositeNeed, Mixer


@MIXERS.register("mixer_sum")
class MixerSum(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if not (len(spec.names) == len(spec.mixers) == len(spec.scales) == 2):
            raise ValueError("a sum of mixers has two children, each with a name and a scale")
        self.children = {name: MIXERS.build(m, env) for name, m in zip(spec.names, spec.mixers)}

    @property
    def graph_safe(self):
        return all(c.graph_safe for c in self.children.values())

    def params(self):
        return {f"{name}.{p}": ps for name, child in self.children.items() for p, ps in child.params().items()}

    def bind(self, tensors):
        for name, child in self.children.items():
            prefix = name + "."
            child.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def cache_need(self):
        return CompositeNeed(tuple((name, child.cache_need()) for name, child in self.children.items()))

    def batch_tilings(self):
        out = {}
        for child in self.children.values():
            out.update(child.batch_tilings())
        return out

    def graph_variant(self, n_tokens, longest_context):
        out = {}
        for child in self.children.values():
            out.update(child.graph_variant(n_tokens, longest_context))
        return out

    def forward_parts(self, x, ctx):
        """((output, scale), (output, scale)) of the two children: a block whose add takes a factor per addend sums them
        itself, and the weighted sum costs no kernel and no pass over memory of its own."""
        outs = []
        for name, child in self.children.items():
            sub = ctx.children[name]
            sub.position, sub.next_block = ctx.position, None
            outs.append(child.forward(x, sub))
        return tuple(zip(outs, (float(s) for s in self.spec.scales)))

    def forward(self, x, ctx):
        outs = [o for o, _ in self.forward_parts(x, ctx)]
        y = ctx.buffer("mixer_sum.y", tuple(outs[0].shape), torch.float32, x.device)
        ops.scaled_sum(outs[0], float(self.spec.scales[0]), outs[1], float(self.spec.scales[1]), y)
        return y
