"""The pre-norm residual block (rollout/monkey_patch/qwen3.py:59-68).

The residual stream is float32 in both precisions.  A block receives the stream and the
"delta" that the block before it still owes the stream, adds it inside its first norm
kernel, and returns its own feed-forward output as the next delta, so each residual add is
fused with the norm that follows it.
"""
from __future__ import annotations

import torch

from ..ext import ops
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, ParamSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.mixer = MIXERS.build(spec.mixer, env)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, env) if spec.feed_forward is not None else None
        self.mixer_norm = NORMS.build(spec.mixer_norm, env)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, env) if spec.feed_forward is not None else None
        self.residual_scale = float(getattr(spec, "residual_scale", 1.0))
        self._children = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            self._children.update({"feed_forward": self.feed_forward, "feed_forward_norm": self.feed_forward_norm})
        # a sublayer's output times a factor, or a layer without a feed-forward: the adds run in the kernel that takes
        # a factor per addend (csrc/recurrent.cu, add_dual_norm), which wants RMSNorms
        self._scaled = (self.residual_scale != 1.0 or self.feed_forward is None or bool(getattr(spec, "float_outputs", False)))
        if self._scaled and any(getattr(n.spec, "kind", None) != "rmsnorm" for n in (self.mixer_norm, self.feed_forward_norm)
                                if n is not None):
            raise ValueError("a pre-norm block with a residual factor, or without a feed-forward, has RMSNorms")

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self._children.values())

    def params(self):
        return {f"{child}.{name}": p for child, part in self._children.items()
                for name, p in part.params().items()}

    def bind(self, tensors):
        for child, part in self._children.items():
            prefix = child + "."
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def cache_need(self):
        return self.mixer.cache_need()

    def batch_tilings(self):
        out = {}
        for part in self._children.values():
            out.update(part.batch_tilings())
        return out

    def graph_variant(self, n_tokens, longest_context):
        out = {}
        for part in self._children.values():
            out.update(part.graph_variant(n_tokens, longest_context))
        return out

    # ------------------------------------------------------------------ few rows: norms and residual adds inside the products
    def first_norm(self):
        """(weight, eps, offset, size) of the RMSNorm that this block applies to the residual stream first, or None.
        The block that runs before this one may then prepare the normed rows in the epilogue of its last product."""
        n = self.mixer_norm
        if getattr(n.spec, "kind", None) == "rmsnorm" and hasattr(n, "p_weight"):
            return n.p_weight, n.spec.eps, n.spec.offset, n.spec.size
        return None

    def _fused_plan(self, stream):
        """For a step of few rows in bfloat16 the two norms and the two residual adds of the block cost no kernel of
        their own: the product before a norm (the mixer's last, the feed-forward's last) adds into the stream
        and leaves v * w and sum(v^2); the product after it (the gated one, the next block's first) scales by
        rstd (csrc/gemm_skinny.cu).  Six launches a layer instead of eight.  That needs a mixer and a feed-forward
        that expose their products, RMSNorms, and sizes the kernel takes; anything else runs part by part."""
        if self.env.act_dtype != torch.bfloat16 or stream.shape[0] > ops.SKINNY_MAX_ROWS or self._scaled:
            return None
        plan = getattr(self, "_fused_parts", None)
        if plan is None:
            plan = False
            mixer, ff = self.mixer, self.feed_forward
            n2 = self.feed_forward_norm
            norms_ok = self.first_norm() is not None and getattr(n2.spec, "kind", None) == "rmsnorm" and hasattr(n2, "p_weight")
            if norms_ok and hasattr(mixer, "in_projection") and hasattr(mixer, "core") and hasattr(ff, "gated_projections"):
                (w_in, in_name), w_out = mixer.in_projection(), mixer.out_projection()
                gate_up, down, interleave = ff.gated_projections()
                weights = (w_in, w_out, gate_up, down)
                if (interleave == 8 and gate_up.shape[0] % 16 == 0 and w_out.shape[0] == stream.shape[1] == down.shape[0]
                        and all(w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0
                                and w.data_ptr() % 16 == 0 for w in weights)):
                    plan = (w_in, in_name, w_out, gate_up, down)
            self._fused_parts = plan
        return plan or None

    def _forward_fused(self, plan, stream, delta, ctx):
        w_in, in_name, w_out, gate_up, down = plan
        T, H = stream.shape
        dev, dt = stream.device, self.env.act_dtype
        n1, n2 = self.mixer_norm, self.feed_forward_norm
        held = ctx.batch.scratch
        # what the block before this one left for this block's first norm (made for this position of the schedule)
        pre = held.pop("block.prenormed", None)
        proj = ctx.buffer(in_name, (T, w_in.shape[0]), dt, dev)
        if delta is None and pre is not None and pre["position"] == ctx.position:
            ops.gemm_skinny_fused(pre["rows"], w_in, proj, scale=(pre["sums"], n1.spec.eps))
        else:
            a = ctx.buffer("block.normed", (T, H), dt, dev)
            n1.add_forward(stream, delta, a)                   # stream += delta; a = norm(stream)
            ops.gemm_skinny(a, w_in, proj)
        mixed = self.mixer.core(proj, ctx)
        rows2 = ctx.buffer("block.rows_mid", (T, H), dt, dev)
        sums2 = ops.RowSums(ctx.buffer("block.sums_mid", (8, ops.RowSums.WIDTH), torch.float32, dev), H)
        ops.gemm_skinny_fused(mixed, w_out, rows2, residual=(stream, (n2.p_weight, n2.spec.offset), sums2))
        act = ctx.buffer("block.gated_act", (T, gate_up.shape[0] // 2), dt, dev)
        ops.gemm_skinny_fused(rows2, gate_up, act, gated=True, scale=(sums2, n2.spec.eps))
        nxt = ctx.next_block.first_norm() if ctx.next_block is not None and hasattr(ctx.next_block, "first_norm") else None
        if nxt is not None and nxt[3] != H:
            nxt = None
        if nxt is None:
            ops.gemm_skinny_fused(act, down, None, residual=(stream, None, None))
        else:
            rows3 = ctx.buffer("block.rows_out", (T, H), dt, dev)
            sums3 = ops.RowSums(ctx.buffer("block.sums_out", (8, ops.RowSums.WIDTH), torch.float32, dev), H)
            ops.gemm_skinny_fused(act, down, rows3, residual=(stream, (nxt[0], nxt[2]), sums3))
            held["block.prenormed"] = {"rows": rows3, "sums": sums3, "position": ctx.position + 1}
        return None                                            # the stream already holds this block's output

    def _forward_scaled(self, stream, delta, ctx):
        """x += m * mixer(norm(x)); x += m * feed_forward(norm(x)).  Every add is fused with the norm that follows it,
        the last one with the first norm of the block that runs next when that block is of this kind (its normed rows
        are left under ``block.prenormed_rows`` in the step's scratch); the block owes the stream nothing."""
        T, H = stream.shape
        m = self.residual_scale
        n1, n2 = self.mixer_norm, self.feed_forward_norm
        held = getattr(ctx.batch, "scratch", None)
        pre = held.pop("block.prenormed_rows", None) if held is not None else None
        a = ctx.buffer("block.normed", (T, H), self.env.act_dtype, stream.device)
        if not (delta is None and pre is not None and pre["position"] == ctx.position and pre["rows"] is a):
            ops.add_dual_norm(stream, (delta,), n1.p_weight, None, n1.spec.eps, n1.spec.offset, a, None)
        if hasattr(self.mixer, "forward_parts"):             # a sum of two mixers: both join the stream in one add
            (y, s1), (y2, s2) = self.mixer.forward_parts(a, ctx)
            ys, scales = (y, y2), (m * s1, m * s2)
        else:
            ys, scales = (self.mixer.forward(a, ctx),), (m, 1.0)
        if self.feed_forward is not None:
            ops.add_dual_norm(stream, ys, n2.p_weight, None, n2.spec.eps, n2.spec.offset, a, None, scales=scales)
            ys, scales = (self.feed_forward.forward(a, ctx),), (m, 1.0)
        nxt = ctx.next_block
        if held is not None and isinstance(nxt, PreNormBlock) and nxt._scaled and nxt.mixer_norm.spec.size == H:
            n = nxt.mixer_norm
            ops.add_dual_norm(stream, ys, n.p_weight, None, n.spec.eps, n.spec.offset, a, None, scales=scales)
            held["block.prenormed_rows"] = {"rows": a, "position": ctx.position + 1}
        else:
            ops.add_dual_norm(stream, ys, None, None, 0.0, 0.0, None, None, scales=scales)
        return None

    def forward(self, stream, delta, ctx):
        if self._scaled:
            return self._forward_scaled(stream, delta, ctx)
        plan = self._fused_plan(stream) if getattr(ctx.batch, "scratch", None) is not None else None
        if plan is not None:
            return self._forward_fused(plan, stream, delta, ctx)
        T, H = stream.shape
        a = ctx.buffer("block.normed", (T, H), self.env.act_dtype, stream.device)
        self.mixer_norm.add_forward(stream, delta, a)             # stream += delta; a = norm(stream)
        mixed = self.mixer.forward(a, ctx)
        self.feed_forward_norm.add_forward(stream, mixed, a)      # stream += mixed; a = norm(stream)
        return self.feed_forward.forward(a, ctx)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """x += mixer(norm_a(x)) + feed_forward(norm_b(x)): both branches read the same stream.

    The two norms are one kernel (they share the row's mean square), fused with the adds that the block before left
    undone: a block of this kind returns its two branch outputs as a pair, and whoever runs next adds them
    (``takes_delta_pair``: this kind does it inside its norm kernel; for any other the model adds them first)."""

    takes_delta_pair = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.mixer = MIXERS.build(spec.mixer, env)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, env) if spec.feed_forward is not None else None
        self.mixer_norm = NORMS.build(spec.mixer_norm, env)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, env) if spec.feed_forward is not None else None
        na, nb = spec.mixer_norm, spec.feed_forward_norm
        if getattr(na, "kind", None) != "rmsnorm" or (nb is not None and (getattr(nb, "kind", None) != "rmsnorm" or
                                                                           (nb.eps, nb.offset, nb.size) != (na.eps, na.offset, na.size))):
            raise ValueError("the two norms of a parallel block are RMSNorms with the same eps, offset and size")
        self._children = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            self._children.update({"feed_forward": self.feed_forward, "feed_forward_norm": self.feed_forward_norm})

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self._children.values())

    def params(self):
        return {f"{child}.{name}": p for child, part in self._children.items()
                for name, p in part.params().items()}

    def bind(self, tensors):
        for child, part in self._children.items():
            prefix = child + "."
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def cache_need(self):
        return self.mixer.cache_need()

    def batch_tilings(self):
        out = {}
        for part in self._children.values():
            out.update(part.batch_tilings())
        return out

    def graph_variant(self, n_tokens, longest_context):
        out = {}
        for part in self._children.values():
            out.update(part.graph_variant(n_tokens, longest_context))
        return out

    def forward(self, stream, delta, ctx):
        T, H = stream.shape
        dt, dev = self.env.act_dtype, stream.device
        n = self.mixer_norm.spec
        deltas = delta if isinstance(delta, tuple) else (delta,)
        a = ctx.buffer("parallel.normed_a", (T, H), dt, dev)
        has_ff = self.feed_forward is not None
        b = ctx.buffer("parallel.normed_b", (T, H), dt, dev) if has_ff else None
        ops.add_dual_norm(stream, deltas, self.mixer_norm.p_weight, self.feed_forward_norm.p_weight if has_ff else None,
                          n.eps, n.offset, a, b)
        mixed = self.mixer.forward(a, ctx)
        if not has_ff:
            return (mixed,)
        return (mixed, self.feed_forward.forward(b, ctx))


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """x += post_a(mixer(pre_a(x))); x += post_b(feed_forward(pre_b(x))): every sublayer is normed on the way in and on
    the way out.

    One kernel sits at every joint: it norms the sublayer's output, adds it to the float32 stream and norms the stream
    for the sublayer that runs next (csrc/elementwise.cu, ``postnorm_add_norm``), also across the border to the next
    block when that block begins with an RMSNorm of the stream (``first_norm``): the normed rows are then left for it
    under ``sandwich.prenormed`` in the step's scratch.  The block owes the stream nothing when it returns."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.mixer = MIXERS.build(spec.mixer, env)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, env) if spec.feed_forward is not None else None
        self._children = {"mixer": self.mixer, "mixer_norm": NORMS.build(spec.mixer_norm, env),
                          "mixer_post_norm": NORMS.build(spec.mixer_post_norm, env)}
        if self.feed_forward is not None:
            self._children.update({"feed_forward": self.feed_forward,
                                   "feed_forward_norm": NORMS.build(spec.feed_forward_norm, env),
                                   "feed_forward_post_norm": NORMS.build(spec.feed_forward_post_norm, env)})
        for name, part in self._children.items():
            if name.endswith("norm") and getattr(part.spec, "kind", None) != "rmsnorm":
                raise ValueError("the norms of a sandwich block are RMSNorms")

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self._children.values())

    def params(self):
        return {f"{child}.{name}": p for child, part in self._children.items()
                for name, p in part.params().items()}

    def bind(self, tensors):
        for child, part in self._children.items():
            prefix = child + "."
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def cache_need(self):
        return self.mixer.cache_need()

    def batch_tilings(self):
        out = {}
        for part in self._children.values():
            out.update(part.batch_tilings())
        return out

    def graph_variant(self, n_tokens, longest_context):
        out = {}
        for part in self._children.values():
            out.update(part.graph_variant(n_tokens, longest_context))
        return out

    def first_norm(self):
        n = self._children["mixer_norm"]
        return (n.p_weight, n.spec.eps, n.spec.offset, n.spec.size) if hasattr(n, "p_weight") else None

    @staticmethod
    def _triple(norm):
        return norm.p_weight, norm.spec.eps, norm.spec.offset

    def forward(self, stream, delta, ctx):
        T, H = stream.shape
        dt, dev = self.env.act_dtype, stream.device
        c = self._children
        held = getattr(ctx.batch, "scratch", None)
        pre = held.pop("sandwich.prenormed", None) if held is not None else None
        if delta is None and pre is not None and pre["position"] == ctx.position:
            a = pre["rows"]                                     # the block before this one normed the stream for us
        else:
            a = ctx.buffer("sandwich.normed_a", (T, H), dt, dev)
            c["mixer_norm"].add_forward(stream, delta, a)       # stream += delta; a = norm(stream)
        mixed = self.mixer.forward(a, ctx)
        last = mixed, c["mixer_post_norm"]
        if self.feed_forward is not None:
            b = ctx.buffer("sandwich.normed_b", (T, H), dt, dev)
            ops.postnorm_add_norm(stream, mixed, self._triple(c["mixer_post_norm"]), self._triple(c["feed_forward_norm"]), b)
            last = self.feed_forward.forward(b, ctx), c["feed_forward_post_norm"]
        nxt = ctx.next_block.first_norm() if ctx.next_block is not None and hasattr(ctx.next_block, "first_norm") else None
        if nxt is not None and nxt[3] == H and held is not None and isinstance(ctx.next_block, SandwichBlock):
            rows = ctx.buffer("sandwich.normed_a", (T, H), dt, dev)      # this block's own normed input is used up by now
            ops.postnorm_add_norm(stream, last[0], self._triple(last[1]), (nxt[0], nxt[1], nxt[2]), rows)
            held["sandwich.prenormed"] = {"rows": rows, "position": ctx.position + 1}
        else:
            ops.postnorm_add_norm(stream, last[0], self._triple(last[1]))
        return None


@BLOCKS.register("hyper")
class HyperBlock(Block):
    """A pre-norm layer over several residual streams (``HyperBlockSpec``).  The stream tensor is float32 [T, S, H].

    Two kernels serve a sublayer (csrc/elementwise.cu): the read (the weighted sum of the streams, normed) and the write
    (every stream becomes a mix of the old ones plus its share of the sublayer's output).  The write also does the read
    of whatever runs next while the row's new streams are in registers: the feed-forward's, or, across the border, the
    next block's first read when that block is of this kind (left under ``hyper.prenormed`` in the step's scratch)."""

    takes_streams = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if not (1 <= spec.streams <= ops.HYPER_MAX_STREAMS):
            raise ValueError(f"streams={spec.streams}: 1 to {ops.HYPER_MAX_STREAMS}")
        self.mixer = MIXERS.build(spec.mixer, env)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, env) if spec.feed_forward is not None else None
        self._children = {"mixer": self.mixer, "mixer_norm": NORMS.build(spec.mixer_norm, env)}
        if self.feed_forward is not None:
            self._children.update({"feed_forward": self.feed_forward,
                                   "feed_forward_norm": NORMS.build(spec.feed_forward_norm, env)})
        for name, part in self._children.items():
            if name.endswith("norm") and getattr(part.spec, "kind", None) != "rmsnorm":
                raise ValueError("the norms of a hyper block are RMSNorms")
        self._sublayers = ("mixer", "feed_forward") if self.feed_forward is not None else ("mixer",)

    @property
    def graph_safe(self):
        return all(part.graph_safe for part in self._children.values())

    def params(self):
        S = self.spec.streams
        p = {f"{child}.{name}": ps for child, part in self._children.items() for name, ps in part.params().items()}
        for sub in self._sublayers if self.spec.learned else ():
            p[f"{sub}_read"] = ParamSpec((S,), role="vector", init="half_to_one")
            p[f"{sub}_write"] = ParamSpec((S,), role="vector", init="half_to_one")
            p[f"{sub}_mix"] = ParamSpec((S, S), role="vector", init="eye_normal")
        return p

    def bind(self, tensors):
        for child, part in self._children.items():
            prefix = child + "."
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})
        # the streams' arithmetic is float32 whatever the checkpoint stores
        if self.spec.learned:
            self.hc = {sub: tuple(tensors[f"{sub}_{n}"].float().contiguous() for n in ("read", "write", "mix"))
                       for sub in self._sublayers}
        else:
            S, dev = self.spec.streams, self.env.device
            ones = (torch.ones(S, dtype=torch.float32, device=dev), torch.ones(S, dtype=torch.float32, device=dev),
                    torch.ones((S, S), dtype=torch.float32, device=dev))
            self.hc = {sub: ones for sub in self._sublayers}

    def cache_need(self):
        return self.mixer.cache_need()

    def batch_tilings(self):
        out = {}
        for part in self._children.values():
            out.update(part.batch_tilings())
        return out

    def graph_variant(self, n_tokens, longest_context):
        out = {}
        for part in self._children.values():
            out.update(part.graph_variant(n_tokens, longest_context))
        return out

    def first_read(self):
        """(read vector, norm weight, eps, offset) of this block's first sublayer: what the block before it needs to do
        that read in its last write."""
        n = self._children["mixer_norm"]
        return self.hc["mixer"][0], n.p_weight, n.spec.eps, n.spec.offset

    def forward(self, streams, delta, ctx):
        if streams.dim() != 3 or streams.shape[1] != self.spec.streams:
            raise ValueError(f"a hyper block of {self.spec.streams} streams was handed a stream tensor of shape {tuple(streams.shape)}")
        if delta is not None:
            raise ValueError("a hyper block takes no pending residual: the block before it must write the streams itself")
        T, S, H = streams.shape
        dt, dev = self.env.act_dtype, streams.device
        c = self._children
        held = getattr(ctx.batch, "scratch", None)
        pre = held.pop("hyper.prenormed", None) if held is not None else None
        if pre is not None and pre["position"] == ctx.position:
            a = pre["rows"]                                     # the block before this one did this read in its last write
        else:
            a = ctx.buffer("hyper.read_a", (T, H), dt, dev)
            n = c["mixer_norm"]
            ops.hyper_read_norm(streams, self.hc["mixer"][0], n.p_weight, n.spec.eps, a, offset=n.spec.offset)
        y = self.mixer.forward(a, ctx)
        _, write, mix = self.hc["mixer"]
        if self.feed_forward is not None:
            n = c["feed_forward_norm"]
            b = ctx.buffer("hyper.read_b", (T, H), dt, dev)
            ops.hyper_write(streams, y, mix, write, nxt=(self.hc["feed_forward"][0], n.p_weight, n.spec.eps, n.spec.offset), out=b)
            y = self.feed_forward.forward(b, ctx)
            _, write, mix = self.hc["feed_forward"]
        nxt = ctx.next_block
        if held is not None and isinstance(nxt, HyperBlock) and nxt.spec.streams == S:
            rows = ctx.buffer("hyper.read_a", (T, H), dt, dev)          # this block's own first read is used up by now
            ops.hyper_write(streams, y, mix, write, nxt=nxt.first_read(), out=rows)
            held["hyper.prenormed"] = {"rows": rows, "position": ctx.position + 1}
        else:
            ops.hyper_write(streams, y, mix, write)
        return None
