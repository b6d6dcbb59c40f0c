"""A decoder made of parts: embedding, a schedule of blocks, final norm, output head.

The model knows nothing of Qwen3.  It is built from a ``DecoderSpec`` and asks each block for
its parameters under the names ``layers.<i>.<part>.<param>``, plus ``embed``, ``final_norm.weight``
and ``lm_head`` (an alias of ``embed`` when the specification ties them).  The forward pass of
one step follows the reference's (rollout/monkey_patch/qwen3.py:71-81): embed, run the layers,
final norm; the head is applied to the rows whose logits are wanted only
(rollout/model.py:286-290).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ext import ops
from ..parts.base import BLOCKS, NORMS, BuildEnv, KVCacheNeed, LayerContext, ParamSpec, StateNeed
from ..parts.spec import DecoderSpec


class DecoderModel:
    def __init__(self, spec: DecoderSpec, env: BuildEnv):
        spec.validate()
        self.spec = spec
        self._graph_safe = None
        self.env = env
        self.blocks = [BLOCKS.build(b, env) for b in spec.layers]
        if spec.streams is not None:
            loose = [i for i, b in enumerate(self.blocks) if not getattr(b, "takes_streams", False)]
            if loose or spec.embedding_norm is not None:
                raise ValueError(f"a model with {spec.streams} residual streams is made of blocks that take them "
                                 f"(layers {loose} do not) and norms no embedding")
        self.final_norm = NORMS.build(spec.final_norm, env)
        self.embedding_norm = NORMS.build(spec.embedding_norm, env) if spec.embedding_norm is not None else None
        self.embed: Optional[torch.Tensor] = None
        # for looking inside a step: called as after_block(schedule index, stream, pending delta) behind every block
        self.after_block = None
        self.lm_head: Optional[torch.Tensor] = None
        self.embed_pairs: Optional[torch.Tensor] = None
        if spec.embedding_pairs is not None and spec.streams is not None:
            raise ValueError("the table of token pairs is added to one residual stream")

    # ------------------------------------------------------------------ parameters
    def params(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"embed": ParamSpec((s.vocab_size, s.hidden_size))}
        if s.embedding_pairs is not None:
            p["embed_pairs"] = ParamSpec((s.embedding_pairs[0] + 1, s.hidden_size))
        for i, block in enumerate(self.blocks):
            for name, ps in block.params().items():
                p[f"layers.{i}.{name}"] = ps
        for name, ps in self.final_norm.params().items():
            p[f"final_norm.{name}"] = ps
        if self.embedding_norm is not None:
            for name, ps in self.embedding_norm.params().items():
                p[f"embedding_norm.{name}"] = ps
        if not s.tie_embeddings:
            p["lm_head"] = ParamSpec((s.vocab_size, s.hidden_size))
        return p

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embed = tensors["embed"]
        self.lm_head = self.embed if self.spec.tie_embeddings else tensors["lm_head"]
        if self.spec.embedding_pairs is not None:
            self.embed_pairs = tensors["embed_pairs"]
        for i, block in enumerate(self.blocks):
            prefix = f"layers.{i}."
            block.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})
        self.final_norm.bind({k[len("final_norm."):]: v for k, v in tensors.items() if k.startswith("final_norm.")})
        if self.embedding_norm is not None:
            self.embedding_norm.bind({k[len("embedding_norm."):]: v for k, v in tensors.items()
                                      if k.startswith("embedding_norm.")})

    @property
    def graph_safe(self) -> bool:
        if self._graph_safe is None:          # the parts do not change after the model is built
            self._graph_safe = all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe
        return self._graph_safe

    def batch_tilings(self):
        """Every table of query-row blocks that some part of the model reads (``Part.batch_tilings``)."""
        out = {}
        for b in self.blocks:
            for name, tiling in b.batch_tilings().items():
                if out.setdefault(name, tiling) != tiling:
                    raise ValueError(f"two parts ask for different tilings under the name {name!r}")
        return out

    def graph_variant(self, n_tokens: int, longest_context: int):
        """What a captured step of single tokens fixes beforehand, over all parts (``Part.graph_variant``)."""
        out = {}
        for b in self.blocks:
            out.update(b.graph_variant(n_tokens, longest_context))
        return out

    # ------------------------------------------------------------------ caches
    def cache_needs(self) -> List[object]:
        """Per schedule entry: what the run's mixer wants cached (None if it owns no cache).  A model whose embedding
        looks at the token before (``DecoderSpec.embedding_pairs``) keeps a request's last token: one more entry
        behind the schedule's, an int per state slot."""
        out = []
        for e in self.spec.schedule:
            out.append(self.blocks[e.layer].cache_need() if e.cache_of is None else None)
        if self.spec.embedding_pairs is not None:
            out.append(StateNeed((1,), torch.int32))
        return out

    @staticmethod
    def _fold(stream, deltas):
        """A block may leave several outputs still to be added to the stream (one per branch); whoever cannot take
        them as they are gets them added here."""
        ops.add_dual_norm(stream, deltas, None, None, 0.0, 0.0, None, None)
        return None

    # ------------------------------------------------------------------ one step
    def forward(self, batch, storage) -> torch.Tensor:
        """Runs the step's tokens through the schedule; returns float32 logits [n_want, vocab]."""
        T = batch.num_tokens
        H = self.spec.hidden_size
        dev = self.env.device
        S = self.spec.streams
        stream = torch.empty((T, H) if S is None else (T, S, H), dtype=torch.float32, device=dev)
        if self.spec.embedding_pairs is None:
            ops.embedding(self.embed, batch.tokens, stream, self.spec.embedding_scale)
        else:
            buckets, mul_prev, mul_cur = self.spec.embedding_pairs
            last = storage.layer_context(len(self.spec.schedule), batch, write=True).state
            ops.embedding_pair(self.embed, self.embed_pairs, batch, last, stream, self.spec.embedding_scale, buckets,
                               mul_prev, mul_cur)
            ops.last_token_update(batch, last)             # after every token of the step has read the old one
        if self.embedding_norm is not None:
            self.embedding_norm.forward(stream, stream)           # in place: a warp reads its row before it writes it
        delta = None
        schedule = self.spec.schedule
        for index, entry in enumerate(schedule):
            owner = index if entry.cache_of is None else entry.cache_of
            ctx = storage.layer_context(owner, batch, write=entry.cache_of is None)
            ctx.position = index
            ctx.next_block = self.blocks[schedule[index + 1].layer] if index + 1 < len(schedule) else None
            block = self.blocks[entry.layer]
            if isinstance(delta, tuple) and not getattr(block, "takes_delta_pair", False):
                delta = self._fold(stream, delta)
            delta = block.forward(stream, delta, ctx)
            if self.after_block is not None:
                self.after_block(index, stream, delta)
        if isinstance(delta, tuple):
            delta = self._fold(stream, delta)
        n_want = batch.num_want
        logits = torch.empty((n_want, self.spec.vocab_size), dtype=torch.float32, device=dev)
        if n_want:
            hidden = torch.empty((n_want, H), dtype=self.env.act_dtype, device=dev)
            if S is None:
                self.final_norm.add_forward(stream, delta, hidden, rows=batch.want_rows)
            else:                                  # the sum of the streams goes to the final norm
                n = self.final_norm
                ops.hyper_read_norm(stream, None, n.p_weight, n.spec.eps, hidden, rows=batch.want_rows, offset=n.spec.offset)
            ops.linear(hidden, self.lm_head, logits)
            if self.spec.logit_softcap is not None:
                ops.softcap(logits, self.spec.logit_softcap)
        return logits
