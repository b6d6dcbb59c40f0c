"""Attention over a paged cache of latents.

Every token leaves one vector in the cache: a normed latent c of ``kv_rank`` numbers and, behind it, a rotated key
part of ``rot_dim`` numbers that all heads share.  A head's key is ``[U_h c | rotated part]`` and its value ``V_h c``.
The engine never expands them: since ``q_h . (U_h c) = (U_h^T q_h) . c`` and ``sum_j a_j V_h c_j = V_h sum_j a_j c_j``,
a head's query is carried into the latent's space once per token (a product per head with U_h^T), the attention
runs over the cached vectors themselves, one kv head for all query heads, and the weighted mean of the latents is carried
to the head's value space afterwards (a product per head with V_h).  The same path serves prompts, portions and
decoded tokens, so the cache is all a request keeps.

Parameters: ``in`` (all projections of the mixer's input, fused: the queries or their latent, the key/value latent
with the rotated part, the gates), ``q_norm.weight`` / ``uq`` (queries through a latent), ``kv_norm.weight``,
``uk`` [heads * key_dim, kv_rank], ``uv`` [heads * value_dim, kv_rank], ``sink`` [heads], ``o``.
"""
from __future__ import annotations

import numpy as np
import torch

from ..ext import ops
from .base import MIXERS, POSITION_ENCODINGS, LatentCacheNeed, Mixer, ParamSpec, Tiling


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if s.rot_dim % 2 or s.rot_dim < 0:
            raise ValueError(f"rot_dim={s.rot_dim} must be even")
        if s.rot_dim and (s.position is None or s.position.rotary_dim != s.rot_dim):
            raise ValueError("a rotated part needs a position encoding of its width")
        if s.window is not None and s.window <= 0:
            raise ValueError("window must be positive")
        if not (0 < s.kv_rank <= ops.LATENT_MAX_RANK):
            raise ValueError(f"kv_rank={s.kv_rank}: the kernels take latents of up to {ops.LATENT_MAX_RANK} numbers")
        self.position = POSITION_ENCODINGS.build(s.position, env) if s.rot_dim else None
        self.q_head = s.key_dim + s.rot_dim
        self.q_size = s.num_heads * self.q_head
        self.first = s.q_rank if s.q_rank is not None else self.q_size          # queries, or their latent
        self.c_off = self.first
        self.g_off = self.first + s.kv_rank + s.rot_dim
        self.in_size = self.g_off + (s.num_heads if s.gate else 0)
        # a cached vector's width: latent and rotated part, padded to whole 16s (the tensor-core kernels' head sizes)
        self.width = (s.kv_rank + s.rot_dim + 15) // 16 * 16

    # ------------------------------------------------------------------ parameters and cache
    def params(self):
        s = self.spec
        p = {"in": ParamSpec((self.in_size, s.hidden_size)),
             "kv_norm.weight": ParamSpec((s.kv_rank,), role="vector", init="ones_normal"),
             "uk": ParamSpec((s.num_heads * s.key_dim, s.kv_rank)),
             "uv": ParamSpec((s.num_heads * s.value_dim, s.kv_rank)),
             "o": ParamSpec((s.hidden_size, s.num_heads * s.value_dim))}
        if s.q_rank is not None:
            p["q_norm.weight"] = ParamSpec((s.q_rank,), role="vector", init="ones_normal")
            p["uq"] = ParamSpec((self.q_size, s.q_rank))
        if s.sink:
            p["sink"] = ParamSpec((s.num_heads,), role="vector", init="normal")
        return p

    def bind(self, tensors):
        s = self.spec
        super().bind(tensors)
        # U_h^T per head, [heads, kv_rank, key_dim]: the map that carries a head's query into the latent's space
        self.uk_t = self.p_uk.view(s.num_heads, s.key_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.uv_h = self.p_uv.view(s.num_heads, s.value_dim, s.kv_rank)
        self.sink_f32 = self.p_sink.float().contiguous() if s.sink else None
        self.ukv = torch.cat([self.p_uk, self.p_uv], dim=0) if self.expanded_head() is not None else None     # [U; V]

    def cache_need(self):
        return LatentCacheNeed(self.width, self.spec.window)

    def _on_tensor_cores(self):
        return ops.latent_on_tensor_cores(self.env.act_dtype, self.width)

    def expanded_head(self):
        """The head size at which portions of prompts run with the heads' keys and values written out, or None: when
        that head (key and rotated part, or value, padded to whole 16s) is one the tcgen05 attention kernel takes and
        is narrower than a cached vector, a head scores and averages fewer numbers a key that way than folded."""
        s = self.spec
        head = (max(s.key_dim + s.rot_dim, s.value_dim) + 15) // 16 * 16
        if self.env.act_dtype == torch.bfloat16 and head in ops.TC5_ATTENTION_HEAD_DIMS and head < self.width:
            return head
        return None

    def batch_tilings(self):
        """The row blocks of the tensor-core attention kernels for prompt portions that this part may run."""
        out = {}
        if self.expanded_head() is not None:
            out[ops.TILES_TC5] = Tiling(ops.TC5_TILE_ROWS, heaviest_first=True)
        if self._on_tensor_cores():
            if self.width in ops.TC5_ATTENTION_HEAD_DIMS:
                out[ops.TILES_TC5] = Tiling(ops.TC5_TILE_ROWS, heaviest_first=True)
            else:
                out[ops.TILES_MMA] = Tiling(ops.MMA_TILE_ROWS)
        return out

    def graph_variant(self, n_tokens, longest_context):
        """A captured step cannot change the grid of the split-KV decode kernel: the number of key splits is fixed per
        captured graph (all query heads share the one key/value head)."""
        if not self._on_tensor_cores():
            return {}
        s = self.spec
        return {ops.decode_splits_key(s.num_heads, 1, s.window): ops.decode_splits_for(n_tokens, longest_context, s.num_heads, 1, s.window)}

    # ------------------------------------------------------------------ portions of prompts, keys and values written out
    EXPANDED_SCRATCH_LIMIT = 2 << 30          # bytes of scratch pools beyond which prompts run folded like decoded tokens

    def _visible_slots(self, ctx):
        """int32 [n]: page * page_size + row of every cached vector that some token of a segment of several tokens sees,
        segment by segment; worked out on the host once per step and group of layers."""
        b, kv, window = ctx.batch, ctx.kv, self.spec.window
        key = ("latent.visible_slots", kv.group, window)
        held = b.scratch
        if key not in held:
            host, P = b.host, kv.page_size
            table = host.block_tables[kv.group]
            runs = []
            for i in range(host.num_segments):
                if int(host.cu_q[i + 1]) - int(host.cu_q[i]) <= 1:
                    continue
                lo = max(0, int(host.seg_pos0[i]) - window + 1) if window else 0
                p = np.arange(lo, int(host.seg_kv_len[i]), dtype=np.int64)
                runs.append(table[i, p // P].astype(np.int64) * P + p % P)
            slots = np.concatenate(runs).astype(np.int32)
            held[key] = torch.from_numpy(slots).to(b.tokens.device, non_blocking=True)
        return held[key]

    def _expanded_ok(self, ctx):
        head = self.expanded_head()
        b = ctx.batch
        if head is None or getattr(b, "scratch", None) is None or b.host.num_multi == 0 or ctx.kv.group < 0:
            return None
        pages = ctx.kv.k.shape[0]
        if 2 * pages * self.spec.num_heads * ctx.kv.page_size * head * 2 > self.EXPANDED_SCRATCH_LIMIT:
            return None
        return head

    def _expanded_prefill(self, head, q, q_abs, ctx, packed):
        """The segments of several tokens: visible latents gathered and carried through [U; V], scattered into scratch
        pools with the request's own pages, the tcgen05 attention with a key/value head per query head, and the
        values taken into ``packed``."""
        s, b, kv = self.spec, ctx.batch, ctx.kv
        T, dev, dt = q_abs.shape[0], q_abs.device, q_abs.dtype
        H, D, R, C, Vd = s.num_heads, s.key_dim, s.rot_dim, s.kv_rank, s.value_dim
        slots = self._visible_slots(ctx)
        n = slots.numel()
        lat = ctx.buffer("latent.x_rows", (n, self.width), dt, dev)
        ops.gather_rows(kv.k.view(-1, self.width), slots, lat)
        expanded = ctx.buffer("latent.x_kv", (n, H * (D + Vd)), dt, dev)
        ops.linear(lat[:, :C], self.ukv, expanded)
        pools = ctx.buffer("latent.x_pools", (2, kv.k.shape[0], H, kv.page_size, head), dt, dev)
        ops.latent_expand_scatter(expanded, lat, C, R, slots, kv.page_size, pools[0], pools[1], H, D, Vd)
        qx = ctx.buffer("latent.x_q", (T, H * head), dt, dev)
        ops.latent_expand_query(q, q_abs, self.width, C, qx, H, D, R)
        ox = ctx.buffer("latent.x_o", (T, H * head), dt, dev)
        ops.attention_prefill_tc5(qx, pools[0], pools[1], b.tiles[ops.TILES_TC5], b.cu_q, b.seg_pos0, kv.block_table,
                                  kv.page_size, ox, H, H, head, s.scale, s.window or 0,
                                  ops._prefill_split_count(b, H, s.window), b.scratch, self.sink_f32)
        ops.latent_take_values(ox, b, packed, H, Vd)

    # ------------------------------------------------------------------ one step
    def forward(self, x, ctx):
        s, b, kv = self.spec, ctx.batch, ctx.kv
        T, dt, dev = x.shape[0], x.dtype, x.device
        H, D, R, C, W = s.num_heads, s.key_dim, s.rot_dim, s.kv_rank, self.width
        proj = ctx.buffer("latent.in", (T, self.in_size), dt, dev)
        ops.linear(x, self.p_in, proj)
        if s.q_rank is not None:
            cq = ctx.buffer("latent.cq", (T, s.q_rank), dt, dev)
            ops.rmsnorm_columns(proj[:, :s.q_rank], self.p_q_norm_weight, s.eps, cq)
            q = ctx.buffer("latent.q", (T, self.q_size), dt, dev)
            ops.linear(cq, self.p_uq, q)
        else:
            q = proj                                             # the queries are the first columns of the projection
        cos, sin, _ = self.position.tables() if self.position is not None else (None, None, 0)
        # a head's query as the attention reads it: [its unrotated part carried into the latent's space | its rotated part]
        q_abs = ctx.buffer("latent.q_abs", (T, H * W), dt, dev)
        ops.latent_write(proj, self.c_off, self.p_kv_norm_weight, s.eps, C, R, cos, sin, b, kv.block_table, kv.page_size,
                         kv.k, ctx.write_cache, q, 0, H, D, q_abs)
        expanded = self._expanded_ok(ctx)
        folded = expanded is None or b.host.decode_segs.shape[0] > 0          # some token runs over the cached vectors themselves
        if folded:
            q_heads = q[:, :self.q_size].view(T, H, self.q_head)[:, :, :D].transpose(0, 1)               # [H, T, D]
            ops.linear_heads(q_heads, self.uk_t, q_abs.view(T, H, W)[:, :, :C].transpose(0, 1))
        o_abs = ctx.buffer("latent.o_abs", (T, H * W), dt, dev)
        packed = ctx.buffer("latent.packed", (T, H * s.value_dim), dt, dev)
        if expanded is None:
            ops.latent_attention(q_abs, kv.k, b, kv.block_table, kv.page_size, self.sink_f32, o_abs, H, C, R, s.scale, s.window)
        elif b.host.decode_segs.shape[0]:
            # portions of prompts run expanded below; the single tokens beside them run folded, over the keys split
            ops.attention_decode_mma(q_abs, kv.k.unsqueeze(1), kv.k.unsqueeze(1), b.decode_segs, b.cu_q, b.seg_kv_len,
                                     kv.block_table, kv.page_size, o_abs, H, 1, W, s.scale, s.window or 0,
                                     ops._decode_split_count(b, H, 1, s.window), b.scratch, self.sink_f32)
        if folded:
            # the weighted means of the latents, head by head, into the heads' value spaces (rows of tokens that run
            # expanded hold nothing yet and are written below)
            ops.linear_heads(o_abs.view(T, H, W)[:, :, :C].transpose(0, 1), self.uv_h, packed.view(T, H, s.value_dim).transpose(0, 1))
        if expanded is not None:
            self._expanded_prefill(expanded, q, q_abs, ctx, packed)
        if s.gate:
            ops.head_gate(packed, proj[:, self.g_off:self.g_off + H], H)
        y = ctx.buffer("latent.y", (T, s.hidden_size), dt, dev)
        ops.linear(packed, self.p_o, y)
        return y
