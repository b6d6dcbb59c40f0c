"""Causal grouped-query attention over the paged cache (rollout/monkey_patch/qwen3.py:25-56).

Projections q, k, v as one fused product (the reference runs three, :29-31; the fused weight is
their row-wise concatenation), per-head RMSNorm of q and k before the rotation (:29-30),
rotation and cache write in one kernel (for a step of single tokens: inside the attention kernel),
attention over the block table, output projection
(:55-56).  Sizes, window, norm and position encoding come from the specification.
"""
from __future__ import annotations

import torch

from ..ext import ops
from .base import MIXERS, NORMS, POSITION_ENCODINGS, KVCacheNeed, Mixer, ParamSpec, Tiling


@MIXERS.register("attention")
class PagedAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_kv_heads={spec.num_kv_heads}")
        if spec.head_dim % 16 or not (16 <= spec.head_dim <= 256):
            raise ValueError(f"head_dim={spec.head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("window must be positive")
        self.q_norm = NORMS.build(spec.qk_norm, env) if spec.qk_norm is not None else None
        self.k_norm = NORMS.build(spec.qk_norm, env) if spec.qk_norm is not None else None
        if spec.qk_norm is not None and (spec.qk_norm.kind != "rmsnorm" or spec.qk_norm.size != spec.head_dim):
            raise ValueError("the fused q/k norm is an RMSNorm over head_dim")
        self.position = POSITION_ENCODINGS.build(spec.position, env) if spec.position is not None else None
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim

    # ------------------------------------------------------------------ parameters and cache
    def params(self):
        s = self.spec
        p = {"qkv": ParamSpec((self.q_size + 2 * self.kv_size, s.hidden_size)),
             "o": ParamSpec((s.hidden_size, self.q_size))}
        if self.q_norm is not None:
            p["q_norm.weight"] = self.q_norm.params()["weight"]
            p["k_norm.weight"] = self.k_norm.params()["weight"]
        return p

    def bind(self, tensors):
        self.p_qkv = tensors["qkv"]
        self.p_o = tensors["o"]
        if self.q_norm is not None:
            self.q_norm.bind({"weight": tensors["q_norm.weight"]})
            self.k_norm.bind({"weight": tensors["k_norm.weight"]})

    def cache_need(self):
        return KVCacheNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def batch_tilings(self):
        """The row blocks of the tensor-core kernel for prompt portions that this head size runs on."""
        if self.env.act_dtype != torch.bfloat16:
            return {}
        if self.spec.head_dim in ops.TC5_ATTENTION_HEAD_DIMS:
            return {ops.TILES_TC5: Tiling(ops.TC5_TILE_ROWS, heaviest_first=True)}
        return {ops.TILES_MMA: Tiling(ops.MMA_TILE_ROWS)}

    def graph_variant(self, n_tokens, longest_context):
        """A captured step cannot change the grid of the split-KV decode kernel: the number of key splits
        is fixed per captured graph."""
        if self.env.act_dtype != torch.bfloat16:
            return {}
        s = self.spec
        return {ops.decode_splits_key(s.num_heads, s.num_kv_heads, s.window):
                ops.decode_splits_for(n_tokens, longest_context, s.num_heads, s.num_kv_heads, s.window)}

    # ------------------------------------------------------------------ one step
    def forward(self, x, ctx):
        T = x.shape[0]
        qkv = ctx.buffer("attention.qkv", (T, self.q_size + 2 * self.kv_size), x.dtype, x.device)
        ops.linear(x, self.p_qkv, qkv)
        o = self.core(qkv, ctx)
        y = ctx.buffer("attention.y", (T, self.spec.hidden_size), x.dtype, x.device)
        ops.linear(o, self.p_o, y)
        return y

    # A mixer that is "product, something in the middle, product" says so, and a block may then run the two
    # products in kernels of its own choosing (fused with the norms around them).
    def in_projection(self):
        """(weight [q + 2 kv, hidden], name of the buffer its output goes to)."""
        return self.p_qkv, "attention.qkv"

    def out_projection(self):
        return self.p_o

    def core(self, qkv, ctx):
        """From the projections [T, q + 2 kv] to the attention output [T, q]: per-head norm, position encoding,
        cache write, attention over the block table."""
        s, b, kv = self.spec, ctx.batch, ctx.kv
        T = qkv.shape[0]
        qw = self.q_norm.p_weight if self.q_norm is not None else None
        kw = self.k_norm.p_weight if self.k_norm is not None else None
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        offset = s.qk_norm.offset if s.qk_norm is not None else 0.0
        tables = self.position.rotary_tables() if self.position is not None else None
        o = ctx.buffer("attention.o", (T, self.q_size), qkv.dtype, qkv.device)
        if (tables is not None or self.position is None) and ops.decode_only(b, qkv.dtype, s.num_heads, s.num_kv_heads, s.window):
            # single decoded tokens only: norm, rotation, cache write and attention are one kernel
            cos, sin, rot = tables if tables is not None else (None, None, 0)
            ops.attention_decode_fused(qkv, qw, kw, eps, offset, cos, sin, rot, kv.k, kv.v, b, kv.block_table,
                                       kv.page_size, o, s.num_heads, s.num_kv_heads, s.head_dim, s.scale, s.window,
                                       write_kv=ctx.write_cache)
            return o
        if tables is not None or self.position is None:
            cos, sin, rot = tables if tables is not None else (None, None, 0)
            ops.qk_norm_rope_write(qkv, qw, kw, eps, cos, sin, rot, b.pos, b.tok_seg, kv.block_table,
                                   kv.page_size, kv.k, kv.v, s.num_heads, s.num_kv_heads, s.head_dim,
                                   write_kv=ctx.write_cache, offset=offset)
        else:
            # an encoding that is not a rotation of pairs: norm, then the encoding's own in-place
            # step on q and k, then the cache write
            ops.qk_norm_rope_write(qkv, qw, kw, eps, None, None, 0, b.pos, b.tok_seg, kv.block_table,
                                   kv.page_size, kv.k, kv.v, s.num_heads, s.num_kv_heads, s.head_dim,
                                   write_kv=False, offset=offset)
            self.position.apply(qkv, b, s.num_heads, s.num_kv_heads, s.head_dim)
            if ctx.write_cache:
                ops.qk_norm_rope_write(qkv, None, None, 0.0, None, None, 0, b.pos, b.tok_seg, kv.block_table,
                                       kv.page_size, kv.k, kv.v, s.num_heads, s.num_kv_heads, s.head_dim,
                                       write_kv=True)
        ops.paged_attention(qkv, kv.k, kv.v, b, kv.block_table, kv.page_size, o, s.num_heads,
                            s.num_kv_heads, s.head_dim, s.scale, s.window)
        return o


@MIXERS.register("gated_attention")
class GatedAttention(Mixer):
    """``GatedAttentionSpec``: one product gives a row [q | k | v | gate] (k and v only if the layer owns its cache; v
    only if it has a value projection); one kernel prepares the row (biases, the norm over a whole projection, the
    rotation of neighbouring pairs, heads padded to the cache's head size, keys and values into their pages); the
    engine's paged attention kernels run with the layer's score options; the gate is applied and the heads are
    projected out.  A layer that reads another run's cache prepares its queries only."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads={s.num_heads} is not a multiple of num_kv_heads={s.num_kv_heads}")
        if s.window is not None and s.chunk is not None:
            raise ValueError("a window and a chunk exclude each other")
        if (s.window is not None and s.window <= 0) or (s.chunk is not None and s.chunk <= 0):
            raise ValueError("window and chunk must be positive")
        if s.gate not in (None, "head", "element"):
            raise ValueError(f"gate={s.gate!r}; known: None, 'head', 'element'")
        if s.values_are_keys and s.value_dim != s.key_dim:
            raise ValueError("values that are the keys have the keys' size")
        self.D = (max(s.key_dim, s.value_dim) + 15) // 16 * 16          # the head size of the cache and the kernels
        if not (16 <= self.D <= 256):
            raise ValueError(f"heads of {max(s.key_dim, s.value_dim)} elements: the attention kernels take up to 256")
        self.position = POSITION_ENCODINGS.build(s.position, env) if s.position is not None else None
        if self.position is not None and not getattr(self.position, "interleaved", False):
            raise ValueError("the row kernel rotates neighbouring pairs: the position encoding must be 'rope_interleaved'")
        if self.position is not None and s.position.rotary_dim > s.key_dim:
            raise ValueError("the rotary width is at most the key size")
        self.nq = s.num_heads * s.key_dim
        self.nk = s.num_kv_heads * s.key_dim if s.own_cache else 0
        self.nv = s.num_kv_heads * s.value_dim if (s.own_cache and not s.values_are_keys) else 0
        self.ng = 0 if s.gate is None else s.num_heads if s.gate == "head" else s.num_heads * s.value_dim
        self._slopes = None
        self._sink = None

    # ------------------------------------------------------------------ parameters and cache
    def params(self):
        s = self.spec
        p = {"in": ParamSpec((self.nq + self.nk + self.nv + self.ng, s.hidden_size)),
             "o": ParamSpec((s.hidden_size, s.num_heads * self.D))}
        if s.bias:
            p["bias"] = ParamSpec((self.nq + self.nk + self.nv,), role="vector", init="normal:0.2")
        if s.whole_norm_eps is not None:
            p["q_norm"] = ParamSpec((self.nq,), role="vector", init="ones_normal")
            if s.own_cache:
                p["k_norm"] = ParamSpec((self.nk,), role="vector", init="ones_normal")
        if s.sink:
            p["sink"] = ParamSpec((s.num_heads,), role="vector", init="normal:0.5")
        return p

    def bind(self, tensors):
        super().bind(tensors)
        s = self.spec
        if s.sink:
            self._sink = self.p_sink.float().contiguous()
        if s.slope_exponent is not None:
            h = torch.arange(1, s.num_heads + 1, dtype=torch.float64)
            self._slopes = torch.exp2(-float(s.slope_exponent) * h / s.num_heads).float().to(self.env.device)

    def cache_need(self):
        s = self.spec
        return KVCacheNeed(s.num_kv_heads, self.D, s.cache_window) if s.own_cache else None

    def batch_tilings(self):
        if self.env.act_dtype != torch.bfloat16:
            return {}
        if self.D in ops.TC5_ATTENTION_HEAD_DIMS:
            return {ops.TILES_TC5: Tiling(ops.TC5_TILE_ROWS, heaviest_first=True)}
        return {ops.TILES_MMA: Tiling(ops.MMA_TILE_ROWS)}

    def graph_variant(self, n_tokens, longest_context):
        if self.env.act_dtype != torch.bfloat16:
            return {}
        s = self.spec
        bound = s.window or s.chunk
        return {ops.decode_splits_key(s.num_heads, s.num_kv_heads, bound):
                ops.decode_splits_for(n_tokens, longest_context, s.num_heads, s.num_kv_heads, bound)}

    def out_projection(self):
        return self.p_o

    # ------------------------------------------------------------------ one step
    def forward(self, x, ctx):
        s, b, kv = self.spec, ctx.batch, ctx.kv
        T, dev, dt = x.shape[0], x.device, x.dtype
        if kv is None:
            raise ValueError("a gated attention needs a paged cache: its own, or the one its schedule entry names")
        if kv.k.shape[-1] != self.D or kv.k.shape[1] != s.num_kv_heads:
            raise ValueError("the cache this layer reads has other heads than the layer")
        proj = ctx.buffer("gated_attention.proj", (T, self.nq + self.nk + self.nv + self.ng), dt, dev)
        ops.linear(x, self.p_in, proj)
        write = bool(ctx.write_cache and s.own_cache)
        biases = None
        if s.bias:
            bq, bk = self.p_bias[:self.nq], self.p_bias[self.nq:self.nq + self.nk]
            biases = (bq, bk if write else None, self.p_bias[self.nq + self.nk:] if write else None)
        norms = None
        if s.whole_norm_eps is not None:
            norms = (self.p_q_norm, self.p_k_norm if write else None)
        q = ctx.buffer("gated_attention.q", (T, s.num_heads * self.D), dt, dev)
        ops.attention_prepare(proj, 0, self.nq, -1 if (s.values_are_keys or not s.own_cache) else self.nq + self.nk,
                              biases, norms, float(s.whole_norm_eps or 0.0),
                              self.position.tables() if self.position is not None else None, b, kv, q,
                              s.num_heads, s.num_kv_heads, s.key_dim, s.value_dim, self.D, write_kv=write)
        o = ctx.buffer("gated_attention.o", (T, s.num_heads * self.D), dt, dev)
        ops.paged_attention(q, kv.k, kv.v, b, kv.block_table, kv.page_size, o, s.num_heads, s.num_kv_heads, self.D,
                            s.scale, s.window, self._sink, s.chunk, s.softcap, self._slopes)
        if s.gate is not None:
            ops.attention_gate(o, proj, self.nq + self.nk + self.nv, s.gate == "head", s.num_heads, s.value_dim, self.D)
        y = ctx.buffer("gated_attention.y", (T, s.hidden_size), torch.float32, dev)
        ops.linear(o, self.p_o, y)
        return y
