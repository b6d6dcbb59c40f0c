"""The Duvadra decoder as a ``DecoderSpec`` plus the map from its checkpoint tensor names to the parts' parameters.

Embedding times a scale plus a row of a table of token pairs; pre-norm layers whose sublayers join the residual stream
times a factor; a layer's mixer is an attention inside blocks of positions with softly capped scores, a distance penalty
per head and a gate per head (optionally on the keys and values of an earlier layer), or the weighted sum of two mixers on
the same input: a windowed attention with a sink beside a gated delta rule, or a windowed attention whose values are its
keys beside a gated linear recurrence.  Feed-forwards are capped gated units or mixtures of experts with logistic scores.
A final norm, an untied head, softly capped logits.

Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head``; ``l<i>.norm1 / norm2``; ``l<i>.mix.{q, k, v, g, o}`` (attention;
no k, v with ``kv_from``); ``l<i>.mix.left.{q, k, v, g, o, sink}`` with ``.b`` biases, or ``left.{q, k, g, o, q.norm, k.norm}``;
``l<i>.mix.right.{q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, norm, g, o}`` or ``right.{y, y.b, x, x.b, conv, conv.b,
ra, ra.b, ri, ri.b, lam, o}``; ``l<i>.mlp.{gate, up, down}`` or ``l<i>.mlp.{router, e<j>.{gate, up, down}}``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..config.duvadra_config import DuvadraConfig
from ..parts.spec import (BlockSpec, ClampedGLUSpec, DecoderSpec, GatedAttentionSpec, GatedDeltaSpec,
                          GatedLinearRecurrenceSpec, InterleavedRopeSpec, MixerSumSpec, MoESpec, NormSpec, ScheduleEntry,
                          SwiGLUSpec)
from ..weights.loader import Source

SLOPE_EXPONENT = 8.0          # a head's distance penalty is 2^(-8 (h + 1) / heads) a position
DECAY_SCALE = 8.0             # log f = -8 r softplus(lam) in the gated linear recurrence
GLU_ALPHA = 1.702             # g sigmoid(1.702 g) in the capped gated unit


def _padded_head(m: dict) -> int:
    return (max(int(m["dim"]), int(m["vdim"])) + 15) // 16 * 16


def _mask(m: dict) -> Optional[int]:
    return int(m["mask"]["size"]) if m.get("mask") else None


def _cache_windows(cfg: DuvadraConfig) -> Dict[int, Optional[int]]:
    """Attention layer that owns keys -> how many of the latest keys its cache must keep: the largest block size among
    the layer and the layers that read its keys, or None (all) if one of them has no mask."""
    spans: Dict[int, list] = {}
    for i, layer in enumerate(cfg.layers):
        if layer["type"] == "attention":
            src = layer["mixer"].get("kv_from")
            spans.setdefault(i if src is None else int(src), []).append(_mask(layer["mixer"]))
    return {i: (None if any(v is None for v in vs) else max(vs)) for i, vs in spans.items()}


def _left_spec(kind: str, m: dict, width: int, eps: float, max_positions: int) -> GatedAttentionSpec:
    common = dict(hidden_size=width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), key_dim=int(m["dim"]),
                  value_dim=int(m["vdim"]), scale=float(m["scale"]), window=_mask(m), cache_window=_mask(m), gate="element")
    if kind == "parallel":
        return GatedAttentionSpec(bias=True, sink=True, **common)
    rot = m.get("rot")
    position = (InterleavedRopeSpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]), max_positions=max_positions)
                if rot and int(rot["dims"]) else None)
    return GatedAttentionSpec(whole_norm_eps=eps, position=position, values_are_keys=True, **common)


def _mixer_spec(cfg: DuvadraConfig, i: int, windows, max_positions: int):
    layer = cfg.layers[i]
    kind, m, W, eps = layer["type"], layer["mixer"], cfg.width, cfg.eps
    if kind == "attention":
        src = m.get("kv_from")
        sc = m.get("softcap")
        return GatedAttentionSpec(hidden_size=W, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                                  key_dim=int(m["dim"]), value_dim=int(m["vdim"]), scale=float(m["scale"]), chunk=_mask(m),
                                  softcap=float(sc) if sc else None, slope_exponent=SLOPE_EXPONENT, gate="head",
                                  own_cache=src is None, cache_window=windows.get(i) if src is None else None)
    left = _left_spec(kind, m["left"], W, eps, max_positions)
    r = m["right"]
    if kind == "parallel":
        right = GatedDeltaSpec(hidden_size=W, num_heads=int(r["heads"]), num_kv_heads=int(r["kv_heads"]),
                               key_dim=int(r["dim"]), value_dim=int(r["vdim"]), conv_taps=int(r["conv"]), eps=eps)
    else:
        right = GatedLinearRecurrenceSpec(hidden_size=W, width=int(r["width"]), blocks=int(r["blocks"]),
                                          conv_taps=int(r["conv"]), decay_scale=DECAY_SCALE)
    return MixerSumSpec(names=("left", "right"), mixers=(left, right),
                        scales=(float(m["left_scale"]), float(m["right_scale"])))


def _mlp_spec(mlp: Optional[dict], width: int):
    if not mlp:
        return None
    if mlp["kind"] == "dense":
        return ClampedGLUSpec(hidden_size=width, intermediate_size=int(mlp["ff"]), limit=float(mlp["limit"]), alpha=GLU_ALPHA)
    r = mlp["router"]
    g = r.get("groups")
    return MoESpec(hidden_size=width, num_experts=int(r["experts"]), top=int(r["top"]),
                   expert=SwiGLUSpec(hidden_size=width, intermediate_size=int(mlp["expert"]["ff"]), interleave=0),
                   groups=int(g["count"]) if g else 1, keep_groups=int(g["keep"]) if g else 1, renorm_tiny=1e-20,
                   score="sigmoid", group_top=2, weight_scale=float(r.get("scale", 1.0)))


def decoder_spec(cfg: DuvadraConfig, max_positions: Optional[int] = None) -> DecoderSpec:
    max_positions = max_positions or 4096
    W = cfg.width
    norm = NormSpec(size=W, eps=cfg.eps)
    windows = _cache_windows(cfg)
    blocks, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        ff = _mlp_spec(layer.get("mlp"), W)
        blocks.append(BlockSpec(mixer=_mixer_spec(cfg, i, windows, max_positions), feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff is not None else None, residual_scale=cfg.residual_mult,
                                float_outputs=True))
        src = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
        schedule.append(ScheduleEntry(i, cache_of=int(src) if src is not None else None))
    return DecoderSpec(vocab_size=cfg.vocab, hidden_size=W, layers=tuple(blocks), schedule=tuple(schedule), final_norm=norm,
                       tie_embeddings=False, logit_softcap=cfg.logit_softcap, embedding_scale=cfg.embedding_scale,
                       embedding_pairs=cfg.bigram)


def weight_sources(cfg: DuvadraConfig) -> Dict[str, Source]:
    m: Dict[str, Source] = {"embed": Source(("embed",)), "final_norm.weight": Source(("final.norm",)),
                            "lm_head": Source(("head",))}
    if cfg.bigram is not None:
        m["embed_pairs"] = Source(("bigram",))
    for i, layer in enumerate(cfg.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        mix, kind, mm = src + "mix.", layer["type"], layer["mixer"]
        m[dst + "mixer_norm.weight"] = Source((src + "norm1",))
        if kind == "attention":
            own = mm.get("kv_from") is None
            m[dst + "mixer.in"] = Source((mix + "q",) + ((mix + "k", mix + "v") if own else ()) + (mix + "g",))
            m[dst + "mixer.o"] = Source((mix + "o",), pad_cols=(int(mm["vdim"]), _padded_head(mm)))
        else:
            l, r = mix + "left.", mix + "right."
            left = mm["left"]
            lo = Source((l + "o",), pad_cols=(int(left["vdim"]), _padded_head(left)))
            if kind == "parallel":
                m[dst + "mixer.left.in"] = Source((l + "q", l + "k", l + "v", l + "g"))
                m[dst + "mixer.left.bias"] = Source((l + "q.b", l + "k.b", l + "v.b"))
                m[dst + "mixer.left.sink"] = Source((l + "sink",))
                m[dst + "mixer.left.o"] = lo
                m[dst + "mixer.right.in"] = Source((r + "q", r + "k", r + "v", r + "g"))
                m[dst + "mixer.right.conv"] = Source((r + "q.conv", r + "k.conv", r + "v.conv"))
                m[dst + "mixer.right.beta"] = Source((r + "b",))
                m[dst + "mixer.right.decay"] = Source((r + "a",))
                for name in ("A_log", "dt_bias", "norm", "o"):
                    m[dst + "mixer.right." + name] = Source((r + name,))
            else:
                m[dst + "mixer.left.in"] = Source((l + "q", l + "k", l + "g"))
                m[dst + "mixer.left.q_norm"] = Source((l + "q.norm",))
                m[dst + "mixer.left.k_norm"] = Source((l + "k.norm",))
                m[dst + "mixer.left.o"] = lo
                m[dst + "mixer.right.in"] = Source((r + "y", r + "x"))
                m[dst + "mixer.right.in_bias"] = Source((r + "y.b", r + "x.b"))
                for ours, theirs in (("conv", "conv"), ("conv_bias", "conv.b"), ("gate_r", "ra"), ("gate_i", "ri"),
                                     ("gate_r_bias", "ra.b"), ("gate_i_bias", "ri.b"), ("lam", "lam"), ("o", "o")):
                    m[dst + "mixer.right." + ours] = Source((r + theirs,))
        mlp = layer.get("mlp")
        if mlp:
            p = src + "mlp."
            m[dst + "feed_forward_norm.weight"] = Source((src + "norm2",))
            if mlp["kind"] == "dense":
                m[dst + "feed_forward.gate_up"] = Source((p + "gate", p + "up"))
                m[dst + "feed_forward.down"] = Source((p + "down",))
            else:
                E = int(mlp["router"]["experts"])
                m[dst + "feed_forward.router"] = Source((p + "router",))
                m[dst + "feed_forward.experts.gate_up"] = Source(tuple(f"{p}e{j}.{n}" for j in range(E) for n in ("gate", "up")))
                m[dst + "feed_forward.experts.down"] = Source(tuple(f"{p}e{j}.down" for j in range(E)))
    return m


def checkpoint_shapes(cfg: DuvadraConfig) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """Every tensor of a checkpoint: name -> (shape, law of its random values).  Matrices are drawn with a deviation of
    fan_in^-1/2 (half that for the maps back into the stream, three times that for the routers: logistic scores far apart
    without running into one), norm weights around one, the others so that gates, decays and sinks are neither shut nor
    open."""
    W, V = cfg.width, cfg.vocab
    out: Dict[str, Tuple[Tuple[int, ...], str]] = {"embed": ((V, W), "normal:1.0"), "final.norm": ((W,), "ones_normal"),
                                                   "head": ((V, W), "fan_in")}
    if cfg.bigram is not None:
        out["bigram"] = ((cfg.bigram[0] + 1, W), "normal:0.5")

    def attention(x: str, a: dict, own: bool, values: bool, gate: int) -> None:
        H, G, D, Vd = int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"])
        out[x + "q"] = ((H * D, W), "fan_in")
        if own:
            out[x + "k"] = ((G * D, W), "fan_in")
            if values:
                out[x + "v"] = ((G * Vd, W), "fan_in")
        out[x + "g"] = ((gate, W), "fan_in")
        out[x + "o"] = ((W, H * Vd), "fan_in:0.5")

    for i, layer in enumerate(cfg.layers):
        p, kind, m = f"l{i}.", layer["type"], layer["mixer"]
        x = p + "mix."
        out[p + "norm1"] = ((W,), "ones_normal")
        if kind == "attention":
            attention(x, m, m.get("kv_from") is None, True, int(m["heads"]))
        else:
            a, r = m["left"], m["right"]
            H, G, D, Vd = int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"])
            attention(x + "left.", a, True, kind == "parallel", H * Vd)
            y = x + "right."
            if kind == "parallel":
                out[x + "left.q.b"] = ((H * D,), "normal:0.3")
                out[x + "left.k.b"] = ((G * D,), "normal:0.3")
                out[x + "left.v.b"] = ((G * Vd,), "normal:0.3")
                out[x + "left.sink"] = ((H,), "normal:1.0")
                RH, RG, RD, RV, K = int(r["heads"]), int(r["kv_heads"]), int(r["dim"]), int(r["vdim"]), int(r["conv"])
                out[y + "q"] = ((RG * RD, W), "fan_in")
                out[y + "k"] = ((RG * RD, W), "fan_in")
                out[y + "v"] = ((RH * RV, W), "fan_in")
                out[y + "q.conv"] = ((RG * RD, K), "normal:0.5")
                out[y + "k.conv"] = ((RG * RD, K), "normal:0.5")
                out[y + "v.conv"] = ((RH * RV, K), "normal:0.5")
                out[y + "b"] = ((RH, W), "fan_in")
                out[y + "a"] = ((RH, W), "fan_in")
                out[y + "A_log"] = ((RH,), "normal:0.5")
                out[y + "dt_bias"] = ((RH,), "normal:0.5")
                out[y + "norm"] = ((RV,), "ones_normal")
                out[y + "g"] = ((RH * RV, W), "fan_in")
                out[y + "o"] = ((W, RH * RV), "fan_in:0.5")
            else:
                out[x + "left.q.norm"] = ((H * D,), "ones_normal")
                out[x + "left.k.norm"] = ((G * D,), "ones_normal")
                RW, B, K = int(r["width"]), int(r["blocks"]), int(r["conv"])
                bs = RW // B
                out[y + "y"] = ((RW, W), "fan_in")
                out[y + "y.b"] = ((RW,), "normal:0.2")
                out[y + "x"] = ((RW, W), "fan_in")
                out[y + "x.b"] = ((RW,), "normal:0.2")
                out[y + "conv"] = ((RW, K), "normal:0.5")
                out[y + "conv.b"] = ((RW,), "normal:0.2")
                out[y + "ra"] = ((B, bs, bs), "fan_in")
                out[y + "ra.b"] = ((B, bs), "normal:0.5")
                out[y + "ri"] = ((B, bs, bs), "fan_in")
                out[y + "ri.b"] = ((B, bs), "normal:0.5")
                out[y + "lam"] = ((RW,), "normal:0.5")
                out[y + "o"] = ((W, RW), "fan_in:0.5")
        mlp = layer.get("mlp")
        if mlp:
            z = p + "mlp."
            out[p + "norm2"] = ((W,), "ones_normal")
            if mlp["kind"] == "dense":
                ff = int(mlp["ff"])
                out[z + "gate"] = ((ff, W), "fan_in")
                out[z + "up"] = ((ff, W), "fan_in")
                out[z + "down"] = ((W, ff), "fan_in:0.5")
            else:
                E, F = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
                out[z + "router"] = ((E, W), "fan_in:3")
                for j in range(E):
                    out[f"{z}e{j}.gate"] = ((F, W), "fan_in")
                    out[f"{z}e{j}.up"] = ((F, W), "fan_in")
                    out[f"{z}e{j}.down"] = ((W, F), "fan_in:0.5")
    return out


def ignorable_tensors(cfg: DuvadraConfig):
    """A layer without a feed-forward never reads a second norm; a file may hold it all the same."""
    return {f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if not layer.get("mlp")}
