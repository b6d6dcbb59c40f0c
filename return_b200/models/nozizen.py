"""The Nozizen decoder as a ``DecoderSpec`` plus the map from its checkpoint tensor names to the parts' parameters.

Embedding times a scale; layers of the pre-norm form over several residual streams (``HyperBlockSpec``; one plain stream
when the configuration names none) whose mixer is a time mix with a decay per token and key row (``wkv``), a state-space
mixer (``mamba2``) or a grouped-query softmax attention with a sliding window and ramped rotary positions, and whose
feed-forward is dense (the square of relu between two products) or a mixture of experts whose weights are the softmax
over the chosen logits; a run of layers may repeat with the same weights (every pass with a cache or state of its own:
the schedule names a layer once per run); a final norm of the streams' sum and the embedding table as the output head.

Tensor names: ``embed``, ``final.norm``; ``l<i>.norm1 / norm2``; ``l<i>.hc1.{in, out, mix}``, ``l<i>.hc2.{in, out, mix}``;
``l<i>.mix.*`` (wkv: ``mu.{r, k, v, g, w}, r, k, v, g, w1, w2, w0, u, norm, o``; mamba2: ``in, conv, conv.b, dt_bias, A_log,
D, norm, o``; attention: ``q, k, v, o``); ``l<i>.mlp.{up, down}`` or ``l<i>.mlp.{router, router.b, e<j>.{gate, up, down}}``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..config.model_config import ConfigError
from ..config.nozizen_config import NozizenConfig
from ..parts.spec import (AttentionSpec, DecoderSpec, DenseMLPSpec, HyperBlockSpec, MoESpec, NormSpec,
                          RampedRopeSpec, ScheduleEntry, StateSpaceSpec, SwiGLUSpec, TimeMixSpec)
from ..weights.loader import Source


def _padded_head(m: dict) -> int:
    """The head size the attention kernels run: key and value sizes padded to one multiple of 16."""
    return (max(int(m["dim"]), int(m["vdim"])) + 15) // 16 * 16


def _rope(m: dict, max_positions: int) -> Optional[RampedRopeSpec]:
    rot = m.get("rot")
    if not rot or not int(rot["dims"]):
        return None
    sc = rot.get("scaling") or None
    return RampedRopeSpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]), max_positions=max_positions,
                          factor=float(sc["factor"]) if sc else None, original=float(sc["original"]) if sc else 0.0,
                          fast=float(sc["fast"]) if sc else 0.0, slow=float(sc["slow"]) if sc else 0.0)


def _mixer_spec(kind: str, m: dict, width: int, eps: float, max_positions: int):
    if kind == "wkv":
        if "decay_rank" not in m:
            raise ConfigError("a wkv mixer's decay rank is a shape of its tensors: read the configuration with "
                              "NozizenConfig.from_model_dir, or give decay_rank in the mixer's entry")
        return TimeMixSpec(hidden_size=width, num_heads=int(m["heads"]), key_dim=int(m["dim"]),
                           decay_rank=int(m["decay_rank"]), eps=eps)
    if kind == "mamba2":
        return StateSpaceSpec(hidden_size=width, num_heads=int(m["heads"]), value_dim=int(m["vdim"]), state_dim=int(m["state"]),
                              groups=int(m["groups"]), conv_taps=int(m["conv"]), norm_groups=int(m["norm_groups"]), eps=eps)
    mask = m.get("mask")
    return AttentionSpec(hidden_size=width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]),
                         head_dim=_padded_head(m), scale=float(m["scale"]), window=int(mask["size"]) if mask else None,
                         qk_norm=None, position=_rope(m, max_positions), key_dim=int(m["dim"]), value_dim=int(m["vdim"]))


def _mlp_spec(mlp: Optional[dict], width: int):
    if not mlp:
        return None
    if mlp["kind"] == "dense":
        return DenseMLPSpec(hidden_size=width, intermediate_size=int(mlp["ff"]), activation="relu2")
    r = mlp["router"]
    return MoESpec(hidden_size=width, num_experts=int(r["experts"]), top=int(r["top"]),
                   expert=SwiGLUSpec(hidden_size=width, intermediate_size=int(mlp["expert"]["ff"]), interleave=0),
                   renorm_tiny=0.0, router_bias=True)


def decoder_spec(cfg: NozizenConfig, max_positions: Optional[int] = None) -> DecoderSpec:
    max_positions = max_positions or 4096
    W, eps, S = cfg.width, cfg.eps, cfg.streams
    norm = NormSpec(size=W, eps=eps)
    blocks = []
    for layer in cfg.layers:
        ff = _mlp_spec(layer.get("mlp"), W)
        mixer = _mixer_spec(layer["type"], layer["mixer"], W, eps, max_positions)
        # without the key there is one stream and the plain residual sum: the same block with connections that are all one
        blocks.append(HyperBlockSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm if ff else None,
                                     streams=S if S is not None else 1, learned=S is not None))
    schedule = tuple(ScheduleEntry(i) for i in cfg.layer_order())
    return DecoderSpec(vocab_size=cfg.vocab, hidden_size=W, layers=tuple(blocks), schedule=schedule, final_norm=norm,
                       tie_embeddings=True, embedding_scale=cfg.embedding_scale, streams=S if S is not None else 1)


def weight_sources(cfg: NozizenConfig) -> Dict[str, Source]:
    m: Dict[str, Source] = {"embed": Source(("embed",)), "final_norm.weight": Source(("final.norm",))}
    hyper = cfg.streams is not None
    for i, layer in enumerate(cfg.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        mix, kind, mm = src + "mix.", layer["type"], layer["mixer"]
        m[dst + "mixer_norm.weight"] = Source((src + "norm1",))
        if hyper:
            for sub, hc in (("mixer", "hc1"), ("feed_forward", "hc2")):
                if sub == "feed_forward" and not layer.get("mlp"):
                    continue
                for ours, theirs in (("read", "in"), ("write", "out"), ("mix", "mix")):
                    m[f"{dst}{sub}_{ours}"] = Source((f"{src}{hc}.{theirs}",))
        if kind == "wkv":
            m[dst + "mixer.mu"] = Source(tuple(mix + "mu." + n for n in ("r", "k", "v", "g", "w")))
            for ours, theirs in (("r", "r"), ("k", "k"), ("v", "v"), ("g", "g"), ("decay_down", "w1"), ("decay_up", "w2"),
                                 ("decay_bias", "w0"), ("bonus", "u"), ("norm", "norm"), ("o", "o")):
                m[dst + "mixer." + ours] = Source((mix + theirs,))
        elif kind == "mamba2":
            for ours, theirs in (("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("dt_bias", "dt_bias"),
                                 ("A_log", "A_log"), ("D", "D"), ("norm", "norm"), ("o", "o")):
                m[dst + "mixer." + ours] = Source((mix + theirs,))
        else:
            D = _padded_head(mm)
            kpad, vpad = (int(mm["dim"]), D), (int(mm["vdim"]), D)
            m[dst + "mixer.qkv"] = Source((mix + "q", mix + "k", mix + "v"), pad_rows=(kpad, kpad, vpad))
            m[dst + "mixer.o"] = Source((mix + "o",), pad_cols=vpad)
        mlp = layer.get("mlp")
        if mlp:
            p = src + "mlp."
            m[dst + "feed_forward_norm.weight"] = Source((src + "norm2",))
            if mlp["kind"] == "dense":
                m[dst + "feed_forward.up"] = Source((p + "up",))
                m[dst + "feed_forward.down"] = Source((p + "down",))
            else:
                E = int(mlp["router"]["experts"])
                m[dst + "feed_forward.router"] = Source((p + "router",))
                m[dst + "feed_forward.router_bias"] = Source((p + "router.b",))
                m[dst + "feed_forward.experts.gate_up"] = Source(tuple(f"{p}e{j}.{n}" for j in range(E) for n in ("gate", "up")))
                m[dst + "feed_forward.experts.down"] = Source(tuple(f"{p}e{j}.down" for j in range(E)))
    return m


def checkpoint_shapes(cfg: NozizenConfig) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """Every tensor of a checkpoint: name -> (shape, law of its random values).  Matrices are drawn with a deviation of
    fan_in^-1/2 (half that for the maps back into the streams, twelve times that for the routers, so that a sublayer adds
    less than the streams hold and rounding seldom turns a choice), norm weights around one, the streams' connections
    positive and near the identity, the others so that gates, decays and steps are neither shut nor open."""
    W, V, S = cfg.width, cfg.vocab, cfg.streams
    out: Dict[str, Tuple[Tuple[int, ...], str]] = {"embed": ((V, W), "normal:0.05"), "final.norm": ((W,), "ones_normal")}
    for i, layer in enumerate(cfg.layers):
        p, kind, m = f"l{i}.", layer["type"], layer["mixer"]
        x = p + "mix."
        out[p + "norm1"] = ((W,), "ones_normal")
        subs = ["hc1"] + (["hc2"] if layer.get("mlp") else [])
        if S is not None:
            for hc in subs:
                out[f"{p}{hc}.in"] = ((S,), "half_to_one")
                out[f"{p}{hc}.out"] = ((S,), "half_to_one")
                out[f"{p}{hc}.mix"] = ((S, S), "eye_normal")
        if kind == "wkv":
            if "decay_rank" not in m:
                raise ConfigError("a wkv mixer needs decay_rank to size its tensors")
            H, D, R = int(m["heads"]), int(m["dim"]), int(m["decay_rank"])
            for n in ("r", "k", "v", "g", "w"):
                out[x + "mu." + n] = ((W,), "uniform01")
            for n in ("r", "k", "v", "g"):
                out[x + n] = ((H * D, W), "fan_in")
            out[x + "w1"] = ((R, W), "fan_in")
            out[x + "w2"] = ((H * D, R), "fan_in")
            out[x + "w0"] = ((H * D,), "normal:0.7")
            out[x + "u"] = ((H, D), "normal:0.5")
            out[x + "norm"] = ((H * D,), "ones_normal")
            out[x + "o"] = ((W, H * D), "fan_in:0.5")
        elif kind == "mamba2":
            H, P, N, G, K = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["conv"])
            C = H * P + 2 * G * N
            out[x + "in"] = ((2 * H * P + 2 * G * N + H, W), "fan_in")
            out[x + "conv"] = ((C, K), "normal:0.5")
            out[x + "conv.b"] = ((C,), "normal:0.2")
            out[x + "dt_bias"] = ((H,), "normal:0.5")
            out[x + "A_log"] = ((H,), "normal:0.5")
            out[x + "D"] = ((H,), "ones_normal")
            out[x + "norm"] = ((H * P,), "ones_normal")
            out[x + "o"] = ((W, H * P), "fan_in:0.5")
        else:
            H, G, D, Vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            out[x + "q"] = ((H * D, W), "fan_in")
            out[x + "k"] = ((G * D, W), "fan_in")
            out[x + "v"] = ((G * Vd, W), "fan_in")
            out[x + "o"] = ((W, H * Vd), "fan_in:0.5")
        mlp = layer.get("mlp")
        if mlp:
            y = p + "mlp."
            out[p + "norm2"] = ((W,), "ones_normal")
            if mlp["kind"] == "dense":
                ff = int(mlp["ff"])
                out[y + "up"] = ((ff, W), "fan_in")
                out[y + "down"] = ((W, ff), "fan_in:0.5")
            else:
                E, F = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
                out[y + "router"] = ((E, W), "fan_in:12")         # choices that rounding seldom turns
                out[y + "router.b"] = ((E,), "normal:4")
                for j in range(E):
                    out[f"{y}e{j}.gate"] = ((F, W), "fan_in")
                    out[f"{y}e{j}.up"] = ((F, W), "fan_in")
                    out[f"{y}e{j}.down"] = ((W, F), "fan_in:0.5")
    return out


def ignorable_tensors(cfg: NozizenConfig):
    """A layer without a feed-forward never reads what belongs to one; a file may hold it all the same."""
    out = set()
    for i, layer in enumerate(cfg.layers):
        if not layer.get("mlp"):
            out.update({f"l{i}.norm2", f"l{i}.hc2.in", f"l{i}.hc2.out", f"l{i}.hc2.mix"})
    return out
