"""Configuration of the Duvadra decoder, read from its own config.json keys.

``vocab``, ``width``, ``norm.eps``, ``embedding`` (optional: ``scale`` and ``bigram`` with ``buckets, mul_prev, mul_cur``: a
table of token pairs added to the embedded token), ``residual_mult`` (optional, 1: the factor on every sublayer's output
as it joins the residual stream), ``logit_softcap`` (optional) and ``layers``: a list of entries with ``type`` (which mixer
the layer has: ``attention``, ``parallel`` or ``parallel_2``), ``mixer`` (its sizes and constants) and ``mlp``
(``{"kind": "dense", "ff": n, "limit": x}``, ``{"kind": "moe", "router": {"experts", "top", "scale", "groups": {"count",
"keep"}}, "expert": {"ff"}}`` or null).

``attention``: ``heads, kv_heads, dim, vdim, scale``, optionally ``softcap``, ``mask.size`` (blocks of that many positions)
and ``kv_from`` (the layer whose keys and values this one reads; it then has no key and value projections of its own).
``parallel`` and ``parallel_2``: ``left`` (an attention: ``heads, kv_heads, dim, vdim, scale``, optionally ``mask.size``, a
sliding window, and for ``parallel_2`` ``rot`` with ``base, dims``), ``right`` (``parallel``: ``heads, kv_heads, dim, vdim, conv``;
``parallel_2``: ``width, blocks, conv``), ``left_scale``, ``right_scale``.
"""
from __future__ import annotations

import copy
from typing import Optional, Tuple

from .model_config import ConfigError

MIXER_TYPES = ("attention", "parallel", "parallel_2")
_ATTENTION_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")
_RIGHT_KEYS = {"parallel": ("heads", "kv_heads", "dim", "vdim", "conv"), "parallel_2": ("width", "blocks", "conv")}


def _need(d, keys, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks {missing}")


def _check_attention(m: dict, where: str, rot_allowed: bool) -> None:
    _need(m, _ATTENTION_KEYS, where)
    if min(int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim")) <= 0:
        raise ConfigError(f"{where}: sizes must be positive")
    if int(m["heads"]) % int(m["kv_heads"]):
        raise ConfigError(f"{where}: heads={m['heads']} is not a multiple of kv_heads={m['kv_heads']}")
    if m.get("mask") is not None:
        _need(m["mask"], ("size",), where + ".mask")
        if int(m["mask"]["size"]) <= 0:
            raise ConfigError(f"{where}.mask.size must be positive")
    rot = m.get("rot")
    if rot is not None:
        if not rot_allowed:
            raise ConfigError(f"{where}: this attention takes no rotation")
        _need(rot, ("base", "dims"), where + ".rot")
        dims = int(rot["dims"])
        if dims < 0 or dims % 2 or dims > int(m["dim"]):
            raise ConfigError(f"{where}.rot.dims={dims} must be even and at most dim={m['dim']}")


class DuvadraConfig:
    def __init__(self, raw: dict):
        self.raw = copy.deepcopy(raw)
        self.validate()

    @classmethod
    def from_dict(cls, raw: dict) -> "DuvadraConfig":
        return cls(raw)

    # ------------------------------------------------------------------ what it holds
    @property
    def vocab(self) -> int:
        return int(self.raw["vocab"])

    vocab_size = vocab

    @property
    def width(self) -> int:
        return int(self.raw["width"])

    @property
    def eps(self) -> float:
        return float(self.raw["norm"]["eps"])

    @property
    def embedding_scale(self) -> float:
        return float((self.raw.get("embedding") or {}).get("scale", 1.0))

    @property
    def bigram(self) -> Optional[Tuple[int, int, int]]:
        """(buckets, mul_prev, mul_cur) of the table of token pairs, or None."""
        b = (self.raw.get("embedding") or {}).get("bigram")
        return (int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])) if b else None

    @property
    def residual_mult(self) -> float:
        return float(self.raw.get("residual_mult", 1.0))

    @property
    def logit_softcap(self) -> Optional[float]:
        c = self.raw.get("logit_softcap")
        return float(c) if c else None

    @property
    def layers(self):
        return self.raw["layers"]

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        raw = self.raw
        _need(raw, ("vocab", "width", "norm", "layers"), "the top level")
        _need(raw["norm"], ("eps",), "norm")
        if self.vocab <= 0 or self.width <= 0 or not (self.eps > 0):
            raise ConfigError("vocab, width and norm.eps must be positive")
        b = (raw.get("embedding") or {}).get("bigram")
        if b is not None:
            _need(b, ("buckets", "mul_prev", "mul_cur"), "embedding.bigram")
            if int(b["buckets"]) <= 0:
                raise ConfigError("embedding.bigram.buckets must be positive")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("layers must be a list with at least one entry")
        for i, layer in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind = layer["type"]
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}.type={kind!r}; known: {list(MIXER_TYPES)}")
            m = layer["mixer"]
            if kind == "attention":
                _check_attention(m, where + ".mixer", rot_allowed=False)
                src = m.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not (0 <= src < i) or raw["layers"][src]["type"] != "attention" \
                            or raw["layers"][src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from={src}: an earlier attention layer with keys of its own")
                    o = raw["layers"][src]["mixer"]
                    if any(int(o[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"{where}.mixer: kv_heads, dim and vdim must equal those of layer {src}")
            else:
                _need(m, ("left", "right", "left_scale", "right_scale"), where + ".mixer")
                _check_attention(m["left"], where + ".mixer.left", rot_allowed=kind == "parallel_2")
                if kind == "parallel_2" and int(m["left"]["vdim"]) != int(m["left"]["dim"]):
                    raise ConfigError(f"{where}.mixer.left: values are the keys, so vdim equals dim")
                r = m["right"]
                _need(r, _RIGHT_KEYS[kind], where + ".mixer.right")
                if min(int(r[k]) for k in _RIGHT_KEYS[kind]) <= 0:
                    raise ConfigError(f"{where}.mixer.right: sizes must be positive")
                if kind == "parallel" and int(r["heads"]) % int(r["kv_heads"]):
                    raise ConfigError(f"{where}.mixer.right: heads is not a multiple of kv_heads")
                if kind == "parallel_2" and int(r["width"]) % int(r["blocks"]):
                    raise ConfigError(f"{where}.mixer.right: width={r['width']} does not form blocks={r['blocks']} equal parts")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] == "dense":
                    _need(mlp, ("ff", "limit"), where + ".mlp")
                elif mlp["kind"] == "moe":
                    _need(mlp, ("router", "expert"), where + ".mlp")
                    r = mlp["router"]
                    _need(r, ("experts", "top"), where + ".mlp.router")
                    _need(mlp["expert"], ("ff",), where + ".mlp.expert")
                    E, top = int(r["experts"]), int(r["top"])
                    g = r.get("groups")
                    count, keep = (int(g["count"]), int(g["keep"])) if g else (1, 1)
                    if g:
                        _need(g, ("count", "keep"), where + ".mlp.router.groups")
                    if count < 1 or E % count or not (1 <= keep <= count) or not (1 <= top <= keep * (E // count)):
                        raise ConfigError(f"{where}.mlp.router: top={top} of {E} experts in {count} groups of which {keep} are kept")
                else:
                    raise ConfigError(f"{where}.mlp.kind={mlp['kind']!r}; known: dense, moe")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = copy.deepcopy(self.raw)
        d.setdefault("architecture", "Duvadra")
        return d
