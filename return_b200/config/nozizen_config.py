"""Configuration of the Nozizen decoder, read from its own config.json keys.

``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (optional, 1), ``streams`` (optional: the number of residual
streams a token has; absent: one stream with plain residual sums), ``loop`` (optional: ``start, stop, times``: layers
start .. stop - 1 run ``times`` times in a row with the same weights, every pass with a cache or state of its own) and
``layers``: a list of entries with ``type`` (which mixer the layer has: ``wkv``, ``mamba2`` or ``attention``), ``mixer``
(its sizes and constants) and ``mlp`` (``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "router": {"experts", "top"},
"expert": {"ff"}}`` or null).

``wkv``: ``heads, dim``.  ``mamba2``: ``heads, vdim, state, groups, conv, norm_groups``.  ``attention``: ``heads, kv_heads,
dim, vdim, scale``, optionally ``mask.size`` (a sliding window) and ``rot`` (``base, dims`` and optionally ``scaling`` with
``factor, original, fast, slow``).

One size of a ``wkv`` mixer is not a config key but a shape of its tensors: the rank of its decay projection.
``from_model_dir`` reads it from the safetensors header and keeps it in the mixer's entry as ``decay_rank``, so that the
configuration alone says every size from then on (``to_dict`` writes it, ``from_dict`` takes it back).
"""
from __future__ import annotations

import copy
import json
import os
from typing import List, Optional

from .model_config import ConfigError

MIXER_TYPES = ("wkv", "mamba2", "attention")
_MIXER_KEYS = {"wkv": ("heads", "dim"),
               "mamba2": ("heads", "vdim", "state", "groups", "conv", "norm_groups"),
               "attention": ("heads", "kv_heads", "dim", "vdim", "scale")}


def _need(d, keys, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks {missing}")


class NozizenConfig:
    def __init__(self, raw: dict):
        self.raw = copy.deepcopy(raw)
        self.validate()

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "NozizenConfig":
        return cls(raw)

    @classmethod
    def from_model_dir(cls, model_dir: str, raw: Optional[dict] = None) -> "NozizenConfig":
        """config.json plus the sizes that only tensor shapes give."""
        if raw is None:
            with open(os.path.join(model_dir, "config.json")) as f:
                raw = json.load(f)
        raw = copy.deepcopy(raw)
        layers = raw.get("layers") or []
        wanted = [i for i, layer in enumerate(layers)
                  if isinstance(layer, dict) and layer.get("type") == "wkv" and isinstance(layer.get("mixer"), dict)
                  and "decay_rank" not in layer["mixer"]]
        if wanted:
            from ..weights.safetensors_io import ModelFiles
            files = ModelFiles(model_dir)
            try:
                for i in wanted:
                    name = f"l{i}.mix.w1"
                    if name not in files:
                        raise ConfigError(f"{model_dir}: tensor {name} is missing; its rows give decay_rank")
                    layers[i]["mixer"]["decay_rank"] = int(files.shape(name)[0])
            finally:
                files.close()
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
    def streams(self) -> Optional[int]:
        s = self.raw.get("streams")
        return int(s) if s is not None else None

    @property
    def layers(self):
        return self.raw["layers"]

    def layer_order(self) -> List[int]:
        """The layers in the order they run."""
        n = len(self.layers)
        loop = self.raw.get("loop")
        if not loop:
            return list(range(n))
        a, b, k = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        return list(range(a)) + list(range(a, b)) * k + list(range(b, n))

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        raw = self.raw
        _need(raw, ("vocab", "width", "norm", "layers"), "the top level")
        _need(raw["norm"], ("eps",), "norm")
        if self.vocab <= 0 or self.width <= 0 or not (self.eps > 0):
            raise ConfigError("vocab, width and norm.eps must be positive")
        if raw.get("embedding") is not None:
            _need(raw["embedding"], ("scale",), "embedding")
        if self.streams is not None and not (1 <= self.streams <= 8):
            raise ConfigError(f"streams={self.streams}: 1 to 8")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("layers must be a list with at least one entry")
        n = len(raw["layers"])
        loop = raw.get("loop")
        if loop:
            _need(loop, ("start", "stop", "times"), "loop")
            a, b, k = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not (0 <= a <= b <= n) or k < 1:
                raise ConfigError(f"loop: layers {a} .. {b - 1}, {k} times, of {n} layers")
        for i, layer in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            kind = layer["type"]
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}.type={kind!r}; known: {list(MIXER_TYPES)}")
            m = layer["mixer"]
            _need(m, _MIXER_KEYS[kind], where + ".mixer")
            if min(int(m[k]) for k in _MIXER_KEYS[kind] if k != "scale") <= 0:
                raise ConfigError(f"{where}.mixer: sizes must be positive")
            if kind == "mamba2":
                H, G = int(m["heads"]), int(m["groups"])
                if H % G:
                    raise ConfigError(f"{where}.mixer: heads={H} is not a multiple of groups={G}")
                if (H * int(m["vdim"])) % int(m["norm_groups"]):
                    raise ConfigError(f"{where}.mixer: heads * vdim does not form norm_groups={m['norm_groups']} equal parts")
            if kind == "attention":
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"{where}.mixer: heads={m['heads']} is not a multiple of kv_heads={m['kv_heads']}")
                if m.get("mask") is not None:
                    _need(m["mask"], ("size",), where + ".mixer.mask")
                    if int(m["mask"]["size"]) <= 0:
                        raise ConfigError(f"{where}.mixer.mask.size must be positive")
                rot = m.get("rot")
                if rot is not None:
                    _need(rot, ("base", "dims"), where + ".mixer.rot")
                    dims = int(rot["dims"])
                    if dims < 0 or dims % 2 or dims > int(m["dim"]):
                        raise ConfigError(f"{where}.mixer.rot.dims={dims} must be even and at most dim={m['dim']}")
                    if rot.get("scaling"):
                        _need(rot["scaling"], ("factor", "original", "fast", "slow"), where + ".mixer.rot.scaling")
                        if not float(rot["scaling"]["factor"]) > 0:
                            raise ConfigError(f"{where}.mixer.rot.scaling.factor must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] == "dense":
                    _need(mlp, ("ff",), where + ".mlp")
                elif mlp["kind"] == "moe":
                    _need(mlp, ("router", "expert"), where + ".mlp")
                    _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
                    _need(mlp["expert"], ("ff",), where + ".mlp.expert")
                    if not (1 <= int(mlp["router"]["top"]) <= int(mlp["router"]["experts"])):
                        raise ConfigError(f"{where}.mlp.router: top={mlp['router']['top']} of {mlp['router']['experts']} experts")
                else:
                    raise ConfigError(f"{where}.mlp.kind={mlp['kind']!r}; known: dense, moe")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = copy.deepcopy(self.raw)
        d.setdefault("architecture", "Nozizen")
        return d
