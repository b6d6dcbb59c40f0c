"""One registry from an architecture's name to its configuration class and its model recipe.

The reference picks its model by a substring test on ``config.model_type``
(rollout/engine_actor.py:24-32) and raises ``ValueError`` for anything else.  Here the key is
``architectures[0]`` of config.json, with ``model_type`` as a fallback.  An architecture gives:
``config_cls`` (typed, ``from_dict``), ``decoder_spec(cfg, max_positions)`` -> DecoderSpec,
``weight_sources(cfg)`` -> {parameter: Source}, ``ignorable_tensors(cfg)`` (names, or name -> twin
it must equal).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Optional


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_cls: type
    decoder_spec: Callable
    weight_sources: Callable
    ignorable_tensors: Callable = lambda cfg: set()
    # rows of each checkpoint tensor inside a fused parameter, or None for an even split
    split_rows: Callable = lambda cfg, param: None
    # checkpoint tensor -> (shape, law of random values), for an architecture whose checkpoint layout is not the
    # parameters' cut into equal or ``split_rows`` pieces (padded heads, tensors of many kinds); None: derived
    checkpoint_shapes: Optional[Callable] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architectures():
    return sorted(_ARCHITECTURES)


def resolve(raw_config: dict) -> Architecture:
    """The architecture a config.json (as a dict) asks for."""
    names = list(raw_config.get("architectures") or [])
    if isinstance(raw_config.get("architecture"), str):      # a config.json that names one architecture, as a string
        names.append(raw_config["architecture"])
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = str(raw_config.get("model_type", "")).lower()
    if not names:
        for arch in _ARCHITECTURES.values():
            if arch.model_type == mt:
                return arch
    raise ValueError(f"no model for architectures={names!r} model_type={mt!r}; known: {architectures()}")


def read_config(model_dir: str):
    """(architecture, typed configuration) of a model folder."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{model_dir} has no config.json")
    with open(path) as f:
        raw = json.load(f)
    arch = resolve(raw)
    if hasattr(arch.config_cls, "from_model_dir"):       # sizes that only the tensors' shapes give
        return arch, arch.config_cls.from_model_dir(model_dir, raw)
    return arch, arch.config_cls.from_dict(raw)


def _register_builtin() -> None:
    from ..models import qwen3
    from .model_config import Qwen3Config
    register_architecture(Architecture(
        name="Qwen3ForCausalLM", model_type="qwen3", config_cls=Qwen3Config,
        decoder_spec=qwen3.decoder_spec, weight_sources=qwen3.weight_sources,
        ignorable_tensors=qwen3.ignorable_tensors, split_rows=qwen3.split_rows))
    from ..models import pisatar
    from .pisatar_config import PisatarConfig
    register_architecture(Architecture(
        name="Pisatar", model_type="pisatar", config_cls=PisatarConfig,
        decoder_spec=pisatar.decoder_spec, weight_sources=pisatar.weight_sources,
        ignorable_tensors=pisatar.ignorable_tensors, checkpoint_shapes=pisatar.checkpoint_shapes))
    from ..models import gonozen
    from .gonozen_config import GonozenConfig
    register_architecture(Architecture(
        name="Gonozen", model_type="gonozen", config_cls=GonozenConfig,
        decoder_spec=gonozen.decoder_spec, weight_sources=gonozen.weight_sources,
        ignorable_tensors=gonozen.ignorable_tensors, checkpoint_shapes=gonozen.checkpoint_shapes))
    from ..models import nozizen
    from .nozizen_config import NozizenConfig
    register_architecture(Architecture(
        name="Nozizen", model_type="nozizen", config_cls=NozizenConfig,
        decoder_spec=nozizen.decoder_spec, weight_sources=nozizen.weight_sources,
        ignorable_tensors=nozizen.ignorable_tensors, checkpoint_shapes=nozizen.checkpoint_shapes))
    from ..models import duvadra
    from .duvadra_config import DuvadraConfig
    register_architecture(Architecture(
        name="Duvadra", model_type="duvadra", config_cls=DuvadraConfig,
        decoder_spec=duvadra.decoder_spec, weight_sources=duvadra.weight_sources,
        ignorable_tensors=duvadra.ignorable_tensors, checkpoint_shapes=duvadra.checkpoint_shapes))


_register_builtin()
