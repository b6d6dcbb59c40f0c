"""Host-side tests of the Duvadra decoder's configuration, specification, weight map and cache needs, and of the plain
implementation against itself (causality, windows and blocks, the router, the rotation, shared keys)."""
import copy
import os

import pytest
import torch

import helpers  # noqa: F401  (paths)
from plain import duvadra_plain as plain
from return_b200.config import registry
from return_b200.config.duvadra_config import DuvadraConfig
from return_b200.config.model_config import ConfigError
from return_b200.models import duvadra
from return_b200.models.decoder import DecoderModel
from return_b200.parts.base import BuildEnv, CompositeNeed, KVCacheNeed, StateNeed
from return_b200.weights import loader


def raw_config():
    moe = {"kind": "moe", "router": {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}, "expert": {"ff": 24}}
    left = {"heads": 3, "kv_heads": 1, "dim": 8, "vdim": 14, "scale": 0.35, "mask": {"size": 21}}
    left2 = {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 10, "scale": 0.3, "mask": {"size": 26}, "rot": {"base": 3000.0, "dims": 6}}
    blocks = {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "softcap": 7.0, "mask": {"size": 13}}
    return {"architecture": "Duvadra", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
            "logit_softcap": 12.0, "embedding": {"scale": 3.0, "bigram": {"buckets": 53, "mul_prev": 31, "mul_cur": 7}}, "layers": [
        {"type": "attention", "mixer": blocks, "mlp": {"kind": "dense", "ff": 56, "limit": 1.25}},
        {"type": "parallel_2", "mixer": {"left": left2, "right": {"width": 24, "blocks": 3, "conv": 3}, "left_scale": 0.9,
                                         "right_scale": 0.4}, "mlp": moe},
        {"type": "attention", "mixer": {**blocks, "heads": 2, "mask": {"size": 29}, "kv_from": 0}, "mlp": None},
        {"type": "parallel", "mixer": {"left": left, "right": {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 6, "conv": 4},
                                       "left_scale": 0.7, "right_scale": 0.6}, "mlp": moe}]}


def test_registry_finds_the_architecture_by_its_name():
    arch = registry.resolve({"architecture": "Duvadra"})
    assert arch.config_cls is DuvadraConfig and "Duvadra" in registry.architectures()


@pytest.mark.parametrize("path,value", [(("layers", 0, "type"), "retention"), (("layers", 0, "mixer", "kv_heads"), 3),
                                        (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 2, "mixer", "kv_from"), 1),
                                        (("layers", 2, "mixer", "kv_from"), 2), (("layers", 2, "mixer", "dim"), 16),
                                        (("layers", 1, "mixer", "left", "rot", "dims"), 7), (("layers", 1, "mixer", "left", "rot", "dims"), 12),
                                        (("layers", 1, "mixer", "left", "vdim"), 12), (("layers", 1, "mixer", "right", "blocks"), 5),
                                        (("layers", 3, "mixer", "right", "kv_heads"), 3), (("layers", 3, "mixer", "left", "rot"), {"base": 10.0, "dims": 4}),
                                        (("layers", 1, "mlp", "router", "top"), 5), (("layers", 1, "mlp", "router", "groups", "count"), 4),
                                        (("layers", 0, "mlp", "kind"), "gated"), (("embedding", "bigram", "buckets"), 0), (("width",), 0)])
def test_configuration_rejects_what_the_design_does_not_have(path, value):
    raw = raw_config()
    d = raw
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError):
        DuvadraConfig(raw)
    missing = raw_config()
    del missing["layers"][3]["mixer"]["right"]["conv"]
    with pytest.raises(ConfigError):
        DuvadraConfig(missing)


def test_optional_keys_may_be_absent():
    raw = raw_config()
    for k in ("residual_mult", "logit_softcap", "embedding"):
        del raw[k]
    del raw["layers"][0]["mixer"]["mask"], raw["layers"][0]["mixer"]["softcap"], raw["layers"][1]["mixer"]["left"]["rot"]
    del raw["layers"][1]["mlp"]["router"]["groups"]
    cfg = DuvadraConfig(raw)
    spec = duvadra.decoder_spec(cfg, 64)
    assert cfg.residual_mult == 1.0 and cfg.bigram is None and spec.logit_softcap is None and spec.embedding_pairs is None
    assert spec.layers[0].mixer.chunk is None and spec.layers[0].mixer.softcap is None and spec.layers[0].mixer.cache_window is None
    assert spec.layers[1].mixer.mixers[0].position is None and spec.layers[1].feed_forward.groups == 1


def test_specification_follows_the_configuration():
    cfg = DuvadraConfig(raw_config())
    spec = duvadra.decoder_spec(cfg, 128)
    assert [e.cache_of for e in spec.schedule] == [None, None, 0, None] and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    first, reader = spec.layers[0].mixer, spec.layers[2].mixer
    assert (first.chunk, first.window, first.softcap, first.gate, first.slope_exponent) == (13, None, 7.0, "head", 8.0)
    assert first.cache_window == 29                       # the cache keeps what the layer that reads it needs: the larger block
    assert not reader.own_cache and reader.chunk == 29 and reader.num_heads == 2
    left2, lru = spec.layers[1].mixer.mixers
    assert left2.values_are_keys and left2.whole_norm_eps == 1e-5 and left2.position.rotary_dim == 6 and left2.gate == "element"
    assert (lru.width, lru.blocks, lru.conv_taps, lru.decay_scale) == (24, 3, 3, 8.0)
    left, delta = spec.layers[3].mixer.mixers
    assert left.bias and left.sink and left.window == 21 and not left.values_are_keys and spec.layers[3].mixer.scales == (0.7, 0.6)
    assert (delta.num_heads, delta.num_kv_heads, delta.key_dim, delta.value_dim, delta.conv_taps) == (4, 2, 10, 6, 4)
    ff = spec.layers[1].feed_forward
    assert (ff.score, ff.group_top, ff.weight_scale, ff.groups, ff.keep_groups, ff.top) == ("sigmoid", 2, 1.5, 3, 2, 2)
    assert spec.layers[0].feed_forward.limit == 1.25 and spec.layers[2].feed_forward is None
    assert all(b.residual_scale == 0.6 for b in spec.layers) and spec.embedding_pairs == (53, 31, 7) and spec.logit_softcap == 12.0


def test_parameters_checkpoint_names_and_cache_needs_fit_together(tmp_path):
    cfg = DuvadraConfig(raw_config())
    arch = registry.resolve(cfg.to_dict())
    model = DecoderModel(arch.decoder_spec(cfg, 64), BuildEnv(torch.float32, torch.device("cpu")))
    params, sources, shapes = model.params(), arch.weight_sources(cfg), loader.checkpoint_shapes(arch, cfg)
    assert set(params) == set(sources)
    named = {n for s in sources.values() for n in s.names}
    assert named == set(shapes)
    assert "l2.mix.k" not in shapes and "l2.mix.v" not in shapes and "l1.mix.left.v" not in shapes and "l2.norm2" not in shapes
    assert shapes["bigram"][0] == (54, 40) and shapes["l1.mix.right.ra"][0] == (3, 8, 8) and shapes["l3.mix.left.sink"][0] == (3,)
    d = loader.write_random_model(str(tmp_path / "m"), cfg, 1, torch.bfloat16)
    loaded = loader.load_parameters(params, sources, {n: s for n, (s, _) in shapes.items()}, d, torch.float32, "cpu",
                                    arch.ignorable_tensors(cfg))
    assert {n: tuple(t.shape) for n, t in loaded.items()} == {n: tuple(p.shape) for n, p in params.items()}
    w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    o = loaded["layers.3.mixer.left.o"].view(40, 3, 16)                       # heads of 14 values padded to the cache's 16
    assert torch.equal(o[:, :, :14].reshape(40, 42), w["l3.mix.left.o"].float()) and float(o[:, :, 14:].abs().max()) == 0.0
    needs = model.cache_needs()
    assert needs[0] == KVCacheNeed(2, 32, 29) and needs[2] is None and needs[4] == StateNeed((1,), torch.int32)
    assert isinstance(needs[1], CompositeNeed) and dict(needs[1].children)["left"] == KVCacheNeed(2, 16, 26)
    assert dict(needs[1].children)["right"] == StateNeed((24 + 24 * 2,), torch.float32)
    assert dict(needs[3].children)["right"] == StateNeed((4 * 16 * 6 + (2 * 2 * 10 + 4 * 6) * 3,), torch.float32)


# ------------------------------------------------------------------------------- the plain implementation against itself

def test_windows_and_blocks_of_the_plain_masks():
    w = plain.visible(12, "window", 4)
    assert w[7].nonzero().flatten().tolist() == [4, 5, 6, 7] and w[2].nonzero().flatten().tolist() == [0, 1, 2]
    b = plain.visible(12, "chunk", 4)
    assert b[7].nonzero().flatten().tolist() == [4, 5, 6, 7] and b[8].nonzero().flatten().tolist() == [8] and b[3].sum() == 4
    assert plain.visible(5, None, 0).sum() == 15


def test_plain_router_keeps_to_the_best_groups():
    z = torch.tensor([[4.0, -9.0, 3.0, 2.9, 3.5, -9.0]], dtype=torch.float64)          # groups (0, 1), (2, 3), (4, 5)
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    picked, wts = plain.route(z, r)                       # the middle group has the largest sum of two, although not the best expert
    assert sorted(picked[0].tolist()) == [2, 3] and abs(float(wts.sum()) - 2.0) < 1e-12
    r["groups"]["keep"] = 3
    assert sorted(plain.route(z, r)[0][0].tolist()) == [0, 4]


def test_plain_rotation_turns_neighbours_and_leaves_the_rest():
    x = torch.randn((5, 2, 10), generator=torch.Generator().manual_seed(0), dtype=torch.float64)
    y = plain.rotate_interleaved(x, 6, 100.0)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    assert torch.allclose(y[..., 0:6].norm(dim=-1), x[..., 0:6].norm(dim=-1))
    assert torch.allclose(y[3, :, 0] ** 2 + y[3, :, 1] ** 2, x[3, :, 0] ** 2 + x[3, :, 1] ** 2)
    assert not torch.allclose(y[3, :, :2], x[3, :, :2])


def test_plain_model_is_causal_and_its_parts_matter(tmp_path):
    cfg = DuvadraConfig(raw_config())
    d = loader.write_random_model(str(tmp_path / "m"), cfg, 2, torch.bfloat16)
    c, w = plain.read_model(d)
    ids = helpers.random_ids(97, 60, 3)
    full = plain.forward(c, w, ids)
    assert torch.allclose(plain.forward(c, w, ids[:31]), full[:31], atol=1e-9)            # nothing looks ahead
    other = list(ids)
    other[0] = (ids[0] + 1) % 97
    assert not torch.allclose(plain.forward(c, w, other)[1], full[1])                    # the token before enters through the pair table
    for change in (lambda c: c["layers"][2]["mixer"].pop("kv_from"),                      # keys of its own would need tensors it has not
                   lambda c: c["layers"][0]["mixer"].update(softcap=0.5),
                   lambda c: c["layers"][3]["mixer"].update(right_scale=0.0),
                   lambda c: c.update(residual_mult=0.5), lambda c: c["layers"][1]["mlp"]["router"].update(scale=1.0)):
        c2 = copy.deepcopy(c)
        change(c2)
        try:
            assert not torch.allclose(plain.forward(c2, w, ids), full, atol=1e-6)
        except KeyError:
            pass
