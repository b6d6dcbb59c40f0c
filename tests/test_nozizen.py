"""Host-side tests of the Nozizen decoder's configuration, specification, weight map and state layout, and of the plain
implementation against itself (causality, the window, a repeated run of layers, streams that reduce to a plain residual)."""
import copy
import json
import os

import pytest
import torch

import helpers  # noqa: F401  (paths)
from plain import nozizen_plain as plain
from return_b200.config import registry
from return_b200.config.model_config import ConfigError
from return_b200.config.nozizen_config import NozizenConfig
from return_b200.models import nozizen
from return_b200.models.decoder import DecoderModel
from return_b200.parts.base import BuildEnv, KVCacheNeed, StateNeed
from return_b200.weights import loader


def raw_config():
    moe = {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24}}
    return {"architecture": "Nozizen", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
            "streams": 3, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
        {"type": "wkv", "mixer": {"heads": 3, "dim": 8, "decay_rank": 6}, "mlp": {"kind": "dense", "ff": 56}},
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 6, "state": 10, "groups": 2, "conv": 4, "norm_groups": 3}, "mlp": moe},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "mask": {"size": 9},
                                        "rot": {"base": 5000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 32,
                                                                                           "fast": 8.0, "slow": 1.0}}},
         "mlp": None},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 16, "decay_rank": 4}, "mlp": moe}]}


def test_registry_finds_the_architecture_by_its_name():
    arch = registry.resolve({"architecture": "Nozizen"})
    assert arch.config_cls is NozizenConfig and "Nozizen" in registry.architectures()


@pytest.mark.parametrize("path,value", [(("layers", 0, "type"), "retention"), (("layers", 1, "mixer", "groups"), 3),
                                        (("layers", 1, "mixer", "norm_groups"), 5), (("layers", 2, "mixer", "kv_heads"), 3),
                                        (("layers", 2, "mixer", "rot", "dims"), 7), (("layers", 2, "mixer", "rot", "dims"), 14),
                                        (("layers", 2, "mixer", "mask", "size"), 0), (("layers", 1, "mlp", "router", "top"), 6),
                                        (("layers", 0, "mlp", "kind"), "gated"), (("loop", "stop"), 5), (("loop", "times"), 0),
                                        (("streams",), 0), (("width",), 0)])
def test_configuration_rejects_what_the_design_does_not_have(path, value):
    raw = raw_config()
    d = raw
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError):
        NozizenConfig(raw)
    missing = raw_config()
    del missing["layers"][1]["mixer"]["state"]
    with pytest.raises(ConfigError):
        NozizenConfig(missing)


def test_specification_follows_the_configuration():
    cfg = NozizenConfig(raw_config())
    assert cfg.layer_order() == [0, 1, 2, 1, 2, 3]
    spec = nozizen.decoder_spec(cfg, 256)
    assert spec.tie_embeddings and spec.embedding_scale == 3.0 and spec.streams == 3 and len(spec.layers) == 4
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    t, s, a = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[2].mixer
    assert (t.kind, t.num_heads, t.key_dim, t.decay_rank) == ("time_mix", 3, 8, 6)
    assert (s.kind, s.num_heads, s.value_dim, s.state_dim, s.groups, s.conv_taps, s.norm_groups) == ("state_space", 4, 6, 10, 2, 4, 3)
    assert (a.num_heads, a.num_kv_heads, a.key_dim, a.value_dim, a.head_dim, a.window, a.scale) == (4, 2, 12, 20, 32, 9, 0.3)
    assert a.position.rotary_dim == 8 and a.position.factor == 4.0 and a.position.max_positions == 256
    assert spec.layers[0].feed_forward.activation == "relu2" and spec.layers[0].feed_forward.intermediate_size == 56
    ff = spec.layers[1].feed_forward
    assert (ff.num_experts, ff.top, ff.groups, ff.router_bias, ff.renorm_tiny, ff.shared) == (5, 2, 1, True, 0.0, None)
    assert spec.layers[2].feed_forward is None and all(b.streams == 3 and b.learned for b in spec.layers)
    # optional keys left out: no window, plain frequencies, no positions at all, no scale, no loop, one plain stream
    raw = raw_config()
    del raw["layers"][2]["mixer"]["mask"], raw["layers"][2]["mixer"]["rot"]["scaling"], raw["embedding"], raw["loop"], raw["streams"]
    spec = nozizen.decoder_spec(NozizenConfig(raw), 64)
    assert spec.layers[2].mixer.window is None and spec.layers[2].mixer.position.factor is None
    assert spec.embedding_scale == 1.0 and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    assert spec.streams == 1 and all(b.streams == 1 and not b.learned for b in spec.layers)
    del raw["layers"][2]["mixer"]["rot"]
    assert nozizen.decoder_spec(NozizenConfig(raw), 64).layers[2].mixer.position is None


def _load(d):
    arch, cfg = registry.read_config(d)
    model = DecoderModel(arch.decoder_spec(cfg, 64), BuildEnv(torch.float32, torch.device("cpu")))
    expected = {n: shape for n, (shape, _) in loader.checkpoint_shapes(arch, cfg).items()}
    params = loader.load_parameters(model.params(), arch.weight_sources(cfg), expected, d, torch.float32, "cpu",
                                    arch.ignorable_tensors(cfg))
    model.bind(params)
    return arch, cfg, model, params, expected


def test_a_random_checkpoint_fills_every_parameter(tmp_path):
    d = loader.write_random_model(str(tmp_path / "m"), NozizenConfig(raw_config()), 1, torch.bfloat16)
    arch, cfg, model, params, expected = _load(d)
    c, w = plain.read_model(d, torch.float32)
    # the five blends of a time mix are one parameter, a row each, in the order the kernel reads them
    mu = params["layers.0.mixer.mu"]
    assert tuple(mu.shape) == (5, 40) and all(torch.equal(mu[i], w[f"l0.mix.mu.{n}"]) for i, n in enumerate("rkvgw"))
    assert torch.equal(params["layers.0.mixer.decay_down"], w["l0.mix.w1"]) and torch.equal(params["layers.0.mixer.bonus"], w["l0.mix.u"])
    # the attention's heads are padded with zeros to one size: keys of 12 and values of 20 in heads of 32
    qkv = params["layers.2.mixer.qkv"].view(4 + 2 + 2, 32, 40)
    assert torch.equal(qkv[1, :12], w["l2.mix.q"][12:24]) and not qkv[:6, 12:].any()
    assert torch.equal(qkv[7, :20], w["l2.mix.v"][20:]) and not qkv[6:, 20:].any()
    o = params["layers.2.mixer.o"].view(40, 4, 32)
    assert torch.equal(o[:, 3, :20], w["l2.mix.o"][:, 60:]) and not o[:, :, 20:].any()
    # an expert's gate rows, then its up rows; the router's bias beside it
    gu = params["layers.1.feed_forward.experts.gate_up"].view(5, 48, 40)
    assert torch.equal(gu[3, :24], w["l1.mlp.e3.gate"]) and torch.equal(gu[3, 24:], w["l1.mlp.e3.up"])
    assert torch.equal(params["layers.1.feed_forward.experts.down"].view(5, 40, 24)[4], w["l1.mlp.e4.down"])
    assert torch.equal(params["layers.1.feed_forward.router_bias"], w["l1.mlp.router.b"])
    assert torch.equal(params["layers.3.feed_forward_mix"], w["l3.hc2.mix"]) and "layers.2.feed_forward_mix" not in params
    assert model.lm_head is model.embed
    bad = dict(expected)
    bad["l0.mix.u"] = (3, 9)
    with pytest.raises(loader.WeightError) as e:
        loader.load_parameters(model.params(), arch.weight_sources(cfg), bad, d, torch.float32, "cpu")
    assert "l0.mix.u" in str(e.value)


def test_the_decay_rank_comes_from_the_tensors_when_the_configuration_lacks_it(tmp_path):
    d = loader.write_random_model(str(tmp_path / "m"), NozizenConfig(raw_config()), 1, torch.bfloat16)
    path = os.path.join(d, "config.json")
    raw = json.load(open(path))
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
    json.dump(raw, open(path, "w"))
    with pytest.raises(ConfigError):
        nozizen.decoder_spec(NozizenConfig(raw))
    _, cfg = registry.read_config(d)
    assert [l["mixer"].get("decay_rank") for l in cfg.layers] == [6, None, None, 4]
    assert NozizenConfig(cfg.to_dict()).layers[3]["mixer"]["decay_rank"] == 4


def test_every_run_of_a_repeated_layer_has_a_state_or_cache_of_its_own(tmp_path):
    d = loader.write_random_model(str(tmp_path / "m"), NozizenConfig(raw_config()), 1, torch.bfloat16)
    _, cfg, model, _, _ = _load(d)
    needs = model.cache_needs()
    assert len(needs) == 6 and needs[1] == needs[3] and needs[2] == needs[4]
    # a time mix keeps its matrices (key rows padded to eights) and the last input; a state-space mixer its matrices
    # (state rows padded to eights, a head's values as columns) and the last taps - 1 inputs of every convolved channel
    assert needs[0] == StateNeed((3 * 8 * 8 + 40,), torch.float32)
    assert needs[1] == StateNeed((4 * 16 * 6 + (4 * 6 + 2 * 2 * 10) * 3,), torch.float32)
    assert needs[2] == KVCacheNeed(2, 32, 9)
    from return_b200.cache.storage import CacheStorage
    st = CacheStorage(needs, page_size=16, num_pages=8, max_reside=2, env=model.env, longest_append=64)
    st.allocate()
    assert len(st.states) == 4 and st.pools[0].shape[0] == 2          # four runs with state, two with keys and values


def _weights(cfg, seed=2):
    return {n: loader.random_tensor(seed, n, shp, law, torch.float64)
            for n, (shp, law) in nozizen.checkpoint_shapes(NozizenConfig(cfg)).items()}


def test_plain_model_is_causal_and_its_window_is_what_it_says():
    cfg = raw_config()
    cfg["layers"], cfg["loop"] = cfg["layers"][2:3], None
    w = _weights(cfg)
    ids = list(range(40))
    whole = plain.forward(cfg, w, ids)[0]
    assert torch.allclose(plain.forward(cfg, w, ids[:25])[0], whole[:25], atol=1e-12)
    other = [96] + ids[1:]                                  # a token farther back than the window does not reach the logits
    assert torch.allclose(plain.forward(cfg, w, other)[0][9:], whole[9:], atol=1e-12)
    assert not torch.allclose(plain.forward(cfg, w, other)[0][8], whole[8], atol=1e-6)


def test_plain_recurrences_carry_the_first_token_to_the_end():
    for keep in (0, 1):
        cfg = raw_config()
        cfg["layers"], cfg["loop"] = cfg["layers"][keep:keep + 1], None
        w = _weights(cfg)
        ids = list(range(30))
        whole = plain.forward(cfg, w, ids)[0]
        assert torch.allclose(plain.forward(cfg, w, ids[:11])[0], whole[:11], atol=1e-12)
        assert not torch.allclose(plain.forward(cfg, w, [96] + ids[1:])[0][-1], whole[-1], atol=1e-9)


def test_plain_loop_and_streams():
    cfg = raw_config()
    w = _weights(cfg)
    ids = [5, 9, 2, 77, 30, 1, 1, 64]
    logits, after = plain.forward(cfg, w, ids, keep_layers=True)
    assert after.shape == (6, 8, 40)
    # the same as the layers written out one after the other, the repeated ones with copies of their tensors
    flat = copy.deepcopy(cfg)
    flat["loop"] = None
    flat["layers"] = [cfg["layers"][i] for i in (0, 1, 2, 1, 2, 3)]
    w2 = {}
    for new, old in enumerate((0, 1, 2, 1, 2, 3)):
        w2.update({f"l{new}." + k.split(".", 1)[1]: v for k, v in w.items() if k.startswith(f"l{old}.")})
    w2.update({k: v for k, v in w.items() if not k.startswith("l")})
    assert torch.equal(plain.forward(flat, w2, ids)[0], logits)
    # one stream whose connections are all one is the plain residual sum
    one = copy.deepcopy(cfg)
    one["streams"] = 1
    w1 = {k: (torch.ones_like(v[:1, :1] if v.dim() == 2 else v[:1]) if ".hc" in k else v) for k, v in w.items()}
    none = copy.deepcopy(cfg)
    del none["streams"]
    assert torch.allclose(plain.forward(one, w1, ids)[0], plain.forward(none, w, ids)[0], atol=1e-12)


def test_plain_router_weighs_the_chosen_logits_only():
    w = {"r.router": torch.eye(4, dtype=torch.float64), "r.router.b": torch.tensor([0.0, 0.0, 5.0, 0.0], dtype=torch.float64)}
    a = torch.tensor([[3.0, 1.0, -3.0, 2.0]], dtype=torch.float64)
    idx, wt = plain.router(w, "r.", {"router": {"experts": 4, "top": 2}}, a)
    assert idx.tolist() == [[0, 2]]                       # the bias lifts the third expert over the fourth
    assert torch.allclose(wt, torch.softmax(torch.tensor([[3.0, 2.0]], dtype=torch.float64), -1))
