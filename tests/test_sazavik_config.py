"""Sazavik without a GPU: registry, schedule and cache plan, tensor names, part parameters, refused configurations."""

import copy

import pytest

from yalis_b200.config.presets import preset
from yalis_b200.config.registry import ConfigError, parse_config
from yalis_b200.engine.model import Model
from yalis_b200.parts.base import PagedKV


def spec_of(name):
    arch, cfg = parse_config(preset(name))
    return arch, cfg, arch.model_spec(cfg)


def test_the_registry_knows_the_design_and_round_trips_its_configuration():
    for which in "ABCD":
        raw = preset(f"sazavik-tiny-{which}")
        arch, cfg = parse_config(raw)
        assert arch.name == "Sazavik" and arch.config_to_dict(cfg) == raw


def test_a_layer_that_reads_anothers_keys_is_a_schedule_entry_that_reads_its_cache():
    _, _, spec = spec_of("sazavik-tiny-A")
    assert [e.cache_of for e in spec.schedule] == [None, None, 0, None, None]
    model = Model(spec)
    reqs = model.cache_requests()
    # the keys of layer 0 are kept for the widest reach among itself (a window of 9) and its reader (23)
    assert reqs[0] == reqs[2] == PagedKV(2, 12, 23, v_head_dim=20)
    assert reqs[1] == PagedKV(2, 16, 11)                                   # a chunk of 11 never looks further back
    assert reqs[3] == PagedKV(1, 24, 13, v_head_dim=8)
    names = set(model.expected_tensors())
    assert {"embed", "embed.norm", "head", "final.norm", "l0.norm1b", "l0.norm2b", "l1.mix.sink", "l1.mix.g"} <= names
    assert {"l0.mix.k", "l0.mix.k.b", "l0.mix.k.norm", "l0.mix.o.b", "l2.mix.q.b", "l2.mix.o.b", "l2.mix.q.norm", "l2.mix.g"} <= names
    assert not {"l2.mix.k", "l2.mix.v", "l2.mix.k.b", "l2.mix.v.b", "l2.mix.k.norm"} & names          # the reader has none
    assert not {"l2.norm2", "l2.norm2b", "l2.mlp.router", "l3.mix.g", "l3.mix.sink", "l1.mix.q.b", "l0.mix.sink"} & names
    assert "l0.mlp.shared.sg" in names and "l3.mlp.shared.up" not in names and "l3.mlp.e3.gate" in names
    assert "l1.mlp.gate" in names and spec.logit_softcap == 12.0 and spec.embedding_norm is not None


def test_what_the_design_fixes_reaches_the_parts_as_parameters():
    _, _, spec = spec_of("sazavik-tiny-A")
    a3, a1, reader, a2 = (spec.layers[i].parts["mixer"].params for i in (0, 1, 2, 3))
    assert a3["window"] == 9 and a3["chunk"] is None and a3["bias"] and a3["out_bias"] and a3["gate"] and not a3["sink"]
    assert a3["distance_slopes"] == tuple(2.0 ** (-8.0 * (h + 1) / 4) for h in range(4)) and a3["rotary"] is None
    assert a3["q_temperature"] == {"coef": 0.4, "every": 5} and a3["cache_window"] == 23
    assert a1["chunk"] == 11 and a1["window"] is None and a1["sink"] == "learned" and a1["gate"] and not a1["bias"]
    assert a1["rotary"] == {"dims": 8, "theta": 100.0, "layout": "interleaved"}
    assert a2["rotary"]["layout"] == "half" and not a2["gate"] and not a2["sink"] and a2["chunk"] == 13
    assert not reader["own_kv"] and reader["window"] == 23 and a3["own_kv"]
    dense, moe = spec.layers[1].parts["feed_forward"], spec.layers[0].parts["feed_forward"]
    assert dense.kind == "swiglu" and dense.params["activation"] == "clamped" and dense.params["limit"] == 1.5
    assert dense.params["alpha"] == 1.702 and dense.params["shift"] == 1.0
    assert moe.kind == "routed_experts" and moe.params["score"] == "sigmoid" and moe.params["weight_on"] == "input"
    assert moe.params["gated"] and not moe.params["renorm"] and moe.params["shared_gate"]
    for layer in spec.layers:
        assert all(layer.parts[n].params["one_plus"] for n in layer.parts if n.startswith("norm"))
    assert spec.final_norm.params["one_plus"] and spec.embedding_norm.params["one_plus"]


def test_page_groups_by_how_long_keys_are_kept():
    from yalis_b200.cache.storage import plan_groups
    _, _, spec = spec_of("sazavik-tiny-A")
    groups = {g.name: g for g in plan_groups(Model(spec).cache_requests(), 16, 64, 1024, 4, 64)}
    assert set(groups) == {"kv_window_23", "kv_window_11", "kv_window_13", "kv_window_7"}


def test_a_model_without_masks_caps_or_optional_parts():
    raw = preset("sazavik-tiny-B")
    for layer in raw["layers"]:
        layer["mixer"].pop("mask")
    raw["layers"][1]["mixer"].pop("q_temp")
    arch, cfg = parse_config(raw)
    spec = arch.model_spec(cfg)
    assert spec.logit_softcap is None
    assert all(r.window is None for r in Model(spec).cache_requests())
    assert spec.layers[1].parts["mixer"].params["q_temperature"] is None


def test_refused_configurations():
    base = preset("sazavik-tiny-A")

    def broken(change):
        raw = copy.deepcopy(base)
        change(raw)
        with pytest.raises(ConfigError):
            parse_config(raw)

    broken(lambda r: r["layers"][2]["mixer"].update(kv_from=4))                       # a later layer
    broken(lambda r: r["layers"][2]["mixer"].update(kv_from=1))                       # keys of another size
    broken(lambda r: r["layers"][2]["mixer"].update(kv_heads=4))
    broken(lambda r: r["layers"][4]["mixer"].update(kv_from=2))                       # a layer that has no keys itself
    broken(lambda r: r["layers"][1]["mixer"].update(kv_heads=3))
    broken(lambda r: r["layers"][0]["mlp"]["router"].update(top=9))
    broken(lambda r: r["layers"][0]["mlp"].update(kind="glu"))
    broken(lambda r: r["layers"][1]["mlp"].update(limit=0.0))
    broken(lambda r: r["layers"][0].update(type="retention"))
    broken(lambda r: r["layers"][1]["mixer"]["rot"].update(dims=18))                  # more sizes than a head has
    broken(lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7))
    broken(lambda r: r["layers"][0]["mixer"]["q_temp"].update(every=0))
    broken(lambda r: r.update(logit_softcap=-1.0))
    broken(lambda r: r.pop("norm"))
    raw = copy.deepcopy(base)
    raw["layers"][0]["mixer"]["kv_from"] = None                                         # spelled out, still its own
    parse_config(raw)


def test_flops_count_the_experts_a_token_uses():
    _, _, spec = spec_of("sazavik-tiny-C")
    ff = Model(spec).blocks[0].feed_forward
    assert ff.matrix_flops_per_token() == 2.0 * 128 * (16 + 3 * 4 * 32 + 3 * 64)
    attention = Model(spec).blocks[0].mixer
    assert attention.keys_seen(0) == 1 and attention.keys_seen(15) == 16 and attention.keys_seen(16) == 1 and attention.keys_seen(40) == 9
    window = Model(spec).blocks[3].mixer
    assert window.keys_seen(10) == 11 and window.keys_seen(49) == 50 and window.keys_seen(50) == 50 and window.keys_seen(700) == 50
