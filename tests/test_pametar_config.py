"""Pametar without a GPU: registry, the order of layer runs and their caches, tensor names, the size that only a tensor
gives, refused configurations, and the plain model's own pieces against sums written out by hand."""

import copy
import math

import pytest
import torch

import plain_pametar as plain
from pametar_models import pametar_dir
from yalis_b200.config.presets import preset
from yalis_b200.config.registry import ConfigError, load_config, parse_config
from yalis_b200.engine.model import Model
from yalis_b200.parts.base import PagedKV, SlotState


def spec_of(name):
    arch, cfg = parse_config(preset(name))
    return arch, cfg, arch.model_spec(cfg)


def test_the_registry_knows_the_design_and_round_trips_its_configuration():
    for which in "ABCD":
        raw = preset(f"pametar-tiny-{which}")
        arch, cfg = parse_config(raw)
        assert arch.name == "Pametar" and arch.config_to_dict(cfg) == raw


def test_looped_layers_run_again_with_the_same_weights_and_caches_of_their_own():
    _, _, spec = spec_of("pametar-tiny-A")
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    model = Model(spec)
    reqs = model.cache_requests()
    # one cache or state for every run, and the previous token of every request for the pair table
    assert reqs == [PagedKV(1, 24 + 8, None, v_head_dim=0), SlotState((2 * 16 * 16,), torch.float32), PagedKV(1, 16 + 4, None, v_head_dim=0),
                    SlotState((2 * 16 * 16,), torch.float32), PagedKV(1, 16 + 4, None, v_head_dim=0), SlotState((4 * 8 * 8,), torch.float32),
                    SlotState((1,), torch.int32)]
    names = set(model.expected_tensors())
    assert {"embed", "bigram", "head", "final.norm", "final.norm.alpha", "final.norm.b"} <= names
    assert {"l1.mix.r", "l1.mix.k", "l1.mix.v", "l1.mix.g", "l1.mix.a", "l1.mix.a.b", "l1.mix.w1", "l1.mix.w2", "l1.mix.w0", "l1.mix.norm",
            "l1.mix.o", "l1.hc1.in", "l1.hc1.out", "l1.hc1.mix", "l1.ls1", "l1.rg1", "l1.rg1.b", "l1.norm1.alpha", "l1.norm1.b"} <= names
    assert {"l0.mix.dq", "l0.mix.dq.norm", "l0.mix.uq", "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.o"} <= names
    assert "l2.norm2" not in names and "l2.hc2.mix" not in names and "l2.mlp.router" not in names      # a layer without feed-forward
    assert "l1.mlp.e5.gate" in names and "l1.mlp.e6.gate" not in names
    shapes = {n: tuple(p.shape) for n, p in model.expected_tensors().items()}
    assert shapes["bigram"] == (509 + 1, 64) and shapes["l0.hc1.mix"] == (2, 2) and shapes["l0.mix.sink"] == (2,)
    assert shapes["l0.mix.dkv"] == (24 + 8, 64) and shapes["l0.mix.uq"] == (2 * (8 + 8), 20) and shapes["l1.mix.w2"] == (32, 8)


def test_without_a_loop_a_pair_table_or_several_copies():
    _, cfg, spec = spec_of("pametar-tiny-C")
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and spec.entry is None and spec.stream_copies == 4
    assert "bigram" not in Model(spec).expected_tensors() and len(Model(spec).cache_requests()) == 4
    _, _, spec = spec_of("pametar-tiny-B")
    assert [e.layer for e in spec.schedule] == [0, 0, 0, 1, 2] and spec.stream_copies == 1
    raw = preset("pametar-tiny-B")
    del raw["streams"], raw["loop"]
    raw["embedding"] = {}
    arch, cfg = parse_config(raw)
    assert cfg.streams == 1 and cfg.loop is None and cfg.embedding_scale == 1.0 and cfg.bigram is None


def test_the_decays_inner_size_comes_from_the_checkpoint():
    d = pametar_dir("D")
    import json, os
    with open(os.path.join(d, "config.json")) as f:
        raw = json.load(f)
    assert all("decay_rank" not in layer["mixer"] for layer in raw["layers"])
    with pytest.raises(ConfigError):
        parse_config(raw)
    arch, cfg = load_config(d)
    assert [l["mixer"].get("decay_rank") for l in cfg.layers] == [6, None, 2]


def test_refused_configurations():
    base = preset("pametar-tiny-A")

    def broken(change):
        raw = copy.deepcopy(base)
        change(raw)
        with pytest.raises(ConfigError):
            parse_config(raw)

    broken(lambda r: r["layers"][0].update(type="retention"))
    broken(lambda r: r["layers"][0]["mlp"]["router"].update(top=5))
    broken(lambda r: r["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda r: r["layers"][0]["mixer"]["rot"].update(dims=10))                  # more sizes than the rotated part
    broken(lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3))
    broken(lambda r: r["layers"][0]["mixer"].pop("q_rank"))
    broken(lambda r: r["layers"][1]["mixer"].update(heads=0))
    broken(lambda r: r["loop"].update(stop=5))
    broken(lambda r: r["loop"].update(start=3, stop=2))
    broken(lambda r: r["loop"].update(times=0))
    broken(lambda r: r.pop("norm"))
    broken(lambda r: r.update(streams=0))
    broken(lambda r: r["embedding"]["bigram"].pop("buckets"))
    with pytest.raises(ValueError):
        arch, cfg = parse_config({**copy.deepcopy(base), "streams": 9})
        Model(arch.model_spec(cfg))


def test_flops_count_the_experts_a_token_uses_and_the_rules_state():
    _, _, spec = spec_of("pametar-tiny-A")
    model = Model(spec)
    assert model.blocks[0].feed_forward.matrix_flops_per_token() == 2.0 * 64 * 4 + 2.0 * 2 * 3 * 64 * 24
    assert model.blocks[1].mixer.mixing_flops(3, 100) == 8.0 * 2 * 16 * 16 * 3
    assert model.blocks[0].connection_1.matrix_flops_per_token() == 2.0 * 64 * 64


# ---- the plain model's pieces against sums by hand ---------------------------------------------------------------

def test_the_plain_pieces_by_hand():
    t = {"n": torch.tensor([2.0, 1.0]), "n.alpha": torch.tensor(0.5), "n.b": torch.tensor([0.0, 1.0])}
    got = plain.dynamic_tanh(torch.tensor([[2.0, -4.0]]), t, "n")
    assert got.flatten().tolist() == pytest.approx([2 * math.tanh(1.0), 1 - math.tanh(2.0)])
    # two copies: read 1 x_0 + 2 x_1; write with mix [from, to] = [[1, 10], [100, 1000]] and out = (1, -1)
    streams = torch.tensor([[[1.0]], [[2.0]]])
    assert plain.read_copies(streams, torch.tensor([1.0, 2.0])).tolist() == [[5.0]]
    new = plain.write_copies(streams, torch.tensor([[1.0, 10.0], [100.0, 1000.0]]), torch.tensor([1.0, -1.0]), torch.tensor([[0.5]]))
    assert new.flatten().tolist() == pytest.approx([1 * 1 + 100 * 2 + 0.5, 10 * 1 + 1000 * 2 - 0.5])
    # the pair table: the first token takes the last row
    cfg = {"embedding": {"scale": 2.0, "bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 2}}}
    tt = {"embed": torch.arange(4.0)[:, None], "bigram": torch.arange(6.0)[:, None] * 100}
    assert plain.embed_tokens([3, 1, 2], tt, cfg).flatten().tolist() == [6 + 500, 2 + 100 * ((9 + 2) % 5), 4 + 100 * ((3 + 4) % 5)]
    # a sink alone halves a single key's weight when it equals the score
    q, k, v = torch.ones(1, 1, 1), torch.full((1, 1, 1), 3.0), torch.full((1, 1, 2), 8.0)
    assert plain.causal_attention_with_sink(q, k, v, 0.5, torch.tensor([1.5])).flatten().tolist() == pytest.approx([4.0, 4.0])
    # pairs of the half-split layout: (x_0, x_2) and (x_1, x_3) of four turning sizes, the fifth passes
    x = torch.tensor([[1.0, 0.0, 0.0, 1.0, 7.0]])
    out = plain.rotate_half_pairs(x, [2], 4, 100.0)
    want = [math.cos(2.0), -math.sin(0.2), math.sin(2.0), math.cos(0.2), 7.0]
    torch.testing.assert_close(out.flatten(), torch.tensor(want))
    # routing: scores of the chosen, times the scale, not brought to sum one
    chosen, weights = plain.routing(torch.tensor([[1.0]]), torch.tensor([[0.0], [math.log(3.0)], [-50.0]]), 1, 2.0)
    assert chosen.tolist() == [[1]] and weights.flatten().tolist() == pytest.approx([2 * 0.75])
