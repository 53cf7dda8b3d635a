"""Small Sazavik model folders for the tests, with weights that make every mechanism show.

The product's random-weights mode draws every matrix from N(0, 0.02) and sets norm scales to one, under which
attention weights are nearly uniform and a router's scores nearly equal: a mask that is one token off, a sink that is
left out or a wrong expert would hardly show.  The folders made here draw matrices wide enough for peaked attention
and decisive routing, norm weights around their neutral value, sinks, biases and gates that matter.  Names and shapes
come from the model's own list of expected tensors; the values are this file's.
"""

import functools
import json
import os
import tempfile

import torch

from yalis_b200.config.presets import preset
from yalis_b200.config.registry import parse_config
from yalis_b200.engine.model import Model
from yalis_b200.weights.safetensors_io import write_safetensors

_ROOT = None


def _root():
    global _ROOT
    if _ROOT is None:
        _ROOT = tempfile.mkdtemp(prefix="yalis_b200_sazavik_")
    return _ROOT


def lively_tensor(name: str, shape, gen: torch.Generator) -> torch.Tensor:
    def normal(std):
        return torch.randn(shape, generator=gen) * std

    if name.endswith((".q.norm", ".k.norm")):
        return 1.0 + normal(0.2)                       # a plain scale
    if name.endswith(("norm1", "norm2", "norm1b", "norm2b", "final.norm", "embed.norm")):
        return normal(0.2)                             # stored around zero
    if name == "embed":
        return normal(1.0)
    if name.endswith(".sink"):
        return 1.0 + normal(1.5)
    if name.endswith(".b"):
        return normal(0.4)
    fan_in = shape[-1]
    if name.endswith((".router", ".sg")):
        return normal(4.0 / fan_in ** 0.5)
    if name.endswith((".q", ".k")):
        return normal(2.5 / fan_in ** 0.5)
    if name.endswith((".gate", ".up", ".g")):
        return normal(2.0 / fan_in ** 0.5)
    return normal(1.3 / fan_in ** 0.5)


def write_model(config: dict, out_dir: str, seed: int, overrides=None) -> str:
    """config.json and model.safetensors (bfloat16) for a Sazavik configuration; ``overrides`` name -> tensor."""
    arch, cfg = parse_config(config)
    expected = Model(arch.model_spec(cfg)).expected_tensors()
    gen = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, ps in expected.items():
        t = lively_tensor(name, tuple(ps.shape), gen)
        if overrides and name in overrides:
            t = overrides[name].reshape(ps.shape).float()
        tensors[name] = t.to(torch.bfloat16)
    os.makedirs(out_dir, exist_ok=True)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(arch.config_to_dict(cfg), f)
    return out_dir


@functools.lru_cache(maxsize=None)
def sazavik_dir(which: str, seed: int = 0) -> str:
    return write_model(preset(f"sazavik-tiny-{which}"), os.path.join(_root(), f"{which}_{seed}"), seed)
