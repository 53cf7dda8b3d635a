"""Small Pametar model folders for the tests, with weights that make every mechanism show.

The product's random-weights mode draws every matrix from N(0, 0.02), sets scales to one and the copies' mixing
to the identity: attention weights would be nearly uniform, a router's scores nearly equal, the copies of the
stream all alike and a lost state hardly visible.  The folders made here draw matrices wide enough for peaked
attention and decisive routing, mixing matrices and read and write weights that tell the copies apart, sinks of
both signs, and biases that spread decays and removal rates over their ranges.  Names and shapes come from the
model's own list of expected tensors; the values are this file's.
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
        _ROOT = tempfile.mkdtemp(prefix="yalis_b200_pametar_")
    return _ROOT


def lively_tensor(name: str, shape, gen: torch.Generator) -> torch.Tensor:
    def normal(std, mean=0.0):
        return mean + torch.randn(shape, generator=gen) * std

    last = name.rsplit(".", 1)[-1]
    if name.endswith(".alpha"):
        return normal(0.02, 0.3)
    if name.endswith((".norm1", ".norm2", "final.norm", ".dq.norm", ".dkv.norm", ".mix.norm")) or last in ("ls1", "ls2"):
        return normal(0.2, 1.0)
    if name.endswith((".norm1.b", ".norm2.b", "final.norm.b", ".rg1.b", ".rg2.b", ".a.b", ".w0")):
        return normal(0.5)
    if name.endswith(".sink"):
        return normal(1.5)
    if last == "mix" and ".hc" in name:
        return torch.eye(shape[0]) * 0.8 + normal(0.25)
    if last == "in" and ".hc" in name:
        return normal(0.3, 1.0 / shape[0] ** 0.5)
    if last == "out" and ".hc" in name:
        return normal(0.4, 0.8)
    if name == "embed":
        return normal(1.0)
    if name == "bigram":
        return normal(0.7)
    fan_in = shape[-1]
    if name.endswith(".router"):
        return normal(4.0 / fan_in ** 0.5)
    if name.endswith((".dq", ".uq", ".dkv", ".uk", ".mix.k", ".mix.r")):
        return normal(2.5 / fan_in ** 0.5)
    if name.endswith((".w1", ".w2", ".mix.a")):
        return normal(3.0 / fan_in ** 0.5)
    return normal(1.3 / fan_in ** 0.5)


def write_model(config: dict, out_dir: str, seed: int, overrides=None) -> str:
    """config.json and model.safetensors (bfloat16) for a Pametar configuration; ``overrides`` name -> tensor."""
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
    written = arch.config_to_dict(cfg)
    for layer in written["layers"]:            # as a folder from elsewhere: the decay's inner size is in the tensors only
        layer["mixer"].pop("decay_rank", None)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(written, f)
    return out_dir


@functools.lru_cache(maxsize=None)
def pametar_dir(which: str, seed: int = 0) -> str:
    return write_model(preset(f"pametar-tiny-{which}"), os.path.join(_root(), f"{which}_{seed}"), seed)
