"""Pametar as an architecture of this engine: a decoder whose residual stream is kept in several copies.

Token rows are scaled as they enter, and a row of a second table, chosen by the token and the one before it, is
added (``embedding.bigram``).  The stream then exists in ``streams`` copies.  Every layer is a pre-norm layer whose
two sub-layers read a weighted sum of the copies and write to all of them, their results scaled by a learned vector
and by a sigmoid gate computed from the sub-layer's input; the norm is a ``dynamic_tanh``.  A layer's mixer is one of

* ``latent_attention``  causal attention over a normed latent of ``kv_rank`` sizes per token and a rotated key part of
                        ``rot_dim`` sizes shared by all heads (half-split pairs), queries through a normed latent of
                        ``q_rank`` sizes, a sink per head in the softmax's denominator;
* ``general_delta``     the generalized delta rule with a decay and a removal rate per head and key channel.

The feed-forward is a mixture of gated silu experts weighted by their softmax scores times ``router.scale`` (not
renormalised), or none.  A range of layers may run several times in a row with the same weights (``loop``); every
pass has a cache and a state of its own.  The output is the final norm of the copies' sum and a matrix of its own.

``config.json`` gives every size and constant but one: the inner size of the decay's low-rank product, which
``sizes_from_tensors`` reads from the checkpoint's header (a configuration written by this package carries it as
``decay_rank``).  Like every architecture here the model is described as data.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from yalis_b200.config.registry import ConfigError, register_architecture
from yalis_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE_NAME = "Pametar"
MAX_POSITION = 1 << 20          # nothing in the design bounds a sequence; block tables are sized by the cache pool
LAYER_TYPES = ("latent_attention", "general_delta")
DECAY_RATE = math.exp(-0.5)     # w = exp(-DECAY_RATE * sigmoid(.)): a channel keeps at least exp(-e^-1/2) per token


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class PametarConfig:
    width: int
    vocab: int
    streams: int
    norm_eps: float
    embedding_scale: float
    bigram: Optional[Mapping[str, int]]       # buckets, mul_prev, mul_cur
    layers: Tuple[Mapping[str, Any], ...]     # validated copies of the config's layer entries
    loop: Optional[Loop]

    @property
    def architecture(self) -> str:
        return ARCHITECTURE_NAME


def _int(d, key: str, where: str, least: int = 1) -> int:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"{where}: `{key}` must be an integer of at least {least}, got {v!r}")
    return v


def _num(d, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: `{key}` must be a number, got {v!r}")
    return float(v)


def _check_mlp(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ConfigError(f"{where}: mlp kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not supported (moe, or null)")
    router = {"experts": _int(mlp.get("router"), "experts", where + ".router"), "top": _int(mlp.get("router"), "top", where + ".router"),
              "scale": _num(mlp.get("router"), "scale", where + ".router")}
    if router["top"] > router["experts"]:
        raise ConfigError(f"{where}.router: top {router['top']} is more than the {router['experts']} experts")
    return {"kind": "moe", "expert": {"ff": _int(mlp.get("expert"), "ff", where + ".expert")}, "router": router}


def _check_layer(i: int, layer) -> Dict[str, Any]:
    where = f"layers[{i}]"
    kind = layer.get("type") if isinstance(layer, Mapping) else None
    if kind not in LAYER_TYPES:
        raise ConfigError(f"{where}: type {kind!r} is not one of {', '.join(LAYER_TYPES)}")
    m = layer.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"{where}: `mixer` must be an object")
    if kind == "general_delta":
        mixer: Dict[str, Any] = {k: _int(m, k, where) for k in ("heads", "dim")}
        if m.get("decay_rank") is None:
            raise ConfigError(f"{where}: the inner size of the decay's product is unknown (no `decay_rank`, and no checkpoint "
                              f"header with l{i}.mix.w1 was read)")
        mixer["decay_rank"] = _int(m, "decay_rank", where)
    else:
        mixer = {k: _int(m, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
        mixer["scale"] = _num(m, "scale", where)
        rot = m.get("rot")
        dims, base = _int(rot, "dims", where + ".rot"), _num(rot, "base", where + ".rot")
        if dims % 2 or dims > mixer["rot_dim"] or base <= 1.0:
            raise ConfigError(f"{where}.rot: dims {dims} must be even and at most rot_dim {mixer['rot_dim']}, base above 1")
        mixer["rot"] = {"dims": dims, "base": base}
    return {"type": kind, "mixer": mixer, "mlp": _check_mlp(layer.get("mlp"), where + ".mlp")}


class PametarArchitecture:
    name = ARCHITECTURE_NAME

    @staticmethod
    def sizes_from_tensors(raw: Dict[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
        """The configuration with the size that only a tensor's shape gives filled in."""
        raw = copy.deepcopy(raw)
        for i, layer in enumerate(raw.get("layers") or []):
            if isinstance(layer, dict) and layer.get("type") == "general_delta" and isinstance(layer.get("mixer"), dict):
                tensor = f"l{i}.mix.w1"
                if tensor in shapes and len(shapes[tensor]) == 2:
                    layer["mixer"]["decay_rank"] = int(shapes[tensor][0])
        return raw

    @staticmethod
    def parse_config(raw: Dict[str, Any]) -> PametarConfig:
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks `layers`")
        eps = _num(raw.get("norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        emb = raw.get("embedding") or {}
        scale = _num(emb, "scale", "embedding") if emb.get("scale") is not None else 1.0
        bigram = None
        if emb.get("bigram") is not None:
            b = emb["bigram"]
            bigram = {"buckets": _int(b, "buckets", "embedding.bigram"), "mul_prev": _int(b, "mul_prev", "embedding.bigram", 0),
                      "mul_cur": _int(b, "mul_cur", "embedding.bigram", 0)}
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            start, stop, times = lp.get("start"), lp.get("stop"), _int(lp, "times", "loop")
            if not all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop)) or not 0 <= start <= stop <= len(layers):
                raise ConfigError(f"loop: start {start!r} and stop {stop!r} must satisfy 0 <= start <= stop <= {len(layers)}")
            loop = Loop(start, stop, times)
        return PametarConfig(width=_int(raw, "width", "config"), vocab=_int(raw, "vocab", "config"),
                             streams=_int(raw, "streams", "config") if raw.get("streams") is not None else 1,
                             norm_eps=eps, embedding_scale=scale, bigram=bigram,
                             layers=tuple(_check_layer(i, l) for i, l in enumerate(layers)), loop=loop)

    @staticmethod
    def config_to_dict(c: PametarConfig) -> Dict[str, Any]:
        emb: Dict[str, Any] = {"scale": c.embedding_scale}
        if c.bigram is not None:
            emb["bigram"] = dict(c.bigram)
        d = {"architecture": ARCHITECTURE_NAME, "embedding": emb, "layers": copy.deepcopy([dict(l) for l in c.layers]),
             "norm": {"eps": c.norm_eps}, "streams": c.streams, "vocab": c.vocab, "width": c.width}
        if c.loop is not None:
            d["loop"] = {"start": c.loop.start, "stop": c.loop.stop, "times": c.loop.times}
        return d

    @staticmethod
    def _norm(c: PametarConfig) -> PartSpec:
        return PartSpec("dynamic_tanh", {"size": c.width})

    @classmethod
    def _layer(cls, c: PametarConfig, i: int, layer: Mapping[str, Any]) -> LayerSpec:
        kind, m = layer["type"], layer["mixer"]
        connection = PartSpec("hyper_connection", {"hidden_size": c.width, "copies": c.streams, "mixing": True,
                                                   "layer_scale": True, "gate": True})
        names: Dict[str, str] = {}

        def sublayer(q: int):
            names.update({f"norm_{q}.weight": f"norm{q}", f"norm_{q}.alpha": f"norm{q}.alpha", f"norm_{q}.bias": f"norm{q}.b",
                          f"connection_{q}.in": f"hc{q}.in", f"connection_{q}.out": f"hc{q}.out", f"connection_{q}.mix": f"hc{q}.mix",
                          f"connection_{q}.scale": f"ls{q}", f"connection_{q}.gate": f"rg{q}", f"connection_{q}.gate_bias": f"rg{q}.b"})

        sublayer(1)
        if kind == "general_delta":
            mixer = PartSpec("general_delta", {"hidden_size": c.width, "heads": m["heads"], "dim": m["dim"],
                                               "decay_rank": m["decay_rank"], "decay_rate": DECAY_RATE, "eps": c.norm_eps,
                                               "out_scale": 1.0})
            names.update({f"mixer.{p}_proj": f"mix.{p}" for p in ("r", "k", "v", "g", "a", "w1", "w2", "o")})
            names.update({"mixer.a_bias": "mix.a.b", "mixer.w_bias": "mix.w0", "mixer.norm": "mix.norm"})
        else:
            rotary = {"head_dim": m["rot"]["dims"], "theta": m["rot"]["base"], "layout": "half", "exact_powers": True,
                      "scaling": None}
            mixer = PartSpec("latent_attention", {
                "hidden_size": c.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"], "rotary": rotary, "scale": m["scale"], "window": None,
                "cache_window": None, "norm_eps": c.norm_eps, "gate": False, "own_latent": True, "q_rank": m["q_rank"],
                "sink": True})
            names.update({"mixer.dq_proj": "mix.dq", "mixer.dq_norm": "mix.dq.norm", "mixer.q_proj": "mix.uq",
                          "mixer.dkv_proj": "mix.dkv", "mixer.dkv_norm": "mix.dkv.norm", "mixer.uk_proj": "mix.uk",
                          "mixer.uv_proj": "mix.uv", "mixer.sink": "mix.sink", "mixer.o_proj": "mix.o"})
        parts = {"norm_1": cls._norm(c), "mixer": mixer, "connection_1": connection}
        mlp = layer["mlp"]
        if mlp is not None:
            sublayer(2)
            parts["norm_2"], parts["connection_2"] = cls._norm(c), connection
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden_size": c.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "expert_size": mlp["expert"]["ff"], "activation": "silu", "gated": True, "shared_size": None,
                "renorm": False, "route_scale": mlp["router"]["scale"]})
            names["feed_forward.router"] = "mlp.router"
            for e in range(mlp["router"]["experts"]):
                for p in ("gate", "up", "down"):
                    names[f"feed_forward.expert_{e}_{p}"] = f"mlp.e{e}.{p}"
        return LayerSpec(block=PartSpec("pre_norm_connected"), parts=parts, weight_prefix=f"l{i}.", weight_names=names)

    @classmethod
    def model_spec(cls, c: PametarConfig) -> ModelSpec:
        n = len(c.layers)
        if c.loop is None:
            order = list(range(n))
        else:
            a, b = c.loop.start, c.loop.stop
            order = list(range(a)) + list(range(a, b)) * c.loop.times + list(range(b, n))
        entry, entry_names = None, {}
        if c.bigram is not None:
            entry = PartSpec("pair_table", {"hidden_size": c.width, "vocab_size": c.vocab, **c.bigram})
            entry_names = {"table": "bigram"}
        return ModelSpec(
            architecture=ARCHITECTURE_NAME, hidden_size=c.width, vocab_size=c.vocab, max_position=MAX_POSITION,
            layers=tuple(cls._layer(c, i, layer) for i, layer in enumerate(c.layers)),
            schedule=tuple(ScheduleEntry(i) for i in order), final_norm=cls._norm(c), embedding_name="embed", head_name="head",
            final_norm_names={"weight": "final.norm", "alpha": "final.norm.alpha", "bias": "final.norm.b"},
            embedding_scale=c.embedding_scale, entry=entry, entry_names=entry_names, stream_copies=c.streams)


register_architecture(ARCHITECTURE_NAME, PametarArchitecture, replace=True)
