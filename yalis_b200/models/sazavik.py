"""Sazavik as an architecture of this engine: a decoder whose token rows are normed as they enter the stream, whose
sub-layers each stand between two norms, x += norm_b(f(norm_a(x))), and whose layers have one of three attention
mixers:

* ``attention``    grouped-query attention with a norm on the heads of q and k, a rotation of the first ``rot.dims``
                   sizes of a head in interleaved pairs (2i, 2i + 1), a chunked mask (a position sees the positions
                   of its own chunk of ``mask.size``, counted from position 0, up to itself), a learned sink per
                   head in the softmax's denominator, and a sigmoid gate on the heads' results;
* ``attention_2``  the same norm, the rotation in half-split pairs (i, i + dims / 2), the chunked mask, a plain
                   softmax, no gate;
* ``attention_3``  biases on all four products, the norm, no rotation: the query grows with the logarithm of its
                   position (``q_temp``), slope_h * distance is taken off every score with
                   slope_h = 2^(-8 (h + 1) / heads), a sliding window of ``mask.size``, and the gate.  A layer with
                   ``kv_from: j`` has no key and value projections and reads what layer j cached.

A feed-forward is dense, down(g sigmoid(1.702 g) (u + 1)) with g and u clamped by ``limit``, or a mixture of experts
(sigmoid router, the ``top`` largest scores as they are, each multiplying its expert's input; silu-gated experts; a
shared expert weighted by one sigmoid per token), or absent.  The logits are squeezed by ``logit_softcap``.
``config.json`` gives every size and every constant that differs between models; like every architecture here the
model is described as data.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from yalis_b200.config.registry import ConfigError, register_architecture
from yalis_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE_NAME = "Sazavik"
MAX_POSITION = 1 << 20          # nothing in the design bounds a sequence; block tables are sized by the cache pool
LAYER_TYPES = ("attention", "attention_2", "attention_3")
# What the design fixes.
ROTARY_LAYOUT = {"attention": "interleaved", "attention_2": "half"}
GATED = {"attention": True, "attention_2": False, "attention_3": True}
SLOPE_EXPONENT = 8.0            # slope of head h (from 0) of H: 2^(-8 (h + 1) / H)
DENSE_ALPHA, DENSE_SHIFT = 1.702, 1.0


@dataclass(frozen=True)
class SazavikConfig:
    width: int
    vocab: int
    norm_eps: float
    logit_softcap: Optional[float]
    layers: Tuple[Mapping[str, Any], ...]     # validated copies of the config's layer entries

    @property
    def architecture(self) -> str:
        return ARCHITECTURE_NAME


def _int(d, key: str, where: str) -> int:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where}: `{key}` must be a positive integer, got {v!r}")
    return v


def _num(d, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: `{key}` must be a number, got {v!r}")
    return float(v)


def _check_mlp(mlp, where: str):
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, Mapping) else None
    if kind == "dense":
        out = {"kind": "dense", "ff": _int(mlp, "ff", where), "limit": _num(mlp, "limit", where)}
        if out["limit"] <= 0:
            raise ConfigError(f"{where}: limit must be positive")
        return out
    if kind != "moe":
        raise ConfigError(f"{where}: mlp kind {kind!r} is not supported (dense, moe, or null)")
    out = {"kind": "moe", "expert": {"ff": _int(mlp.get("expert"), "ff", where + ".expert")},
           "router": {"experts": _int(mlp.get("router"), "experts", where + ".router"),
                      "top": _int(mlp.get("router"), "top", where + ".router")}}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"{where}.router: top {out['router']['top']} is more than the {out['router']['experts']} experts")
    if mlp.get("shared") is not None:
        out["shared"] = {"ff": _int(mlp["shared"], "ff", where + ".shared")}
    return out


def _check_layer(i: int, layer) -> Dict[str, Any]:
    where = f"layers[{i}]"
    kind = layer.get("type") if isinstance(layer, Mapping) else None
    if kind not in LAYER_TYPES:
        raise ConfigError(f"{where}: type {kind!r} is not one of {', '.join(LAYER_TYPES)}")
    m = layer.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"{where}: `mixer` must be an object")
    mixer: Dict[str, Any] = {k: _int(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim")}
    if mixer["heads"] % mixer["kv_heads"]:
        raise ConfigError(f"{where}: heads {mixer['heads']} is not a multiple of kv_heads {mixer['kv_heads']}")
    mixer["scale"] = _num(m, "scale", where)
    if m.get("mask") is not None:
        mixer["mask"] = {"size": _int(m["mask"], "size", where + ".mask")}
    if kind in ROTARY_LAYOUT:
        rot = m.get("rot")
        if rot is not None:
            dims, base = _int(rot, "dims", where + ".rot"), _num(rot, "base", where + ".rot")
            if dims % 2 or dims > mixer["dim"] or base <= 0:
                raise ConfigError(f"{where}.rot: dims {dims} must be even and at most {mixer['dim']}, base positive")
            mixer["rot"] = {"dims": dims, "base": base}
    else:
        qt = m.get("q_temp")
        if qt is not None:
            mixer["q_temp"] = {"coef": _num(qt, "coef", where + ".q_temp"), "every": _int(qt, "every", where + ".q_temp")}
    if m.get("kv_from") is not None:
        j = m["kv_from"]
        if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
            raise ConfigError(f"{where}: kv_from {j!r} must name an earlier layer")
        mixer["kv_from"] = j
    return {"type": kind, "mixer": mixer, "mlp": _check_mlp(layer.get("mlp"), where + ".mlp")}


def _reach(layer: Mapping[str, Any]) -> Optional[int]:
    """How many positions back a layer's queries reach at most (None: to the start): a window of W sees W positions,
    a chunk of C at most C."""
    mask = layer["mixer"].get("mask")
    return None if mask is None else mask["size"]


class SazavikArchitecture:
    name = ARCHITECTURE_NAME

    @staticmethod
    def parse_config(raw: Dict[str, Any]) -> SazavikConfig:
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks `layers`")
        eps = _num(raw.get("norm"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        checked = tuple(_check_layer(i, l) for i, l in enumerate(layers))
        for i, layer in enumerate(checked):
            j = layer["mixer"].get("kv_from")
            if j is None:
                continue
            src, m = checked[j]["mixer"], layer["mixer"]
            if src.get("kv_from") is not None:
                raise ConfigError(f"layers[{i}]: kv_from {j} must name a layer with keys of its own")
            if any(src.get(k) != m.get(k) for k in ("kv_heads", "dim", "vdim", "rot")):
                raise ConfigError(f"layers[{i}]: kv_heads, dim, vdim and rot must equal those of layer {j}, whose keys it reads")
        cap = raw.get("logit_softcap")
        if cap is not None:
            cap = _num(raw, "logit_softcap", "config")
            if cap <= 0:
                raise ConfigError("logit_softcap must be positive")
        return SazavikConfig(width=_int(raw, "width", "config"), vocab=_int(raw, "vocab", "config"), norm_eps=eps,
                             logit_softcap=cap, layers=checked)

    @staticmethod
    def config_to_dict(c: SazavikConfig) -> Dict[str, Any]:
        out = {"architecture": ARCHITECTURE_NAME, "layers": copy.deepcopy([dict(l) for l in c.layers]),
               "norm": {"eps": c.norm_eps}, "vocab": c.vocab, "width": c.width}
        if c.logit_softcap is not None:
            out["logit_softcap"] = c.logit_softcap
        return out

    @staticmethod
    def _kept(c: SazavikConfig, owner: int) -> Optional[int]:
        """How many positions back the keys of layer ``owner`` must be kept: the widest reach among the layer itself
        and the layers that read its keys (None: for ever)."""
        reaches = [_reach(l) for i, l in enumerate(c.layers) if i == owner or l["mixer"].get("kv_from") == owner]
        return None if any(r is None for r in reaches) else max(reaches)

    @classmethod
    def _norm(cls, c: SazavikConfig) -> PartSpec:
        return PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps, "one_plus": True})

    @classmethod
    def _layer(cls, c: SazavikConfig, i: int, layer: Mapping[str, Any]) -> LayerSpec:
        kind, m = layer["type"], layer["mixer"]
        own = m.get("kv_from") is None
        size = None if m.get("mask") is None else m["mask"]["size"]
        biased = kind == "attention_3"
        rot = m.get("rot")
        params = {
            "hidden_size": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "bias": biased, "out_bias": biased, "qk_norm_eps": c.norm_eps, "scale": m["scale"],
            "rotary": None if rot is None else {"dims": rot["dims"], "theta": rot["base"], "layout": ROTARY_LAYOUT[kind]},
            "softcap": None, "sink": "learned" if kind == "attention" else False, "gate": GATED[kind], "own_kv": own,
            "window": size if kind == "attention_3" else None, "chunk": None if kind == "attention_3" else size,
            "cache_window": cls._kept(c, i if own else m["kv_from"]), "out_scale": 1.0,
            "q_temperature": m.get("q_temp"),
            "distance_slopes": tuple(2.0 ** (-SLOPE_EXPONENT * (h + 1) / m["heads"]) for h in range(m["heads"]))
            if kind == "attention_3" else None}
        names = {"norm_1.weight": "norm1", "norm_1_post.weight": "norm1b", "mixer.q_proj": "mix.q", "mixer.o_proj": "mix.o",
                 "mixer.q_norm": "mix.q.norm"}
        if own:
            names.update({"mixer.k_proj": "mix.k", "mixer.v_proj": "mix.v", "mixer.k_norm": "mix.k.norm"})
        if biased:
            names.update({"mixer.q_bias": "mix.q.b", "mixer.o_bias": "mix.o.b"})
            if own:
                names.update({"mixer.k_bias": "mix.k.b", "mixer.v_bias": "mix.v.b"})
        if GATED[kind]:
            names["mixer.g_proj"] = "mix.g"
        if kind == "attention":
            names["mixer.sink"] = "mix.sink"
        parts = {"norm_1": cls._norm(c), "mixer": PartSpec("general_attention", params), "norm_1_post": cls._norm(c)}
        mlp = layer["mlp"]
        if mlp is not None:
            parts["norm_2"], parts["norm_2_post"] = cls._norm(c), cls._norm(c)
            names.update({"norm_2.weight": "norm2", "norm_2_post.weight": "norm2b"})
            if mlp["kind"] == "dense":
                parts["feed_forward"] = PartSpec("swiglu", {
                    "hidden_size": c.width, "intermediate_size": mlp["ff"], "activation": "clamped", "limit": mlp["limit"],
                    "alpha": DENSE_ALPHA, "shift": DENSE_SHIFT})
                names.update({f"feed_forward.{p}_proj": f"mlp.{p}" for p in ("gate", "up", "down")})
            else:
                shared = mlp.get("shared")
                parts["feed_forward"] = PartSpec("routed_experts", {
                    "hidden_size": c.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                    "expert_size": mlp["expert"]["ff"], "activation": "silu", "gated": True, "score": "sigmoid",
                    "renorm": False, "weight_on": "input", "shared_size": None if shared is None else shared["ff"],
                    "shared_gate": shared is not None})
                names["feed_forward.router"] = "mlp.router"
                for e in range(mlp["router"]["experts"]):
                    names.update({f"feed_forward.expert_{e}_{p}": f"mlp.e{e}.{p}" for p in ("gate", "up", "down")})
                if shared is not None:
                    names.update({"feed_forward.shared_gate_proj": "mlp.shared.gate", "feed_forward.shared_up": "mlp.shared.up",
                                  "feed_forward.shared_down": "mlp.shared.down", "feed_forward.shared_gate": "mlp.shared.sg"})
        return LayerSpec(block=PartSpec("pre_norm_residual"), parts=parts, weight_prefix=f"l{i}.", weight_names=names)

    @classmethod
    def model_spec(cls, c: SazavikConfig) -> ModelSpec:
        # a layer that reads another layer's keys is a schedule entry that reads that entry's cache
        schedule = tuple(ScheduleEntry(i, cache_of=layer["mixer"].get("kv_from")) for i, layer in enumerate(c.layers))
        return ModelSpec(
            architecture=ARCHITECTURE_NAME, hidden_size=c.width, vocab_size=c.vocab, max_position=MAX_POSITION,
            layers=tuple(cls._layer(c, i, layer) for i, layer in enumerate(c.layers)), schedule=schedule,
            final_norm=cls._norm(c), embedding_name="embed", head_name="head", final_norm_names={"weight": "final.norm"},
            logit_softcap=c.logit_softcap, embedding_norm=cls._norm(c), embedding_norm_names={"weight": "embed.norm"})


register_architecture(ARCHITECTURE_NAME, SazavikArchitecture, replace=True)
