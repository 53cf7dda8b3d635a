"""Mixers that keep a matrix per head instead of keys and values, and mixers side by side.

``retention``    S_t = d_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t  with a fixed decay d_h per head; rotated q
                 and k; the read-out of each head divided by its root mean square and gated.
``gated_delta``  S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t  with q, k, v passed
                 through a short causal convolution and silu, q and k brought to unit length, a decay g_t
                 per head or per head and key channel computed from the input, and a normed, gated read-out.
``general_delta``  S <- diag(w_t) S - (a_t * u_t)(u_t^T S) + k_t v_t^T (both terms read the old S);  o_t = S^T r_t  with
                 the unit key u_t = k_t / |k_t|, a decay w_t per head and key channel through a low-rank product and a
                 removal rate a_t per head and key channel; a normed, sigmoid-gated read-out.
``sum_of_mixers``  several mixers that read the same input; their results are added, each times its factor.

All three are ``Projected``: an arrangement may run their input and output products together with those of its
other parts.  What the recurrences keep (state matrices in float32, the convolution's last inputs) is one row
of slot memory per request; the kernels walk a request's tokens in order, so the result at a position does not
depend on how the request was cut into steps.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops import recurrent as rec_ops
from yalis_b200.ops.elementwise import activation, qkv_prepare
from yalis_b200.ops.linear import linear
from .base import Mixer, ParamSpec, PositionEncoding, Projected, SlotState, SlotStateCache, make_part, register_part, stack_rows


def position_part(params) -> Optional[PositionEncoding]:
    """The position part a mixer builds for itself from its ``rotary`` parameter ({"dims", "theta"} and optionally
    "layout"; None: none)."""
    rot = params.get("rotary")
    if rot is None:
        return None
    return make_part("position", PartSpec("rotary", {"head_dim": int(rot["dims"]), "theta": float(rot["theta"]),
                                                     "scaling": None, "exact_powers": True,
                                                     "layout": rot.get("layout", "half")}))


class _ProjectedMixer(Mixer, Projected):
    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec, position)
        self.w_in: Optional[torch.Tensor] = None
        self.w_out: Optional[torch.Tensor] = None
        self.out_scale = float(spec.params.get("out_scale", 1.0))

    def in_weight(self) -> torch.Tensor:
        return self.w_in

    def out_weight(self) -> torch.Tensor:
        return self.w_out

    def release_projections(self) -> None:
        self.w_in = self.w_out = None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        return self.project_and_mix(x, ctx, cache)

    def capture_key(self, host):
        # the kernels read the step's arrays on the device and their grids follow the shapes alone; only the tile of
        # tokens that the recurrence stages at a time follows the longest portion, up to 16
        return min(host.max_q_len, 16)


class Retention(_ProjectedMixer):
    """Parameters: ``hidden_size``, ``heads``, ``dim`` (of q and k), ``vdim``, ``decay`` (one number per head),
    ``rotary`` ({"dims", "theta"} or None), ``eps`` (of the read-out's norm), ``out_scale``.
    Keys are multiplied by dim^(-1/2) after the rotation; the gate is silu."""

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec, position or position_part(spec.params))
        p = spec.params
        self.hidden, self.h, self.d, self.vd = int(p["hidden_size"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.eps = float(p["eps"])
        self.decay_values = [float(x) for x in p["decay"]]
        if len(self.decay_values) != self.h:
            raise ValueError(f"retention: {len(self.decay_values)} decays for {self.h} heads")
        self.layout = rec_ops.StateLayout(self.h, self.d, self.vd)
        self.hidden_width = self.h * self.vd
        self.decay: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        hd, hv = self.h * self.d, self.h * self.vd
        return {"q_proj": ParamSpec((hd, self.hidden)), "k_proj": ParamSpec((hd, self.hidden)),
                "v_proj": ParamSpec((hv, self.hidden)), "g_proj": ParamSpec((hv, self.hidden)),
                "o_proj": ParamSpec((self.hidden, hv))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_in = torch.cat([t["q_proj"], t["k_proj"], t["v_proj"], t["g_proj"]], dim=0).contiguous()
        self.w_out = t["o_proj"].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(self.w_out.device)

    def cache_request(self) -> SlotState:
        return SlotState((self.layout.total,), torch.float32)

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        return 4.0 * self.h * self.d * self.vd * q_len

    def mix(self, z: torch.Tensor, ctx, cache: SlotStateCache, y: torch.Tensor) -> None:
        hd, hv = self.h * self.d, self.h * self.vd
        freq = self.position.rotary_frequencies(self.position.head_dim, z.device) if self.position is not None else None
        q, k, v = qkv_prepare(z, (0, hd, 2 * hd), self.h, self.h, self.d, self.vd, ctx.positions, ctx.req_of_token,
                              out_dtype=torch.float32, inv_freq=freq, k_scale=self.d ** -0.5)
        o = rec_ops.state_scan(q, k, v, cache.state, self.layout, ctx.q_start, ctx.slots, kv_heads=self.h, decay=self.decay,
                               max_q_len=ctx.host.max_q_len)
        rec_ops.head_norm_gate(o, self.h, self.vd, self.eps, ctx.req_of_token, y, gate=z[:, 2 * hd + hv:2 * hd + 2 * hv],
                               gate_kind=rec_ops.GATE_SILU, out_scale=self.out_scale)


class GatedDelta(_ProjectedMixer):
    """Parameters: ``hidden_size``, ``heads`` (of v and of the state), ``kv_heads`` (of q and k; value head h uses
    q/k head h // (heads / kv_heads)), ``dim``, ``vdim``, ``conv`` (taps of the short convolution), ``eps`` (of the
    read-out's norm), ``decay`` ("head": g = exp(-exp(A_log) softplus(W_a x + dt_bias)), one per head; "channel":
    the same over W_a2 W_a1 x, one per head and key channel, ``decay_rank`` rows in W_a1), ``gate`` ("silu": silu(W_g x);
    "sigmoid_low_rank": sigmoid(W_g2 W_g1 x), ``gate_rank`` rows in W_g1), ``out_scale``.
    q is multiplied by dim^(-1/2) after it is brought to unit length (x / sqrt(sum x^2 + 1e-6))."""

    UNIT_EPS = 1e-6

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec, position)
        p = spec.params
        self.hidden, self.h, self.g = int(p["hidden_size"]), int(p["heads"]), int(p["kv_heads"])
        self.d, self.vd, self.taps = int(p["dim"]), int(p["vdim"]), int(p["conv"])
        self.eps = float(p["eps"])
        self.decay_kind, self.gate_kind = str(p.get("decay", "head")), str(p.get("gate", "silu"))
        if self.h % self.g:
            raise ValueError(f"gated_delta: heads {self.h} is not a multiple of kv_heads {self.g}")
        if self.decay_kind not in ("head", "channel") or self.gate_kind not in ("silu", "sigmoid_low_rank"):
            raise ValueError(f"gated_delta: unknown decay {self.decay_kind!r} or gate {self.gate_kind!r}")
        self.decay_rank = int(p["decay_rank"]) if self.decay_kind == "channel" else 0
        self.gate_rank = int(p["gate_rank"]) if self.gate_kind == "sigmoid_low_rank" else 0
        self.channels = 2 * self.g * self.d + self.h * self.vd
        self.layout = rec_ops.StateLayout(self.h, self.d, self.vd, self.channels, self.taps)
        self.hidden_width = self.h * self.vd
        self.spans: Dict[str, tuple] = {}

    def param_specs(self) -> Dict[str, ParamSpec]:
        gd, hv, hid = self.g * self.d, self.h * self.vd, self.hidden
        specs = {"q_proj": ParamSpec((gd, hid)), "q_conv": ParamSpec((gd, self.taps), keep_float32=True),
                 "k_proj": ParamSpec((gd, hid)), "k_conv": ParamSpec((gd, self.taps), keep_float32=True),
                 "v_proj": ParamSpec((hv, hid)), "v_conv": ParamSpec((hv, self.taps), keep_float32=True),
                 "b_proj": ParamSpec((self.h, hid)), "A_log": ParamSpec((self.h,), init="zeros", keep_float32=True),
                 "norm": ParamSpec((self.vd,), init="ones", keep_float32=True), "o_proj": ParamSpec((hid, hv))}
        if self.decay_kind == "head":
            specs["a_proj"] = ParamSpec((self.h, hid))
            specs["dt_bias"] = ParamSpec((self.h,), init="zeros", keep_float32=True)
        else:
            specs["a1_proj"] = ParamSpec((self.decay_rank, hid))
            specs["a2_proj"] = ParamSpec((self.h * self.d, self.decay_rank))
            specs["dt_bias"] = ParamSpec((self.h * self.d,), init="zeros", keep_float32=True)
        if self.gate_kind == "silu":
            specs["g_proj"] = ParamSpec((hv, hid))
        else:
            specs["g1_proj"] = ParamSpec((self.gate_rank, hid))
            specs["g2_proj"] = ParamSpec((hv, self.gate_rank))
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        # q, k, v first and without gaps: the convolution runs over them as one block of channels
        qkv = torch.cat([t["q_proj"], t["k_proj"], t["v_proj"]], dim=0)
        names = ["qkv", "g" if self.gate_kind == "silu" else "g1"] + (["a1"] if self.decay_kind == "channel" else []) + ["b"] \
            + (["a"] if self.decay_kind == "head" else [])
        blocks = [qkv] + [t[f"{n}_proj"] for n in names[1:]]
        self.w_in, spans = stack_rows(blocks)
        self.spans = dict(zip(names, spans))
        self.w_out = t["o_proj"].contiguous()
        self.conv_w = torch.cat([t["q_conv"], t["k_conv"], t["v_conv"]], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = t["A_log"].contiguous(), t["dt_bias"].contiguous(), t["norm"].contiguous()
        self.w_a2 = t["a2_proj"].contiguous() if self.decay_kind == "channel" else None
        self.w_g2 = t["g2_proj"].contiguous() if self.gate_kind == "sigmoid_low_rank" else None

    def cache_request(self) -> SlotState:
        return SlotState((self.layout.total,), torch.float32)

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        return 6.0 * self.h * self.d * self.vd * q_len

    def _block(self, z: torch.Tensor, name: str) -> torch.Tensor:
        a, b = self.spans[name]
        return z[:, a:b]

    def mix(self, z: torch.Tensor, ctx, cache: SlotStateCache, y: torch.Tensor) -> None:
        gd = self.g * self.d
        a_raw = linear(self._block(z, "a1"), self.w_a2) if self.decay_kind == "channel" else self._block(z, "a")
        conv, decay, beta = rec_ops.delta_prepare(
            self._block(z, "qkv"), self.conv_w, cache.state, self.layout.state_floats, ctx.req_of_token, ctx.q_start, ctx.slots,
            unit_heads=self.g, dim=self.d, q_scale=self.d ** -0.5, unit_eps=self.UNIT_EPS, a_raw=a_raw, a_log=self.a_log,
            dt_bias=self.dt_bias, b_raw=self._block(z, "b"))
        o = rec_ops.state_scan(conv[:, :gd], conv[:, gd:2 * gd], conv[:, 2 * gd:], cache.state, self.layout, ctx.q_start,
                               ctx.slots, kv_heads=self.g, decay=decay, beta=beta, max_q_len=ctx.host.max_q_len)
        if self.gate_kind == "silu":
            gate, kind = self._block(z, "g"), rec_ops.GATE_SILU
        else:
            gate, kind = linear(self._block(z, "g1"), self.w_g2), rec_ops.GATE_SIGMOID
        rec_ops.head_norm_gate(o, self.h, self.vd, self.eps, ctx.req_of_token, y, weight=self.norm_w, gate=gate,
                               gate_kind=kind, out_scale=self.out_scale)


class GeneralDelta(_ProjectedMixer):
    """The generalized delta rule.  Parameters: ``hidden_size``, ``heads``, ``dim`` (of r, k and v alike), ``decay_rank``
    (rows of the first matrix of the decay's low-rank product), ``decay_rate`` (c in w = exp(-c sigmoid(.))), ``eps`` (of
    the read-out's norm), ``out_scale``.

        r, k, v = W_r x, W_k x, W_v x            w = exp(-c sigmoid(W_w2 tanh(W_w1 x) + w0))     a = sigmoid(W_a x + b_a)
        u = k / sqrt(sum k^2 + 1e-6) per head    S <- diag(w) S - (a * u)(u^T S) + k v^T          o = S^T r
        y = W_o (o / rms(o) per head * n * sigmoid(W_g x))

    Everything between the projections and the output product is float32; the state [heads, dim, dim] is a float32
    slot row."""

    UNIT_EPS = 1e-6

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec, position)
        p = spec.params
        self.hidden, self.h, self.d = int(p["hidden_size"]), int(p["heads"]), int(p["dim"])
        self.rank, self.rate, self.eps = int(p["decay_rank"]), float(p["decay_rate"]), float(p["eps"])
        self.layout = rec_ops.StateLayout(self.h, self.d, self.d)
        self.hidden_width = self.h * self.d
        self.spans: Dict[str, tuple] = {}

    def param_specs(self) -> Dict[str, ParamSpec]:
        hd, hid = self.h * self.d, self.hidden
        return {"r_proj": ParamSpec((hd, hid)), "k_proj": ParamSpec((hd, hid)), "v_proj": ParamSpec((hd, hid)),
                "g_proj": ParamSpec((hd, hid)), "a_proj": ParamSpec((hd, hid)),
                "a_bias": ParamSpec((hd,), init="zeros", keep_float32=True),
                "w1_proj": ParamSpec((self.rank, hid)), "w2_proj": ParamSpec((hd, self.rank)),
                "w_bias": ParamSpec((hd,), init="zeros", keep_float32=True),
                "norm": ParamSpec((hd,), init="ones", keep_float32=True), "o_proj": ParamSpec((hid, hd))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        rkv = torch.cat([t["r_proj"], t["k_proj"], t["v_proj"]], dim=0)
        self.w_in, spans = stack_rows([rkv, t["g_proj"], t["a_proj"], t["w1_proj"]])
        self.spans = dict(zip(("rkv", "g", "a", "w1"), spans))
        self.w_out = t["o_proj"].contiguous()
        self.w_w2 = t["w2_proj"].contiguous()
        self.a_bias, self.w_bias, self.norm_w = t["a_bias"].contiguous(), t["w_bias"].contiguous(), t["norm"].contiguous()

    def cache_request(self) -> SlotState:
        return SlotState((self.layout.total,), torch.float32)

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        return 8.0 * self.h * self.d * self.d * q_len

    def mix(self, z: torch.Tensor, ctx, cache: SlotStateCache, y: torch.Tensor) -> None:
        hd = self.h * self.d
        a0, _ = self.spans["rkv"]
        blk = lambda name: z[:, self.spans[name][0]:self.spans[name][1]]
        w_raw = linear(activation(blk("w1"), "tanh"), self.w_w2)
        q, k, v, decay, unit, removal = rec_ops.general_delta_prepare(
            z[:, a0:a0 + hd], z[:, a0 + hd:a0 + 2 * hd], z[:, a0 + 2 * hd:a0 + 3 * hd], blk("a"), self.a_bias, w_raw,
            self.w_bias, self.h, self.d, self.rate, self.UNIT_EPS, ctx.req_of_token)
        o = rec_ops.state_scan(q, k, v, cache.state, self.layout, ctx.q_start, ctx.slots, kv_heads=self.h, decay=decay,
                               unit=unit, removal=removal, max_q_len=ctx.host.max_q_len)
        rec_ops.head_norm_gate(o, self.h, self.d, self.eps, ctx.req_of_token, y, weight=self.norm_w, gate=blk("g"),
                               gate_kind=rec_ops.GATE_SIGMOID, out_scale=self.out_scale)


class SumOfMixers(_ProjectedMixer):
    """Parameters: ``mixers``: name -> PartSpec of a ``Projected`` mixer (its ``out_scale`` is its factor in the sum).
    All read the same input.  Tensors of mixer ``name`` are named ``<name>.<its own name>``; what the mixers keep
    is asked for and handed out as a dictionary by mixer name."""

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec, position)
        self.subs: Dict[str, Mixer] = {name: make_part("mixer", sub) for name, sub in spec.params["mixers"].items()}
        for name, m in self.subs.items():
            if not isinstance(m, Projected):
                raise ValueError(f"sum_of_mixers: mixer {name!r} ({m.spec.kind}) cannot share its products")
        self.hidden_width = sum(m.hidden_width for m in self.subs.values())
        self.in_spans: List[tuple] = []

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {f"{name}.{local}": ps for name, m in self.subs.items() for local, ps in m.param_specs().items()}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        for name, m in self.subs.items():
            m.load({local: t[f"{name}.{local}"] for local in m.param_specs()})
        self.w_in, self.in_spans = stack_rows([m.in_weight() for m in self.subs.values()])
        self.w_out = torch.cat([m.out_weight() for m in self.subs.values()], dim=1).contiguous()
        for m in self.subs.values():
            m.release_projections()

    def cache_request(self):
        req = {name: m.cache_request() for name, m in self.subs.items()}
        return {name: r for name, r in req.items() if r is not None} or None

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        return sum(m.mixing_flops(q_len, ctx_before) for m in self.subs.values())

    def capture_key(self, host):
        from .base import NOT_CAPTURABLE
        keys = []
        for m in self.subs.values():
            key = m.capture_key(host)
            if key is NOT_CAPTURABLE:
                return NOT_CAPTURABLE
            keys.append(key)
        return tuple(keys)

    def mix(self, z: torch.Tensor, ctx, cache, y: torch.Tensor) -> None:
        at = 0
        for (name, m), (a, b) in zip(self.subs.items(), self.in_spans):
            m.mix(z[:, a:b], ctx, (cache or {}).get(name), y[:, at:at + m.hidden_width])
            at += m.hidden_width


register_part("mixer", "retention", Retention)
register_part("mixer", "gated_delta", GatedDelta)
register_part("mixer", "general_delta", GeneralDelta)
register_part("mixer", "sum_of_mixers", SumOfMixers)
