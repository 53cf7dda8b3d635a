"""A routed feed-forward: every token runs ``top`` of ``experts`` small feed-forwards, chosen and weighted by a
router, and optionally a shared one that every token runs.

    s = softmax(W_r x) over all experts (float32);  chosen = the ``top`` largest s;  w_j = s_j / (sum chosen s + eps)
    y = sum_j w_j  D_j act(U_j x)  +  D_s act(U_s x)

With ``renorm`` off the weights are the chosen scores themselves, and ``route_scale`` multiplies them either way.  A
``gated`` expert has a second input matrix G_j and computes D_j (act(G_j x) * (U_j x)).  With ``score`` = ``sigmoid`` the
scores are sigmoid(W_r x), each on its own.  With ``weight_on`` = ``input`` a weight multiplies what its expert reads,
y = sum_j expert_j(w_j x), which is not the same for an expert that is not linear.  With ``shared_gate`` the shared
expert's result is multiplied by sigmoid(g . x), one learned vector g and one number per token.

The router's matrix is held in float32 and its product, softmax and choice are one float32 kernel.  The experts' products are one
launch each way over all experts (tokens sorted by expert on the device, nothing read back), so a step with
routed layers launches the same kernels whatever the routing and can be recorded.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops import experts as ops
from yalis_b200.ops.elementwise import ACTIVATIONS, activation, silu_mul
from yalis_b200.ops.linear import linear
from .base import FeedForward, ParamSpec, register_part

_GROUPED_ACT = {"relu2": ops.ACT_RELU2, "none": ops.ACT_NONE}


class RoutedExperts(FeedForward):
    """Parameters: ``hidden_size``, ``experts``, ``top``, ``expert_size`` (inner size of an expert), ``activation``
    (``relu2``: the square of relu; ``silu`` with ``gated``), ``gated`` (experts of the form down(act(gate x) * (up x));
    default False), ``shared_size`` (inner size of the shared expert; None: none), ``renorm`` (divide the chosen scores by
    their sum; default True), ``renorm_eps`` (added to that sum; default 1e-20), ``route_scale`` (a factor on every
    weight; default 1), ``score`` (``softmax``, the default, or ``sigmoid``), ``weight_on`` (``output``, the default, or
    ``input``), ``shared_gate`` (default False)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden, self.n_experts, self.top = int(p["hidden_size"]), int(p["experts"]), int(p["top"])
        self.inner = int(p["expert_size"])
        self.act = str(p.get("activation", "relu2"))
        self.shared = int(p["shared_size"]) if p.get("shared_size") is not None else None
        self.eps = float(p.get("renorm_eps", 1e-20)) if bool(p.get("renorm", True)) else None
        self.route_scale = float(p.get("route_scale", 1.0))
        self.gated = bool(p.get("gated", False))
        self.score = str(p.get("score", "softmax"))
        self.weight_on = str(p.get("weight_on", "output"))
        self.shared_gate = bool(p.get("shared_gate", False))
        if self.score not in ("softmax", "sigmoid") or self.weight_on not in ("output", "input"):
            raise ValueError(f"score {self.score!r} / weight_on {self.weight_on!r}: softmax or sigmoid, output or input")
        if self.shared_gate and self.shared is None:
            raise ValueError("a gate on the shared expert needs a shared expert")
        if self.gated:
            if self.act != "silu":
                raise ValueError(f"a gated expert's activation is silu, not {self.act!r}")
        elif self.act not in _GROUPED_ACT or self.act not in ACTIVATIONS:
            raise ValueError(f"activation {self.act!r} is not one the routed feed-forward has ({', '.join(_GROUPED_ACT)})")
        if not 0 < self.top <= min(self.n_experts, ops.MAX_TOP) or self.n_experts > ops.MAX_EXPERTS:
            raise ValueError(f"top {self.top} of {self.n_experts} experts is not supported "
                             f"(top <= {ops.MAX_TOP}, experts <= {ops.MAX_EXPERTS})")
        self.router: Optional[torch.Tensor] = None
        self.w_up = self.w_down = self.s_up = self.s_down = self.s_gate = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"router": ParamSpec((self.n_experts, self.hidden), keep_float32=True)}
        for i in range(self.n_experts):
            if self.gated:
                specs[f"expert_{i}_gate"] = ParamSpec((self.inner, self.hidden))
            specs[f"expert_{i}_up"] = ParamSpec((self.inner, self.hidden))
            specs[f"expert_{i}_down"] = ParamSpec((self.hidden, self.inner))
        if self.shared is not None:
            if self.gated:
                specs["shared_gate_proj"] = ParamSpec((self.shared, self.hidden))
            specs["shared_up"] = ParamSpec((self.shared, self.hidden))
            specs["shared_down"] = ParamSpec((self.hidden, self.shared))
        if self.shared_gate:
            specs["shared_gate"] = ParamSpec((1, self.hidden), keep_float32=True)
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.router = t["router"].float().contiguous()
        if self.gated:      # per expert the gate's rows, then the up-projection's: one product, then silu(gate) * up
            self.w_up = torch.stack([torch.cat([t[f"expert_{i}_gate"], t[f"expert_{i}_up"]], dim=0)
                                     for i in range(self.n_experts)]).contiguous()
        else:
            self.w_up = torch.stack([t[f"expert_{i}_up"] for i in range(self.n_experts)]).contiguous()
        self.w_down = torch.stack([t[f"expert_{i}_down"] for i in range(self.n_experts)]).contiguous()
        if self.shared is not None:
            self.s_up, self.s_down = t["shared_up"].contiguous(), t["shared_down"].contiguous()
            if self.gated:
                self.s_up = torch.cat([t["shared_gate_proj"], t["shared_up"]], dim=0).contiguous()
        if self.shared_gate:
            self.s_gate = t["shared_gate"].float().reshape(-1).contiguous()

    def capture_key(self, host):
        return None

    def matrix_flops_per_token(self) -> float:
        # the products a token runs: the router, ``top`` experts and the shared one
        per = 3 if self.gated else 2
        return 2.0 * self.hidden * (self.n_experts + per * self.top * self.inner + per * (self.shared or 0))

    def expected_unused_bytes(self, tokens: int) -> float:
        """Bytes of the experts that a step of ``tokens`` tokens is expected to leave unread when every choice is
        uniformly random (for rooflines)."""
        unused = self.n_experts * (1.0 - self.top / self.n_experts) ** tokens
        return unused * (self.w_up[0].numel() + self.w_down[0].numel()) * self.w_up.element_size()

    def _aligned(self, x: torch.Tensor) -> bool:
        return (x.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.inner % 8 == 0 and x.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0)

    def row_tile(self, x: torch.Tensor, wstream: bool) -> int:
        """Rows of a tile of the experts' products, from the step's shape alone.  tcgen05 form: the smallest of 16 ... 256
        that holds twice the rows an expert gets on average (a tile is the N side of the MMA: a half-empty one costs
        nothing where the weights set the pace, and few experts then need a second tile).  mma form: 128 when an
        expert gets about that many, 16 when at most 8, else 32.  The float32 form has tiles of 32."""
        entries = x.shape[0] * self.top
        if wstream:
            for tile in ops.WSTREAM_TILES:
                if 2 * entries <= tile * self.n_experts:
                    return tile
            return ops.WSTREAM_TILES[-1]
        if not self._aligned(x):
            return 32
        return 128 if entries >= 96 * self.n_experts else (16 if entries <= 8 * self.n_experts else 32)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        routed = ops.route(x, self.router, self.top, self.eps, ctx.req_of_token if ctx is not None else None,
                           factor=self.route_scale, score=self.score, side=self.s_gate)
        ids, weights = routed[0], routed[1]
        shared_scale = routed[2] if self.shared_gate else None
        on_input = self.weight_on == "input"
        act = ops.ACT_NONE if self.gated else _GROUPED_ACT[self.act]
        wstream = self._aligned(x) and ops.wstream_form(x, self.w_up)
        plan = ops.expert_plan(ids, self.n_experts, self.row_tile(x, wstream))
        if wstream:
            # the rows in slot order, each times its choice's weight where the weight belongs to the input
            rows = ops.gather_scale_rows(x, plan, self.top, weights) if on_input else ops.gather_rows(x, plan, self.top)
            inner = ops.grouped_gemm_wstream(rows, self.w_up, plan, act=act)
            if self.gated:
                inner = silu_mul(inner)
            y = ops.grouped_gemm_wstream(inner, self.w_down, plan)
        else:
            if on_input:
                inner = ops.grouped_gemm(ops.gather_scale_rows(x, plan, self.top, weights), self.w_up, plan, act=act)
            else:
                inner = ops.grouped_gemm(x, self.w_up, plan, gather_top=self.top, act=act)
            if self.gated:
                inner = silu_mul(inner)
            y = ops.grouped_gemm(inner, self.w_down, plan)
        shared = None
        if self.shared is not None:
            hidden = linear(x, self.s_up)
            shared = linear(silu_mul(hidden) if self.gated else activation(hidden, self.act), self.s_down)
        return ops.expert_combine(y, plan, None if on_input else weights, shared, top=self.top, shared_scale=shared_scale)


register_part("feed_forward", "routed_experts", RoutedExperts)
