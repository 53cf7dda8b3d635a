"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)) (yalis/external/model.py:710-744).

gate and up are stored as one matrix [Wgate; Wup] so that one product feeds the
activation kernel (the reference interleaves their rows instead, model.py:741).

With ``activation`` = ``clamped`` the gate is bounded from above and the up part from both sides before they meet:
g <- min(g, limit), u <- clamp(u, -limit, limit), y = g * sigmoid(alpha g) * (u + shift).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.elementwise import GATED_CLAMPED, gated_activation
from yalis_b200.ops.linear import linear, linear_partial, linear_silu_mul
from .base import FeedForward, ParamSpec, register_part


class SwiGLU(FeedForward):
    """Parameters: ``hidden_size``, ``intermediate_size``, ``activation`` (``silu``, the default, or ``clamped`` with
    ``limit``, ``alpha`` and ``shift``)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.act = str(spec.params.get("activation", "silu"))
        if self.act not in ("silu", "clamped"):
            raise ValueError(f"unknown gated activation {self.act!r} (silu or clamped)")
        if self.act == "clamped":
            self.limit, self.alpha, self.shift = (float(spec.params[k]) for k in ("limit", "alpha", "shift"))
            if not self.limit > 0:
                raise ValueError("the limit of a clamped activation must be positive")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "gate_proj": ParamSpec((self.inter, self.hidden)),
            "up_proj": ParamSpec((self.inter, self.hidden)),
            "down_proj": ParamSpec((self.hidden, self.inter)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj"], tensors["up_proj"]], dim=0).contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        if self.act == "clamped":
            inner = gated_activation(linear(x, self.w_gate_up), 0, self.inter, self.inter, kind=GATED_CLAMPED, limit=self.limit,
                                     alpha=self.alpha, shift=self.shift)
            return linear_partial(inner, self.w_down)
        return linear_partial(linear_silu_mul(x, self.w_gate_up), self.w_down)

    def capture_key(self, host):
        return None


register_part("feed_forward", "swiglu", SwiGLU)
