"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * weight, all in float32
(yalis/external/model.py:957-989), fused with the residual add before it."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.elementwise import add_normed_rmsnorm, add_rmsnorm
from .base import Norm, NormedSum, ParamSpec, PendingWrite, ResidualStream, register_part


class RMSNorm(Norm):
    """Parameters: ``size`` (width of the stream), ``eps``, ``one_plus`` (the stored tensor w lies around
    zero and the scale is 1 + w; default False: the tensor is the scale).  The scale is held in float32."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.one_plus = bool(spec.params.get("one_plus", False))
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), init="zeros" if self.one_plus else "ones", keep_float32=True)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors["weight"].contiguous()
        self.weight = (1.0 + w) if self.one_plus else w       # float32: the sum is exact to one rounding

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if stream.copies > 1:
            raise ValueError("rms_norm reads a stream of one copy")
        stream.materialize()
        if isinstance(stream.pending, PendingWrite):
            stream.flush()
        if isinstance(stream.pending, NormedSum):      # a result with a bias or a norm of its own: the same single pass
            pend = stream.pending
            y = add_normed_rmsnorm(stream.x, pend.y, bias=pend.bias, delta_norm=pend.norm, weight=self.weight, eps=self.eps,
                                   out_dtype=stream.dtype, rows=rows)
        else:
            y = add_rmsnorm(stream.x, stream.pending, self.weight, self.eps, stream.dtype, rows=rows)
        if rows is None:
            stream.pending = None   # the kernel has written x + delta back
        return y

    def normalize(self, y: torch.Tensor) -> torch.Tensor:
        # the same kernel over a zero stream with y as its pending delta: float32 math, one rounding
        zero = torch.zeros(y.shape, dtype=torch.float32, device=y.device)
        return add_rmsnorm(zero, y.contiguous(), self.weight, self.eps, y.dtype)

    def rms_parameters(self):
        return self.weight, self.eps

    def capture_key(self, host):
        return None


class DynamicTanh(Norm):
    """A norm without statistics: y = tanh(alpha x) * weight + bias with one learned number alpha, element by element.
    Parameters: ``size``.  All three tensors are held in float32.  It reads a stream of one copy or of several (the sum
    of the copies, after whatever write is pending), in the same pass that applies the pending write."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.alpha = self.weight = self.bias = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), init="ones", keep_float32=True),
                "alpha": ParamSpec((), init="const:0.5", keep_float32=True),
                "bias": ParamSpec((self.size,), init="zeros", keep_float32=True)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight, self.bias = tensors["weight"].contiguous(), tensors["bias"].contiguous()
        self.alpha = tensors["alpha"].reshape(1).contiguous()

    def triple(self):
        return (self.alpha, self.weight, self.bias)

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                in_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``in_weights`` [copies]: the weights of the copies in the sum that is normed (None: the plain sum)."""
        from yalis_b200.ops.streams import stream_step
        if isinstance(stream.pending, NormedSum):
            stream.flush()
        pending = stream.pending
        write = pending.arguments() if isinstance(pending, PendingWrite) else ({"y": pending} if pending is not None else {})
        h = stream_step(stream.x, norm=self.triple(), in_weights=in_weights, rows=rows, out_dtype=stream.dtype,
                        source=stream.take_source(stores=rows is None), **write)
        if rows is None:
            stream.pending = None   # the kernel has stored the written copies
        return h

    def normalize(self, y: torch.Tensor) -> torch.Tensor:
        from yalis_b200.ops.streams import stream_step
        return stream_step(y.float().contiguous(), norm=self.triple(), out_dtype=y.dtype)

    def capture_key(self, host):
        return None


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
