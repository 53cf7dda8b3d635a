"""A residual stream kept in several copies, and the arrangement of a pre-norm layer around it.

``hyper_connection`` (category ``connection``): a sub-layer reads u = sum_s in_s x_s and its result y is written to
all copies at once, x_t <- sum_s mix[s, t] x_s + out_t y.  Before the write y may be multiplied, element by element,
by a learned vector (``layer_scale``) and by a gate sigmoid(W_g h + b_g) computed from what the sub-layer read
(``gate``).  With one copy and no mixing this is the plain residual sum with those two factors.

``pre_norm_connected`` (category ``block``): x <- write_1(mixer(norm_1(read_1 x))), then the same with the
feed-forward, if the layer has one.  The norm reads the copies, applies the pending write of the sub-layer before
and norms in one pass (``ops/streams.stream_step``).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.linear import linear
from yalis_b200.ops.streams import MAX_COPIES
from .base import Block, Connection, ParamSpec, PendingWrite, ResidualStream, register_part


class HyperConnection(Connection):
    """Parameters: ``hidden_size``, ``copies`` (of the stream), ``mixing`` (bool: learned read weights, write weights
    and a matrix that mixes the copies; False: the plain sum), ``layer_scale`` (bool), ``gate`` (bool)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden, self.copies = int(p["hidden_size"]), int(p.get("copies", 1))
        self.mixing = bool(p.get("mixing", self.copies > 1))
        self.has_scale, self.has_gate = bool(p.get("layer_scale", False)), bool(p.get("gate", False))
        if not 1 <= self.copies <= MAX_COPIES:
            raise ValueError(f"a stream has 1 to {MAX_COPIES} copies, not {self.copies}")
        if self.copies > 1 and not self.mixing:
            raise ValueError("a stream of several copies needs the mixing weights")
        self.w_in = self.w_out = self.mix = self.scale = self.gate_w = self.gate_b = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        s, specs = self.copies, {}
        if self.mixing:
            specs["in"] = ParamSpec((s,), init=f"const:{1.0 / s}", keep_float32=True)
            specs["out"] = ParamSpec((s,), init="ones", keep_float32=True)
            specs["mix"] = ParamSpec((s, s), init="identity", keep_float32=True)
        if self.has_scale:
            specs["scale"] = ParamSpec((self.hidden,), init="ones", keep_float32=True)
        if self.has_gate:
            specs["gate"] = ParamSpec((self.hidden, self.hidden))
            specs["gate_bias"] = ParamSpec((self.hidden,), init="zeros", keep_float32=True)
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        if self.mixing:
            self.w_in, self.w_out, self.mix = t["in"].contiguous(), t["out"].contiguous(), t["mix"].contiguous()
        if self.has_scale:
            self.scale = t["scale"].contiguous()
        if self.has_gate:
            self.gate_w, self.gate_b = t["gate"].contiguous(), t["gate_bias"].contiguous()

    def read_weights(self) -> Optional[torch.Tensor]:
        return self.w_in

    def write(self, h: torch.Tensor, y: torch.Tensor) -> PendingWrite:
        gate = linear(h, self.gate_w) if self.has_gate else None
        return PendingWrite(y, gate=gate, gate_bias=self.gate_b, layer_scale=self.scale, mix=self.mix, out_weights=self.w_out)

    def matrix_flops_per_token(self) -> float:
        return 2.0 * self.hidden * self.hidden if self.has_gate else 0.0

    def capture_key(self, host):
        return None


class PreNormConnectedBlock(Block):
    """h = norm_1(read_1(x)); x <- write_1(h, mixer(h)); h = norm_2(read_2(x)); x <- write_2(h, feed_forward(h)).
    Reads and writes are the layer's ``connection`` parts; the norms must read a stream of several copies with
    weights (``forward(stream, rows, in_weights=)``).  A layer may leave out the position part and the feed-forward
    with its norm and connection."""

    slots = {"position": "position", "norm_1": "norm", "mixer": "mixer", "connection_1": "connection",
             "norm_2": "norm", "feed_forward": "feed_forward", "connection_2": "connection"}
    optional = ("position", "norm_2", "feed_forward", "connection_2")

    def __init__(self, spec, parts):
        super().__init__(spec, parts)
        present = [n in self.parts for n in ("norm_2", "feed_forward", "connection_2")]
        if any(present) != all(present):
            raise ValueError("a connected pre-norm block has a feed-forward with its norm and connection, or none of them")

    @staticmethod
    def _read(norm, stream: ResidualStream, connection: Connection) -> torch.Tensor:
        weights = connection.read_weights()
        return norm.forward(stream) if weights is None else norm.forward(stream, in_weights=weights)

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        h = self._read(self.norm_1, stream, self.connection_1)
        stream.add(self.connection_1.write(h, self.mixer.forward(h, ctx, cache)))
        if "feed_forward" in self.parts:
            h = self._read(self.norm_2, stream, self.connection_2)
            stream.add(self.connection_2.write(h, self.feed_forward.forward(h, ctx)))


register_part("connection", "hyper_connection", HyperConnection)
register_part("block", "pre_norm_connected", PreNormConnectedBlock)
