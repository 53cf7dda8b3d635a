"""What joins the token rows as they enter the stream.

``pair_table``  a row of a table chosen by a token and the one before it: row (previous * mul_prev + token * mul_cur)
                mod buckets; the first token of a sequence takes the table's last row (number ``buckets``).  The
                previous token of a portion's first token is part of the request's state: one int32 per request slot.
"""

from __future__ import annotations

from typing import Dict

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.streams import pair_rows_add, remember_last_tokens
from .base import Entry, ParamSpec, SlotState, SlotStateCache, register_part


class PairTable(Entry):
    """Parameters: ``hidden_size``, ``vocab_size``, ``buckets``, ``mul_prev``, ``mul_cur``."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden, self.vocab, self.buckets = int(p["hidden_size"]), int(p["vocab_size"]), int(p["buckets"])
        self.mul_prev, self.mul_cur = int(p["mul_prev"]), int(p["mul_cur"])
        if self.buckets <= 0:
            raise ValueError("a pair table needs at least one bucket")
        self.table = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"table": ParamSpec((self.buckets + 1, self.hidden))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.table = t["table"].contiguous()

    def cache_request(self) -> SlotState:
        return SlotState((1,), torch.int32)

    def forward(self, x: torch.Tensor, ctx, cache: SlotStateCache) -> None:
        from_slot = ctx.token_from_slot
        chosen = ctx.chosen if from_slot is not None else None
        last = cache.state.view(-1)
        pair_rows_add(x, self.table, self.buckets, self.mul_prev, self.mul_cur, ctx.token_ids, ctx.positions,
                      ctx.req_of_token, ctx.q_start, ctx.slots, last, self.vocab, from_slot=from_slot, chosen=chosen)
        remember_last_tokens(ctx.token_ids, ctx.q_start, ctx.slots, last, from_slot=from_slot, chosen=chosen)

    def matrix_flops_per_token(self) -> float:
        return 0.0

    def capture_key(self, host):
        return None


register_part("entry", "pair_table", PairTable)
