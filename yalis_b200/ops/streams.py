"""Wrappers of csrc/streams.cu: the step between two sub-layers of a residual stream kept in one or several copies
(write of a sub-layer's result, read and norm for the next), and the embedding rows chosen by pairs of tokens."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from ._lib import check, dtype_code, i32, i64, lib, need, need_cuda, ptr, stream

MAX_COPIES = 8


def stream_step(x: torch.Tensor, *, y: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                gate_bias: Optional[torch.Tensor] = None, layer_scale: Optional[torch.Tensor] = None,
                mix: Optional[torch.Tensor] = None, out_weights: Optional[torch.Tensor] = None,
                in_weights: Optional[torch.Tensor] = None,
                norm: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
                rows: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                read: bool = True, source: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One pass over the stream ``x`` float32 [N, S, D] (S copies; [N, D] counts as one copy).

    Write, when ``y`` is given ([N, D] in float32 or bfloat16, or float32 partial sums [P, N, D] added in order):
    y <- y * layer_scale * sigmoid(gate + gate_bias) (each factor optional; ``gate`` [N, D] float32 or bfloat16), then
    x_t <- sum_s mix[s, t] x_s + out_weights[t] y for all copies from the old ones (without ``mix``: x_t += y).
    Read, when ``read``: u = sum_s in_weights[s] x_s (without ``in_weights``: the sum), h = tanh(alpha u) w + b with
    ``norm`` = (alpha [1], w [D], b [D]), else h = u; returned as [N, D] in ``out_dtype``.

    With ``rows`` (int32 row indices, -1: skip) only those rows are read, into [len(rows), D], and the written copies are
    not stored: the stream stays as it was.

    ``source`` float32 [N, D]: the stream's first pass.  ``x`` holds nothing yet; every copy of row n equals
    ``source[n]``, and (without ``rows``) the copies are stored to ``x`` whether or not there is a write."""
    name = "stream_step"
    need_cuda(name, x, y, gate, gate_bias, layer_scale, mix, out_weights, in_weights, rows, source, *(norm or ()))
    need(x.dtype == torch.float32 and x.dim() in (2, 3) and x.is_contiguous(), name, "x must be contiguous float32 [N, S, D] or [N, D]")
    n, d = x.shape[0], x.shape[-1]
    s = x.shape[1] if x.dim() == 3 else 1
    need(1 <= s <= MAX_COPIES, name, f"1 to {MAX_COPIES} copies of the stream")
    y_parts = y_part_stride = y_stride = 0
    if y is not None:
        need(y.stride(-1) == 1 and ((y.dim() == 2 and y.shape == (n, d) and y.dtype in (torch.float32, torch.bfloat16))
                                    or (y.dim() == 3 and y.shape[1:] == (n, d) and y.dtype == torch.float32)), name,
             "y must be [N, D] (float32 or bfloat16) or float32 partial sums [P, N, D]")
        y_parts = y.shape[0] if y.dim() == 3 else 1
        y_part_stride = y.stride(0) if y.dim() == 3 else 0
        y_stride = y.stride(-2)
    else:
        need(gate is None and layer_scale is None and mix is None, name, "gate, layer_scale and mix belong to a write")
    if gate is not None:
        need(gate.shape == (n, d) and gate.stride(1) == 1 and gate.dtype in (torch.float32, torch.bfloat16), name,
             "gate must be [N, D] float32 or bfloat16")
    for t, shape, what in ((gate_bias, (d,), "gate_bias"), (layer_scale, (d,), "layer_scale"), (mix, (s, s), "mix"),
                           (out_weights, (s,), "out_weights"), (in_weights, (s,), "in_weights")):
        need(t is None or (t.dtype == torch.float32 and tuple(t.shape) == shape and t.is_contiguous()), name,
             f"{what} must be contiguous float32 {list(shape)}")
    need((mix is None) == (out_weights is None), name, "mix and out_weights come together")
    need(gate_bias is None or gate is not None, name, "a gate bias needs a gate")
    alpha = w = b = None
    if norm is not None:
        alpha, w, b = norm
        need(alpha.dtype == torch.float32 and alpha.numel() == 1 and w.dtype == b.dtype == torch.float32
             and w.shape == b.shape == (d,) and w.is_contiguous() and b.is_contiguous(), name,
             "norm must be (alpha float32 [1], w float32 [D], b float32 [D])")
    if rows is not None:
        need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), name, "rows must be int32 [R]")
    count = n if rows is None else rows.numel()
    h = None
    if read:
        need(out_dtype in (torch.float32, torch.bfloat16), name, "the result is float32 or bfloat16")
        h = torch.empty((count, d), dtype=out_dtype, device=x.device)
    need(read or y is not None or source is not None, name, "nothing to do")
    need(source is None or (source.dtype == torch.float32 and source.shape == (n, d) and source.is_contiguous()), name,
         "source must be contiguous float32 [N, D]")
    check(lib().yalis_stream_step(
        ptr(x), i32(n), i32(s), i32(d), ptr(y), i32(y_parts), i64(y_part_stride), i64(y_stride),
        i32(int(y is not None and y.dtype == torch.float32)), ptr(gate), i64(gate.stride(0) if gate is not None else 0),
        ptr(gate_bias), i32(int(gate is not None and gate.dtype == torch.float32)), ptr(layer_scale), ptr(mix), ptr(out_weights),
        ptr(in_weights), ptr(alpha), ptr(w), ptr(b), ptr(rows), i32(0 if rows is None else rows.numel()), ptr(h),
        i64(h.stride(0) if h is not None else 0), i32(int(h is not None and h.dtype == torch.float32)), ptr(source), stream()), name)
    return h


def pair_rows_add(x: torch.Tensor, table: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int, ids: torch.Tensor,
                  positions: torch.Tensor, req_of_token: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
                  last_token: torch.Tensor, vocab: int, from_slot: Optional[torch.Tensor] = None,
                  chosen: Optional[torch.Tensor] = None) -> None:
    """x[n, :] += table[(previous * mul_prev + token * mul_cur) mod buckets, :] for every token of a request, in place
    (float32 [N, D]); a token at position 0 takes row ``buckets``, the table's last.  The token before a portion's
    first one is ``last_token[slot]`` (int32 per request slot, see ``remember_last_tokens``).  ``from_slot`` / ``chosen``
    as in the embedding: tokens that an earlier step chose and left on the device."""
    name = "pair_rows_add"
    need_cuda(name, x, table, ids, positions, req_of_token, q_start, slots, last_token, from_slot, chosen)
    n, d = x.shape
    need(x.dtype == torch.float32 and x.is_contiguous(), name, "x must be contiguous float32 [N, D]")
    need(table.dim() == 2 and table.shape == (buckets + 1, d) and table.is_contiguous(), name, "table must be contiguous [buckets + 1, D]")
    for t in (ids, positions, req_of_token):
        need(t.dtype == torch.int32 and t.shape == (n,) and t.is_contiguous(), name, "ids, positions, req_of_token: int32 [N]")
    need(q_start.dtype == slots.dtype == last_token.dtype == torch.int32 and slots.numel() == q_start.numel() - 1
         and last_token.is_contiguous(), name, "q_start int32 [R + 1], slots int32 [R], last_token int32 per slot")
    need((from_slot is None) == (chosen is None), name, "from_slot and chosen come together")
    check(lib().yalis_pair_rows_add(ptr(x), i32(n), i32(d), ptr(table), i32(dtype_code(table.dtype)), i32(buckets), i64(mul_prev),
                                    i64(mul_cur), ptr(ids), ptr(from_slot), ptr(chosen), ptr(positions), ptr(req_of_token),
                                    ptr(q_start), ptr(slots), ptr(last_token), i32(vocab), stream()), name)


def remember_last_tokens(ids: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, last_token: torch.Tensor,
                         from_slot: Optional[torch.Tensor] = None, chosen: Optional[torch.Tensor] = None) -> None:
    """last_token[slots[r]] = the last token request r brings in this step (requests without tokens keep theirs)."""
    name = "remember_last_tokens"
    need_cuda(name, ids, q_start, slots, last_token, from_slot, chosen)
    need(ids.dtype == q_start.dtype == slots.dtype == last_token.dtype == torch.int32 and slots.numel() == q_start.numel() - 1,
         name, "int32 arrays: ids [N], q_start [R + 1], slots [R], last_token per slot")
    check(lib().yalis_remember_last_tokens(ptr(ids), ptr(from_slot), ptr(chosen), ptr(q_start), ptr(slots), i32(slots.numel()),
                                           ptr(last_token), stream()), name)
