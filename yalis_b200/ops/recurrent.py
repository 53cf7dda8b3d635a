"""Wrappers of the kernels for mixers that keep a matrix per head (csrc/recurrent.cu).

The per-request memory of such a mixer is one row of float32 numbers in the slot
memory of the cache manager; ``StateLayout`` says where in the row the state matrices
and the convolution's tail lie.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ._lib import check, dtype_code, f32, i32, i64, lib, need, need_cuda, ptr, stream

DECAY_CONSTANT, DECAY_PER_TOKEN, DECAY_PER_CHANNEL = 0, 1, 2
GATE_NONE, GATE_SILU, GATE_SIGMOID = 0, 1, 2


@dataclass(frozen=True)
class StateLayout:
    """A slot row of a state-keeping mixer: ``heads * vdim * dim_padded`` floats of state (per head a
    matrix [vdim, dim_padded], the rows over ``dim`` padded to a multiple of four), then the
    convolution's tail ``[channels, taps - 1]`` (nothing when there is no convolution)."""

    heads: int
    dim: int
    vdim: int
    conv_channels: int = 0
    taps: int = 0

    @property
    def dim_padded(self) -> int:
        return -(-self.dim // 4) * 4

    @property
    def state_floats(self) -> int:
        return self.heads * self.vdim * self.dim_padded

    @property
    def tail_floats(self) -> int:
        return self.conv_channels * max(self.taps - 1, 0)

    @property
    def total(self) -> int:
        return -(-(self.state_floats + self.tail_floats) // 4) * 4


def _index_arrays(name, n, req_of_token, q_start, slots):
    need(req_of_token.dtype == torch.int32 and req_of_token.shape == (n,) and req_of_token.is_contiguous(), name,
         "req_of_token must be int32 [N]")
    need(q_start.dtype == torch.int32 and q_start.dim() == 1 and q_start.is_contiguous(), name, "q_start must be int32 [R + 1]")
    need(slots.dtype == torch.int32 and slots.shape == (q_start.numel() - 1,) and slots.is_contiguous(), name,
         "slots must be int32 [R]")


def delta_prepare(x: torch.Tensor, weight: torch.Tensor, slot_rows: torch.Tensor, tail_offset: int,
                  req_of_token: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, *, unit_heads: int = 0,
                  dim: int = 0, q_scale: float = 1.0, unit_eps: float = 1e-6, a_raw: Optional[torch.Tensor] = None,
                  a_log: Optional[torch.Tensor] = None, dt_bias: Optional[torch.Tensor] = None,
                  b_raw: Optional[torch.Tensor] = None):
    """What a delta rule reads, in one kernel: silu of a causal convolution over time, per channel, continuing each
    request from the tail its slot keeps; the heads of q and k brought to unit length; decay and write strength.

    ``x`` [N, C] (a column block of a wider matrix is fine), ``weight`` float32 [C, taps] with the current token's
    tap last, ``slot_rows`` float32 [slots, row] with the tail [C, taps - 1] at ``tail_offset`` of each row.  With
    ``unit_heads`` = G > 0 the first 2 G ``dim`` channels are G heads of q and G of k: each becomes
    x / sqrt(sum x^2 + unit_eps), q times ``q_scale``.  With ``a_raw`` ([N, heads] or [N, heads * dim]), ``a_log``
    [heads], ``dt_bias`` (one per column of a_raw) and ``b_raw`` [N, heads]: g = exp(-exp(a_log) softplus(a_raw +
    dt_bias)) and beta = sigmoid(b_raw).  Returns (float32 [N, C], g, beta), g and beta float32 or None; afterwards
    the tails hold the last ``taps - 1`` inputs of every request."""
    name = "delta_prepare"
    need_cuda(name, x, weight, slot_rows, req_of_token, q_start, slots, a_raw, a_log, dt_bias, b_raw)
    need(x.dim() == 2 and x.stride(1) == 1, name, "x must be [N, C] with unit inner stride")
    n, c = x.shape
    need(weight.dtype == torch.float32 and weight.dim() == 2 and weight.shape[0] == c and weight.is_contiguous(), name,
         "weight must be contiguous float32 [C, taps]")
    taps = weight.shape[1]
    need(1 <= taps <= 16, name, f"{taps} taps are not supported (1 to 16)")
    need(slot_rows.dtype == torch.float32 and slot_rows.dim() == 2 and slot_rows.is_contiguous()
         and tail_offset + c * (taps - 1) <= slot_rows.shape[1], name, "slot rows must be float32 [slots, row] that hold the tail")
    need(unit_heads == 0 or (dim > 0 and 2 * unit_heads * dim <= c), name, "the heads of q and k must lie within the channels")
    _index_arrays(name, n, req_of_token, q_start, slots)
    out = torch.empty((n, c), dtype=torch.float32, device=x.device)
    g = beta = None
    heads = a_cols = 0
    if a_raw is not None:
        need(a_log is not None and dt_bias is not None and b_raw is not None, name, "a_raw comes with a_log, dt_bias and b_raw")
        heads = a_log.numel()
        need(a_raw.dim() == 2 and a_raw.shape[0] == n and a_raw.stride(1) == 1 and a_raw.dtype == x.dtype
             and a_raw.shape[1] % heads == 0, name, "a_raw must be [N, heads] or [N, heads * dim] in the dtype of x")
        a_cols = a_raw.shape[1]
        need(a_log.dtype == torch.float32 and a_log.is_contiguous() and dt_bias.dtype == torch.float32
             and dt_bias.shape == (a_cols,) and dt_bias.is_contiguous(), name, "a_log float32 [heads], dt_bias float32 per column of a_raw")
        need(b_raw.shape == (n, heads) and b_raw.stride(1) == 1 and b_raw.dtype == x.dtype, name, "b_raw must be [N, heads] in the dtype of x")
        g = torch.empty((n, a_cols), dtype=torch.float32, device=x.device)
        beta = torch.empty((n, heads), dtype=torch.float32, device=x.device)
    tail = slot_rows.view(-1)[tail_offset:]
    check(lib().yalis_delta_prepare(
        ptr(x), i32(dtype_code(x.dtype)), i32(x.stride(0)), ptr(weight), ptr(tail), i64(slot_rows.stride(0)),
        ptr(req_of_token), ptr(q_start), ptr(slots), ptr(out), i32(c), i32(n), i32(slots.numel()), i32(c), i32(taps),
        i32(unit_heads), i32(dim), f32(q_scale), f32(unit_eps), ptr(a_raw), i32(a_raw.stride(0) if a_raw is not None else 0),
        i32(a_cols), ptr(a_log), ptr(dt_bias), ptr(b_raw), i32(b_raw.stride(0) if b_raw is not None else 0), i32(heads),
        ptr(g), ptr(beta), stream()), name)
    return out, g, beta


def short_conv_silu(x: torch.Tensor, weight: torch.Tensor, slot_rows: torch.Tensor, tail_offset: int,
                    req_of_token: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """The convolution of ``delta_prepare`` alone: float32 [N, C]."""
    return delta_prepare(x, weight, slot_rows, tail_offset, req_of_token, q_start, slots)[0]


def state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, slot_rows: torch.Tensor, layout: StateLayout,
               q_start: torch.Tensor, slots: torch.Tensor, *, kv_heads: int, decay: torch.Tensor,
               beta: Optional[torch.Tensor] = None, unit: Optional[torch.Tensor] = None,
               removal: Optional[torch.Tensor] = None, max_q_len: int = 0) -> torch.Tensor:
    """Walks every request's tokens in order through the recurrence, from and to the state in its slot.

    Per head (S is [dim, vdim]):  S <- g S;  u = beta (v - S^T k) with ``beta`` (the delta rule), else u = v;
    S <- S + k u^T;  o = S^T q.  ``q``, ``k`` float32 [N, kv_heads * dim], ``v`` float32 [N, heads * vdim] (column
    blocks are fine).  ``decay`` float32: [heads] (constant), [N, heads] (per token) or [N, heads * dim] (per key
    channel too); ``beta`` float32 [N, heads].  With ``unit`` and ``removal`` (float32 [N, heads * dim]) the rule is the generalized delta rule instead:
    S <- diag(g) S - removal (unit^T S) + k v^T, both terms reading the old state; it needs a decay per key channel
    and kv_heads = heads, and ``decay``, ``unit``, ``removal`` contiguous.  ``max_q_len``: the longest portion of the step if known (it bounds
    the tile of tokens staged in shared memory, nothing else).  Returns float32 [N, heads * vdim]."""
    name = "state_scan"
    need_cuda(name, q, k, v, slot_rows, q_start, slots, decay, beta)
    h, d, vd = layout.heads, layout.dim, layout.vdim
    n = q.shape[0]
    for t, width, what in ((q, kv_heads * d, "q"), (k, kv_heads * d, "k"), (v, h * vd, "v")):
        need(t.dtype == torch.float32 and t.dim() == 2 and t.shape == (n, width) and t.stride(1) == 1, name,
             f"{what} must be float32 [N, {width}] with unit inner stride")
    need(h % kv_heads == 0, name, "heads must be a multiple of kv_heads")
    need(slot_rows.dtype == torch.float32 and slot_rows.dim() == 2 and slot_rows.is_contiguous()
         and slot_rows.shape[1] >= layout.state_floats and slot_rows.stride(0) % 4 == 0, name,
         "slot rows must be float32 [slots, row], rows a multiple of four floats that hold the state")
    need(q_start.dtype == torch.int32 and slots.dtype == torch.int32 and slots.numel() == q_start.numel() - 1, name,
         "q_start int32 [R + 1], slots int32 [R]")
    need(decay.dtype == torch.float32 and decay.is_contiguous(), name, "decay must be contiguous float32")
    if decay.dim() == 1:
        need(decay.shape == (h,), name, "a constant decay has one entry per head")
        kind = DECAY_CONSTANT
    else:
        need(decay.shape in ((n, h), (n, h * d)), name, "decay must be [heads], [N, heads] or [N, heads * dim]")
        kind = DECAY_PER_TOKEN if decay.shape[1] == h else DECAY_PER_CHANNEL
    if beta is not None:
        need(beta.dtype == torch.float32 and beta.shape == (n, h) and beta.is_contiguous(), name, "beta must be float32 [N, heads]")
    rule = 1 if beta is not None else 0
    if unit is not None or removal is not None:
        need(beta is None and unit is not None and removal is not None and kind == DECAY_PER_CHANNEL and kv_heads == h, name,
             "the generalized rule takes unit keys and removal vectors, a decay per key channel, kv_heads = heads and no beta")
        for t, what in ((unit, "unit"), (removal, "removal")):
            need(t.dtype == torch.float32 and t.shape == (n, h * d) and t.is_contiguous(), name,
                 f"{what} must be contiguous float32 [N, heads * dim]")
        rule = 2
    out = torch.empty((n, h * vd), dtype=torch.float32, device=q.device)
    check(lib().yalis_state_scan(
        ptr(q), i32(q.stride(0)), ptr(k), i32(k.stride(0)), ptr(v), i32(v.stride(0)), ptr(decay), i32(kind), ptr(beta),
        ptr(unit), ptr(removal), ptr(slot_rows), i64(slot_rows.stride(0)), ptr(out), i32(out.stride(0)), ptr(q_start), ptr(slots),
        i32(slots.numel()), i32(h), i32(kv_heads), i32(d), i32(vd), i32(rule), i32(max_q_len), stream()), name)
    return out


def head_norm_gate(o: torch.Tensor, heads: int, vdim: int, eps: float, req_of_token: torch.Tensor,
                   out: torch.Tensor, weight: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                   gate_kind: int = GATE_NONE, out_scale: float = 1.0) -> torch.Tensor:
    """out[n, h, :] = o / sqrt(mean(o^2) + eps) * weight * act(gate[n, h, :]) * out_scale, per token and head.

    ``o`` float32 [N, heads * vdim]; ``weight`` float32 [vdim] or None; ``gate`` [N, heads * vdim] in the dtype
    of ``out`` with silu or sigmoid applied; ``out`` [N, heads * vdim] (a column block of a wider matrix is fine)."""
    name = "head_norm_gate"
    need_cuda(name, o, req_of_token, out, weight, gate)
    n = o.shape[0]
    need(o.dtype == torch.float32 and o.shape == (n, heads * vdim) and o.stride(1) == 1, name, "o must be float32 [N, heads * vdim]")
    need(out.shape == (n, heads * vdim) and out.stride(1) == 1, name, "out must be [N, heads * vdim] with unit inner stride")
    per_head = False
    if weight is not None:
        need(weight.dtype == torch.float32 and weight.shape in ((vdim,), (heads * vdim,)) and weight.is_contiguous(), name,
             "weight must be float32 [vdim] or [heads * vdim]")
        per_head = weight.shape == (heads * vdim,) and heads > 1
    if gate_kind != GATE_NONE:
        need(gate is not None and gate.shape == (n, heads * vdim) and gate.stride(1) == 1 and gate.dtype == out.dtype, name,
             "gate must be [N, heads * vdim] in the output's dtype")
    check(lib().yalis_head_norm_gate(ptr(o), i32(o.stride(0)), ptr(weight), ptr(gate),
                                     i32(gate.stride(0) if gate is not None else 0), i32(gate_kind), ptr(out),
                                     i32(out.stride(0)), i32(dtype_code(out.dtype)), ptr(req_of_token), i32(n), i32(heads),
                                     i32(vdim), f32(eps), f32(out_scale), i32(int(per_head)), stream()), name)
    return out


def general_delta_prepare(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a_raw: torch.Tensor, a_bias: torch.Tensor,
                          w_raw: torch.Tensor, w_bias: torch.Tensor, heads: int, dim: int, rate: float, unit_eps: float,
                          req_of_token: torch.Tensor):
    """What the generalized delta rule reads, six contiguous float32 matrices [N, heads * dim]:
    (q, k, v, decay, unit, removal) with decay = exp(-rate * sigmoid(w_raw + w_bias)), unit = k / sqrt(sum k^2 +
    unit_eps) per head and removal = sigmoid(a_raw + a_bias) * unit.  ``q``, ``k``, ``v`` [N, heads * dim] are column
    blocks of one matrix (one row stride) in the model's dtype, ``a_raw`` and ``w_raw`` [N, heads * dim] in that dtype
    too; the biases are float32 [heads * dim]."""
    name = "general_delta_prepare"
    need_cuda(name, q, k, v, a_raw, a_bias, w_raw, w_bias, req_of_token)
    n, width = q.shape[0], heads * dim
    for t in (q, k, v, a_raw, w_raw):
        need(t.dim() == 2 and t.shape == (n, width) and t.stride(1) == 1 and t.dtype == q.dtype, name,
             f"q, k, v, a_raw, w_raw must be [N, {width}] of one dtype with unit inner stride")
    need(q.stride(0) == k.stride(0) == v.stride(0), name, "q, k, v must share a row stride")
    for t in (a_bias, w_bias):
        need(t.dtype == torch.float32 and t.shape == (width,) and t.is_contiguous(), name, "biases must be float32 [heads * dim]")
    need(req_of_token.dtype == torch.int32 and req_of_token.shape == (n,), name, "req_of_token must be int32 [N]")
    out = torch.empty((6, n, width), dtype=torch.float32, device=q.device)
    check(lib().yalis_general_delta_prepare(ptr(q), ptr(k), ptr(v), i32(q.stride(0)), ptr(a_raw), i32(a_raw.stride(0)), ptr(a_bias),
                                            ptr(w_raw), i32(w_raw.stride(0)), ptr(w_bias), f32(rate), f32(unit_eps),
                                            ptr(req_of_token), i32(n), i32(heads), i32(dim), i32(dtype_code(q.dtype)), ptr(out),
                                            stream()), name)
    return tuple(out[i] for i in range(6))
