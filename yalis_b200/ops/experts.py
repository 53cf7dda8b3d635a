"""Wrappers of csrc/experts.cu: the kernels of a routed feed-forward (router, grouping by expert, one product
over all experts, weighted sum).  Nothing here reads the routing on the host."""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from ._lib import check, dtype_code, f32, i32, i64, lib, need, need_cuda, ptr, stream

MAX_EXPERTS, MAX_TOP = 1024, 32
ACT_NONE, ACT_RELU2 = 0, 1


def route_topk(logits: torch.Tensor, top: int, eps: Optional[float] = 1e-20, req_of_token: Optional[torch.Tensor] = None,
               factor: float = 1.0, score: str = "softmax"):
    """(ids int32 [N, top], weights float32 [N, top]): the ``top`` largest of softmax(logits) per row (ties to the
    smaller index) and those scores divided by their sum + eps (``eps`` None: the scores as they are), times
    ``factor``.  ``score`` = ``sigmoid``: the scores are sigmoid(logits), each on its own.  Rows of no request get
    ids -1."""
    name = "route_topk"
    need_cuda(name, logits, req_of_token)
    need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(), name, "logits must be contiguous float32 [N, E]")
    n, e = logits.shape
    need(0 < top <= min(e, MAX_TOP) and e <= MAX_EXPERTS, name, f"needs top <= min(E, {MAX_TOP}) and E <= {MAX_EXPERTS}")
    ids = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    check(lib().yalis_route_topk(ptr(logits), i32(n), i32(e), i32(top), f32(-1.0 if eps is None else eps), f32(factor), ptr(req_of_token), ptr(ids), ptr(weights),
                                 i32(_score_code(name, score)), stream()), name)
    return ids, weights


def _score_code(name: str, score: str) -> int:
    need(score in ("softmax", "sigmoid"), name, f"unknown score {score!r} (softmax or sigmoid)")
    return int(score == "sigmoid")


def route(x: torch.Tensor, router: torch.Tensor, top: int, eps: Optional[float] = 1e-20, req_of_token: Optional[torch.Tensor] = None,
          factor: float = 1.0, score: str = "softmax", side: Optional[torch.Tensor] = None):
    """``route_topk`` of the logits ``x router^T`` in one launch: ``x`` [N, K] (float32 or bfloat16, unit inner stride),
    ``router`` float32 [E, K].  The logits are float32 sums in a fixed order per (token, expert).  With ``side``
    (float32 [K]) a third result is returned: float32 [N], sigmoid(x . side), a gate per token from the same rows."""
    name = "route"
    need_cuda(name, x, router, req_of_token, side)
    side_out = None
    if side is not None:
        need(side.dtype == torch.float32 and side.shape == (x.shape[1],) and side.is_contiguous(), name, "side must be float32 [K]")
        side_out = torch.zeros(x.shape[0], dtype=torch.float32, device=x.device)
    need(x.dim() == 2 and x.stride(1) == 1 and router.dtype == torch.float32 and router.dim() == 2 and router.is_contiguous()
         and router.shape[1] == x.shape[1], name, "x [N, K], router contiguous float32 [E, K]")
    n, e = x.shape[0], router.shape[0]
    need(0 < top <= min(e, MAX_TOP) and e <= MAX_EXPERTS, name, f"needs top <= min(E, {MAX_TOP}) and E <= {MAX_EXPERTS}")
    ids = torch.empty((n, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=x.device)
    check(lib().yalis_route(ptr(x), i32(dtype_code(x.dtype)), i64(x.stride(0)), ptr(router), i32(n), i32(e), i32(x.shape[1]), i32(top),
                            f32(-1.0 if eps is None else eps), f32(factor), ptr(req_of_token), ptr(ids), ptr(weights),
                            i32(_score_code(name, score)), ptr(side), ptr(side_out), stream()), name)
    return (ids, weights) if side is None else (ids, weights, side_out)


@dataclass
class ExpertPlan:
    """The entries (token, choice) of a step sorted by expert: ``offsets`` [E + 1], ``perm`` slot -> entry, ``inv``
    entry -> slot (-1: none), and the row tiles (expert, first slot) of ``bm`` slots, ``n_tiles`` of them (at most
    ``max_tiles``, which only the shapes give)."""

    offsets: torch.Tensor
    perm: torch.Tensor
    inv: torch.Tensor
    tile_expert: torch.Tensor
    tile_slot: torch.Tensor
    n_tiles: torch.Tensor
    max_tiles: int
    bm: int
    entries: int


def expert_plan(ids: torch.Tensor, n_experts: int, bm: int) -> ExpertPlan:
    name = "expert_plan"
    need_cuda(name, ids)
    need(ids.dtype == torch.int32 and ids.dim() == 2 and ids.is_contiguous(), name, "ids must be contiguous int32 [N, top]")
    entries = ids.numel()
    max_tiles = entries // bm + min(n_experts, entries)
    buf = torch.empty(n_experts + 1 + 2 * entries + 2 * max_tiles + 1, dtype=torch.int32, device=ids.device)
    o = 0

    def take(count):
        nonlocal o
        view = buf[o:o + count]
        o += count
        return view

    plan = ExpertPlan(take(n_experts + 1), take(entries), take(entries), take(max_tiles), take(max_tiles), take(1),
                      max_tiles, bm, entries)
    check(lib().yalis_expert_plan(ptr(ids), i32(entries), i32(n_experts), i32(bm), ptr(plan.offsets), ptr(plan.perm),
                                  ptr(plan.inv), ptr(plan.tile_expert), ptr(plan.tile_slot), ptr(plan.n_tiles), stream()), name)
    return plan


def tensor_core_form(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the product takes the mma form: bfloat16, K a multiple of 8, rows on 16-byte boundaries."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, plan: ExpertPlan, *, gather_top: Optional[int] = None,
                 act: int = ACT_NONE, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[s, :] = act(A[row(s), :] . w[expert(s)]^T) for every slot s of the plan; row(s) = perm[s] // gather_top
    when ``gather_top`` is given (A holds one row per token), else s (A holds one row per slot).  ``w`` [E, n_out, K]."""
    name = "grouped_gemm"
    need_cuda(name, a, w, out)
    need(a.dim() == 2 and w.dim() == 3 and w.is_contiguous() and a.stride(1) == 1 and a.shape[1] == w.shape[2]
         and a.dtype == w.dtype, name, "A [rows, K], w [E, n_out, K] contiguous, one dtype")
    n_out, k = w.shape[1], w.shape[2]
    if out is None:
        out = torch.empty((plan.entries, n_out), dtype=a.dtype, device=a.device)
    need(out.shape == (plan.entries, n_out) and out.dtype == a.dtype and out.stride(1) == 1, name, "bad out tensor")
    tc = tensor_core_form(a, w) and plan.bm in (16, 32, 128)
    need(tc or plan.bm == 32, name, "the plan's row tile does not fit the kernel that takes these operands")
    check(lib().yalis_grouped_gemm(ptr(a), i64(a.stride(0)), ptr(plan.perm if gather_top else None), i32(gather_top or 1),
                                   ptr(w), ptr(out), i64(out.stride(0)), i32(dtype_code(a.dtype)), ptr(plan.offsets),
                                   ptr(plan.tile_expert), ptr(plan.tile_slot), ptr(plan.n_tiles), i32(plan.max_tiles),
                                   i32(n_out), i32(k), i32(act), i32(plan.bm), i32(1 if tc else 0), stream()), name)
    return out


WSTREAM_TILES = (16, 32, 64, 128, 256)      # row tiles of the tcgen05 form


def wstream_form(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the experts' product takes the tcgen05 form: bfloat16, K a multiple of 8, rows on 16-byte boundaries
    (``YALIS_B200_NO_GROUPED_TCGEN05=1`` keeps every product on the mma form)."""
    return os.environ.get("YALIS_B200_NO_GROUPED_TCGEN05", "0") != "1" and tensor_core_form(a, w)


def gather_rows(x: torch.Tensor, plan: ExpertPlan, top: int) -> torch.Tensor:
    """[entries, K]: row ``perm[slot] // top`` of ``x`` for every slot in use (bfloat16, K % 8 == 0)."""
    name = "gather_rows"
    need_cuda(name, x)
    need(x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
         and x.data_ptr() % 16 == 0, name, "x must be bfloat16 [N, K] with K % 8 == 0 and rows on 16-byte boundaries")
    out = torch.empty((plan.entries, x.shape[1]), dtype=x.dtype, device=x.device)
    check(lib().yalis_gather_rows(ptr(x), i64(x.stride(0)), ptr(plan.perm), i32(top), ptr(plan.offsets),
                                  i32(plan.offsets.numel() - 1), ptr(out), i32(plan.entries), i32(x.shape[1]), stream()), name)
    return out


def gather_scale_rows(x: torch.Tensor, plan: ExpertPlan, top: int, weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[entries, K]: row ``perm[slot] // top`` of ``x`` for every slot in use, times ``weights[perm[slot]]`` (float32
    [N, top]; None: as it is): what an expert reads when a choice's weight multiplies its input.  Any dtype."""
    name = "gather_scale_rows"
    need_cuda(name, x, weights)
    need(x.dim() == 2 and x.stride(1) == 1, name, "x must be [N, K] with unit inner stride")
    need(weights is None or (weights.dtype == torch.float32 and weights.is_contiguous() and weights.numel() == plan.entries), name,
         "weights must be contiguous float32 [N, top]")
    out = torch.empty((plan.entries, x.shape[1]), dtype=x.dtype, device=x.device)
    check(lib().yalis_gather_scale_rows(ptr(x), i64(x.stride(0)), i32(dtype_code(x.dtype)), ptr(plan.perm), i32(top), ptr(weights),
                                        ptr(plan.offsets), i32(plan.offsets.numel() - 1), ptr(out), i32(plan.entries),
                                        i32(x.shape[1]), stream()), name)
    return out


def grouped_gemm_wstream(a: torch.Tensor, w: torch.Tensor, plan: ExpertPlan, *, act: int = ACT_NONE) -> torch.Tensor:
    """C[s, :] = act(A[s, :] . w[expert(s)]^T) on tcgen05 tensor cores with TMA-streamed operands: ``a`` [entries, K]
    holds one row per slot (see ``gather_rows``), ``w`` [E, n_out, K]; the plan's row tile is one of ``WSTREAM_TILES``."""
    name = "grouped_gemm_wstream"
    need_cuda(name, a, w)
    need(a.dim() == 2 and w.dim() == 3 and w.is_contiguous() and a.shape == (plan.entries, w.shape[2]) and a.stride(1) == 1
         and tensor_core_form(a, w) and plan.bm in WSTREAM_TILES, name,
         "A bfloat16 [entries, K] in slot order, w bfloat16 [E, n_out, K], K % 8 == 0, a row tile the kernel has")
    out = torch.empty((plan.entries, w.shape[1]), dtype=a.dtype, device=a.device)
    from ._lib import error_word
    check(lib().yalis_grouped_gemm_wstream(ptr(a), i64(a.stride(0)), i32(plan.entries), ptr(w), i32(w.shape[0]), i32(w.shape[1]),
                                           i32(w.shape[2]), ptr(out), i64(out.stride(0)), ptr(plan.offsets), ptr(plan.tile_expert),
                                           ptr(plan.tile_slot), ptr(plan.n_tiles), i32(plan.max_tiles), i32(plan.bm), i32(act),
                                           ptr(error_word(a.device)), stream()), name)
    return out


def expert_combine(y: torch.Tensor, plan: ExpertPlan, weights: Optional[torch.Tensor], shared: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None, top: Optional[int] = None,
                   shared_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[n, :] = sum_j weights[n, j] * y[inv[n, j], :] (+ shared_scale[n] * shared[n, :]), float32 sums in the order of
    j.  ``weights`` None (then ``top`` says how many choices a token has): every choice counts once."""
    name = "expert_combine"
    need_cuda(name, y, weights, shared, out, shared_scale)
    if weights is None:
        need(top is not None and top > 0 and plan.entries % top == 0, name, "without weights, top must be given")
        n = plan.entries // top
    else:
        n, top = weights.shape
        need(weights.dtype == torch.float32 and weights.is_contiguous() and n * top == plan.entries, name, "weights: float32 [N, top]")
    need(shared_scale is None or (shared is not None and shared_scale.dtype == torch.float32 and shared_scale.shape == (n,)
                                  and shared_scale.is_contiguous()), name, "shared_scale: float32 [N], with shared")
    need(y.dim() == 2 and y.shape[0] == plan.entries and y.stride(1) == 1, name, "y must be [N * top, C]")
    cols = y.shape[1]
    if shared is not None:
        need(shared.shape == (n, cols) and shared.dtype == y.dtype and shared.stride(1) == 1, name, "shared must be [N, C] like y")
    if out is None:
        out = torch.empty((n, cols), dtype=y.dtype, device=y.device)
    need(out.shape == (n, cols) and out.dtype == y.dtype and out.stride(1) == 1, name, "bad out tensor")
    check(lib().yalis_expert_combine(ptr(y), i64(y.stride(0)), ptr(plan.inv), ptr(weights), i32(top), ptr(shared),
                                     i64(shared.stride(0) if shared is not None else 0), ptr(out), i64(out.stride(0)),
                                     i32(dtype_code(y.dtype)), i32(n), i32(cols), ptr(shared_scale), stream()), name)
    return out
