"""Wrappers of csrc/latent_attention.cu: attention over one cached row per token (a normed latent and a rotated
key part shared by all heads), in the form that never expands keys and values per head."""

from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, dtype_code, f32, i32, i64, lib, need, need_cuda, ptr, stream


def latent_prepare(src: torch.Tensor, q_off: int, kv_off: Optional[int], heads: int, d: int, r: int, p: int,
                   norm_w: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], interleaved: bool,
                   magnitude: float, qc: torch.Tensor, pool: Optional[torch.Tensor], block_table: torch.Tensor,
                   positions: torch.Tensor, req_of_token: torch.Tensor, bad_flag: Optional[torch.Tensor] = None,
                   q_src: Optional[torch.Tensor] = None) -> None:
    """From the input projection ``src`` [N, ...] (model dtype; per head [d plain | p rotated] from column ``q_off``,
    and from ``kv_off`` the token's [r | p]): writes every head's rotated query part into the last p columns of
    ``qc`` [N, heads, r + p] (float32) and, when ``kv_off`` and ``pool`` are given, the row
    [c / sqrt(mean(c^2) + eps) * norm_w | rotated key part] into the token's place in ``pool``
    [pages, 1, page_size, r + p].  The rotation turns the first 2 * len(inv_freq) of the p sizes by
    position * inv_freq, pairs (2i, 2i + 1) when ``interleaved`` else (i, i + len(inv_freq)), with cosine and sine
    multiplied by ``magnitude``.  With ``q_src`` [N, ...] (dtype of ``src``) the heads' queries are its columns from
    ``q_off`` instead of columns of ``src``."""
    name = "latent_prepare"
    need_cuda(name, src, norm_w, inv_freq, qc, pool, block_table, positions, req_of_token, bad_flag, q_src)
    n = src.shape[0]
    need(src.dim() == 2 and src.stride(1) == 1, name, "src must be [N, ...] with unit inner stride")
    qs = src if q_src is None else q_src
    need(qs.dim() == 2 and qs.stride(1) == 1 and qs.shape[0] == n and qs.dtype == src.dtype, name, "q_src must be [N, ...] like src")
    need(q_off + heads * (d + p) <= qs.shape[1] and (kv_off is None or kv_off + r + p <= src.shape[1]), name,
         "columns lie outside src")
    need(qc.dtype == torch.float32 and qc.shape == (n, heads, r + p) and qc.is_contiguous(), name,
         "qc must be contiguous float32 [N, heads, r + p]")
    for t in (positions, req_of_token):
        need(t.dtype == torch.int32 and t.shape == (n,) and t.is_contiguous(), name, "positions/req_of_token: int32 [N]")
    rot_dims = 0
    if inv_freq is not None:
        need(inv_freq.dtype == torch.float32 and inv_freq.dim() == 1 and inv_freq.is_contiguous()
             and 2 * inv_freq.numel() <= p, name, "inv_freq must be float32 [rot_dims / 2], rot_dims <= p")
        rot_dims = 2 * inv_freq.numel()
    page_size = num_pages = 0
    if kv_off is not None and pool is not None:
        need(norm_w is not None and norm_w.dtype == torch.float32 and norm_w.shape == (r,) and norm_w.is_contiguous(), name,
             "the latent's norm scale must be float32 [r]")
        need(pool.dtype == src.dtype and pool.dim() == 4 and pool.shape[1] == 1 and pool.shape[3] == r + p
             and pool.is_contiguous(), name, "pool must be contiguous [pages, 1, page_size, r + p] in the dtype of src")
        num_pages, page_size = pool.shape[0], pool.shape[2]
    need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), name,
         "block_table must be contiguous int32 [R, width]")
    check(lib().yalis_latent_prepare(
        ptr(src), i32(dtype_code(src.dtype)), i32(src.stride(0)), i32(q_off), i32(-1 if kv_off is None else kv_off),
        i32(heads), i32(d), i32(r), i32(p), ptr(norm_w), f32(eps), ptr(inv_freq), i32(rot_dims), i32(1 if interleaved else 0),
        f32(magnitude), ptr(qc), ptr(pool if kv_off is not None else None), ptr(block_table), i32(block_table.shape[1]),
        i32(page_size), i32(num_pages), ptr(positions), ptr(req_of_token), i32(n), ptr(bad_flag), ptr(q_src),
        i32(q_src.stride(0) if q_src is not None else 0), stream()), name)


def norm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight per row of ``x`` [N, width] (a column block of a wider matrix is fine), float32
    arithmetic; contiguous, in the dtype of ``x``."""
    name = "norm_rows"
    need_cuda(name, x, weight)
    need(x.dim() == 2 and x.stride(1) == 1 and weight.dtype == torch.float32 and weight.shape == (x.shape[1],)
         and weight.is_contiguous(), name, "x [N, width] with unit inner stride, weight float32 [width]")
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    check(lib().yalis_norm_rows(ptr(x), i64(x.stride(0)), ptr(weight), f32(eps), i32(x.shape[1]), ptr(y), i64(y.stride(0)),
                                i32(x.shape[0]), i32(dtype_code(x.dtype)), stream()), name)
    return y


def head_project(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None,
                 req_of_token: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[n, h, :] = w[h] x[n, h, :] for ``x`` [N, H, K] and ``out`` [N, H, O] (any strides over n and h, unit inner
    stride; float32 or the dtype of ``w``) and ``w`` [H, O, K] contiguous; with ``gate`` [N, H * O] (dtype of w)
    the result is multiplied by sigmoid(gate).  float32 sums on the CUDA cores in a fixed order."""
    name = "head_project"
    need_cuda(name, x, w, out, gate, req_of_token)
    need(x.dim() == 3 and w.dim() == 3 and out.dim() == 3 and w.is_contiguous(), name, "x [N, H, K], w [H, O, K], out [N, H, O]")
    n, h, k = x.shape
    o = w.shape[1]
    need(w.shape == (h, o, k) and out.shape == (n, h, o) and x.stride(2) == 1 and out.stride(2) == 1, name, "shapes do not agree")
    gs = 0
    if gate is not None:
        need(gate.dtype == w.dtype and gate.shape == (n, h * o) and gate.stride(1) == 1, name, "gate must be [N, H * O] in the dtype of w")
        gs = gate.stride(0)
    check(lib().yalis_head_project(ptr(x), i32(dtype_code(x.dtype)), i64(x.stride(0)), i64(x.stride(1)), ptr(w),
                                   i32(dtype_code(w.dtype)), i32(h), i32(o), i32(k), ptr(out), i32(dtype_code(out.dtype)),
                                   i64(out.stride(0)), i64(out.stride(1)), ptr(gate), i64(gs), ptr(req_of_token), i32(n),
                                   stream()), name)
    return out


def sigmoid_gate(x: torch.Tensor, g: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y[n, h * e + c] = x[n, h, c] * sigmoid(g[n, h * e + c]): ``x`` [N, H, e] with any strides over n and h (float32
    or the dtype of g and y), ``g`` and ``y`` [N, H * e] with unit inner stride."""
    name = "sigmoid_gate"
    need_cuda(name, x, g, y)
    need(x.dim() == 3 and g.dim() == 2 and x.stride(2) == 1 and g.shape == y.shape == (x.shape[0], x.shape[1] * x.shape[2])
         and g.stride(1) == y.stride(1) == 1 and g.dtype == y.dtype, name, "x [N, H, e]; g, y [N, H * e] of one dtype")
    check(lib().yalis_sigmoid_gate(ptr(x), i32(dtype_code(x.dtype)), i64(x.stride(0)), i64(x.stride(1)), i32(x.shape[2]), ptr(g),
                                   i64(g.stride(0)), ptr(y), i64(y.stride(0)), i32(dtype_code(y.dtype)), i32(g.shape[0]),
                                   i32(g.shape[1]), stream()), name)
    return y


MAX_ROW = 640      # r + p the exact kernel takes


def latent_attention_exact(qc: torch.Tensor, pool: torch.Tensor, positions: torch.Tensor, req_of_token: torch.Tensor,
                           block_table: torch.Tensor, r: int, scale: float, window: Optional[int],
                           out: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[n, h, :] = sum_j softmax_j((qc[n, h] . row_j) * scale) row_j[:r] over the rows j of the token's request
    with 0 <= position - j < window (None: all j <= position).  ``qc`` float32 [N, H, r + p]; float32 [N, H, r].
    ``sink`` float32 [H]: exp(sink_h) joins every denominator of head h (a score without key and value, not scaled)."""
    name = "latent_attention_exact"
    need_cuda(name, qc, pool, positions, req_of_token, block_table, out, sink)
    need(sink is None or (sink.dtype == torch.float32 and sink.shape == (qc.shape[1],) and sink.is_contiguous()), name,
         "sink must be float32 [H]")
    n, h, w = qc.shape
    need(qc.dtype == torch.float32 and qc.is_contiguous() and 0 < r <= w <= MAX_ROW, name,
         f"qc must be contiguous float32 [N, H, r + p] with r + p <= {MAX_ROW}")
    need(pool.dim() == 4 and pool.shape[1] == 1 and pool.shape[3] == w and pool.is_contiguous(), name,
         "pool must be contiguous [pages, 1, page_size, r + p]")
    need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), name,
         "block_table must be contiguous int32 [R, width]")
    if out is None:
        out = torch.empty((n, h, r), dtype=torch.float32, device=qc.device)
    need(out.dtype == torch.float32 and out.shape == (n, h, r) and out.is_contiguous(), name, "bad out tensor")
    check(lib().yalis_latent_attention_exact(ptr(qc), ptr(out), ptr(pool), i32(dtype_code(pool.dtype)), ptr(positions),
                                             ptr(req_of_token), ptr(block_table), i32(block_table.shape[1]),
                                             i32(pool.shape[2]), i32(pool.shape[0]), i32(n), i32(h), i32(r), i32(w - r),
                                             f32(scale), i32(window or 0), ptr(sink), stream()), name)
    return out


def mma_supports(r: int, p: int) -> bool:
    """Whether the tensor-core form takes a latent of ``r`` and a rotated part of ``p`` sizes."""
    return bool(lib().yalis_latent_attention_mma_supports(i32(r), i32(p)))


def latent_attention_mma(q_lat: torch.Tensor, q_rot: torch.Tensor, out: torch.Tensor, pool: torch.Tensor,
                         positions: torch.Tensor, q_start: torch.Tensor, req_of_token: torch.Tensor, block_table: torch.Tensor,
                         n_requests: int, max_q_len: int, scale: float, window: Optional[int], n_splits: int = 1,
                         sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same sums as ``latent_attention_exact`` on the tensor cores, for bfloat16 rows.  ``q_lat`` [N, H, r]
    (float32 or bfloat16) and ``q_rot`` [N, H, p] (float32) are the two parts of the queries and ``out`` [N, H, r]
    (float32 or bfloat16) the result, each with any strides over n and h and unit inner stride.  ``q_start`` int32
    [R + 1] gives each request's token range; ``max_q_len`` bounds the grid.  Queries and rows meet as bfloat16 with
    float32 sums; the weights meet the rows in two bfloat16 halves.  ``n_splits`` > 1 deals the rows a request's
    queries see to that many blocks in turn and merges their shares in order (for steps of single tokens)."""
    name = "latent_attention_mma"
    need_cuda(name, q_lat, q_rot, out, pool, positions, q_start, req_of_token, block_table, sink)
    need(sink is None or (sink.dtype == torch.float32 and sink.shape == (q_lat.shape[1],) and sink.is_contiguous()), name,
         "sink must be float32 [H]")
    n, h, r = q_lat.shape
    p = q_rot.shape[2]
    need(q_rot.shape == (n, h, p) and out.shape == (n, h, r) and q_rot.dtype == torch.float32
         and q_lat.stride(2) == q_rot.stride(2) == out.stride(2) == 1, name, "q_lat [N, H, r], q_rot float32 [N, H, p], out [N, H, r]")
    need(q_lat.dtype in (torch.float32, torch.bfloat16) and out.dtype in (torch.float32, torch.bfloat16), name, "float32 or bfloat16")
    need(pool.dtype == torch.bfloat16 and pool.dim() == 4 and pool.shape[1] == 1 and pool.shape[3] == r + p and pool.is_contiguous(),
         name, "pool must be contiguous bfloat16 [pages, 1, page_size, r + p]")
    need(mma_supports(r, p), name, f"r = {r}, p = {p} is not a shape of the tensor-core form")
    need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous() and q_start.dtype == torch.int32
         and q_start.numel() >= n_requests + 1, name, "block_table int32 [R, width], q_start int32 [R + 1]")
    need(n_splits >= 1, name, "n_splits must be positive")
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((n_splits, n * h, r), dtype=torch.float32, device=q_lat.device)
        part_ml = torch.full((n_splits, n * h, 2), float("-inf"), dtype=torch.float32, device=q_lat.device)
    check(lib().yalis_latent_attention_mma(
        ptr(q_lat), i32(q_lat.dtype == torch.bfloat16), i64(q_lat.stride(0)), i64(q_lat.stride(1)), ptr(q_rot),
        i64(q_rot.stride(0)), i64(q_rot.stride(1)), ptr(out), i32(out.dtype == torch.bfloat16), i64(out.stride(0)),
        i64(out.stride(1)), ptr(pool), ptr(positions), ptr(q_start), ptr(req_of_token), ptr(block_table), i32(block_table.shape[1]),
        i32(pool.shape[2]), i32(pool.shape[0]), i32(n_requests), i32(n), i32(max_q_len), i32(h), i32(r), i32(p), f32(scale),
        i32(window or 0), ptr(sink), i32(n_splits), ptr(part_o), ptr(part_ml), stream()), name)
    return out
