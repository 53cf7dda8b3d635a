"""Wrappers of the memory-bound kernels (csrc/elementwise.cu)."""

from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, dtype_code, f32, i32, i64, lib, need, need_cuda, ptr, stream


def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None,
              bad_flag: Optional[torch.Tensor] = None, scale: Optional[float] = None,
              from_slot: Optional[torch.Tensor] = None, chosen: Optional[torch.Tensor] = None,
              norm=None) -> torch.Tensor:
    """out[t] = float32(table[ids[t]]) (times ``scale`` if given).  ids int32 [N]; table [vocab, width].
    ``norm`` = (weight float32 [width], eps): the rows enter normed, v / sqrt(mean(v^2) + eps) * weight.
    With ``from_slot`` (int32 [N]) and ``chosen`` (int32 vector), token t takes its id from
    ``chosen[from_slot[t]]`` where ``from_slot[t]`` is not negative."""
    name = "embedding"
    need_cuda(name, table, ids, out, bad_flag, from_slot, chosen)
    need((from_slot is None) == (chosen is None), name, "from_slot and chosen come together")
    if from_slot is not None:
        need(from_slot.dtype == torch.int32 and from_slot.shape == ids.shape and from_slot.is_contiguous()
             and chosen.dtype == torch.int32 and chosen.dim() == 1 and chosen.is_contiguous(), name,
             "from_slot must be int32 [N] and chosen a contiguous int32 vector")
    need(ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(), name, "ids must be contiguous int32 [N]")
    need(table.dim() == 2 and table.is_contiguous(), name, "table must be contiguous [vocab, width]")
    n, (vocab, width) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, width), dtype=torch.float32, device=table.device)
    need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (n, width), name, "out must be float32 [N, width]")
    norm_w, norm_eps = (None, 0.0) if norm is None else norm
    if norm_w is not None:
        need_cuda(name, norm_w)
        need(norm_w.dtype == torch.float32 and norm_w.shape == (width,) and norm_w.is_contiguous(), name,
             "the norm's weight must be float32 [width]")
    check(lib().yalis_embedding(ptr(table), i32(dtype_code(table.dtype)), ptr(ids), ptr(from_slot), ptr(chosen),
                                ptr(out), i32(n), i32(width),
                                i32(vocab), f32(1.0 if scale is None else scale), ptr(bad_flag), ptr(norm_w), f32(norm_eps),
                                stream()), name)
    return out


def softcap_(values: torch.Tensor, cap: float) -> torch.Tensor:
    """values <- cap * tanh(values / cap), in place (float32, contiguous)."""
    name = "softcap"
    need_cuda(name, values)
    need(values.dtype == torch.float32 and values.is_contiguous(), name, "values must be contiguous float32")
    need(cap > 0, name, "the cap must be positive")
    check(lib().yalis_softcap_f32(ptr(values), i64(values.numel()), f32(cap), stream()), name)
    return values


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(x + delta) * weight, with x (float32 residual stream) updated in place.

    ``delta`` is None, [N, width], or split partial sums [S, N, width] (added in order).
    With ``rows`` (int32 indices) only those rows are normed and x is left untouched.
    """
    name = "add_rmsnorm"
    need_cuda(name, x, delta, weight, rows, out)
    need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), name, "x must be contiguous float32 [N, width]")
    n, width = x.shape
    need(weight.dtype == torch.float32 and weight.shape == (width,) and weight.is_contiguous(), name,
         "weight must be float32 [width]")
    n_delta, d_stride, d_code = 0, 0, 0
    if delta is not None:
        need(delta.is_contiguous(), name, "delta must be contiguous")
        if delta.dim() == 2:
            need(delta.shape == (n, width), name, f"delta shape {tuple(delta.shape)} != {(n, width)}")
            n_delta, d_stride = 1, 0
        else:
            need(delta.dim() == 3 and delta.shape[1:] == (n, width), name, "split delta must be [S, N, width]")
            n_delta, d_stride = delta.shape[0], n * width
        d_code = dtype_code(delta.dtype)
    n_out = n
    if rows is not None:
        need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), name, "rows must be int32 [R]")
        n_out = rows.numel()
    if out is None:
        out = torch.empty((n_out, width), dtype=out_dtype, device=x.device)
    need(out.shape == (n_out, width) and out.dtype == out_dtype and out.is_contiguous(), name, "bad out tensor")
    check(lib().yalis_add_rmsnorm(ptr(x), ptr(delta), i32(d_code), i32(n_delta), i64(d_stride), ptr(weight), ptr(out),
                                  i32(dtype_code(out_dtype)), ptr(rows), i32(n_out), i32(width), f32(eps),
                                  i32(0 if rows is not None else 1), stream()), name)
    return out


def add_normed_rmsnorm(x: torch.Tensor, delta: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                       delta_norm=None, weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                       out_dtype: Optional[torch.dtype] = None, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """A sub-layer's result that is normed on its way into the stream, and the norm that follows, in one pass:

        d = delta (the sum of split partial sums [S, N, width], in order) + bias
        d <- d / sqrt(mean(d^2) + e_d) * w_d          with ``delta_norm`` = (w_d, e_d)
        x <- x + d;  returns rmsnorm(x) * weight in ``out_dtype``        (nothing without ``weight``)

    all float32.  With ``rows`` only those rows are computed and x is left untouched."""
    name = "add_normed_rmsnorm"
    d_w, d_eps = (None, 0.0) if delta_norm is None else delta_norm
    need_cuda(name, x, delta, bias, d_w, weight, rows)
    need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), name, "x must be contiguous float32 [N, width]")
    n, width = x.shape
    for v in (bias, d_w, weight):
        need(v is None or (v.dtype == torch.float32 and v.shape == (width,) and v.is_contiguous()), name,
             "bias and norm weights must be float32 [width]")
    need(delta.is_contiguous(), name, "delta must be contiguous")
    if delta.dim() == 2:
        need(delta.shape == (n, width), name, f"delta shape {tuple(delta.shape)} != {(n, width)}")
        n_delta, d_stride = 1, 0
    else:
        need(delta.dim() == 3 and delta.shape[1:] == (n, width), name, "split delta must be [S, N, width]")
        n_delta, d_stride = delta.shape[0], n * width
    n_out = n
    if rows is not None:
        need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), name, "rows must be int32 [R]")
        n_out = rows.numel()
    out = None
    if weight is not None:
        need(out_dtype is not None, name, "the output needs a dtype")
        out = torch.empty((n_out, width), dtype=out_dtype, device=x.device)
    check(lib().yalis_add_normed_rmsnorm(ptr(x), ptr(delta), i32(dtype_code(delta.dtype)), i32(n_delta), i64(d_stride), ptr(bias),
                                         ptr(d_w), f32(d_eps), ptr(weight), ptr(out),
                                         i32(dtype_code(out_dtype if out is not None else torch.float32)), ptr(rows), i32(n_out),
                                         i32(width), f32(eps), i32(0 if rows is not None else 1), stream()), name)
    return out


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    """x += delta (or the sum of split partials [S, ...]) in float32, in place."""
    name = "residual_add"
    need_cuda(name, x, delta)
    need(x.dtype == torch.float32 and x.is_contiguous() and delta.is_contiguous(), name, "x float32, both contiguous")
    if delta.dim() == x.dim():
        need(delta.shape == x.shape, name, "shape mismatch")
        n_delta, stride = 1, 0
    else:
        need(delta.shape[1:] == x.shape, name, "split delta must be [S, *x.shape]")
        n_delta, stride = delta.shape[0], x.numel()
    check(lib().yalis_residual_add(ptr(x), ptr(delta), i32(dtype_code(delta.dtype)), i32(n_delta), i64(stride),
                                   i64(x.numel()), stream()), name)


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, req_of_token: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                  block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                  out_dtype: Optional[torch.dtype] = None, bad_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotate Q and K of the fused qkv rows, store K and V into their pages, return Q.

    ``qkv`` is [N, (nh + 2g) * hs] in the model dtype, or float32 partial sums
    [S, N, (nh + 2g) * hs] of a split product (summed in order).  Pools are
    [num_pages, g, page_size, hs]; block_table int32 [R, width].  Returns the rotated
    Q [N, nh * hs] in ``out_dtype`` (default: qkv's dtype).
    """
    name = "rope_kv_write"
    need_cuda(name, qkv, positions, req_of_token, inv_freq, k_pool, v_pool, block_table, bad_flag)
    width = (num_heads + 2 * num_kv_heads) * head_dim
    need(qkv.is_contiguous() and qkv.shape[-1] == width and qkv.dim() in (2, 3), name,
         "qkv must be contiguous [N, (heads + 2*kv_heads) * head_dim] or [S, N, ...]")
    parts = qkv.shape[0] if qkv.dim() == 3 else 1
    n = qkv.shape[-2]
    need(qkv.dim() == 2 or qkv.dtype == torch.float32, name, "split partial sums must be float32")
    out_dtype = out_dtype or qkv.dtype
    need(qkv.dim() == 3 or qkv.dtype == out_dtype, name, "an unsplit qkv must have the output dtype")
    need(head_dim % 2 == 0, name, f"head_dim {head_dim} must be even")
    for t in (positions, req_of_token):
        need(t.dtype == torch.int32 and t.shape == (n,) and t.is_contiguous(), name, "positions/req_of_token: int32 [N]")
    if inv_freq is not None:
        need(inv_freq.dtype == torch.float32 and inv_freq.shape == (head_dim // 2,) and inv_freq.is_contiguous(), name,
             "inv_freq must be float32 [head_dim / 2]")
    need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), name,
         "block_table must be contiguous int32 [R, width]")
    page_size, num_pages = 1, 0
    if k_pool is not None:
        need(v_pool is not None and k_pool.shape == v_pool.shape and k_pool.dtype == out_dtype == v_pool.dtype, name,
             "pools must match each other and the output dtype")
        need(k_pool.dim() == 4 and k_pool.shape[1] == num_kv_heads and k_pool.shape[3] == head_dim
             and k_pool.is_contiguous() and v_pool.is_contiguous(), name,
             "pools must be contiguous [pages, kv_heads, page_size, head_dim]")
        num_pages, page_size = k_pool.shape[0], k_pool.shape[2]
    q_out = torch.empty((n, num_heads * head_dim), dtype=out_dtype, device=qkv.device)
    check(lib().yalis_rope_kv_write(ptr(qkv), i32(dtype_code(qkv.dtype)), i32(width), i32(parts), i64(n * width),
                                    ptr(q_out), i32(dtype_code(out_dtype)), ptr(positions), ptr(req_of_token),
                                    ptr(inv_freq), ptr(k_pool), ptr(v_pool), ptr(block_table),
                                    i32(block_table.shape[1]), i32(page_size), i32(num_pages), i32(num_heads),
                                    i32(num_kv_heads), i32(head_dim), i32(n), ptr(bad_flag), stream()), name)
    return q_out


def silu_mul(x: torch.Tensor, interleaved: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate) * up for rows [gate | up] (or gate0, up0, gate1, ... when interleaved)."""
    name = "silu_mul"
    need_cuda(name, x, out)
    need(x.dim() == 2 and x.is_contiguous() and x.shape[1] % 2 == 0, name, "input must be contiguous [N, 2*inter]")
    n, inter = x.shape[0], x.shape[1] // 2
    if out is None:
        out = torch.empty((n, inter), dtype=x.dtype, device=x.device)
    need(out.shape == (n, inter) and out.dtype == x.dtype and out.is_contiguous(), name, "bad out tensor")
    check(lib().yalis_silu_mul(ptr(x), ptr(out), i32(dtype_code(x.dtype)), i32(n), i32(inter), i32(int(interleaved)),
                               stream()), name)
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    name = "gather_rows"
    need_cuda(name, x, rows)
    need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), name, "x must be float32 [N, width]")
    need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), name, "rows must be int32 [R]")
    out = torch.empty((rows.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    check(lib().yalis_gather_rows_f32(ptr(x), ptr(rows), ptr(out), i32(rows.numel()), i32(x.shape[1]), stream()), name)
    return out


GATED_SILU, GATED_CLAMPED = 0, 1


def gated_activation(x: torch.Tensor, gate_off: int, up_off: int, width: int, *, kind: int = GATED_SILU, limit: float = 0.0,
                     alpha: float = 1.0, shift: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A gated activation over rows that hold a gate part g = x[:, gate_off : gate_off + width] and an up part
    u = x[:, up_off : up_off + width]: ``GATED_SILU`` silu(g) * u; ``GATED_CLAMPED`` with g <- min(g, limit) and
    u <- clamp(u, -limit, limit): g * sigmoid(alpha g) * (u + shift).  float32 arithmetic, one rounding."""
    name = "gated_activation"
    need_cuda(name, x, out)
    need(x.dim() == 2 and x.stride(1) == 1 and max(gate_off, up_off) + width <= x.shape[1] and min(gate_off, up_off) >= 0,
         name, "x must be [N, C] with unit inner stride and hold both parts")
    if out is None:
        out = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
    need(out.shape == (x.shape[0], width) and out.dtype == x.dtype and out.stride(1) == 1, name, "bad out tensor")
    check(lib().yalis_gated_activation(ptr(x), i64(x.stride(0)), i32(gate_off), i32(up_off), ptr(out), i64(out.stride(0)),
                                       i32(dtype_code(x.dtype)), i32(x.shape[0]), i32(width), i32(kind), f32(limit), f32(alpha),
                                       f32(shift), stream()), name)
    return out


ACT_GELU_ERF, ACT_GELU_TANH, ACT_SILU, ACT_RELU2, ACT_TANH = 0, 1, 2, 3, 4
ACTIVATIONS = {"gelu": ACT_GELU_ERF, "gelu_erf": ACT_GELU_ERF, "gelu_tanh": ACT_GELU_TANH, "silu": ACT_SILU,
               "relu2": ACT_RELU2, "tanh": ACT_TANH}


def activation(x: torch.Tensor, kind: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x) element by element in float32: ``gelu_erf`` 0.5 z (1 + erf(z / sqrt 2)), ``gelu_tanh``
    0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))), ``silu``, ``relu2`` (max(z, 0)^2) or ``tanh``.  ``x`` and ``out`` are [N, C] with unit inner
    stride (column blocks of wider matrices are fine)."""
    name = "activation"
    need_cuda(name, x, out)
    need(kind in ACTIVATIONS, name, f"unknown activation {kind!r} (one of {', '.join(ACTIVATIONS)})")
    need(x.dim() == 2 and x.stride(1) == 1, name, "x must be [N, C] with unit inner stride")
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    need(out.shape == x.shape and out.dtype == x.dtype and out.stride(1) == 1, name, "bad out tensor")
    check(lib().yalis_activation(ptr(x), i32(x.stride(0)), ptr(out), i32(out.stride(0)), i32(dtype_code(x.dtype)),
                                 i32(x.shape[0]), i32(x.shape[1]), i32(ACTIVATIONS[kind]), stream()), name)
    return out


def add_rows_vector(x: torch.Tensor, other: Optional[torch.Tensor] = None, vec: Optional[torch.Tensor] = None) -> None:
    """x[n, :] += other[n, :] + vec[:] in place, float32 (either addend may be absent)."""
    name = "add_rows_vector"
    need_cuda(name, x, other, vec)
    need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), name, "x must be contiguous float32 [N, width]")
    if other is not None:
        need(other.dtype == torch.float32 and other.shape == x.shape and other.is_contiguous(), name, "other must match x")
    if vec is not None:
        need(vec.dtype == torch.float32 and vec.shape == (x.shape[1],) and vec.is_contiguous(), name, "vec must be float32 [width]")
    check(lib().yalis_add_rows_vector(ptr(x), ptr(other), ptr(vec), i32(x.shape[0]), i32(x.shape[1]), stream()), name)


def qkv_prepare(src: torch.Tensor, offsets, nq: int, nk: int, dim: int, vdim: int, positions: torch.Tensor,
                req_of_token: torch.Tensor, *, out_dtype: torch.dtype, biases=(None, None, None),
                q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None, norm_eps: float = 0.0,
                inv_freq: Optional[torch.Tensor] = None, q_scale: float = 1.0, k_scale: float = 1.0,
                k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
                block_table: Optional[torch.Tensor] = None, store: bool = True,
                bad_flag: Optional[torch.Tensor] = None, interleaved: bool = False, q_temperature=None):
    """Prepares the heads of a mixer from its input projection ``src`` [N, ...] (model dtype), whose query,
    key and value heads start at the columns ``offsets`` = (q, k, v):

        x <- x + bias;  q, k <- x / sqrt(mean(x^2) + norm_eps) * norm (where a norm is given);
        q, k <- rotation of their first 2 * len(inv_freq) sizes by the angle position * inv_freq (size i paired
        with i + len(inv_freq); with ``interleaved`` size 2i with 2i + 1), the other sizes unchanged;
        q <- q * q_scale, k <- k * k_scale;  with ``q_temperature`` = (coef, every) also
        q <- q * (1 + coef * ln(floor((position + 1) / every) + 1)).

    With pools, keys [pages, nk, page_size, dim] and values [pages, nk, page_size, vdim] are written to the pages
    of ``block_table`` (not at all when ``store`` is False) and the queries [N, nq * dim] are returned.  Without
    pools (q, k, v) are returned as plain matrices in ``out_dtype``."""
    name = "qkv_prepare"
    need_cuda(name, src, positions, req_of_token, q_norm, k_norm, inv_freq, k_pool, v_pool, block_table, bad_flag, *biases)
    need(src.dim() == 2 and src.stride(1) == 1, name, "src must be [N, ...] with unit inner stride")
    n = src.shape[0]
    q_off, k_off, v_off = (int(o) for o in offsets)
    need(max(q_off + nq * dim, k_off + nk * dim, v_off + nk * vdim) <= src.shape[1], name, "head columns lie outside src")
    for t in (positions, req_of_token):
        need(t.dtype == torch.int32 and t.shape == (n,) and t.is_contiguous(), name, "positions/req_of_token: int32 [N]")
    for b, width in zip(biases, (nq * dim, nk * dim, nk * vdim)):
        need(b is None or (b.dtype == src.dtype and b.shape == (width,) and b.is_contiguous()), name,
             "a bias must be a contiguous vector over its heads in the dtype of src")
    for w in (q_norm, k_norm):
        need(w is None or (w.dtype == torch.float32 and w.shape == (dim,) and w.is_contiguous()), name,
             "a norm scale must be float32 [dim]")
    rot_dims = 0
    if inv_freq is not None:
        need(inv_freq.dtype == torch.float32 and inv_freq.dim() == 1 and inv_freq.is_contiguous()
             and 2 * inv_freq.numel() <= dim, name, "inv_freq must be float32 [rot_dims / 2], rot_dims <= dim")
        rot_dims = 2 * inv_freq.numel()
    need(q_temperature is None or int(q_temperature[1]) > 0, name, "the query temperature's period must be positive")
    paged = k_pool is not None
    q_out = torch.empty((n, nq * dim), dtype=out_dtype, device=src.device)
    k_out = v_out = None
    page_size = num_pages = table_width = 0
    if paged:
        need(out_dtype == src.dtype, name, "with pools the queries keep the dtype of src")
        need(v_pool is not None and block_table is not None and k_pool.dtype == v_pool.dtype == src.dtype
             and k_pool.dim() == 4 and v_pool.dim() == 4 and k_pool.shape[:3] == v_pool.shape[:3]
             and k_pool.shape[1] == nk and k_pool.shape[3] == dim and v_pool.shape[3] == vdim
             and k_pool.is_contiguous() and v_pool.is_contiguous(), name,
             "pools must be contiguous [pages, kv_heads, page_size, dim] and [..., vdim] in the dtype of src")
        need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), name,
             "block_table must be contiguous int32 [R, width]")
        num_pages, page_size, table_width = k_pool.shape[0], k_pool.shape[2], block_table.shape[1]
    else:
        k_out = torch.empty((n, nk * dim), dtype=out_dtype, device=src.device)
        v_out = torch.empty((n, nk * vdim), dtype=out_dtype, device=src.device)
    # (with pools but ``store`` False - a layer that reads another entry's cache - the blocks of the key and
    # value heads find no destination and return)
    check(lib().yalis_qkv_prepare(
        ptr(src), i32(dtype_code(src.dtype)), i32(src.stride(0)), i32(q_off), i32(k_off), i32(v_off),
        ptr(biases[0]), ptr(biases[1]), ptr(biases[2]), ptr(q_norm), ptr(k_norm), f32(norm_eps), ptr(inv_freq),
        i32(rot_dims), i32(int(interleaved)), f32(q_scale), f32(k_scale),
        f32(q_temperature[0] if q_temperature is not None else 0.0), i32(q_temperature[1] if q_temperature is not None else 0),
        ptr(q_out), i32(q_out.stride(0)), ptr(k_out),
        i32(k_out.stride(0) if k_out is not None else 0), ptr(v_out), i32(v_out.stride(0) if v_out is not None else 0),
        i32(dtype_code(out_dtype)), ptr(k_pool if store else None), ptr(v_pool if store else None), ptr(block_table),
        i32(table_width), i32(page_size), i32(num_pages), ptr(positions), ptr(req_of_token), i32(n), i32(nq), i32(nk),
        i32(dim), i32(vdim), ptr(bad_flag), stream()), name)
    return q_out if paged else (q_out, k_out, v_out)
