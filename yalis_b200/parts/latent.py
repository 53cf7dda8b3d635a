"""Attention over a latent: keys and values of all heads are linear maps of one small normed vector per token.

    q_h = [plain (d) | rotated (p)] of W_q x;   W_dkv x = [c~ (r) | k~ (p)]
    c = c~ / sqrt(mean(c~^2) + eps) * n;        k_rot = rotation of k~ (one for all heads)
    key_h(j) = [U_k,h c(j) | k_rot(j)],  value_h(j) = U_v,h c(j)
    o_h(i) = sum_j softmax_j(q_h(i) . key_h(j) * scale) value_h(j)  over the j a window lets i see
    y = W_o (o * sigmoid(W_g x))                (the gate is optional)

Options: the queries may pass through a normed latent of their own (``q_rank``: q = W_uq (W_dq x / rms * n_q)), and
every head may have a sink, a learned score without key and value whose exponential joins the softmax's denominator.

Only the row [c | k_rot] of a token is cached (one "key head" of width r + p without values).  Keys and values
are never expanded: U_k,h^T is applied to the plain part of the query and U_v,h to the weighted sum of the
latents, which turns every head into a query over the same rows (see csrc/latent_attention.cu).  A layer may read
the rows another layer wrote (``own_latent`` False; the schedule entry names the other with ``cache_of``).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops import latent as ops
from yalis_b200.ops.linear import linear
from .base import Mixer, PagedKV, PagedKVCache, ParamSpec, PositionEncoding, Projected, make_part, register_part, stack_rows


class LatentAttention(Mixer, Projected):
    """Parameters: ``hidden_size``, ``num_heads``, ``head_dim`` (d, the plain part of a query and key),
    ``rot_dim`` (p, the rotated part), ``v_head_dim`` (e), ``kv_rank`` (r), ``rotary`` (the parameters of a
    ``rotary`` position part whose ``head_dim`` is the number of sizes that turn, at most p; None: no rotation),
    ``scale``, ``window`` (None: all keys), ``cache_window`` (how long rows are kept: at least ``window`` and the
    windows of the layers that read them; None: for ever), ``norm_eps``, ``gate`` (bool), ``own_latent`` (bool),
    ``q_rank`` (size of the queries' latent; None: queries are one product of the input), ``sink`` (bool)."""

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        p = spec.params
        if position is None and p.get("rotary") is not None:
            position = make_part("position", PartSpec("rotary", dict(p["rotary"])))
        super().__init__(spec, position)
        self.hidden, self.nh = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.p, self.e, self.r = int(p["head_dim"]), int(p["rot_dim"]), int(p["v_head_dim"]), int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        self.cache_window = p.get("cache_window", self.window)
        self.eps = float(p["norm_eps"])
        self.gate = bool(p.get("gate", False))
        self.own = bool(p.get("own_latent", True))
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") is not None else None
        self.has_sink = bool(p.get("sink", False))
        if self.r + self.p > ops.MAX_ROW:
            raise ValueError(f"kv_rank + rot_dim = {self.r + self.p} is more than the kernels take ({ops.MAX_ROW})")
        if self.position is not None and self.position.head_dim > self.p:
            raise ValueError(f"{self.position.head_dim} sizes are to turn, but the rotated part has {self.p}")
        if self.window is not None and self.cache_window is not None and self.cache_window < self.window:
            raise ValueError("cache_window must not be smaller than window")
        self.hidden_width = self.nh * self.e
        self.w_in: Optional[torch.Tensor] = None
        self.w_out: Optional[torch.Tensor] = None
        self.uk = self.uk_t = self.uv = self.uv_t = self.norm_w = None
        self.w_uq = self.q_norm_w = self.sink = None
        self.q_off = self.kv_off = self.g_off = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"q_proj": ParamSpec((self.nh * (self.d + self.p), self.hidden if self.q_rank is None else self.q_rank)),
                 "uk_proj": ParamSpec((self.nh * self.d, self.r)), "uv_proj": ParamSpec((self.nh * self.e, self.r)),
                 "o_proj": ParamSpec((self.hidden, self.nh * self.e))}
        if self.own:
            specs["dkv_proj"] = ParamSpec((self.r + self.p, self.hidden))
            specs["dkv_norm"] = ParamSpec((self.r,), init="ones", keep_float32=True)
        if self.gate:
            specs["g_proj"] = ParamSpec((self.nh * self.e, self.hidden))
        if self.q_rank is not None:
            specs["dq_proj"] = ParamSpec((self.q_rank, self.hidden))
            specs["dq_norm"] = ParamSpec((self.q_rank,), init="ones", keep_float32=True)
        if self.has_sink:
            specs["sink"] = ParamSpec((self.nh,), init="zeros", keep_float32=True)
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        if self.q_rank is None:
            blocks, names = [t["q_proj"]], ["q"]
        else:       # the input product makes the queries' latent; the queries are a second product of its normed rows
            blocks, names = [t["dq_proj"]], ["q"]
            self.w_uq, self.q_norm_w = t["q_proj"].contiguous(), t["dq_norm"].contiguous()
        if self.has_sink:
            self.sink = t["sink"].float().contiguous()
        if self.own:
            blocks.append(t["dkv_proj"])
            names.append("kv")
            self.norm_w = t["dkv_norm"].contiguous()
        if self.gate:
            blocks.append(t["g_proj"])
            names.append("g")
        self.w_in, spans = stack_rows(blocks)
        at = {n: s[0] for n, s in zip(names, spans)}
        self.q_off, self.kv_off, self.g_off = at["q"], at.get("kv"), at.get("g")
        self.w_out = t["o_proj"].contiguous()
        # U_k,h^T as [H, r, d] (it maps a query's plain part to the latent's size); U_v,h as stored, [H, e, r]
        self.uk = t["uk_proj"].reshape(self.nh, self.d, self.r).contiguous()
        self.uk_t = self.uk.transpose(1, 2).contiguous()
        self.uv = t["uv_proj"].reshape(self.nh, self.e, self.r).contiguous()
        self.uv_t = self.uv.transpose(1, 2).contiguous()

    def in_weight(self) -> torch.Tensor:
        return self.w_in

    def out_weight(self) -> torch.Tensor:
        return self.w_out

    def release_projections(self) -> None:
        self.w_in = self.w_out = None

    def cache_request(self) -> PagedKV:
        return PagedKV(1, self.r + self.p, self.cache_window, v_head_dim=0)

    def _tensor_core_form(self, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16 and ops.mma_supports(self.r, self.p)

    def capture_key(self, host):
        # the exact kernel launches the same for every step; the tensor-core one sizes its grid by the longest portion
        return ("latent_attention", host.max_q_len)

    def _splits(self, ctx) -> int:
        """Blocks that share the rows of one request in a step of single tokens: enough to fill the GPU twice, at most
        16 (a function of the step's shape alone, so a recording keeps it)."""
        if ctx.host.max_q_len != 1:
            return 1
        from yalis_b200.ops.attention import sm_count
        tiles = ctx.n_requests * -(-self.nh // 32)
        return max(1, min(16, (2 * sm_count(ctx.positions.device)) // max(1, tiles)))

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        keys = sum(min(ctx_before + t + 1, self.window or (ctx_before + t + 1)) for t in range(q_len)) if self.window \
            else q_len * ctx_before + q_len * (q_len + 1) / 2
        return 2.0 * self.nh * (2 * self.r + self.p) * keys

    def mix(self, z: torch.Tensor, ctx, cache: PagedKVCache, y: torch.Tensor) -> None:
        n, nh, d, p, e, r = z.shape[0], self.nh, self.d, self.p, self.e, self.r
        pos = self.position
        freq = pos.frequencies(pos.head_dim, z.device) if pos is not None else None
        table = ctx.block_tables[cache.group]
        qc = torch.empty((n, nh, r + p), dtype=torch.float32, device=z.device)
        q_all, q_off = None, self.q_off
        if self.q_rank is not None:
            q_all = linear(ops.norm_rows(z[:, self.q_off:self.q_off + self.q_rank], self.q_norm_w, self.eps), self.w_uq)
            q_off = 0
        ops.latent_prepare(z, q_off, self.kv_off if (self.own and cache.writable) else None, nh, d, r, p, self.norm_w,
                           self.eps, freq, bool(pos.interleaved) if pos is not None else False,
                           float(pos.magnitude) if pos is not None else 1.0, qc, cache.k, table, ctx.positions,
                           ctx.req_of_token, bad_flag=ctx.error_flag, q_src=q_all)
        q = (z[:, self.q_off:self.q_off + nh * (d + p)] if q_all is None else q_all).unflatten(1, (nh, d + p))
        gate = z[:, self.g_off:self.g_off + nh * e] if self.gate else None
        if self._tensor_core_form(z.dtype):
            # bfloat16 rows of a shape the tensor-core attention takes: the two per-head maps are batched library
            # products (at 8 tokens, 16 heads of 128 x 256, the engine's own kernel took 41 us a map, the library 4),
            # with the absorbed queries, the attention's result and the values head-major [H, N, .] in bfloat16
            q_lat = torch.bmm(q[:, :, :d].transpose(0, 1), self.uk)                       # [H, N, r]
            mixed = torch.empty((nh, n, r), dtype=z.dtype, device=z.device)
            ops.latent_attention_mma(q_lat.transpose(0, 1), qc[:, :, r:], mixed.transpose(0, 1), cache.k, ctx.positions,
                                     ctx.q_start, ctx.req_of_token, table, ctx.n_requests, ctx.host.max_q_len, self.scale,
                                     self.window, n_splits=self._splits(ctx), sink=self.sink)
            o = torch.bmm(mixed, self.uv_t)                                               # [H, N, e]
            if gate is not None:
                ops.sigmoid_gate(o.transpose(0, 1), gate, y)
            else:
                y.unflatten(1, (nh, e)).copy_(o.transpose(0, 1))
            return
        # the float32 path, and shapes the tensor-core form does not take: exact kernels throughout
        ops.head_project(q[:, :, :d], self.uk_t, qc[:, :, :r], req_of_token=ctx.req_of_token)
        mixed = ops.latent_attention_exact(qc, cache.k, ctx.positions, ctx.req_of_token, table, r, self.scale, self.window, sink=self.sink)
        ops.head_project(mixed, self.uv, y.unflatten(1, (nh, e)), gate=gate, req_of_token=ctx.req_of_token)

    def forward(self, x: torch.Tensor, ctx, cache: PagedKVCache) -> torch.Tensor:
        return self.project_and_mix(x, ctx, cache)


register_part("mixer", "latent_attention", LatentAttention)
