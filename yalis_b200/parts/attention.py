"""Grouped-query causal attention over the paged cache.

qkv = x Wqkv^T; positions are encoded into Q and K and K, V stored (the position
part does both in one kernel); every token attends to the cached keys of its
request up to its own position; the heads are projected back with Wo
(yalis/external/model.py:540-608).  The three projections are stored
concatenated [Wq; Wk; Wv] (the reference interleaves them per KV group,
model.py:544-557, which only serves its tensor-parallel split).
"""

from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops import attention as attn_ops
from yalis_b200.ops.linear import linear_partial
from yalis_b200.ops.elementwise import qkv_prepare
from .base import NOT_ROTARY, Mixer, NormedSum, PagedKV, PagedKVCache, ParamSpec, PositionEncoding, Projected, register_part


class PagedAttention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``window`` (None = all keys), ``scale`` (None = 1/sqrt(head_dim))."""

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec, position)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.g = int(p["num_kv_heads"])
        self.hs = int(p["head_dim"])
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hs)
        if self.nh % self.g:
            raise ValueError(f"num_heads {self.nh} is not a multiple of num_kv_heads {self.g}")
        if self.hs % 2 or self.hs > 256:
            raise ValueError(f"head_dim {self.hs} is not supported (even, at most 256)")
        if position is None:
            raise ValueError("paged_attention needs a position part (use kind 'none' for no encoding)")
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "q_proj": ParamSpec((self.nh * self.hs, self.hidden)),
            "k_proj": ParamSpec((self.g * self.hs, self.hidden)),
            "v_proj": ParamSpec((self.g * self.hs, self.hidden)),
            "o_proj": ParamSpec((self.hidden, self.nh * self.hs)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0).contiguous()
        self.w_o = tensors["o_proj"].contiguous()

    def cache_request(self) -> PagedKV:
        return PagedKV(self.g, self.hs, self.window)

    def capture_key(self, host):
        # everything the choice of kernel and its launch depend on besides the shapes of the step's tensors
        per = self.nh // self.g
        if host.max_q_len == 1:
            return host.once(("decode_step_kind",), lambda: attn_ops.decode_step_kind([b + 1 for b in host.ctx_before]))
        return host.once(("portion_step_kind", per, self.g, self.hs),
                         lambda: attn_ops.portion_step_kind(host, per, self.g, self.hs))

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        # QK^T and PV over the keys each token sees (causal; a window bounds them)
        keys = sum(min(ctx_before + t + 1, self.window or (ctx_before + t + 1)) for t in range(q_len)) if self.window \
            else q_len * ctx_before + q_len * (q_len + 1) / 2
        return 4.0 * self.nh * self.hs * keys

    def forward(self, x: torch.Tensor, ctx, cache: PagedKVCache) -> torch.Tensor:
        qkv = linear_partial(x, self.w_qkv)          # [N, width], or float32 partial sums [S, N, width]
        if (attn_ops.USE_FUSED_ROPE and ctx.n_requests * self.g <= 2 * attn_ops.sm_count(x.device)
                and attn_ops.decode_tma_applicable(x.dtype, ctx, self.hs, cache.k.shape[2], self.nh // self.g, self.window)
                and not attn_ops.decode_lean_preferred(ctx.n_requests, self.g, self.hs, attn_ops.step_kind(ctx)[0])):
            # A decode step whose attention blocks fit the GPU at once: the attention kernel rotates Q and the new K
            # itself and stores K, V (one launch less).  With more blocks than that the extra work at the start of
            # every block costs more than the launch (measured at batch 64: 59.5 against 57 us per layer).
            freq = self.position.rotary_frequencies(self.hs, x.device)
            if freq is not NOT_ROTARY:
                y = attn_ops.decode_attention_tma_fused(
                    qkv, freq, cache.writable, cache.k, cache.v, ctx.positions, ctx.q_start,
                    ctx.block_tables[cache.group], self.nh, self.g, self.hs, scale=self.scale,
                    n_splits=attn_ops.decode_tma_splits(ctx.n_requests, self.g, attn_ops.step_kind(ctx)[1]),
                    error_flag=ctx.error_flag,
                    early_fetch=bool(getattr(ctx, "settled", False)))
                return linear_partial(y, self.w_o)
        q = self.position.encode_and_store(qkv, self.nh, self.g, self.hs, ctx, cache, dtype=x.dtype)
        y = attn_ops.paged_attention(q, cache.k, cache.v, ctx, cache.group, self.nh, self.g, self.hs,
                                     scale=self.scale, window=self.window)
        return linear_partial(y, self.w_o)             # the residual stream adds the partial sums


class GeneralAttention(Mixer, Projected):
    """Grouped-query causal attention over the paged cache with the variations that the fast kernels of
    ``paged_attention`` do not take.  Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``
    (of q and k), ``v_head_dim`` (None: head_dim), ``bias`` (q, k, v = W x + b), ``qk_norm_eps`` (None: no norm;
    else q and k of every head become x / sqrt(mean(x^2) + eps) * scale before the rotation, one learned scale
    [head_dim] for q and one for k), ``rotary`` ({"dims", "theta", "layout"}: the first ``dims`` sizes of a head turn,
    size i paired with i + dims / 2, or with layout ``interleaved`` size 2i with 2i + 1; None: no rotation), ``scale``
    (None: 1/sqrt(head_dim)), ``softcap`` (c: scores become c tanh(s / c)), ``sink`` (True: 1 is added to the
    softmax's denominator; ``"learned"``: exp(z_h) with a learned z per head, the tensor ``sink``), ``window`` (position
    p sees the W positions up to itself), ``chunk`` (position p sees only its own chunk of C positions, counted from
    position 0, up to itself), ``distance_slopes`` (one number per head: slope_h * (p - j) is taken off the scaled
    score of key j), ``q_temperature`` ({"coef", "every"}: the query at position p is multiplied by
    1 + coef ln(floor((p + 1) / every) + 1)), ``gate`` (the heads' results are multiplied by sigmoid(W_g x), one more
    matrix over the mixer's input), ``out_bias`` (a bias on the output product), ``own_kv`` (False: the mixer has no
    key and value projections and reads the cache of the schedule entry it is pointed at; default True),
    ``cache_window`` (how many positions back the keys are kept, when that is not the mixer's own ``window`` or
    ``chunk``: the widest reach among this mixer and the mixers that read its cache), ``out_scale``.  Scores, weights
    and the weighted sum are float32 in every dtype."""

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        if position is None:
            from .recurrent import position_part
            position = position_part(spec.params)
        super().__init__(spec, position)
        p = spec.params
        self.hidden, self.nh, self.g, self.hs = int(p["hidden_size"]), int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.vd = int(p["v_head_dim"]) if p.get("v_head_dim") is not None else self.hs
        self.bias = bool(p.get("bias", False))
        self.norm_eps = float(p["qk_norm_eps"]) if p.get("qk_norm_eps") is not None else None
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hs)
        self.softcap = float(p["softcap"]) if p.get("softcap") is not None else None
        self.learned_sink = p.get("sink") == "learned"
        self.sink = bool(p.get("sink", False))
        self.window = p.get("window")
        self.chunk = int(p["chunk"]) if p.get("chunk") is not None else None
        self.slopes_host = tuple(float(v) for v in p["distance_slopes"]) if p.get("distance_slopes") is not None else None
        qt = p.get("q_temperature")
        self.q_temperature = (float(qt["coef"]), int(qt["every"])) if qt is not None else None
        self.gated = bool(p.get("gate", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.own_kv = bool(p.get("own_kv", True))
        self.cache_window = p.get("cache_window", self.window if self.window is not None else self.chunk)
        if p.get("cache_window") is None and self.window is not None and self.chunk is not None:
            self.cache_window = min(self.window, self.chunk)
        self.out_scale = float(p.get("out_scale", 1.0))
        if self.slopes_host is not None and len(self.slopes_host) != self.nh:
            raise ValueError(f"{len(self.slopes_host)} distance slopes for {self.nh} heads")
        if self.chunk is not None and self.chunk <= 0 or self.q_temperature is not None and self.q_temperature[1] <= 0:
            raise ValueError("chunk and the query temperature's period must be positive")
        if self.nh % self.g:
            raise ValueError(f"num_heads {self.nh} is not a multiple of num_kv_heads {self.g}")
        if max(self.hs, self.vd) > 256:
            raise ValueError(f"head sizes {self.hs}, {self.vd} are not supported (at most 256)")
        self.hidden_width = self.nh * self.vd
        self.w_in: Optional[torch.Tensor] = None
        self.w_out: Optional[torch.Tensor] = None
        self.biases = (None, None, None)
        self.q_norm = self.k_norm = None
        self.sink_logits = self.slopes = self.o_bias = None
        self.spans = {}

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"q_proj": ParamSpec((self.nh * self.hs, self.hidden)), "o_proj": ParamSpec((self.hidden, self.nh * self.vd))}
        if self.own_kv:
            specs.update({"k_proj": ParamSpec((self.g * self.hs, self.hidden)), "v_proj": ParamSpec((self.g * self.vd, self.hidden))})
        if self.bias:
            specs["q_bias"] = ParamSpec((self.nh * self.hs,), init="zeros")
            if self.own_kv:
                specs.update({"k_bias": ParamSpec((self.g * self.hs,), init="zeros"), "v_bias": ParamSpec((self.g * self.vd,), init="zeros")})
        if self.norm_eps is not None:
            specs["q_norm"] = ParamSpec((self.hs,), init="ones", keep_float32=True)
            if self.own_kv:
                specs["k_norm"] = ParamSpec((self.hs,), init="ones", keep_float32=True)
        if self.learned_sink:
            specs["sink"] = ParamSpec((self.nh,), init="zeros", keep_float32=True)
        if self.gated:
            specs["g_proj"] = ParamSpec((self.nh * self.vd, self.hidden))
        if self.out_bias:
            specs["o_bias"] = ParamSpec((self.hidden,), init="zeros", keep_float32=True)
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        # the input matrices stacked, each block of the product's columns on a 16-byte boundary
        names = ["q_proj"] + (["k_proj", "v_proj"] if self.own_kv else []) + (["g_proj"] if self.gated else [])
        plain = not self.gated and self.own_kv
        if plain:
            self.w_in = torch.cat([t[n] for n in names], dim=0).contiguous()
            qd, kd = self.nh * self.hs, self.g * self.hs
            spans = [(0, qd), (qd, qd + kd), (qd + kd, qd + kd + self.g * self.vd)]
        else:
            from .base import stack_rows
            self.w_in, spans = stack_rows([t[n] for n in names])
        self.spans = dict(zip(names, spans))
        self.w_out = t["o_proj"].contiguous()
        if self.bias:
            self.biases = tuple(t[n].to(self.w_in.dtype).contiguous() if n in t else None for n in ("q_bias", "k_bias", "v_bias"))
        if self.norm_eps is not None:
            self.q_norm = t["q_norm"].contiguous()
            self.k_norm = t["k_norm"].contiguous() if self.own_kv else None
        if self.learned_sink:
            self.sink_logits = t["sink"].float().contiguous()
        if self.slopes_host is not None:
            self.slopes = torch.tensor(self.slopes_host, dtype=torch.float32, device=self.w_in.device)
        if self.out_bias:
            self.o_bias = t["o_bias"].float().contiguous()

    def in_weight(self) -> torch.Tensor:
        return self.w_in

    def out_weight(self) -> torch.Tensor:
        return self.w_out

    def release_projections(self) -> None:
        if self.out_bias:
            raise ValueError("an arrangement that adds several output products into one cannot carry this mixer's output bias")
        self.w_in = self.w_out = None

    def cache_request(self) -> PagedKV:
        return PagedKV(self.g, self.hs, self.cache_window, v_head_dim=None if self.vd == self.hs else self.vd)

    def _tensor_core_form(self, dtype: torch.dtype) -> bool:
        """bfloat16 steps whose keys and values have one head size the kernel is built for go to the tensor cores
        (scores and the sum of weights in float32, the weights against V in two bfloat16 halves); float32 steps
        and other shapes go to the exact kernel."""
        return dtype == torch.bfloat16 and self.vd == self.hs and attn_ops.mma_supports(self.hs)

    def _launch_shape(self, host):
        """(longest portion, key splits): a step in which a request's rows fill at most one tile of 16 (single
        tokens of up to 16 heads per group) may divide each request's keys among blocks."""
        rows = host.max_q_len * (self.nh // self.g)
        return host.max_q_len, (attn_ops.decode_splits(len(host.slots), self.g) if rows <= 16 else 1)

    def capture_key(self, host):
        # the exact kernel launches the same for every step; the tensor-core one by the longest portion
        return ("general_attention",) + self._launch_shape(host)

    def keys_seen(self, position: int) -> int:
        """How many keys the query at ``position`` sees."""
        lo = max(0, position - self.window + 1) if self.window else 0
        if self.chunk:
            lo = max(lo, position // self.chunk * self.chunk)
        return position - lo + 1

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        keys = sum(self.keys_seen(ctx_before + t) for t in range(q_len)) if self.window or self.chunk \
            else q_len * ctx_before + q_len * (q_len + 1) / 2
        return 2.0 * self.nh * (self.hs + self.vd) * keys

    def mix(self, z: torch.Tensor, ctx, cache: PagedKVCache, y: torch.Tensor) -> None:
        if self.position is None:
            freq, interleaved = None, False
        else:
            interleaved = bool(getattr(self.position, "interleaved", False))
            freq = self.position.frequencies(self.position.head_dim, z.device) if interleaved \
                else self.position.rotary_frequencies(self.position.head_dim, z.device)
        table = ctx.block_tables[cache.group]
        if self.own_kv != cache.writable:
            raise ValueError("a mixer with key and value projections writes its own cache; one without reads another's")
        q_at = self.spans["q_proj"][0]
        k_at, v_at = (self.spans["k_proj"][0], self.spans["v_proj"][0]) if self.own_kv else (q_at, q_at)
        q = qkv_prepare(z, (q_at, k_at, v_at), self.nh, self.g, self.hs, self.vd, ctx.positions, ctx.req_of_token,
                        out_dtype=z.dtype, biases=self.biases, q_norm=self.q_norm, k_norm=self.k_norm,
                        norm_eps=self.norm_eps or 0.0, inv_freq=freq, k_pool=cache.k, v_pool=cache.v, block_table=table,
                        store=cache.writable, bad_flag=ctx.error_flag, interleaved=interleaved,
                        q_temperature=self.q_temperature)
        gate = None
        if self.gated:
            a, b = self.spans["g_proj"]
            gate = z[:, a:b]
        extras = dict(chunk=self.chunk, sink_logits=self.sink_logits, slopes=self.slopes, gate=gate)
        if self._tensor_core_form(z.dtype):
            longest, splits = self._launch_shape(ctx.host)
            direct = y.data_ptr() % 16 == 0 and y.stride(0) % 2 == 0
            out = attn_ops.paged_attention_mma(q, cache.k, cache.v, ctx.positions, ctx.q_start, ctx.req_of_token, table, longest,
                                               self.nh, self.g, self.hs, scale=self.scale, window=self.window, n_splits=splits,
                                               out=y if direct else None, softcap=self.softcap, sink=self.sink,
                                               out_scale=self.out_scale, exact_weights=True, **extras)
            if not direct:
                y.copy_(out)
            return
        attn_ops.paged_attention_generic(q, cache.k, cache.v, ctx.positions, ctx.req_of_token, table, self.nh, self.g, self.hs,
                                         scale=self.scale, window=self.window, out=y, v_head_dim=self.vd,
                                         softcap=self.softcap, sink=self.sink, out_scale=self.out_scale, **extras)

    def forward(self, x: torch.Tensor, ctx, cache: PagedKVCache):
        out = self.project_and_mix(x, ctx, cache)
        return NormedSum(out, bias=self.o_bias) if self.out_bias else out


register_part("mixer", "paged_attention", PagedAttention)
register_part("mixer", "general_attention", GeneralAttention)
