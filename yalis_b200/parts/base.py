"""Interfaces of the parts a layer is put together from, and their registry.

Seven categories, each with one small interface:

``norm``          ``forward(stream, rows=None) -> Tensor``: applies the pending
                  residual delta, returns the normed rows in the model dtype.
``position``      ``encode_and_store(qkv, heads, kv_heads, head_dim, ctx, cache, dtype) -> q``:
                  encodes positions into Q and K of a fused qkv matrix (given in
                  the model dtype or as float32 partial sums [S, N, width]), puts
                  K, V into the layer's cache pages and returns Q [N, heads*head_dim].
``mixer``         ``cache_request() -> PagedKV | SlotState | None`` and
                  ``forward(x, ctx, cache) -> Tensor [N, hidden]``.
``feed_forward``  ``forward(x, ctx) -> Tensor [N, hidden]``.
``connection``    ``write(h, y) -> PendingWrite`` and ``read_weights()``: how a
                  sub-layer's result enters a stream kept in one or several copies
                  (factors, a gate computed from the sub-layer's input, the mixing of
                  the copies) and with which weights the copies are read.
``entry``         ``cache_request()`` and ``forward(x, ctx, cache) -> None``: what is added
                  to the token rows as they enter the stream (one per model, optional);
                  it may keep a state per request like a mixer.
``block``         ``forward(stream, ctx, cache) -> None``: the arrangement of the
                  others around the residual stream.  A block kind declares the
                  places it has (``slots``: place name -> category); a layer's
                  ``LayerSpec.parts`` fills exactly those.

Every part is constructed from a ``PartSpec`` (kind + parameters) alone, names
its tensors with ``param_specs()`` and receives them in ``load()``.  A part
never sees the model configuration, the architecture's name or another layer.
New kinds are added with ``register_part(category, kind, cls)``; nothing else in
the package has to change.

A step can be recorded once (a CUDA graph) and replayed: steps in which every
request brings one token share a recording per bucket of requests, other steps
get one at their exact counts when their shape comes again.  A replay runs no
Python, so whatever a part decides on the
host from the step's facts has to be the same for every step that replays one
recording: ``capture_key(host)`` returns a hashable that determines all such
decisions (kernel choice, grid sizes), or ``NOT_CAPTURABLE`` (the default) for a
part whose ``forward`` works on the host per request, synchronises or allocates
by data.  The engine records one step per distinct tuple of keys and sends
steps with a part that cannot be captured to the launched path.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Hashable, Mapping, Optional, Tuple

import torch

from yalis_b200.config.spec import PartSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "connection", "entry", "block")


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs.

    ``init`` says what the random-weights mode writes: ``normal`` = N(0, 0.02)
    (the reference's GPT._init_weights, yalis/external/model.py:113-120),
    ``ones``, ``zeros``, ``identity`` (a square matrix) or ``const:<value>``.  ``keep_float32``: held in float32 whatever the
    engine's dtype (norm scales).  ``integer``: an integer table, held as int32.
    """

    shape: Tuple[int, ...]
    init: str = "normal"
    keep_float32: bool = False
    integer: bool = False


# ---- what a mixer may ask of the cache manager ---------------------------------

@dataclass(frozen=True)
class PagedKV:
    """Keys and values in pages. ``window`` None keeps every key; W keeps, for a
    query at position p, the keys at positions > p - W."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None      # head size of the values when it is not the keys'

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class SlotState:
    """A tensor of fixed shape per request (zeroed when the request is admitted)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


def cache_leaves(request):
    """A part that keeps several things (keys in pages and a state, say) asks for them as a dictionary
    name -> request, nested as deep as its own parts are; the storage answers with the same dictionary of caches.
    This yields the ``PagedKV`` and ``SlotState`` requests of such a tree (or of a single request)."""
    if request is None:
        return
    if isinstance(request, Mapping):
        for sub in request.values():
            yield from cache_leaves(sub)
    else:
        yield request


class PagedKVCache:
    """What a paged mixer gets for one schedule entry: its two pools
    [pages, kv_heads, page_size, head_dim] and the name of its page group, under
    which the step context holds the block tables.  ``writable`` is False for an
    entry that reads the cache of another entry."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor, group: str, writable: bool = True):
        self.k, self.v, self.group, self.writable = k, v, group, writable

    @property
    def page_size(self) -> int:
        return self.k.shape[2]


class SlotStateCache:
    """What a stateful mixer gets: ``state`` [max_slots + 1, *shape]; rows are indexed
    by the step context's ``slots``.  The last row belongs to no request: the padding
    rows of a recorded step point there, so a kernel may update ``state[ctx.slots]``
    for every row of the step without a test."""

    def __init__(self, state: torch.Tensor, writable: bool = True):
        self.state, self.writable = state, writable


# ---- the residual stream ----------------------------------------------------------

@dataclass
class PendingWrite:
    """A sub-layer's result on its way into a stream kept in several copies, with everything the write does to it:
    y <- y * layer_scale * sigmoid(gate + gate_bias), then x_t <- sum_s mix[s, t] x_s + out_weights[t] y.  ``y`` is
    [N, hidden] or float32 partial sums [P, N, hidden]; every other field may be None (without ``mix``: x_t += y)."""

    y: torch.Tensor
    gate: Optional[torch.Tensor] = None
    gate_bias: Optional[torch.Tensor] = None
    layer_scale: Optional[torch.Tensor] = None
    mix: Optional[torch.Tensor] = None
    out_weights: Optional[torch.Tensor] = None

    def arguments(self) -> Dict[str, Optional[torch.Tensor]]:
        return {"y": self.y, "gate": self.gate, "gate_bias": self.gate_bias, "layer_scale": self.layer_scale, "mix": self.mix,
                "out_weights": self.out_weights}


@dataclass
class NormedSum:
    """A sub-layer's result that is not added as it is: ``bias`` (float32 [hidden]) is added to it, and with ``norm`` =
    (weight float32 [hidden], eps) the sum is normed, d / sqrt(mean(d^2) + eps) * weight, before it joins the stream
    (an arrangement with a norm behind each sub-layer).  ``y`` is [N, hidden] in the model dtype or float32 partial
    sums [P, N, hidden].  All of it is float32 arithmetic inside the pass that adds it."""

    y: torch.Tensor
    bias: Optional[torch.Tensor] = None
    norm: Optional[Tuple[torch.Tensor, float]] = None


class ResidualStream:
    """The float32 residual stream [N, hidden] with one pending delta.

    A sub-layer's output is not added at once: it is parked in ``pending`` and
    the next norm adds it while it reads the stream (one pass instead of two).
    ``pending`` is [N, hidden] in the model dtype, or float32 split partial sums
    [S, N, hidden] that are added in order, or a ``NormedSum`` (such a tensor with a bias, a norm of its own
    or both).

    A model may keep the stream in several copies: ``x`` is then [N, copies, hidden], what is parked is a
    ``PendingWrite``, and the norms and arrangements that know such streams read and write all copies in one pass.
    At the start all copies equal the entering rows: ``source`` [N, hidden] holds them and ``x`` nothing, until the
    first pass over the stream stores the copies (``take_source`` hands the rows to that pass).
    """

    def __init__(self, x: torch.Tensor, dtype: torch.dtype, source: Optional[torch.Tensor] = None):
        self.x = x
        self.dtype = dtype
        self.pending = None       # a tensor (see above), a NormedSum or a PendingWrite
        self.source = source

    def take_source(self, stores: bool = True) -> Optional[torch.Tensor]:
        """The entering rows, if the copies are not stored yet; ``stores``: the pass that gets them stores the copies."""
        source = self.source
        if stores:
            self.source = None
        return source

    def materialize(self) -> None:
        if self.source is not None:
            from yalis_b200.ops.streams import stream_step
            stream_step(self.x, source=self.take_source(), read=False)

    @property
    def copies(self) -> int:
        return self.x.shape[1] if self.x.dim() == 3 else 1

    def add(self, delta) -> None:
        self.flush()
        if self.x.dim() == 3 and not isinstance(delta, PendingWrite):
            raise ValueError("a stream kept in several copies takes a PendingWrite, not a plain sum")
        if isinstance(delta, NormedSum) and delta.bias is None and delta.norm is None:
            delta = delta.y
        self.pending = delta

    def flush(self) -> None:
        if self.pending is None:
            return
        if isinstance(self.pending, PendingWrite):
            from yalis_b200.ops.streams import stream_step
            stream_step(self.x, read=False, source=self.take_source(), **self.pending.arguments())
        elif isinstance(self.pending, NormedSum):
            from yalis_b200.ops.elementwise import add_normed_rmsnorm
            add_normed_rmsnorm(self.x, self.pending.y, bias=self.pending.bias, delta_norm=self.pending.norm)
        else:
            from yalis_b200.ops.elementwise import residual_add
            residual_add(self.x, self.pending)
        self.pending = None

    def total(self) -> torch.Tensor:
        """float32 [N, hidden]: the stream, or the sum of its copies, with what is pending applied."""
        self.flush()
        if self.x.dim() == 2:
            return self.x
        from yalis_b200.ops.streams import stream_step
        return stream_step(self.x, out_dtype=torch.float32, source=self.take_source())

    def add_rows(self, other: Optional[torch.Tensor] = None, vector: Optional[torch.Tensor] = None) -> None:
        """x[n, :] += other[n, :] + vector[:] (float32; either may be absent), after what is pending."""
        from yalis_b200.ops.elementwise import add_rows_vector
        self.flush()
        if self.x.dim() == 3:
            raise ValueError("rows are added to a stream of one copy only")
        add_rows_vector(self.x, other, vector)


# ---- parts ---------------------------------------------------------------------------

class _NotCapturable:
    def __repr__(self) -> str:
        return "NOT_CAPTURABLE"


NOT_CAPTURABLE = _NotCapturable()   # answer of Part.capture_key: run this part's steps launch by launch


class Part:
    category = ""

    def __init__(self, spec: PartSpec):
        self.spec = spec

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the tensors named by param_specs(), on the device, in the engine's dtype."""

    def capture_key(self, host) -> Hashable:
        """What a recorded step of this part depends on beyond the shapes of its tensors (see the module
        docstring).  ``host`` is the step's ``HostStep``.  Return None when ``forward`` launches the same
        kernels whatever the requests' lengths are."""
        return NOT_CAPTURABLE

    def matrix_flops_per_token(self) -> float:
        """Floating-point operations per token in this part's matrix products (2 per weight of every 2-D tensor)."""
        return float(sum(2 * ps.shape[0] * ps.shape[1] for ps in self.param_specs().values() if len(ps.shape) == 2))


class Norm(Part):
    category = "norm"

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def normalize(self, y: torch.Tensor) -> torch.Tensor:
        """The norm of a plain tensor [N, width] in its own dtype (for arrangements that norm a sub-layer's
        output rather than the stream)."""
        raise NotImplementedError

    def rms_parameters(self) -> Optional[Tuple[torch.Tensor, float]]:
        """(weight float32 [width], eps) if the norm is x / sqrt(mean(x^2) + eps) * weight and nothing else, so that a
        kernel which produces or consumes the rows can apply it itself; None (the default) otherwise."""
        return None


NOT_ROTARY = object()     # answer of PositionEncoding.rotary_frequencies for encodings a mixer's kernel cannot apply itself


class PositionEncoding(Part):
    category = "position"

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, ctx, cache: PagedKVCache, dtype=None):
        raise NotImplementedError

    def rotary_frequencies(self, head_dim: int, device):
        """For mixers whose kernel can encode positions itself (one launch less): the float32 inverse
        frequencies [head_dim / 2] of a half-split rotary encoding with angle position * frequency, ``None``
        for "store and use Q, K unrotated", or ``NOT_ROTARY`` (the default) for anything else - the mixer
        then calls ``encode_and_store``."""
        return NOT_ROTARY


class Mixer(Part):
    category = "mixer"

    def __init__(self, spec: PartSpec, position: Optional[PositionEncoding] = None):
        super().__init__(spec)
        self.position = position

    def cache_request(self):
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError

    def mixing_flops(self, q_len: int, ctx_before: int) -> float:
        """Floating-point operations, beyond the matrix products, of ``q_len`` tokens fed after ``ctx_before``
        cached ones (for rooflines; 0 when the mixer has none worth counting)."""
        return 0.0


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Connection(Part):
    category = "connection"

    def read_weights(self) -> Optional[torch.Tensor]:
        """float32 [copies]: the weights of the stream's copies in the sum a sub-layer reads (None: the plain sum)."""
        return None

    def write(self, h: torch.Tensor, y: torch.Tensor) -> "PendingWrite":
        """The sub-layer's result ``y`` (as a mixer or feed-forward returns it) on its way into the stream; ``h`` is
        what the sub-layer read."""
        raise NotImplementedError


class Entry(Part):
    category = "entry"

    def cache_request(self):
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> None:
        """Adds to the token rows ``x`` float32 [N, hidden] in place."""
        raise NotImplementedError


class Projected:
    """What a mixer or feed-forward of the form  W_out core(W_in x)  can say about itself, so that an arrangement
    in which several of them read one input and add into one sum (a parallel block, mixers side by side) runs
    ONE product for all their inputs and ONE for all their outputs (the output matrices side by side along K):

    ``in_weight()``    the input matrix [rows, hidden] (after ``load``);
    ``hidden_width``   columns of the core's result;
    ``out_weight()``   the output matrix [hidden, hidden_width];
    ``mix(z, ctx, cache, y)``  the core: reads its rows ``z`` [N, rows] of the input product and writes
                       ``y`` [N, hidden_width]; both may be column blocks of wider matrices.  A factor on the
                       part's result is applied to ``y``.
    ``release_projections()``  the arrangement has copied both matrices into its own: drop them.
    """

    hidden_width = 0

    def in_weight(self) -> torch.Tensor:
        raise NotImplementedError

    def out_weight(self) -> torch.Tensor:
        raise NotImplementedError

    def mix(self, z: torch.Tensor, ctx, cache, y: torch.Tensor) -> None:
        raise NotImplementedError

    def release_projections(self) -> None:
        raise NotImplementedError

    def project_and_mix(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        """The part on its own: W_out core(W_in x), the last product as partial sums where the kernel splits K."""
        from yalis_b200.ops.linear import linear, linear_partial
        z = linear(x, self.in_weight())
        y = torch.empty((x.shape[0], self.hidden_width), dtype=x.dtype, device=x.device)
        self.mix(z, ctx, cache, y)
        return linear_partial(y, self.out_weight())


def stack_rows(blocks, multiple: int = 8):
    """The matrices [rows_i, K] stacked into one, each starting at a row that is a multiple of ``multiple`` (zero rows
    between them), so that each block of the product's columns starts on a 16-byte boundary.  Returns the matrix and
    the (start, stop) of every block."""
    spans, rows, at = [], [], 0
    for w in blocks:
        pad = (-at) % multiple
        if pad:
            rows.append(torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device))
            at += pad
        rows.append(w)
        spans.append((at, at + w.shape[0]))
        at += w.shape[0]
    if at % multiple:           # rows of the product start on the boundary too
        rows.append(torch.zeros(((-at) % multiple, rows[0].shape[1]), dtype=rows[0].dtype, device=rows[0].device))
    return torch.cat(rows, dim=0).contiguous(), spans


class Block(Part):
    """An arrangement of parts around the residual stream.

    ``slots`` names the places of the arrangement and the category of part each takes; the layer's
    ``LayerSpec.parts`` must fill exactly these.  The built parts arrive as a dictionary and are also set as
    attributes (``self.mixer`` ...).  A place of category ``position`` is built first and handed to the
    block's mixers.  A block keeps at most one cache: what its ``cache_request`` returns (by default its
    mixer's request, or nothing when it has no mixer).
    """

    category = "block"
    slots: Mapping[str, str] = {}
    optional: Tuple[str, ...] = ()      # places a layer may leave empty

    def __init__(self, spec: PartSpec, parts: Dict[str, Part]):
        super().__init__(spec)
        self.parts = dict(parts)
        for name, part in self.parts.items():
            setattr(self, name, part)

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        raise NotImplementedError

    def cache_request(self):
        mixers = [p for p in self.parts.values() if isinstance(p, Mixer)]
        if len(mixers) > 1:
            raise NotImplementedError("a block with several mixers must say itself what it caches")
        return mixers[0].cache_request() if mixers else None

    def capture_key(self, host) -> Hashable:
        keys = []
        for part in self.parts.values():
            key = part.capture_key(host)
            if key is NOT_CAPTURABLE:
                return NOT_CAPTURABLE
            keys.append(key)
        return tuple(keys)


def build_block(layer) -> Block:
    """The block of a ``LayerSpec`` with all its parts."""
    _ensure_builtin()
    try:
        factory = _REGISTRY["block"][layer.block.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY["block"])) or "none"
        raise ValueError(f"no block of kind {layer.block.kind!r} is registered (known: {known})") from None
    slots = dict(getattr(factory, "slots", {}))
    optional = tuple(getattr(factory, "optional", ()))
    missing = [n for n in slots if n not in layer.parts and n not in optional]
    slots = {n: c for n, c in slots.items() if n in layer.parts or n not in optional}
    unknown = [n for n in layer.parts if n not in slots]
    if missing or unknown:
        raise ValueError(f"block kind {layer.block.kind!r} has the places {sorted(slots)}: "
                         + (f"the layer fills none of {missing}" if missing else "")
                         + ("; " if missing and unknown else "")
                         + (f"the layer names {unknown}, which the block does not have" if unknown else ""))
    built: Dict[str, Part] = {}
    positions = [n for n, c in slots.items() if c == "position"]
    for name in positions:
        built[name] = make_part("position", layer.parts[name])
    position = built[positions[0]] if len(positions) == 1 else None
    for name, category in slots.items():
        if category == "position":
            continue
        extra = {"position": position} if category == "mixer" else {}
        built[name] = make_part(category, layer.parts[name], **extra)
    ordered = {name: built[name] for name in slots}
    return factory(layer.block, ordered)


# ---- registry ---------------------------------------------------------------------------

_REGISTRY: Dict[str, Dict[str, Callable[..., Part]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, factory: Callable[..., Part], *, replace: bool = False) -> None:
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r} (one of {', '.join(CATEGORIES)})")
    if kind in _REGISTRY[category] and not replace:
        raise ValueError(f"{category} kind {kind!r} is already registered")
    _REGISTRY[category][kind] = factory


def make_part(category: str, spec: PartSpec, **kwargs: Any) -> Part:
    _ensure_builtin()
    try:
        factory = _REGISTRY[category][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {}))) or "none"
        raise ValueError(f"no {category} of kind {spec.kind!r} is registered (known: {known})") from None
    return factory(spec, **kwargs)


def registered(category: str) -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_REGISTRY[category]))


def _ensure_builtin() -> None:
    from yalis_b200.parts import attention, block, dense, entry, experts, hyper, latent, norm, recurrent, rotary, swiglu  # noqa: F401
