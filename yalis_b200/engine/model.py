"""A model built from a ``ModelSpec``: blocks of registered parts run in schedule order.

Nothing here is specific to an architecture.  The class names every tensor it
expects (for the loader and for the random-weights mode), asks every mixer what
cache it wants, and runs embedding -> schedule -> final norm -> output matrix
(yalis/external/model.py:137-197), with the output computed only for the rows
whose logits are wanted (the reference computes all positions, model.py:184).
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from yalis_b200.config.spec import ModelSpec
from yalis_b200.ops.elementwise import embedding, softcap_
from yalis_b200.ops.linear import linear
from yalis_b200.parts.base import NOT_CAPTURABLE, Block, ParamSpec, ResidualStream, build_block, make_part


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks: List[Block] = [build_block(layer) for layer in spec.layers]
        self.final_norm = make_part("norm", spec.final_norm)
        self.entry = make_part("entry", spec.entry) if spec.entry is not None else None
        self.embedding_norm = make_part("norm", spec.embedding_norm) if spec.embedding_norm is not None else None
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None
        self.extra: Dict[str, torch.Tensor] = {}
        self._keeps_embedding = any(e.before is not None and e.before.embedding for e in spec.schedule)

    # ---- tensors ---------------------------------------------------------------------
    def _layer_tensor_names(self, li: int) -> Dict[str, Dict[str, str]]:
        """part slot -> {local parameter name -> tensor name in the checkpoint}."""
        layer, block = self.spec.layers[li], self.blocks[li]
        out: Dict[str, Dict[str, str]] = {}
        for slot, part in block.parts.items():
            names = {}
            for local in part.param_specs():
                key = f"{slot}.{local}"
                if key not in layer.weight_names:
                    raise KeyError(f"layer {li}: the architecture names no tensor for {key}")
                names[local] = layer.weight_prefix + layer.weight_names[key]
            out[slot] = names
        return out

    def expected_tensors(self) -> Dict[str, ParamSpec]:
        """Every tensor of the checkpoint by name, in a fixed order."""
        s = self.spec
        out: Dict[str, ParamSpec] = {s.embedding_name: ParamSpec((s.vocab_size, s.hidden_size))}

        def put(name: str, ps: ParamSpec):
            if name in out and out[name] != ps:
                raise ValueError(f"tensor {name} is expected with two different specs: {out[name]} and {ps}")
            out[name] = ps

        for li, block in enumerate(self.blocks):
            names = self._layer_tensor_names(li)
            for slot, part in block.parts.items():
                for local, ps in part.param_specs().items():
                    put(names[slot][local], ps)
        for local, ps in self.final_norm.param_specs().items():
            put(s.final_norm_names[local], ps)
        if self.entry is not None:
            for local, ps in self.entry.param_specs().items():
                put(s.entry_names[local], ps)
        if self.embedding_norm is not None:
            for local, ps in self.embedding_norm.param_specs().items():
                put(s.embedding_norm_names[local], ps)
        for tensor_name, shape in s.extra_tensors.values():
            put(tensor_name, ParamSpec(tuple(shape), keep_float32=True))
        if s.head_name is not None:
            put(s.head_name, ParamSpec((s.vocab_size, s.hidden_size)))
        return out

    def load(self, fetch: Callable[[str], torch.Tensor], dtype: torch.dtype) -> None:
        """``fetch(name)`` returns the named tensor on the device in its final dtype."""
        s = self.spec
        self.dtype = dtype
        self.embedding = fetch(s.embedding_name).contiguous()
        for li, block in enumerate(self.blocks):
            names = self._layer_tensor_names(li)
            for slot, part in block.parts.items():
                part.load({local: fetch(name) for local, name in names[slot].items()})
        self.final_norm.load({local: fetch(s.final_norm_names[local]) for local in self.final_norm.param_specs()})
        if self.entry is not None:
            self.entry.load({local: fetch(s.entry_names[local]) for local in self.entry.param_specs()})
        if self.embedding_norm is not None:
            self.embedding_norm.load({local: fetch(s.embedding_norm_names[local]) for local in self.embedding_norm.param_specs()})
        self.head = self.embedding if s.head_name is None else fetch(s.head_name).contiguous()
        self.extra = {local: fetch(tensor_name).contiguous() for local, (tensor_name, _) in s.extra_tensors.items()}

    # ---- cache -------------------------------------------------------------------------
    def cache_requests(self) -> List[Optional[object]]:
        """What the block of each schedule entry wants to keep (an entry that reads another
        entry's cache still says what it expects to find there); behind them what the model's entry part keeps,
        if there is one."""
        requests = [self.blocks[e.layer].cache_request() for e in self.spec.schedule]
        if self.entry is not None:
            requests.append(self.entry.cache_request())
        return requests

    def cache_sources(self) -> List[Optional[int]]:
        """For each item of ``cache_requests``: the index of the item whose cache it reads instead of its own."""
        return [e.cache_of for e in self.spec.schedule] + ([None] if self.entry is not None else [])

    def capture_key(self, host):
        """The keys of all parts that run in a step, or ``NOT_CAPTURABLE`` if one of them cannot be recorded."""
        keys = []
        parts = [self.blocks[i] for i in sorted({e.layer for e in self.spec.schedule})] + [self.final_norm]
        for part in parts + [p for p in (self.entry, self.embedding_norm) if p is not None]:
            key = part.capture_key(host)
            if key is NOT_CAPTURABLE:
                return NOT_CAPTURABLE
            keys.append(key)
        return tuple(keys)

    # ---- forward -----------------------------------------------------------------------
    def forward(self, ctx, caches: List[Optional[object]], tap: Optional[Callable] = None) -> ResidualStream:
        """``tap(i, x)``, if given, sees the float32 stream [N, hidden] (the sum of its copies, if it has several)
        after schedule entry ``i`` (every pending addition applied): for comparisons layer by layer."""
        # a norm of the plain root-mean-square kind is applied by the kernel that gathers the rows
        fused = self.embedding_norm.rms_parameters() if self.embedding_norm is not None else None
        x = embedding(self.embedding, ctx.token_ids, bad_flag=ctx.error_flag, scale=self.spec.embedding_scale,
                      from_slot=ctx.token_from_slot, chosen=ctx.chosen if ctx.token_from_slot is not None else None,
                      norm=fused)
        if self.embedding_norm is not None and fused is None:
            x = self.embedding_norm.normalize(x)
        if self.entry is not None:
            self.entry.forward(x, ctx, caches[len(self.spec.schedule)])
        entered = x.clone() if self._keeps_embedding else None
        if self.spec.stream_copies is not None:
            # the copies are stored by the first pass over the stream, which reads the entering rows for all of them
            copies = torch.empty((x.shape[0], self.spec.stream_copies, x.shape[1]), dtype=torch.float32, device=x.device)
            stream = ResidualStream(copies, self.dtype, source=x)
        else:
            stream = ResidualStream(x, self.dtype)
        for i, (entry, cache) in enumerate(zip(self.spec.schedule, caches)):
            if entry.before is not None:
                b = entry.before
                stream.add_rows(entered if b.embedding else None, self.extra[b.vector][b.row] if b.vector is not None else None)
            self.blocks[entry.layer].forward(stream, ctx, cache)
            if tap is not None:
                tap(i, stream.total())
        return stream

    def logits(self, stream: ResidualStream, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] of the given token rows."""
        h = self.final_norm.forward(stream, rows=rows)
        out = linear(h, self.head, out_dtype=torch.float32)
        if self.spec.logit_softcap is not None:
            softcap_(out, self.spec.logit_softcap)
        return out

    def weight_bytes(self) -> int:
        """Bytes of every tensor on the device that the model's parts hold (each counted once)."""
        seen, visited, total = set(), set(), 0

        def walk(obj, depth=0):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.is_cuda and obj.untyped_storage().data_ptr() not in seen:
                    seen.add(obj.untyped_storage().data_ptr())
                    total += obj.untyped_storage().nbytes()
                return
            if depth > 6 or id(obj) in visited:
                return
            if isinstance(obj, (list, tuple)):
                for v in obj:
                    walk(v, depth + 1)
            elif isinstance(obj, dict):
                for v in obj.values():
                    walk(v, depth + 1)
            elif hasattr(obj, "spec") and hasattr(obj, "__dict__"):      # a part
                visited.add(id(obj))
                for v in vars(obj).values():
                    walk(v, depth + 1)

        walk(self.embedding)
        walk(self.head)
        walk(self.extra)
        walk(self.blocks)
        walk(self.final_norm)
        walk(self.entry)
        walk(self.embedding_norm)
        return total
