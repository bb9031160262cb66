"""A decoder assembled from a ``ModelSpec``: embedding, blocks run in the order
of the schedule, final norm and output projection (src/model.rs:646-687, 637-643).

Nothing here names an architecture; the spec says which parts each layer has.
"""
from __future__ import annotations

from collections.abc import Mapping
from typing import Dict, List, Optional

import torch

from ..cache.kv import KVRequest, StateRequest
from ..config.spec import ModelSpec
from ..parts import block as block_mod
from ..parts.base import Part, Runtime, TensorSpec, delta_for, make_part
from ..weights.store import WeightStore


def _named_parts(spec: ModelSpec):
    """Yield (part, prefix) for every part of the model, unbound."""
    emb = make_part("embedding", spec.embedding)
    blocks = [block_mod.make_block(l) for l in spec.layers]
    final_norm = make_part("norm", spec.final_norm)
    head = make_part("head", spec.head)
    return emb, blocks, final_norm, head


def _joins(spec: ModelSpec):
    return [make_part("join", j) for j in spec.joins]


class PartTensors(Mapping):
    """The tensors of one part, by local name, fetched from the store when they are asked for and
    not kept: a part that re-lays its weights out (one slab for all experts, say) holds a tensor of
    the store only while it copies it.  ``pop`` is a fetch too."""

    def __init__(self, store: WeightStore, prefix: str, names, dtype, device):
        self._store, self._prefix, self._names = store, prefix, list(names)
        self._dtype, self._device = dtype, device

    def __getitem__(self, local):
        if local not in self._names:
            raise KeyError(local)
        return self._store.get(self._prefix + local, self._dtype, self._device)

    def pop(self, local, *default):
        if local not in self._names and default:
            return default[0]
        return self[local]

    def __iter__(self):
        return iter(self._names)

    def __len__(self):
        return len(self._names)


def _tensors_of(part: Part, store: Optional[WeightStore]) -> Dict[str, TensorSpec]:
    if store is None:
        return part.tensors()
    return part.tensors_in(lambda local: store.has(part.spec.prefix + local))


def expected_tensors(spec: ModelSpec, store: Optional[WeightStore] = None) -> Dict[str, TensorSpec]:
    """Checkpoint name -> shape of every tensor the model needs; with a ``store``, in the layout
    that each part finds there (a part may take several, ``Part.tensors_in``)."""
    emb, blocks, final_norm, head = _named_parts(spec)
    out: Dict[str, TensorSpec] = {}
    parts: List[Part] = [emb, final_norm, head] + _joins(spec)
    for b in blocks:
        parts.extend(b.parts())
    for p in parts:
        for local, ts in _tensors_of(p, store).items():
            out[p.spec.prefix + local] = ts
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, store: WeightStore, rt: Runtime, check: bool = True):
        self.spec = spec
        self.rt = rt
        self.embedding, self.blocks, self.final_norm, self.head = _named_parts(spec)
        self.joins = _joins(spec)
        # a list: every step appends the 32-bit stream after each scheduled layer (a copy, with what
        # the layer left pending added); for tests and debugging, not under a captured graph
        self.stream_tap = None
        if check:
            exp = expected_tensors(spec, store)
            store.check({n: ts.shape for n, ts in exp.items()}, spec.ignorable,
                        integer=[n for n, ts in exp.items() if ts.integer])
        self._validate_schedule()

        def bind(part: Part, **kw):
            part.bind(PartTensors(store, part.spec.prefix, _tensors_of(part, store), rt.compute_dtype, rt.device),
                      rt, **kw)

        bind(self.embedding)
        for b in self.blocks:
            for p in b.parts():
                bind(p)
        for j in self.joins:
            bind(j)
        bind(self.final_norm)
        bind(self.head, embedding=self.embedding)
        self.num_parameters = sum(
            int(torch.tensor(ts.shape).prod()) for ts in expected_tensors(spec).values()
        )

    # ---- cache needs -------------------------------------------------------------
    def _validate_schedule(self):
        writers: Dict[int, int] = {}
        for i, e in enumerate(self.spec.schedule):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer} of {len(self.blocks)}")
            if e.join is not None and not 0 <= e.join < len(self.joins):
                raise ValueError(f"schedule entry {i} names join {e.join} of {len(self.joins)}")
            mixer = self.blocks[e.layer].mixer
            own = getattr(mixer, "own_kv", True)
            if e.writes_cache:
                if e.cache in writers:
                    raise ValueError(f"cache entry {e.cache} is written by schedule entries {writers[e.cache]} and {i}")
                if not own:
                    raise ValueError(f"schedule entry {i} writes cache {e.cache} but its mixer projects no keys")
                writers[e.cache] = i
            else:
                if e.cache not in writers:
                    raise ValueError(f"schedule entry {i} reads cache {e.cache} before any entry wrote it")
                if own:
                    raise ValueError(f"schedule entry {i} reads another layer's cache but its mixer has keys of its own")
                a = mixer.kv_request()
                b = self.blocks[self.spec.schedule[writers[e.cache]].layer].mixer.kv_request()
                if a != b:
                    raise ValueError(f"schedule entry {i} reads cache {e.cache} with a different record shape")

    def kv_requests(self) -> Dict[int, Optional[KVRequest]]:
        out: Dict[int, Optional[KVRequest]] = {}
        for e in self.spec.schedule:
            if e.writes_cache:
                out[e.cache] = self.blocks[e.layer].mixer.kv_request()
        return out

    def state_requests(self) -> Dict[object, Optional[StateRequest]]:
        """State of fixed size per sequence, by key: a cache entry's number for its mixer,
        ("block", number) for what the block itself carries beside its mixer (every scheduled run of a
        layer has its own), "embedding" for the embedding."""
        out: Dict[object, Optional[StateRequest]] = {}
        for e in self.spec.schedule:
            if e.writes_cache:
                out[e.cache] = self.blocks[e.layer].mixer.state_request()
            own = getattr(self.blocks[e.layer], "state_request", None)
            if own is not None:
                if ("block", e.cache) in out:
                    raise ValueError(f"cache entry {e.cache} is used by two runs of blocks with state of their own")
                out[("block", e.cache)] = own()
        own = getattr(self.embedding, "state_request", None)
        if own is not None:
            out["embedding"] = own()
        return out

    # ---- one step ------------------------------------------------------------------
    def forward(self, batch, cache) -> Optional[torch.Tensor]:
        """Run the batch's tokens through every scheduled layer, appending to the cache;
        return float32 logits [len(want_rows), vocab], or None if no row is wanted."""
        rt = self.rt
        if hasattr(self.embedding, "state_request"):
            x = self.embedding.forward(rt, batch.token_ids, batch.num_tokens, batch, state=cache.state("embedding"))
        else:
            x = self.embedding.forward(rt, batch.token_ids, batch.num_tokens, batch)
        pending = None
        for j in self.joins:
            j.remember(rt, x)
        for e in self.spec.schedule:
            if e.join is not None:
                x, pending = self.joins[e.join].forward(rt, x, pending), None
            block = self.blocks[e.layer]
            if hasattr(block, "state_request"):
                x, pending = block.forward(rt, x, pending, batch, cache.view(e.cache), cache.state(e.cache),
                                           block_state=cache.state(("block", e.cache)))
            else:
                x, pending = block.forward(rt, x, pending, batch, cache.view(e.cache), cache.state(e.cache))
            if self.stream_tap is not None:
                d = pending.materialize(rt) if hasattr(pending, "materialize") else pending
                self.stream_tap.append(x.clone() if d is None else x + d)
        if batch.num_want == 0:
            return None
        h = self.final_norm.forward(rt, x, delta=delta_for(self.final_norm, pending, rt), rows=batch.want_rows,
                                    write_back=False)
        return self.head.forward(rt, h)
