"""A decoder put together from parts, and the order in which its layers run.

``DecoderModel`` holds an embedding, a list of blocks, a final norm and a head.
The order of execution is data: ``schedule`` is a list of ``LayerCall``; a call
names the block to run and the call whose cache it uses.  By default call i runs
block i on a cache of its own.  A schedule may name a block twice (each call
that owns a cache gets its own), or let a call read the cache an earlier call
wrote (the reference's ``kv_src`` layers, ``lua/lgml/transformer.lua:1829-1830``,
``:592``).  mischief/lgml's loop over layers is ``M:forward``
(``:2285-2365``): embedding (``:2303``), the layers (``:2312-2345``), the rows
whose logits are wanted (``:2349-2350``), the final norm and the head
(``:2095-2096``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..weights import TensorSpec


@dataclass(frozen=True)
class LayerCall:
    block: int                    # index into DecoderModel.blocks
    cache: Optional[int] = None   # index of the call that owns the cache used; None = this call


class DecoderModel:
    def __init__(self, config, embedding, blocks, final_norm, head, schedule: Optional[List[LayerCall]] = None,
                 block_prefix: str = "model.layers.{}", final_norm_prefix: str = "model.norm",
                 embed_scale: Optional[float] = None, logit_scale: Optional[float] = None, logit_softcap: Optional[float] = None,
                 ignored_tensors: Sequence[str] = ()):
        self.config = config
        self.embedding = embedding
        self.blocks = list(blocks)
        self.final_norm = final_norm
        self.head = head
        self.block_prefix = block_prefix
        self.final_norm_prefix = final_norm_prefix
        # name patterns of tensors that a folder of this architecture may carry unread
        self.ignored_tensors = tuple(ignored_tensors)
        # scales that other families of the reference apply and Llama does not (None = no kernel):
        # on the embedding's rows (``embd_scale``, ``lua/lgml/transformer.lua:2303-2306``), on the
        # logits, and the logits' cap (``logit_scale``, ``softcap``, ``:2097-2102``)
        self.embed_scale, self.logit_scale, self.logit_softcap = embed_scale, logit_scale, logit_softcap
        self.schedule = list(schedule) if schedule is not None else [LayerCall(i) for i in range(len(self.blocks))]
        for ci, call in enumerate(self.schedule):
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"schedule entry {ci} names block {call.block}, but there are {len(self.blocks)}")
            if call.cache is not None:
                if not 0 <= call.cache < ci:
                    raise ValueError(f"schedule entry {ci} reads the cache of entry {call.cache}, which does not run before it")
                if self.schedule[call.cache].cache is not None:
                    raise ValueError(f"schedule entry {ci} reads the cache of entry {call.cache}, which has none of its own")
        self.vocab_size = head.vocab
        parts = [embedding, final_norm, head] + self.blocks
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in parts)
        self.max_position = getattr(config, "max_position_embeddings", None)

    # ---- weights -----------------------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        specs = list(self.embedding.tensor_specs(""))
        for i, b in enumerate(self.blocks):
            specs += b.tensor_specs(self.block_prefix.format(i))
        specs += self.final_norm.tensor_specs(self.final_norm_prefix)
        specs += self.head.tensor_specs("")
        seen = {}
        for s in specs:          # a tensor two parts share (e.g. frequency factors) is listed once
            seen.setdefault(s.name, s)
        return list(seen.values())

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.embedding.bind("", tensors, rt)
        for i, b in enumerate(self.blocks):
            b.bind(self.block_prefix.format(i), tensors, rt)
        self.final_norm.bind(self.final_norm_prefix, tensors, rt)
        self.head.bind("", tensors, rt)

    # ---- cache -------------------------------------------------------------------------
    def cache_layout(self) -> Dict[int, object]:
        """schedule index -> the cache spec of the calls that own a cache."""
        out = {}
        for ci, call in enumerate(self.schedule):
            if call.cache is None:
                spec = self.blocks[call.block].cache_spec()
                if spec is not None:
                    out[ci] = spec
        return out

    # ---- the forward pass of one step --------------------------------------------------
    def forward(self, rt, batch) -> torch.Tensor:
        """float32 logits [len(batch.logit_rows), vocab] for the tokens of ``batch``."""
        x = self.embedding.forward(rt, batch.token_ids)
        if self.embed_scale is not None:
            ops.scale_cap(x, self.embed_scale)
        pending = None
        for ci, call in enumerate(self.schedule):
            owner = ci if call.cache is None else call.cache
            cache = batch.cache_view(owner, writable=call.cache is None)
            x, pending = self.blocks[call.block].forward(rt, x, pending, batch, cache)
        h = self.final_norm.forward(rt, x, rt.dtype, delta=pending, rows=batch.logit_rows)
        logits = self.head.forward(rt, h)
        if self.logit_scale is not None or self.logit_softcap:
            ops.scale_cap(logits, 1.0 if self.logit_scale is None else self.logit_scale, self.logit_softcap or 0.0)
        return logits
