"""The arrangement of a layer's parts.

``PreNormBlock`` is the Llama layer (``lua/lgml/transformer.lua:2312-2345``):
x = x + mixer(norm(x)); x = x + ffn(norm(x)).  The residual stream x stays
float32 and every sum into it is a float32 add.  A sum and the norm that follows
it are one kernel, so a block hands its last delta on as ``pending`` and the next
norm (the next block's, or the model's final norm) adds it.
"""
from __future__ import annotations

from .. import ops
from .base import Part, register_part


class PreNormBlock(Part):
    def __init__(self, mixer_norm, mixer, ffn_norm, ffn, names=None):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        # tensor-name stems of the four parts under the layer's prefix
        self.names = names or {"mixer_norm": "input_layernorm", "mixer": "self_attn",
                               "ffn_norm": "post_attention_layernorm", "ffn": "mlp"}

    def _parts(self, prefix):
        for key in ("mixer_norm", "mixer", "ffn_norm", "ffn"):
            part = getattr(self, key)
            if part is not None:
                yield part, f"{prefix}.{self.names[key]}"

    def tensor_specs(self, prefix):
        return [s for part, p in self._parts(prefix) for s in part.tensor_specs(p)]

    def bind(self, prefix, tensors, rt):
        for part, p in self._parts(prefix):
            part.bind(p, tensors, rt)

    def cache_spec(self):
        return self.mixer.cache_spec() if self.mixer is not None else None

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    def forward(self, rt, x, pending, batch, cache):
        if self.mixer is not None:
            h = self.mixer_norm.forward(rt, x, rt.dtype, delta=pending)
            if self.ffn is not None:
                first = getattr(self.ffn, "first_weights", None)
                if first is not None:
                    rt.ahead(first())       # read after the mixer: L2 may fetch their head meanwhile
            pending = self.mixer.forward(rt, h, batch, cache)
        if self.ffn is not None:
            h = self.ffn_norm.forward(rt, x, rt.dtype, delta=pending)
            pending = self.ffn.forward(rt, h)
        return x, pending


register_part("block", "pre_norm", PreNormBlock)
