"""Block arrangements: how a layer's mixer, feed-forward and norms are wired.

``prenorm``: ``hs += mixer(norm_1(hs)); hs += feed_forward(norm_2(hs))`` with the
residual stream ``hs`` in float32 (model/DecoderLayer.cajeta:38-75,
model/CausalLM.cajeta:1445-1446,1506,1512-1517,1575).  Parameters: the tensor-name
pieces ``mixer_norm_name``, ``feed_forward_norm_name``, ``mixer_name``,
``feed_forward_name`` under the layer's prefix.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import Part, make_part, register_part
from .plan import LayerSpec, ParamSpec


@register_part("block", "prenorm")
class PreNormBlock(Part):
    def __init__(self, spec, prefix, runtime, layer: LayerSpec):
        super().__init__(spec, prefix, runtime)
        self.mixer_norm = make_part("norm", layer.mixer_norm, self.name(spec["mixer_norm_name"]), runtime)
        self.mixer = make_part("mixer", layer.mixer, self.name(spec["mixer_name"]), runtime)
        self.feed_forward_norm = make_part("norm", layer.feed_forward_norm, self.name(spec["feed_forward_norm_name"]), runtime)
        self.feed_forward = make_part("feed_forward", layer.feed_forward, self.name(spec["feed_forward_name"]), runtime)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.params())
        return out

    def libraries(self) -> set:
        out = set()
        for p in self.parts():
            out |= p.libraries()
        return out

    def load(self, source) -> None:
        for p in self.parts():
            p.load(source)

    def forward(self, hs: torch.Tensor, ctx, entry) -> None:
        x, _ = self.mixer_norm.forward(hs)
        # a mixer may return partial sums it still owes the residual stream ([S, rows, H]
        # float32, from a product split along K); the next norm adds them as it reads hs
        pending = self.mixer.forward(x, hs, ctx, entry)
        # the feed-forward may want its input once more in float32 (a router), or, for many
        # rows, as three bfloat16 terms that a tensor-core product can sum to the same grade
        ff = self.feed_forward
        wants_split = getattr(ff, "wants_split_input", None)
        split = bool(wants_split and wants_split(hs.shape[0]))
        x, x_exact = self.feed_forward_norm.forward(hs, want_f32=getattr(ff, "needs_f32_input", False) and not split,
                                                    pending=pending, want_split=split)
        ff.forward(x, x_exact, hs, ctx)
