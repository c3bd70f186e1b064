"""The two ends of a model: token embedding and language-model head.

``token_embedding`` (category ``embedding``): ``hs[t, :] = W[token_t, :]`` widened to the
float32 residual stream, times ``scale`` when one is given (the reference's
``embedScale``, 0 = none: model/Embedding.cajeta:73-81, model/HostOps.cajeta:32-49).
Parameters: ``scale`` (optional).  Must offer ``forward(token_ids int32 [T]) -> float32
[T, hidden]`` and ``table`` (the ``[vocab, hidden]`` tensor, which a tied head reads).

``linear_head`` (category ``head``): ``logits = x W^T (+ b)`` in float32 on the rows it is
given (the final norm has already picked and normed the wanted rows:
model/CausalLM.cajeta:1712-1718); ``W`` is the embedding table when the plan names no
head tensor (model/CausalLM.cajeta:625-631).  Parameters: ``bias`` (optional, default
false; its tensor is the head's name with ``weight`` replaced by ``bias``).  Must offer
``forward(x [rows, hidden]) -> float32 [rows, vocab]``.

Both are built by the model with the plan's sizes and tensor names as keyword arguments
(``vocab_size``, ``hidden_size``, ``weight_name``; the head also gets ``embedding``, the
embedding part), so that a kind of its own - a scaled or factorised embedding, a head with a
soft cap - needs no change to the model class.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import kernels as K
from .base import Part, register_part
from .linear import project
from .plan import ParamSpec


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, spec, prefix, runtime, vocab_size: int, hidden_size: int, weight_name: str):
        super().__init__(spec, prefix, runtime)
        self.vocab = int(vocab_size)
        self.hidden = int(hidden_size)
        self.weight_name = weight_name
        self.scale = float(spec.get("scale", 0.0) or 0.0)
        self.table: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.vocab, self.hidden))}

    def libraries(self) -> set:
        return {"rowwise"}

    def load(self, source) -> None:
        self.table = self.fetch(source, self.weight_name)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        hs = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        K.tag = "embedding"
        K.embed_gather(hs, self.table, token_ids, self.scale)
        K.tag = None
        return hs


@register_part("head", "linear_head")
class LinearHead(Part):
    def __init__(self, spec, prefix, runtime, vocab_size: int, hidden_size: int, weight_name: Optional[str], embedding: Part):
        super().__init__(spec, prefix, runtime)
        self.vocab = int(vocab_size)
        self.hidden = int(hidden_size)
        self.weight_name = weight_name               # None: tied to the embedding table
        self.embedding = embedding
        self.has_bias = bool(spec.get("bias", False))
        if self.has_bias and weight_name is None:
            raise ValueError("a head tied to the embedding table has no tensor name to derive its bias from")
        self.bias_name = weight_name[: -len("weight")] + "bias" if self.has_bias and weight_name.endswith("weight") else (
            f"{weight_name}.bias" if self.has_bias else None)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        if self.weight_name is not None:
            out[self.weight_name] = ParamSpec((self.vocab, self.hidden))
        if self.bias_name is not None:
            out[self.bias_name] = ParamSpec((self.vocab,), role="vector")
        return out

    def libraries(self) -> set:
        libs = {"gemm_simt"}
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs.add("gemm_tc")
        return libs

    def load(self, source) -> None:
        self.weight = self.fetch(source, self.weight_name) if self.weight_name is not None else self.embedding.table
        if self.bias_name is not None:
            self.bias = self.fetch(source, self.bias_name)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.vocab), dtype=torch.float32, device=x.device)
        K.tag = "head"
        project(self.runtime, x, self.weight, out, bias=self.bias)
        K.tag = None
        return out
