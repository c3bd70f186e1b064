"""A model built from a plan: embedding, blocks, final norm, language-model head.

The model class is the same for every architecture; what differs is the
:class:`cajeta_llm_b200.parts.plan.ModelPlan` the architecture's registry entry builds
from ``config.json`` (the reference likewise serves every family with one ``CausalLM``
over ``DecoderModel``/``DecoderLayer``, model/DecoderModel.cajeta:17-48,
model/CausalLM.cajeta:64-94; the head is tied to the embedding when the plan says so,
model/CausalLM.cajeta:625-631).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.base import ModelConfig, get_architecture, load_config
from ..csrc import kernels as K
from ..parts.base import KvNeed, Runtime, StateNeed, make_part
from ..parts.linear import project
from ..parts.plan import ModelPlan, ParamSpec
from ..weights.sources import RandomWeights, SafetensorsWeights


class Model:
    def __init__(self, plan: ModelPlan, runtime: Runtime):
        plan.validate()
        self.plan = plan
        self.runtime = runtime
        self.hidden = plan.hidden_size
        self.vocab = plan.vocab_size
        self.blocks = [make_part("block", layer.block, layer.prefix, runtime, layer=layer) for layer in plan.layers]
        self.final_norm = make_part("norm", plan.final_norm, plan.final_norm_prefix, runtime)
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None

    # -- tensors ---------------------------------------------------------------------
    def params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {self.plan.embedding_name: ParamSpec((self.vocab, self.hidden))}
        for b in self.blocks:
            out.update(b.params())
        out.update(self.final_norm.params())
        if self.plan.lm_head_name is not None:
            out[self.plan.lm_head_name] = ParamSpec((self.vocab, self.hidden))
        return out

    def libraries(self) -> set:
        """The kernel libraries this model's steps will call (embedding, norms and head included)."""
        out = {"rowwise", "gemm_simt", "sampling"}
        for b in self.blocks:
            out |= b.libraries()
        out |= self.final_norm.libraries()
        if self.runtime.fast_kernels and self.hidden >= 128:
            out.add("gemm_tc")
        return out

    def load(self, source) -> None:
        schema = self.params()
        source.check(schema)
        rt = self.runtime
        name = self.plan.embedding_name
        self.embedding = rt.place(source.get(name, schema[name]), schema[name])
        for b in self.blocks:
            b.load(source)
        self.final_norm.load(source)
        if self.plan.lm_head_name is not None:
            name = self.plan.lm_head_name
            self.lm_head = rt.place(source.get(name, schema[name]), schema[name])
        else:
            self.lm_head = self.embedding

    # -- what the cache manager must provide, per schedule entry ---------------------
    def kv_needs(self) -> List[Optional[KvNeed]]:
        return [self.blocks[e.layer].mixer.cache_need() for e in self.plan.schedule]

    def state_needs(self) -> List[Optional[StateNeed]]:
        return [self.blocks[e.layer].mixer.state_need() for e in self.plan.schedule]

    def cache_from(self) -> List[Optional[int]]:
        return [e.cache_from for e in self.plan.schedule]

    # -- the pieces of a step outside the blocks -------------------------------------
    def embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        hs = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        K.embed_gather(hs, self.embedding, token_ids)
        return hs

    def logits(self, hs: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Final norm and head on the wanted rows only; float32 ``[len(rows), vocab]``
        (model/CausalLM.cajeta:1712-1718)."""
        x, _ = self.final_norm.forward(hs, row_index=rows)
        out = torch.empty((rows.numel(), self.vocab), dtype=torch.float32, device=hs.device)
        project(self.runtime, x, self.lm_head, out)
        return out

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self._tensors():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _tensors(self):
        yield self.embedding
        yield self.lm_head
        stack = list(self.blocks) + [self.final_norm]
        while stack:
            p = stack.pop()
            for v in vars(p).values():
                if isinstance(v, torch.Tensor):
                    yield v
                elif hasattr(v, "params") and hasattr(v, "runtime"):
                    stack.append(v)


def build_model(config: ModelConfig, runtime: Runtime) -> Model:
    """The model class is chosen by the configuration's architecture name."""
    arch = get_architecture(config.architecture)
    return Model(arch.build_plan(config), runtime)


def load_model(model_dir: str, runtime: Runtime) -> "tuple[Model, ModelConfig]":
    """config.json -> architecture -> plan -> model, then the weights by tensor name."""
    config = load_config(model_dir)
    model = build_model(config, runtime)
    source = SafetensorsWeights(model_dir)
    try:
        model.load(source)
    finally:
        source.close()
    return model, config


def random_model(config: ModelConfig, runtime: Runtime, seed: int, store_dtype: torch.dtype = torch.bfloat16,
                 on_device: bool = True) -> Model:
    """A model with seeded random weights drawn in place (no file)."""
    model = build_model(config, runtime)
    model.load(RandomWeights(seed, store_dtype=store_dtype, device=str(runtime.device) if on_device else "cpu"))
    return model
