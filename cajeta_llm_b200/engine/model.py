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
from ..parts.base import KvNeed, Runtime, StateNeed, make_part
from ..parts.plan import ModelPlan, ParamSpec
from ..weights.sources import RandomWeights, SafetensorsWeights


class Model:
    def __init__(self, plan: ModelPlan, runtime: Runtime):
        plan.validate()
        self.plan = plan
        self.runtime = runtime
        self.hidden = plan.hidden_size
        self.vocab = plan.vocab_size
        # both ends are parts like the layers' parts: the plan names their kinds
        self.embedding_part = make_part("embedding", plan.embedding, "", runtime, vocab_size=self.vocab,
                                        hidden_size=self.hidden, weight_name=plan.embedding_name)
        self.blocks = [make_part("block", layer.block, layer.prefix, runtime, layer=layer) for layer in plan.layers]
        self.final_norm = make_part("norm", plan.final_norm, plan.final_norm_prefix, runtime)
        self.head_part = make_part("head", plan.head, "", runtime, vocab_size=self.vocab, hidden_size=self.hidden,
                                   weight_name=plan.lm_head_name, embedding=self.embedding_part)

    def parts(self):
        return [self.embedding_part] + list(self.blocks) + [self.final_norm, self.head_part]

    @property
    def embedding(self) -> Optional[torch.Tensor]:
        """The embedding table (a tied head reads the same tensor)."""
        return getattr(self.embedding_part, "table", None)

    @property
    def lm_head(self) -> Optional[torch.Tensor]:
        return getattr(self.head_part, "weight", None)

    # -- tensors ---------------------------------------------------------------------
    def params(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for p in self.parts():
            out.update(p.params())
        return out

    def libraries(self) -> set:
        """The kernel libraries this model's steps will call (embedding, norms and head included)."""
        out = {"rowwise", "gemm_simt", "sampling"}
        for p in self.parts():
            out |= p.libraries()
        return out

    def load(self, source) -> None:
        source.check(self.params())
        for p in self.parts():
            p.load(source)

    # -- what the cache manager must provide, per schedule entry ---------------------
    def kv_needs(self) -> List[Optional[KvNeed]]:
        return [self.blocks[e.layer].mixer.cache_need() for e in self.plan.schedule]

    def state_needs(self) -> List[Optional[StateNeed]]:
        return [self.blocks[e.layer].mixer.state_need() for e in self.plan.schedule]

    def cache_from(self) -> List[Optional[int]]:
        return [e.cache_from for e in self.plan.schedule]

    # -- the pieces of a step outside the blocks -------------------------------------
    def embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.embedding_part.forward(token_ids)

    def logits(self, hs: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Final norm and head on the wanted rows only; float32 ``[len(rows), vocab]``
        (model/CausalLM.cajeta:1712-1718)."""
        x, _ = self.final_norm.forward(hs, row_index=rows)
        return self.head_part.forward(x)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self._tensors():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _tensors(self):
        stack = self.parts()
        while stack:
            p = stack.pop()
            for v in vars(p).values():
                if isinstance(v, torch.Tensor):
                    yield v
                elif hasattr(v, "params") and hasattr(v, "runtime") and v is not getattr(p, "embedding", None):
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
