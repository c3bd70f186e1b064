"""The data that describes a model: part specs, layer specs, run order, tensor names.

A model is not a class per architecture.  An architecture's ``build_plan`` turns its
configuration into a :class:`ModelPlan`, which is plain data:

* every part (mixer, feed-forward, norm, position encoding) is a :class:`PartSpec`:
  a registered ``kind`` plus the sizes and constants that part needs, chosen layer
  by layer;
* ``schedule`` is the order in which layers run: a list of :class:`ScheduleEntry`,
  which may name a layer twice or let an entry read the cache another entry wrote.

The reference varies one set of classes by configuration flags
(model/DecoderLayer.cajeta:38-75 picks ``mlp`` or ``moe`` for all layers alike,
model/ModelConfig.cajeta:151-164 gives a window per layer); here the choice is per
layer and the result is data the engine walks.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A registered part ``kind`` with its parameters (sizes, constants, nested specs)."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "params", MappingProxyType(dict(self.params)))

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part reads from the weight file.

    ``role`` decides how the engine holds it: ``"matrix"`` follows the engine dtype
    (bfloat16 when serving, float32 on the 32-bit path); ``"vector"`` (norm weights,
    biases, router and gate rows: small, used in 32-bit arithmetic) is held in
    float32, which is exact for a bfloat16 file and leaves a 32-bit file as it is;
    ``"table"`` is an integer table held as int32.
    ``init`` is what the random-weights mode draws: ``"normal"`` N(0, std), ``"ones"``
    or ``"zeros"``.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    std: float = 0.02


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer, a feed-forward and norms.

    ``prefix`` is the tensor-name prefix of the layer (for example
    ``model.layers.3``); each part appends its own tensor names.
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelPlan.layers``.  ``cache_from`` is None when the entry
    owns a cache plane (it writes keys and values and reads them); otherwise it is
    the index of an earlier schedule entry whose plane this entry reads without
    writing.
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    """Everything the engine needs to build and run one model."""

    architecture: str
    hidden_size: int
    vocab_size: int
    embedding_name: str
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str
    lm_head_name: Optional[str]          # None: tied to the embedding table
    eog_token_ids: Tuple[int, ...] = ()
    max_position: Optional[int] = None
    embedding: PartSpec = PartSpec("token_embedding")     # how token ids become rows of the residual stream
    head: PartSpec = PartSpec("linear_head")              # how the normed wanted rows become logits

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}; the plan has {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which does not run before it")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which owns none")
