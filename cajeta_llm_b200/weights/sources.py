"""Where a model's tensors come from: a folder of safetensors, or a seed.

Both sources answer ``get(name) -> host-or-device tensor`` for the names a model's
parts declare (:class:`cajeta_llm_b200.parts.plan.ParamSpec`).  Before anything is
loaded :func:`check_schema` compares the declared names and shapes with what the
source holds and raises ONE error that lists every missing tensor, every unexpected
tensor and every wrong shape (the reference names one tensor at a time:
io/Checkpoint.cajeta:495-499, model/Linear.cajeta:1857-1867, model/RMSNorm.cajeta:45-48).

The random-weights mode draws bell-shaped values of mean 0 and a given standard deviation
for matrices, biases and router rows, ones for norm weights (the reference has such weights
only as test fixtures, selftest/ToyModel.cajeta:116-120); a value depends on (seed, tensor
name, element index) only, so neither the order of generation nor the device matters.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Tuple

import torch

from ..parts.plan import ParamSpec
from . import random_fill
from .safetensors_io import Checkpoint, write_safetensors


class WeightError(ValueError):
    """The weights do not fit the model; lists every problem found."""


def check_schema(schema: Mapping[str, ParamSpec], have: Mapping[str, Tuple[int, ...]], where: str) -> None:
    missing = [n for n in schema if n not in have]
    unexpected = [n for n in have if n not in schema]
    wrong = [(n, tuple(schema[n].shape), tuple(have[n])) for n in schema
             if n in have and tuple(have[n]) != tuple(schema[n].shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not fit the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}):")
        lines += [f"    {n} {list(schema[n].shape)}" for n in missing]
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}):")
        lines += [f"    {n} {list(have[n])}" for n in unexpected]
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}):")
        lines += [f"    {n}: expected {list(e)}, found {list(f)}" for n, e, f in wrong]
    raise WeightError("\n".join(lines))


class SafetensorsWeights:
    """Tensors of a model folder, by name, in the dtype the file stores."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.checkpoint = Checkpoint(model_dir)

    def check(self, schema: Mapping[str, ParamSpec]) -> None:
        have = {n: self.checkpoint.shape_of(n) for n in self.checkpoint.names()}
        check_schema(schema, have, self.model_dir)

    def get(self, name: str, spec: ParamSpec) -> torch.Tensor:
        return self.checkpoint.load(name)

    def close(self) -> None:
        self.checkpoint.close()


class RandomWeights:
    """Seeded random tensors by name.

    A value depends on (seed, tensor name, element index) only
    (:mod:`cajeta_llm_b200.weights.random_fill`): ``device`` chooses where the values are
    computed - on the host when a model folder is written, by a kernel to fill a large model
    in place without a file - and both give the same bits, so that whoever knows the seed can
    rebuild any tensor of a model drawn on the device.  ``store_dtype`` is the dtype a file of
    these weights would store (values are rounded to it, to nearest even).
    """

    def __init__(self, seed: int, store_dtype: torch.dtype = torch.bfloat16, device: str = "cpu"):
        if store_dtype not in (torch.bfloat16, torch.float32):
            raise WeightError(f"random weights are stored as bfloat16 or float32, not {store_dtype}")
        self.seed = int(seed)
        self.store_dtype = store_dtype
        self.device = torch.device(device)

    def check(self, schema: Mapping[str, ParamSpec]) -> None:
        return None

    def get(self, name: str, spec: ParamSpec) -> torch.Tensor:
        if spec.role == "table":
            raise WeightError(f"random weights cannot draw the integer table '{name}'")
        if spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=self.device)
        elif spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=torch.float32, device=self.device)
        elif spec.init == "normal":
            key = random_fill.tensor_key(self.seed, name)
            count = 1
            for n in spec.shape:
                count *= int(n)
            if self.device.type == "cuda":
                from ..csrc import kernels as K
                t = torch.empty(spec.shape, dtype=self.store_dtype, device=self.device)
                with torch.cuda.device(self.device):
                    K.random_fill(t, key, float(random_fill.scale_for(spec.std)))
                return t
            t = torch.from_numpy(random_fill.fill(count, key, spec.std)).reshape(spec.shape)
        else:
            raise WeightError(f"tensor '{name}': unknown init '{spec.init}'")
        return t.to(self.store_dtype)

    def close(self) -> None:
        return None


def write_model_folder(model_dir: str, config, schema: Mapping[str, ParamSpec], seed: int,
                       store_dtype: torch.dtype = torch.bfloat16) -> None:
    """The random-weights mode: ``config.json`` and ``model.safetensors`` from a
    configuration and a seed."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_json_dict(), f, indent=2)
    src = RandomWeights(seed, store_dtype=store_dtype, device="cpu")
    tensors: Dict[str, torch.Tensor] = {name: src.get(name, spec) for name, spec in schema.items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
