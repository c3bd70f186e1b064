"""Interfaces of the parts a layer is put together from, and their registry.

A part is built from a :class:`PartSpec` (its sizes and constants), the tensor-name
prefix it lives under and the :class:`Runtime` (device, dtypes).  It declares the
tensors it reads (:meth:`Part.params`), loads them (:meth:`Part.load`) and runs on the
rows of one step.  No part knows which model it is in: everything it needs arrives in
its spec or in the step's context.

Categories and what each must offer
-----------------------------------
``norm``          ``forward(x_f32, want_f32=False, row_index=None, pending=None) -> (y, y_f32 | None)``
``position``      ``rotary_dim`` and ``inv_freq`` (float32 device tensor, rotary_dim / 2)
``mixer``         ``cache_need()``, ``state_need()``, ``forward(x, residual, ctx, entry) -> None | pending``
``feed_forward``  ``needs_f32_input``, ``forward(x, x_f32, residual, ctx)``
``block``         ``forward(hs, ctx, entry)`` over its mixer, feed-forward and norms
``embedding``     ``forward(token_ids) -> float32 [T, hidden]``, ``table``
``head``          ``forward(x [rows, hidden]) -> float32 [rows, vocab]``

``x`` is the normed input in the activation dtype, ``residual`` the float32 residual
stream the part adds its result into (the residual sum is always 32-bit; a mixer may
instead return ``pending``, float32 partial sums [S, rows, H] that the next norm adds), ``ctx`` the
:class:`cajeta_llm_b200.engine.step.StepContext` of the step and ``entry`` the
:class:`cajeta_llm_b200.engine.step.EntryContext` of the schedule entry being run
(its cache plane, block table and state slots).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple, Type

import torch

from .plan import ParamSpec, PartSpec

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class Runtime:
    """Device and dtypes of one engine instance.

    ``dtype == "bfloat16"``: matrices, activations between kernels and the cache are
    bfloat16; statistics, sums, the residual stream, router inputs and logits are
    float32.  ``dtype == "float32"``: everything is float32 and every product runs on
    the FMA pipe (no reduced-precision matrix mode).
    """

    def __init__(self, dtype: str = "bfloat16", device: str = "cuda:0", fast_kernels: bool = True):
        if dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {sorted(DTYPES)}, found '{dtype}'")
        self.dtype_name = dtype
        self.act_dtype = DTYPES[dtype]
        self.matrix_dtype = DTYPES[dtype]
        self.cache_dtype = DTYPES[dtype]
        self.device = torch.device(device)
        self.fast_kernels = fast_kernels and dtype == "bfloat16"
        self._decode_scratch = None
        self._sm_count = None

    @property
    def sm_count(self) -> int:
        """Streaming multiprocessors of the device (148 on a B200), asked of the device once;
        tile and split choices that aim at filling the machine use this, never a constant."""
        if self._sm_count is None:
            self._sm_count = (torch.cuda.get_device_properties(self.device).multi_processor_count
                              if self.device.type == "cuda" else 1)
        return self._sm_count

    @property
    def decode_scratch(self):
        """Scratch of the split-KV decode attention, shared by all layers (one stream)."""
        if self._decode_scratch is None:
            from ..csrc.kernels import DecodeScratch
            self._decode_scratch = DecodeScratch()
        return self._decode_scratch

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=self.matrix_dtype).contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def table(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.int32).contiguous()

    def place(self, t: torch.Tensor, spec: ParamSpec) -> torch.Tensor:
        if spec.role == "matrix":
            return self.matrix(t)
        if spec.role == "vector":
            return self.vector(t)
        if spec.role == "table":
            return self.table(t)
        raise ValueError(f"unknown tensor role '{spec.role}'")

    def empty(self, *shape: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.act_dtype, device=self.device)


@dataclass(frozen=True)
class KvNeed:
    """A mixer that caches keys and values: pages of ``kv_heads x head_dim`` per token;
    ``window`` > 0 means only the last ``window`` positions are ever read."""

    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps per-request state of fixed size (one slot per request)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    category = ""

    def __init__(self, spec: PartSpec, prefix: str, runtime: Runtime):
        self.spec = spec
        self.prefix = prefix
        self.runtime = runtime

    def name(self, suffix: str) -> str:
        return f"{self.prefix}.{suffix}" if self.prefix else suffix

    def params(self) -> Dict[str, ParamSpec]:
        """Tensor name -> what the weight file must hold under it."""
        return {}

    def libraries(self) -> set:
        """Names of the kernel libraries (``csrc/build.py``) this part's steps will call: a hint,
        so that a model's libraries can be compiled side by side before its first step instead
        of one after the other as they are first wanted.  Nothing breaks if a part names none."""
        return set()

    def load(self, source: Any) -> None:
        """Fetch the declared tensors from ``source.get(name, spec)`` onto the device."""
        return None

    def fetch(self, source: Any, name: str) -> torch.Tensor:
        cache = getattr(self, "_params_cache", None)
        if cache is None:
            cache = self._params_cache = self.params()
        spec = cache[name]
        return self.runtime.place(source.get(name, spec), spec)


_REGISTRY: Dict[Tuple[str, str], Type[Part]] = {}
CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")


def register_part(category: str, kind: str, cls: Optional[Type[Part]] = None, replace: bool = False):
    """Register a part class; usable as a decorator: ``@register_part("mixer", "toy")``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category '{category}'; categories: {', '.join(CATEGORIES)}")

    def do(c: Type[Part]) -> Type[Part]:
        if (category, kind) in _REGISTRY and not replace:
            raise ValueError(f"{category} '{kind}' is already registered")
        c.category = category
        _REGISTRY[(category, kind)] = c
        return c

    return do(cls) if cls is not None else do


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.pop((category, kind), None)


def registered_parts(category: str) -> Tuple[str, ...]:
    return tuple(sorted(k for c, k in _REGISTRY if c == category))


def make_part(category: str, spec: PartSpec, prefix: str, runtime: Runtime, **extra: Any) -> Part:
    cls = _REGISTRY.get((category, spec.kind))
    if cls is None:
        raise ValueError(f"no {category} of kind '{spec.kind}' is registered; registered: "
                         f"{', '.join(registered_parts(category)) or '(none)'}")
    return cls(spec, prefix, runtime, **extra)
