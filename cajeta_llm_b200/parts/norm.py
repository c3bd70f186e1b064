"""RMSNorm part.

``ss = sum x_i^2; scale = 1 / sqrt(ss / dim + eps); y_i = x_i * scale * w_i`` with the
statistics in float32 (model/Prim.cajeta:120-151; weight and eps held per norm,
model/RMSNorm.cajeta:14-53).  Parameters: ``dim``, ``eps``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..csrc import kernels as K
from .base import Part, register_part
from .plan import ParamSpec


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.dim = int(spec["dim"])
        self.eps = float(spec["eps"])
        self.weight: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        return {self.name("weight"): ParamSpec((self.dim,), role="vector", init="ones")}

    def libraries(self) -> set:
        return {"rowwise"}

    def load(self, source) -> None:
        self.weight = self.fetch(source, self.name("weight"))

    def forward(self, x: torch.Tensor, want_f32: bool = False, row_index: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, pending: Optional[torch.Tensor] = None,
                want_split: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Normalise rows of the float32 residual stream.

        Returns the result in the activation dtype and, when ``want_f32``, also in
        float32 (the same tensor on the 32-bit path).  ``row_index`` (int32) picks the
        rows to normalise.  ``pending`` ([S, rows, dim] float32) are partial sums still
        owed to the residual stream by the part before: they are added to ``x`` (in
        order, ``x`` keeps the sum) in the same pass.  ``want_split`` (instead of
        ``want_f32``): the second result is bfloat16 ``[rows, 3 * dim]``, the float32 value
        as three bfloat16 terms hi | mid | lo whose sum is the value to 2^-24 - the form a
        tensor-core product needs to give float32-grade sums."""
        rt = self.runtime
        rows = x.shape[0] if row_index is None else row_index.numel()
        dtype = out_dtype or rt.act_dtype
        out = torch.empty((rows, self.dim), dtype=dtype, device=x.device)
        out_f32 = None
        if want_split:
            split = torch.empty((rows, 3 * self.dim), dtype=torch.bfloat16, device=x.device)
            K.rmsnorm(x, self.weight, self.eps, out, None, row_index, pending, out_split=split)
            return out, split
        if want_f32:
            out_f32 = out if dtype == torch.float32 else torch.empty((rows, self.dim), dtype=torch.float32, device=x.device)
        K.rmsnorm(x, self.weight, self.eps, out, out_f32 if out_f32 is not out else None, row_index, pending)
        return out, out_f32
