"""Feed-forward parts: the dense SwiGLU MLP and the sparse mixture of experts.

``dense_swiglu``: ``W_d (silu(W_g x) * (W_u x))``, ``silu(x) = x / (1 + exp(-x))``
(model/Prim.cajeta:1822-1847, model/CausalLM.cajeta:1556-1566).  Parameters:
``hidden_size``, ``intermediate_size``.

``sparse_moe``: router logits ``l_e = Wr[e] . x`` in float32, softmax over all experts,
top-k by repeated strict-``>`` argmax (ties to the lower index), weights = the picked
probabilities, optionally renormalised with the divisor clamped at 2^-14
(model/MoeFfn.cajeta:908-988); each picked expert is a SwiGLU MLP of
``expert_intermediate_size``, summed per token in selection order
(model/MoeFfn.cajeta:1849-1916); an optional shared expert of
``shared_intermediate_size`` is added, scaled by ``sigma(g . x)`` when it has a gate
(model/MoeFfn.cajeta:1925-1964).  Tokens are grouped by expert with a counting sort and
each expert multiplies its own rows (model/MoeFfn.cajeta:2064-2099,2644-2777).  When the
shared expert's width is a multiple of the experts' width it is cut into chunks of that
width which ride through the same two grouped products as extra groups that every token
belongs to (their partial down-projections are summed in chunk order by the combine):
one launch streams all expert weights of the layer.
Parameters: ``hidden_size``, ``num_experts``, ``top_k``, ``expert_intermediate_size``,
``shared_intermediate_size`` (0 = none), ``shared_gate``, ``norm_topk_prob``.

The file stores one tensor per expert and projection
(``experts.{e}.gate_proj.weight`` ...); they are stacked into ``[E, I, H]`` and
``[E, H, I]`` slabs at load, as the reference binds merged slabs
(model/ExpertBank.cajeta:243-308).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import kernels as K
from .base import Part, register_part
from .linear import project
from .plan import ParamSpec


@register_part("feed_forward", "dense_swiglu")
class DenseSwiGLU(Part):
    needs_f32_input = False

    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.w_gate = self.w_up = self.w_down = None

    def params(self) -> Dict[str, ParamSpec]:
        return {
            self.name("gate_proj.weight"): ParamSpec((self.inter, self.hidden)),
            self.name("up_proj.weight"): ParamSpec((self.inter, self.hidden)),
            self.name("down_proj.weight"): ParamSpec((self.hidden, self.inter)),
        }

    def libraries(self) -> set:
        libs = {"gemm_simt"}
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs |= {"gemm_tc", "gemm_tc2"}
        return libs

    def load(self, source) -> None:
        self.w_gate = self.fetch(source, self.name("gate_proj.weight"))
        self.w_up = self.fetch(source, self.name("up_proj.weight"))
        self.w_down = self.fetch(source, self.name("down_proj.weight"))

    def forward(self, x: torch.Tensor, x_f32: Optional[torch.Tensor], residual: torch.Tensor, ctx) -> None:
        T = x.shape[0]
        act = torch.empty((T, self.inter), dtype=self.runtime.act_dtype, device=x.device)
        K.tag = "dense gate/up"
        project(self.runtime, x, self.w_gate, act, w_up=self.w_up)
        K.tag = "dense down"
        project(self.runtime, act, self.w_down, residual, accumulate=True)
        K.tag = None


@register_part("feed_forward", "sparse_moe")
class SparseMoE(Part):
    needs_f32_input = True      # the router reads the normed row in float32

    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.num_experts = int(spec["num_experts"])
        self.top_k = int(spec["top_k"])
        self.inter = int(spec["expert_intermediate_size"])
        self.shared_inter = int(spec.get("shared_intermediate_size", 0) or 0)
        self.shared_gate = bool(spec.get("shared_gate", False)) and self.shared_inter > 0
        self.norm_topk = bool(spec.get("norm_topk_prob", False))
        if not 1 <= self.top_k <= self.num_experts:
            raise ValueError(f"top_k must be between 1 and num_experts ({self.num_experts}), found {self.top_k}")
        if self.num_experts > 1024:
            raise ValueError(f"num_experts {self.num_experts} is more than the router kernel takes (1024)")
        self.router = None
        self.w_gate = self.w_up = self.w_down = None
        self.ws_gate = self.ws_up = self.ws_down = None
        self.shared_gate_w = None
        self.router_split = None        # [cols, 3 hidden] bfloat16: router rows (and the gate's) three times over
        # chunks of the shared expert that run as extra groups of the grouped products
        self.shared_chunks = 0
        if self.shared_inter > 0 and self.shared_inter % self.inter == 0 and self.shared_inter // self.inter <= 64:
            self.shared_chunks = self.shared_inter // self.inter

    def params(self) -> Dict[str, ParamSpec]:
        p = {self.name("gate.weight"): ParamSpec((self.num_experts, self.hidden), role="vector")}
        for e in range(self.num_experts):
            p[self.name(f"experts.{e}.gate_proj.weight")] = ParamSpec((self.inter, self.hidden))
            p[self.name(f"experts.{e}.up_proj.weight")] = ParamSpec((self.inter, self.hidden))
            p[self.name(f"experts.{e}.down_proj.weight")] = ParamSpec((self.hidden, self.inter))
        if self.shared_inter > 0:
            p[self.name("shared_expert.gate_proj.weight")] = ParamSpec((self.shared_inter, self.hidden))
            p[self.name("shared_expert.up_proj.weight")] = ParamSpec((self.shared_inter, self.hidden))
            p[self.name("shared_expert.down_proj.weight")] = ParamSpec((self.hidden, self.shared_inter))
            if self.shared_gate:
                p[self.name("shared_expert_gate.weight")] = ParamSpec((1, self.hidden), role="vector")
        return p

    def libraries(self) -> set:
        libs = {"rowwise", "moe_route", "gemm_simt"}
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs |= {"gemm_tc", "gemm_tc2"}
        return libs

    def load(self, source) -> None:
        rt = self.runtime
        self.router = self.fetch(source, self.name("gate.weight"))

        E, C, I = self.num_experts, self.shared_chunks, self.inter

        def slab(proj: str, rows: int, cols: int) -> torch.Tensor:
            out = torch.empty((E + C, rows, cols), dtype=rt.matrix_dtype, device=rt.device)
            for e in range(E):
                out[e].copy_(self.fetch(source, self.name(f"experts.{e}.{proj}.weight")))
            return out

        self.w_gate = slab("gate_proj", I, self.hidden)
        self.w_up = slab("up_proj", I, self.hidden)
        self.w_down = slab("down_proj", self.hidden, I)
        if self.shared_inter > 0:
            ws_gate = self.fetch(source, self.name("shared_expert.gate_proj.weight"))
            ws_up = self.fetch(source, self.name("shared_expert.up_proj.weight"))
            ws_down = self.fetch(source, self.name("shared_expert.down_proj.weight"))
            if C > 0:
                # chunk c of the shared expert: rows [c I, (c + 1) I) of gate and up, columns of down
                self.w_gate[E:].copy_(ws_gate.view(C, I, self.hidden))
                self.w_up[E:].copy_(ws_up.view(C, I, self.hidden))
                self.w_down[E:].copy_(ws_down.view(self.hidden, C, I).permute(1, 0, 2))
                if rt.fast_kernels:
                    # steps with many rows run the shared expert as dense products of its own (see
                    # forward): gate and up are then the chunks' rows seen as one matrix, the down
                    # projection is held a second time, whole
                    self.ws_down = ws_down
            else:
                self.ws_gate, self.ws_up, self.ws_down = ws_gate, ws_up, ws_down
            if self.shared_gate:
                self.shared_gate_w = self.fetch(source, self.name("shared_expert_gate.weight")).reshape(-1).contiguous()

        self._prepare_split_router()

    # Router logits on the tensor cores, float32-grade.  The normed row arrives as three
    # bfloat16 terms hi | mid | lo (their sum is the float32 value to 2^-24); the router's
    # weights, when they are exactly representable in bfloat16 (a bfloat16 checkpoint), are
    # laid three times side by side, so one bfloat16 product over K = 3 hidden, accumulated in
    # float32 and cut along K into partial sums, gives sum_j w[e, j] (hi + mid + lo)[j] with
    # every product exact.  Used for many rows; few rows take the fused float32 kernel.
    SPLIT_ROUTER_MIN_ROWS = 64

    def _prepare_split_router(self) -> None:
        rt = self.runtime
        self.router_split = None
        if not rt.fast_kernels or self.hidden % 8 != 0 or self.hidden < 128:
            return
        rows = [self.router]
        if self.shared_gate:
            rows.append(self.shared_gate_w.view(1, -1))
        w = torch.cat(rows, dim=0)
        wb = w.to(torch.bfloat16)
        if not torch.equal(wb.to(torch.float32), w):
            return                              # weights with more than 8 bits of mantissa: the float32 kernel
        cols = -(-w.shape[0] // 16) * 16
        padded = torch.zeros((cols, self.hidden), dtype=torch.bfloat16, device=w.device)
        padded[:w.shape[0]] = wb
        self.router_split = torch.cat([padded, padded, padded], dim=1).contiguous()

    # From this many rows on, the shared expert leaves the grouped products: as extra groups it
    # costs a copy of every row per chunk in the gather, a float32 partial result per chunk out of
    # the down product and as many reads in the combine - bytes that a step with few rows does not
    # notice beside the weights, and a step with many rows does.
    SHARED_DENSE_MIN_ROWS = 512

    def wants_split_input(self, rows: int) -> bool:
        return self.router_split is not None and rows >= self.SPLIT_ROUTER_MIN_ROWS

    def _route(self, x_exact: torch.Tensor, sel, wts, shared_scale, pin=None, gap=None) -> None:
        k = self.top_k
        if x_exact.dtype == torch.bfloat16:
            # the three-term form: one tensor-core product, cut along K so that the machine is
            # occupied and the float32 sums stay short
            T = x_exact.shape[0]
            cols, Kd = self.router_split.shape
            k_blocks = Kd // 64
            tiles = -(-T // 128) * -(-cols // 128)
            rt_sms = self.runtime.sm_count
            splits = max(1, min(8, k_blocks // 8, -(-rt_sms // tiles)))
            logits = torch.empty((splits, T, cols), dtype=torch.float32, device=x_exact.device)
            K.gemm_tc(x_exact, self.router_split, logits if splits > 1 else logits[0], K.EPI_STORE_F32, False, 128,
                      k_splits=splits)
            K.router_select(logits, self.num_experts, k, self.norm_topk, sel, wts, shared_scale, pin=pin, gap=gap)
        else:
            K.router_topk(x_exact, self.router, self.shared_gate_w, k, self.norm_topk, sel, wts, shared_scale, pin=pin, gap=gap)

    def forward(self, x: torch.Tensor, x_exact: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        rt = self.runtime
        dev = x.device
        T = x.shape[0]
        k, E = self.top_k, self.num_experts
        sel = torch.empty((T, k), dtype=torch.int32, device=dev)
        wts = torch.empty((T, k), dtype=torch.float32, device=dev)
        shared_scale = torch.empty((T,), dtype=torch.float32, device=dev) if self.shared_gate else None
        # a step may bring the experts of its rows with it (``ctx.routing_pin``: this part's tensor-name
        # prefix -> int32 [rows, k]; the weights stay the rows' own probabilities), or ask for what was
        # picked and how narrowly (``ctx.routing_dump``: prefix -> (experts, margins))
        pins, dump = getattr(ctx, "routing_pin", None), getattr(ctx, "routing_dump", None)
        pin = pins.get(self.prefix) if pins else None
        gap = torch.empty((T,), dtype=torch.float32, device=dev) if dump is not None and pin is None else None
        K.tag = "router"
        self._route(x_exact, sel, wts, shared_scale, pin, gap)
        if dump is not None:
            dump[self.prefix] = (sel, gap)

        shared_dense = self.ws_down is not None and self.shared_chunks > 0 and T >= self.SHARED_DENSE_MIN_ROWS
        C = 0 if shared_dense else self.shared_chunks
        n_slots = T * k + C * T
        offsets = torch.empty((E + C + 1,), dtype=torch.int32, device=dev)
        slot_token = torch.empty((n_slots,), dtype=torch.int32, device=dev)
        slot_of_pick = torch.empty((T * k,), dtype=torch.int32, device=dev)
        K.tag = "grouping"
        K.moe_group(sel, k, E, offsets, slot_token, slot_of_pick, extra_groups=C)

        act = torch.empty((n_slots, self.inter), dtype=rt.act_dtype, device=dev)
        G = E + C
        K.tag = "experts gate/up"
        project(rt, x, self.w_gate[:G], act, w_up=self.w_up[:G], group_offsets=offsets, a_row_index=slot_token,
                max_group_rows=T)
        y = torch.empty((n_slots, self.hidden), dtype=torch.float32, device=dev)
        K.tag = "experts down"
        project(rt, act, self.w_down[:G], y, group_offsets=offsets, max_group_rows=T, offsets_settled=True)

        shared = None
        if C > 0:
            shared = y[T * k:].view(C, T, self.hidden)
        elif self.shared_inter > 0:
            sact = torch.empty((T, self.shared_inter), dtype=rt.act_dtype, device=dev)
            if shared_dense:
                ws_gate = self.w_gate[E:].view(self.shared_inter, self.hidden)
                ws_up = self.w_up[E:].view(self.shared_inter, self.hidden)
            else:
                ws_gate, ws_up = self.ws_gate, self.ws_up
            K.tag = "shared gate/up"
            project(rt, x, ws_gate, sact, w_up=ws_up)
            shared = torch.empty((T, self.hidden), dtype=torch.float32, device=dev)
            K.tag = "shared down"
            project(rt, sact, self.ws_down, shared)
        K.tag = "combine"
        K.moe_combine(residual, y, slot_of_pick, wts, k, shared, shared_scale)
        K.tag = None
