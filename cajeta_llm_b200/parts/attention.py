"""Grouped-query attention over the paged cache.

Per row at absolute position ``p``: ``q = x Wq^T + bq``, ``k = x Wk^T + bk``,
``v = x Wv^T + bv`` (bias after the product, none on the output projection:
model/Attention.cajeta:48-56,102-111, model/Linear.cajeta:1883-1898); the position
encoding rotates q and k; rotated k and raw v are appended to the cache at ``p``
(model/CausalLM.cajeta:1454-1485); head ``h`` attends with kv head
``h / (heads / kv_heads)`` over keys ``[from, p]``, ``from = p + 1 - window`` when a
window is set and exceeded, else 0, scale ``1 / sqrt(head_dim)`` unless given
(model/PagedKvCache.cajeta:374-470, model/Attention.cajeta:67-71); the output
projection is added into the residual stream (model/CausalLM.cajeta:1498,1506).

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``window``,
``qkv_bias``, ``out_bias``, ``scale``, ``position`` (a position PartSpec).

An entry that reads another entry's cache (``entry.writes_cache`` false) projects and
rotates only q.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import kernels as K
from .base import KvNeed, Part, make_part, register_part
from .linear import project, project_split
from .plan import ParamSpec


@register_part("mixer", "attention")
class PagedAttention(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = int(spec.get("window", 0) or 0)
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.out_bias = bool(spec.get("out_bias", False))
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"num_heads {self.heads} is not a multiple of num_kv_heads {self.kv_heads}")
        if self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is larger than the attention kernels take (256)")
        self.position = make_part("position", spec["position"], prefix, runtime)
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim
        self.w_qkv: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None

    # -- what the cache manager must provide ----------------------------------------
    def cache_need(self) -> Optional[KvNeed]:
        return KvNeed(self.kv_heads, self.head_dim, self.window)

    def state_need(self):
        return None

    # -- tensors ---------------------------------------------------------------------
    def params(self) -> Dict[str, ParamSpec]:
        p = {
            self.name("q_proj.weight"): ParamSpec((self.q_dim, self.hidden)),
            self.name("k_proj.weight"): ParamSpec((self.kv_dim, self.hidden)),
            self.name("v_proj.weight"): ParamSpec((self.kv_dim, self.hidden)),
            self.name("o_proj.weight"): ParamSpec((self.hidden, self.q_dim)),
        }
        if self.qkv_bias:
            p[self.name("q_proj.bias")] = ParamSpec((self.q_dim,), role="vector")
            p[self.name("k_proj.bias")] = ParamSpec((self.kv_dim,), role="vector")
            p[self.name("v_proj.bias")] = ParamSpec((self.kv_dim,), role="vector")
        if self.out_bias:
            p[self.name("o_proj.bias")] = ParamSpec((self.hidden,), role="vector")
        return p

    def libraries(self) -> set:
        libs = {"rowwise", "gemm_simt"}
        if self.runtime.fast_kernels and self.head_dim in (64, 128):
            libs |= {"attention_decode", "attention_prefill_tc" if self.head_dim == 128 else "attention_prefill"}
        else:
            libs.add("attention_paged")
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs |= {"gemm_tc", "gemm_tc2"}
        return libs

    def load(self, source) -> None:
        # q, k and v rows are stacked so that one product yields all three
        self.w_qkv = torch.cat([self.fetch(source, self.name(f"{n}_proj.weight")) for n in ("q", "k", "v")], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([self.fetch(source, self.name(f"{n}_proj.bias")) for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = self.fetch(source, self.name("o_proj.weight"))
        if self.out_bias:
            self.b_o = self.fetch(source, self.name("o_proj.bias"))

    # -- one step --------------------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> Optional[torch.Tensor]:
        rt = self.runtime
        T = x.shape[0]
        pos = self.position
        write = entry.writes_cache
        n_out = self.q_dim + (2 * self.kv_dim if write else 0)
        qkv = torch.empty((T, n_out), dtype=torch.float32, device=x.device)
        K.tag = "qkv"
        project(rt, x, self.w_qkv[:n_out], qkv, bias=None if self.b_qkv is None else self.b_qkv[:n_out])
        q = torch.empty((T, self.heads, self.head_dim), dtype=rt.act_dtype, device=x.device)
        K.tag = "rope + cache write"
        K.rope_kv_write(qkv, 0, self.q_dim, self.q_dim + self.kv_dim, q, entry.k_plane, entry.v_plane,
                        ctx.positions, ctx.row_req, entry.block_table, entry.page_tokens, self.heads, self.kv_heads,
                        self.head_dim, pos.rotary_dim, pos.inv_freq, write)
        out = torch.empty_like(q)
        K.tag = "attention"
        if rt.fast_kernels and getattr(ctx, "all_single", False) and self.head_dim in (64, 128):
            # every request brings one token: the split-KV decode kernel
            K.decode_attention(q, out, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table,
                               entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale,
                               ctx.max_context, getattr(ctx, "decode_scratch", None) or rt.decode_scratch)
        elif rt.fast_kernels and self.head_dim == 128 and entry.page_tokens == 16 and hasattr(ctx, "req_start"):
            # portions of prompts (and whatever single tokens ride along): both products on tcgen05,
            # scores and output in tensor memory
            K.prefill_attention_tc(q, out, entry.k_plane, entry.v_plane, ctx.req_start, ctx.req_prior, entry.block_table,
                                   entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale)
        elif rt.fast_kernels and self.head_dim in (64, 128) and hasattr(ctx, "req_start"):
            # other page sizes, head size 64: query tiles on mma.sync
            K.prefill_attention(q, out, entry.k_plane, entry.v_plane, ctx.req_start, ctx.req_prior, entry.block_table,
                                entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale)
        else:
            K.paged_attention(q, out, entry.k_plane, entry.v_plane, ctx.positions, ctx.row_req, entry.block_table,
                              entry.page_tokens, self.heads, self.kv_heads, self.head_dim, self.window, self.scale)
        K.tag = "o"
        parts = project_split(rt, out.view(T, self.q_dim), self.w_o, bias=self.b_o)
        if parts is None:
            project(rt, out.view(T, self.q_dim), self.w_o, residual, bias=self.b_o, accumulate=True)
        K.tag = None
        return parts                         # partial sums owed to the residual stream (the next norm adds them), or None
