"""Grouped-query attention over the paged cache.

Per row at absolute position ``p``: ``q = x Wq^T + bq``, ``k = x Wk^T + bk``,
``v = x Wv^T + bv`` (bias after the product, none on the output projection:
model/Attention.cajeta:48-56,102-111, model/Linear.cajeta:1883-1898); the position
encoding rotates q and k; rotated k and raw v are appended to the cache at ``p``
(model/CausalLM.cajeta:1454-1485; on the tensor-core path both happen in the epilogue of the
q/k/v product, on the others in a kernel of their own); head ``h`` attends with kv head
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
from .linear import project, project_rope_cache, project_split, rope_cache_ok, rope_pairs_order
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
        # On the tensor-core path the rotation and the cache write happen in the q/k/v product's own
        # epilogue; the weight rows are laid out for it at load (``qkv_row_order[new] = old``, else None).
        self.fused_rope = (self.position.rotary_dim > 0 and
                           rope_cache_ok(runtime, self.hidden, self.q_dim))
        self.qkv_row_order: Optional[torch.Tensor] = None
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
        if self.fused_rope:
            # the two halves of every rotation pair side by side (csrc/rope_epilogue.cuh)
            self.qkv_row_order = rope_pairs_order(self.heads, self.kv_heads, self.head_dim, self.position.rotary_dim)
            order = self.qkv_row_order.to(self.w_qkv.device)
            self.w_qkv = self.w_qkv[order].contiguous()
            if self.b_qkv is not None:
                self.b_qkv = self.b_qkv[order].contiguous()
            self._rope_key = ("rope table", self.position.rotary_dim, tuple(self.position.inv_freq.cpu().tolist()))

    # -- one step --------------------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, entry) -> Optional[torch.Tensor]:
        rt = self.runtime
        T = x.shape[0]
        pos = self.position
        write = entry.writes_cache
        n_out = self.q_dim + (2 * self.kv_dim if write else 0)
        q = torch.empty((T, self.heads, self.head_dim), dtype=rt.act_dtype, device=x.device)
        if self.fused_rope:
            # one kernel: the product's epilogue rotates q and k and puts k and v into the cache pages.
            # cos / sin of the rows' angles are worked out once a step (the same for every layer), the
            # rows' places in the cache once a step and cache group.
            scratch = getattr(ctx, "scratch", None)
            cos_sin = scratch.get(self._rope_key) if scratch is not None else None
            if cos_sin is None:
                cos_sin = torch.empty((T, pos.rotary_dim // 2, 2), dtype=torch.float32, device=x.device)
                K.tag = "rope table"
                K.rope_table(ctx.positions, pos.inv_freq, cos_sin)
                if scratch is not None:
                    scratch[self._rope_key] = cos_sin
            kv_base = None
            if write:
                key = ("cache rows", entry.block_table.data_ptr(), self.kv_heads, self.head_dim)
                kv_base = scratch.get(key) if scratch is not None else None
                if kv_base is None:
                    kv_base = torch.empty((T,), dtype=torch.int64, device=x.device)
                    K.tag = "rope table"
                    K.kv_rows(ctx.positions, ctx.row_req, entry.block_table, entry.page_tokens, self.kv_heads, self.head_dim, kv_base)
                    if scratch is not None:
                        scratch[key] = kv_base
            K.tag = "qkv"
            project_rope_cache(rt, x, self.w_qkv[:n_out], None if self.b_qkv is None else self.b_qkv[:n_out],
                               q.view(T, self.q_dim), entry.k_plane if write else None, entry.v_plane if write else None,
                               cos_sin, kv_base, self.q_dim, self.kv_dim, self.head_dim, pos.rotary_dim, entry.page_tokens)
        else:
            qkv = torch.empty((T, n_out), dtype=torch.float32, device=x.device)
            K.tag = "qkv"
            project(rt, x, self.w_qkv[:n_out], qkv, bias=None if self.b_qkv is None else self.b_qkv[:n_out])
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
