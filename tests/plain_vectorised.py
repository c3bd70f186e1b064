"""The plain implementation once more, with whole tensors instead of Python loops over rows.

``tests/plain_qwen2moe.py`` walks rows, heads and experts in Python: right for tiny models,
hopeless for 24 layers of 60 experts and a vocabulary of 151,936.  This file restates the
same formulas (the same reference lines: model/Prim.cajeta:120-151 RMSNorm, :1866-1940
RoPE, model/PagedKvCache.cajeta:374-470 attention, model/MoeFfn.cajeta:908-988 routing,
:1849-1964 experts and shared expert, model/CausalLM.cajeta:1424-1608,1712-1718 the layer
and the head) as batched tensor operations in float64 by default, on whatever device the
weights live on.  It is held to the row-by-row implementation on the small configurations
(``tests/test_plain.py``); the full-size tests then hold the engine to it.

Weights come from ``get(name) -> tensor`` with the checkpoint's tensor names, so the caller
can hand out views of the tensors an engine already holds instead of a second copy; every
tensor is widened to the working dtype only while it is used.  No code is shared with the
package.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import torch

import plain_qwen2moe as P


def _first_argmax(p: torch.Tensor) -> torch.Tensor:
    """Index of the first largest entry of every row (ties to the lower index)."""
    E = p.shape[-1]
    top = p.max(dim=-1, keepdim=True).values
    idx = torch.arange(E, device=p.device).expand_as(p)
    return torch.where(p == top, idx, torch.full_like(idx, E)).min(dim=-1).values


def route(logits: torch.Tensor, top_k: int, norm_topk: bool):
    """Rows of router logits [T, E] -> (picked experts [T, k] int64, their weights [T, k],
    each row's margin (p_k - p_{k+1}) / p_k): softmax over all experts, k times the first
    largest, renormalisation with the divisor clamped at 2^-14."""
    p = torch.exp(logits - logits.max(dim=-1, keepdim=True).values)
    p = p / p.sum(dim=-1, keepdim=True)
    left = p.clone()
    sel, wts = [], []
    rows = torch.arange(p.shape[0], device=p.device)
    for _ in range(top_k):
        j = _first_argmax(left)
        sel.append(j)
        wts.append(left[rows, j])
        left[rows, j] = -1.0
    sel_t, w = torch.stack(sel, dim=1), torch.stack(wts, dim=1)
    if top_k < p.shape[1]:
        nxt = left.max(dim=-1).values
        margin = (w[:, -1] - nxt) / w[:, -1]
    else:
        margin = torch.ones(p.shape[0], dtype=p.dtype, device=p.device)
    if norm_topk:
        w = w / torch.clamp(w.sum(dim=-1, keepdim=True), min=0.00006103515625)
    return sel_t, w, margin


def rope(t: torch.Tensor, positions: torch.Tensor, inv: torch.Tensor) -> torch.Tensor:
    half = t.shape[-1] // 2
    ang = (positions.to(torch.float32)[:, None] * inv.to(torch.float32)[None, :]).to(t.dtype)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = t[..., :half], t[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int, scale: float) -> torch.Tensor:
    """q [T, heads, hd], k and v [T, kv_heads, hd] of one whole sequence."""
    T, heads, hd = q.shape
    group = heads // k.shape[1]
    pos = torch.arange(T, device=q.device)
    allowed = pos[None, :] <= pos[:, None]
    if window > 0:
        allowed &= pos[None, :] > pos[:, None] - window
    out = torch.empty_like(q)
    for h in range(heads):
        s = (q[:, h, :] @ k[:, h // group, :].t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        out[:, h, :] = (e @ v[:, h // group, :]) * (1.0 / e.sum(dim=-1, keepdim=True))
    return out


def _swiglu(x, wg, wu, wd):
    g = x @ wg.t()
    return ((g / (1.0 + torch.exp(-g))) * (x @ wu.t())) @ wd.t()


def forward(config: dict, get: Callable[[str], torch.Tensor], tokens: Sequence[int], dtype: torch.dtype = torch.float64,
            device: Optional[torch.device] = None, margins: Optional[List[float]] = None,
            selections: Optional[Dict[int, torch.Tensor]] = None, vocab_chunk: int = 16384) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``margins`` (a list of T ones) receives each
    row's smallest routing margin over the layers; ``selections`` (a dict) each sparse layer's
    picked experts [T, k]."""
    def W(name: str) -> torch.Tensor:
        t = get(name)
        return t.to(device=device if device is not None else t.device, dtype=dtype)

    heads = config["num_attention_heads"]
    kv_heads = config.get("num_key_value_heads", heads)
    hd = config.get("head_dim") or config["hidden_size"] // heads
    eps = config["rms_norm_eps"]
    T = len(tokens)
    emb = get("model.embed_tokens.weight")
    dev = device if device is not None else emb.device
    ids = torch.tensor(list(tokens), dtype=torch.long, device=emb.device)
    hs = emb[ids].to(device=dev, dtype=dtype)
    positions = torch.arange(T, device=dev)
    inv = P.inv_freq(hd, config.get("rope_theta", 10000.0), dtype).to(dev)
    worst = torch.ones(T, dtype=dtype, device=dev)
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}"
        xn = P.rmsnorm(hs, W(f"{p}.input_layernorm.weight"), eps)
        q = (xn @ W(f"{p}.self_attn.q_proj.weight").t() + W(f"{p}.self_attn.q_proj.bias")).reshape(T, heads, hd)
        k = (xn @ W(f"{p}.self_attn.k_proj.weight").t() + W(f"{p}.self_attn.k_proj.bias")).reshape(T, kv_heads, hd)
        v = (xn @ W(f"{p}.self_attn.v_proj.weight").t() + W(f"{p}.self_attn.v_proj.bias")).reshape(T, kv_heads, hd)
        ao = attention(rope(q, positions, inv), rope(k, positions, inv), v, P.layer_window(config, l), 1.0 / math.sqrt(hd))
        hs = hs + ao.reshape(T, heads * hd) @ W(f"{p}.self_attn.o_proj.weight").t()
        xn = P.rmsnorm(hs, W(f"{p}.post_attention_layernorm.weight"), eps)
        if P.layer_is_sparse(config, l):
            kk = config["num_experts_per_tok"]
            sel, wts, margin = route(xn @ W(f"{p}.mlp.gate.weight").t(), kk, config.get("norm_topk_prob", False))
            worst = torch.minimum(worst, margin)
            if selections is not None:
                selections[l] = sel
            picks = torch.zeros((T, kk, hs.shape[1]), dtype=dtype, device=dev)
            for e in range(config["num_experts"]):
                t_idx, j_idx = torch.nonzero(sel == e, as_tuple=True)
                if t_idx.numel() == 0:
                    continue
                y = _swiglu(xn[t_idx], W(f"{p}.mlp.experts.{e}.gate_proj.weight"), W(f"{p}.mlp.experts.{e}.up_proj.weight"),
                            W(f"{p}.mlp.experts.{e}.down_proj.weight"))
                picks[t_idx, j_idx] = wts[t_idx, j_idx][:, None] * y
            ff = torch.zeros_like(hs)
            for j in range(kk):                                   # the picks are added in selection order
                ff = ff + picks[:, j]
            if config.get("shared_expert_intermediate_size", 0) > 0:
                s = _swiglu(xn, W(f"{p}.mlp.shared_expert.gate_proj.weight"), W(f"{p}.mlp.shared_expert.up_proj.weight"),
                            W(f"{p}.mlp.shared_expert.down_proj.weight"))
                z = xn @ W(f"{p}.mlp.shared_expert_gate.weight").reshape(-1)
                ff = ff + (1.0 / (1.0 + torch.exp(-z)))[:, None] * s
        else:
            ff = _swiglu(xn, W(f"{p}.mlp.gate_proj.weight"), W(f"{p}.mlp.up_proj.weight"), W(f"{p}.mlp.down_proj.weight"))
        hs = hs + ff
    xn = P.rmsnorm(hs, W("model.norm.weight"), eps)
    head = get("model.embed_tokens.weight" if config.get("tie_word_embeddings", False) else "lm_head.weight")
    out = torch.empty((T, head.shape[0]), dtype=dtype, device=dev)
    for lo in range(0, head.shape[0], vocab_chunk):                # the head in slices: it is the one large matrix
        out[:, lo:lo + vocab_chunk] = xn @ head[lo:lo + vocab_chunk].to(device=dev, dtype=dtype).t()
    if margins is not None:
        for t, m in enumerate(worst.tolist()):
            margins[t] = min(margins[t], m)
    return out


def engine_views(model) -> Callable[[str], torch.Tensor]:
    """``get(name)`` over the tensors a built engine model holds, by the checkpoint's names and
    without copies where the engine's layout allows: q, k and v are row ranges of the stacked
    projection, an expert is a slice of its slab, the shared expert is the slab's extra groups
    seen as one matrix (or the engine's separate tensors where it keeps them)."""
    plan = model.plan
    views: Dict[str, Callable[[], torch.Tensor]] = {plan.embedding_name: lambda: model.embedding}
    if plan.lm_head_name is not None:
        views[plan.lm_head_name] = lambda: model.lm_head
    views[model.final_norm.name("weight")] = lambda: model.final_norm.weight
    for block in model.blocks:
        for norm in (block.mixer_norm, block.feed_forward_norm):
            views[norm.name("weight")] = (lambda n=norm: n.weight)
        a = block.mixer
        bounds = {"q": (0, a.q_dim), "k": (a.q_dim, a.q_dim + a.kv_dim), "v": (a.q_dim + a.kv_dim, a.q_dim + 2 * a.kv_dim)}
        for n, (lo, hi) in bounds.items():
            views[a.name(f"{n}_proj.weight")] = (lambda a=a, lo=lo, hi=hi: a.w_qkv[lo:hi])
            views[a.name(f"{n}_proj.bias")] = (lambda a=a, lo=lo, hi=hi: a.b_qkv[lo:hi])
        views[a.name("o_proj.weight")] = (lambda a=a: a.w_o)
        f = block.feed_forward
        if hasattr(f, "num_experts"):
            E, C, I, H = f.num_experts, f.shared_chunks, f.inter, f.hidden
            views[f.name("gate.weight")] = (lambda f=f: f.router)
            for e in range(E):
                views[f.name(f"experts.{e}.gate_proj.weight")] = (lambda f=f, e=e: f.w_gate[e])
                views[f.name(f"experts.{e}.up_proj.weight")] = (lambda f=f, e=e: f.w_up[e])
                views[f.name(f"experts.{e}.down_proj.weight")] = (lambda f=f, e=e: f.w_down[e])
            if f.shared_inter > 0:
                if C > 0:
                    views[f.name("shared_expert.gate_proj.weight")] = (lambda f=f: f.w_gate[f.num_experts:].reshape(-1, f.hidden))
                    views[f.name("shared_expert.up_proj.weight")] = (lambda f=f: f.w_up[f.num_experts:].reshape(-1, f.hidden))
                    views[f.name("shared_expert.down_proj.weight")] = (
                        lambda f=f: f.w_down[f.num_experts:].permute(1, 0, 2).reshape(f.hidden, -1))
                else:
                    views[f.name("shared_expert.gate_proj.weight")] = (lambda f=f: f.ws_gate)
                    views[f.name("shared_expert.up_proj.weight")] = (lambda f=f: f.ws_up)
                    views[f.name("shared_expert.down_proj.weight")] = (lambda f=f: f.ws_down)
                if f.shared_gate:
                    views[f.name("shared_expert_gate.weight")] = (lambda f=f: f.shared_gate_w.view(1, -1))
        else:
            views[f.name("gate_proj.weight")] = (lambda f=f: f.w_gate)
            views[f.name("up_proj.weight")] = (lambda f=f: f.w_up)
            views[f.name("down_proj.weight")] = (lambda f=f: f.w_down)
    return lambda name: views[name]()
