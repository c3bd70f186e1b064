"""Plain, slow implementation of Qwen2-MoE: whole sequences, no cache, no batching.

It rests on the reference's formulas: the reference's model code is cajeta source and
there is no cajeta toolchain on this machine, so it cannot be imported or compiled
here.  Each function cites the reference's float32 host path (paths are relative to
``src/main/cajeta/dev/cajeta/llm/``).  The router and the shared-expert gate are
additionally checked against constants that the reference's own test asserts
(tests/golden/).

It shares no code with the engine: it reads ``config.json`` and ``model.safetensors``
itself, and imports nothing from the package.  Arithmetic runs in the dtype given
(float64 by default, so that a difference from the engine is the engine's rounding).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ----------------------------------------------------------------------------------
# reading a model folder (own reader: header length, JSON header, raw payload;
# io/SafetensorsFile.cajeta:59-139)
# ----------------------------------------------------------------------------------
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    base = 8 + n
    out: Dict[str, torch.Tensor] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = blob[base + b: base + e]
        dt = info["dtype"]
        if dt == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        elif dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif dt == "F16":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f2").astype(np.float32))
        else:
            raise ValueError(f"{path}: dtype {dt} of '{name}' not handled by the plain reader")
        out[name] = t.reshape(info["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        config = json.load(f)
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return config, weights


# ----------------------------------------------------------------------------------
# parts, one function each
# ----------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """hs[t, :] = W_emb[token_t, :], no scale (model/Embedding.cajeta:73-81,
    model/HostOps.cajeta:32-49)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x_i^2; scale = 1/sqrt(ss/dim + eps); y_i = x_i * scale * w_i
    (model/Prim.cajeta:120-151)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    scale = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * scale * w


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T, bias added after the product (model/Linear.cajeta:1883-1898; the file
    stores torch's [out, in], model/Linear.cajeta:1856-1873)."""
    y = x @ w.t()
    if b is not None:
        y = y + b
    return y


def inv_freq(head_dim: int, theta: float, dtype: torch.dtype) -> torch.Tensor:
    """inv[d] = theta^(-2d/head_dim), d in [0, head_dim/2), computed in float32 as the
    reference does (model/Prim.cajeta:1866-1880), then widened."""
    half = head_dim // 2
    vals = [np.float32(np.power(np.float32(theta), np.float32(0.0 - 2.0 * d) / np.float32(head_dim)))
            for d in range(half)]
    return torch.tensor(np.array(vals, dtype=np.float32)).to(dtype)


def rope(t: torch.Tensor, positions: torch.Tensor, inv: torch.Tensor) -> torch.Tensor:
    """Half-split pairs (d, d + half): ang = p * inv[d]; a' = a cos - b sin;
    b' = a sin + b cos; t is [T, heads, head_dim] (model/Prim.cajeta:1917-1940)."""
    half = t.shape[-1] // 2
    # the angle is a float32 product in the reference; cos and sin are then taken in
    # the working dtype
    ang = (positions.to(torch.float32)[:, None] * inv.to(torch.float32)[None, :]).to(t.dtype)   # [T, half]
    c = torch.cos(ang)[:, None, :]
    s = torch.sin(ang)[:, None, :]
    a, b = t[..., :half], t[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int, scale: float) -> torch.Tensor:
    """Causal attention of one whole sequence, row by row.

    For head h, kvh = h / (heads / kv_heads); keys t in [from, p] with
    from = p + 1 - w if w > 0 and p + 1 > w else 0; s_t = (q . k_t) * scale;
    e_t = exp(s_t - max s); o = (sum_t e_t v_t) * (1 / sum_t e_t)
    (model/PagedKvCache.cajeta:374-470).  q is [T, heads, hd]; k, v are [T, kv_heads, hd].
    """
    T, heads, hd = q.shape
    group = heads // k.shape[1]
    out = torch.zeros_like(q)
    for p in range(T):
        start = p + 1 - window if (window > 0 and p + 1 > window) else 0
        for h in range(heads):
            kvh = h // group
            s = (k[start:p + 1, kvh, :] @ q[p, h, :]) * scale
            e = torch.exp(s - s.max())
            out[p, h, :] = (e[:, None] * v[start:p + 1, kvh, :]).sum(dim=0) * (1.0 / e.sum())
    return out


def route(logits: torch.Tensor, top_k: int, norm_topk: bool):
    """Softmax over all experts, top-k by repeated strict-> argmax (ties to the lower
    index), optional renormalisation with the divisor clamped at 2^-14
    (model/MoeFfn.cajeta:908-988).  logits is one row [E]."""
    p = torch.exp(logits - logits.max())
    p = p / p.sum()
    probs = p.clone()
    sel: List[int] = []
    w: List[torch.Tensor] = []
    for _ in range(top_k):
        best, bp = -1, None
        for e in range(probs.shape[0]):
            if probs[e] >= 0 and (best < 0 or probs[e] > bp):
                best, bp = e, probs[e]
        if best < 0:
            raise ValueError("router logits are not finite")
        sel.append(best)
        w.append(bp.clone())
        probs[best] = -1.0
    wt = torch.stack(w)
    if norm_topk:
        ws = wt.sum()
        ws = torch.clamp(ws, min=0.00006103515625)
        wt = wt / ws
    return sel, wt


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x)) (model/Prim.cajeta:1822-1847)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """W_d (silu(W_g x) * (W_u x)) (model/Prim.cajeta:1822-1847,
    model/CausalLM.cajeta:1556-1566)."""
    return linear(silu(linear(x, wg)) * linear(x, wu), wd)


def routing_margin(logits: torch.Tensor, top_k: int) -> float:
    """How far the row is from another choice of experts: (p_k - p_{k+1}) / p_k of the
    k-th and (k+1)-th largest router probabilities (1.0 when every expert is picked).
    The reference measures the same gap behind a routing flip
    (model/MoeFfn.cajeta:135-149); a row with a tiny margin changes discontinuously
    under rounding, which a comparison in reduced precision has to know."""
    if top_k >= logits.shape[0]:
        return 1.0
    p = torch.softmax(logits.double(), dim=0).sort(descending=True).values
    return float((p[top_k - 1] - p[top_k]) / p[top_k - 1])


def sparse_moe(x: torch.Tensor, weights: Dict[str, torch.Tensor], prefix: str, num_experts: int, top_k: int,
               norm_topk: bool, has_shared: bool, margins: Optional[List[float]] = None,
               picked: Optional[List[List[int]]] = None) -> torch.Tensor:
    """Per row: router, selected experts accumulated in selection order, then the
    sigmoid-gated shared expert (model/MoeFfn.cajeta:1849-1916 and :1925-1964).
    ``margins`` (one entry per row, updated in place) keeps the smallest routing margin;
    ``picked`` (a list) receives each row's experts in selection order."""
    out = torch.zeros_like(x)
    router_w = weights[f"{prefix}.gate.weight"]
    for t in range(x.shape[0]):
        row = x[t]
        logits = linear(row, router_w)
        if margins is not None:
            margins[t] = min(margins[t], routing_margin(logits, top_k))
        sel, wt = route(logits, top_k, norm_topk)
        if picked is not None:
            picked.append(list(sel))
        acc = torch.zeros_like(row)
        for j, e in enumerate(sel):
            y = swiglu_mlp(row, weights[f"{prefix}.experts.{e}.gate_proj.weight"],
                           weights[f"{prefix}.experts.{e}.up_proj.weight"],
                           weights[f"{prefix}.experts.{e}.down_proj.weight"])
            acc = acc + wt[j] * y
        if has_shared:
            s = swiglu_mlp(row, weights[f"{prefix}.shared_expert.gate_proj.weight"],
                           weights[f"{prefix}.shared_expert.up_proj.weight"],
                           weights[f"{prefix}.shared_expert.down_proj.weight"])
            z = (weights[f"{prefix}.shared_expert_gate.weight"].reshape(-1) * row).sum()
            acc = acc + (1.0 / (1.0 + torch.exp(-z))) * s
        out[t] = acc
    return out


# ----------------------------------------------------------------------------------
# which feed-forward and which window a layer has (this engine's reading of the HF
# keys; the reference has neither decoder_sparse_step nor max_window_layers)
# ----------------------------------------------------------------------------------
def layer_is_sparse(config: dict, layer: int) -> bool:
    return (layer not in config.get("mlp_only_layers", []) and config.get("num_experts", 0) > 0
            and (layer + 1) % config.get("decoder_sparse_step", 1) == 0)


def layer_window(config: dict, layer: int) -> int:
    if config.get("use_sliding_window", False) and layer >= config.get("max_window_layers", config["num_hidden_layers"]):
        return int(config["sliding_window"])
    return 0


# ----------------------------------------------------------------------------------
# the whole model
# ----------------------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int],
            dtype: torch.dtype = torch.float64, margins: Optional[List[float]] = None,
            selections: Optional[Dict[int, List[List[int]]]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (model/CausalLM.cajeta:1424-1608 per
    layer, :1712-1718 for the head).  ``margins``: a list of T ones that receives each
    row's smallest routing margin over the layers.  ``selections``: a dict that receives,
    per sparse layer, each row's picked experts."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    heads = config["num_attention_heads"]
    kv_heads = config.get("num_key_value_heads", heads)
    hd = config.get("head_dim") or config["hidden_size"] // heads
    eps = config["rms_norm_eps"]
    T = len(tokens)
    positions = torch.arange(T)
    inv = inv_freq(hd, config.get("rope_theta", 10000.0), dtype)
    hs = embed(W["model.embed_tokens.weight"], tokens)
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}"
        xn = rmsnorm(hs, W[f"{p}.input_layernorm.weight"], eps)
        q = linear(xn, W[f"{p}.self_attn.q_proj.weight"], W[f"{p}.self_attn.q_proj.bias"]).reshape(T, heads, hd)
        k = linear(xn, W[f"{p}.self_attn.k_proj.weight"], W[f"{p}.self_attn.k_proj.bias"]).reshape(T, kv_heads, hd)
        v = linear(xn, W[f"{p}.self_attn.v_proj.weight"], W[f"{p}.self_attn.v_proj.bias"]).reshape(T, kv_heads, hd)
        q = rope(q, positions, inv)
        k = rope(k, positions, inv)
        ao = attention(q, k, v, layer_window(config, l), 1.0 / math.sqrt(hd)).reshape(T, heads * hd)
        hs = hs + linear(ao, W[f"{p}.self_attn.o_proj.weight"])
        xn = rmsnorm(hs, W[f"{p}.post_attention_layernorm.weight"], eps)
        if layer_is_sparse(config, l):
            picked = [] if selections is not None else None
            ff = sparse_moe(xn, W, f"{p}.mlp", config["num_experts"], config["num_experts_per_tok"],
                            config.get("norm_topk_prob", False),
                            config.get("shared_expert_intermediate_size", 0) > 0, margins, picked)
            if selections is not None:
                selections[l] = picked
        else:
            ff = swiglu_mlp(xn, W[f"{p}.mlp.gate_proj.weight"], W[f"{p}.mlp.up_proj.weight"],
                            W[f"{p}.mlp.down_proj.weight"])
        hs = hs + ff
    xn = rmsnorm(hs, W["model.norm.weight"], eps)
    head = W["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else W["lm_head.weight"]
    return linear(xn, head)


# ----------------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------------
def argmax_first(logits: torch.Tensor) -> int:
    """First-occurrence argmax (model/HostOps.cajeta:107-122)."""
    best, bl = 0, logits[0]
    for i in range(1, logits.shape[0]):
        if logits[i] > bl:
            best, bl = i, logits[i]
    return best


def prepared_distribution(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                          repeat_penalty: float, history: Sequence[int]) -> torch.Tensor:
    """The post-filter distribution by token id (gen/Sampler.cajeta:60-179): repetition
    penalty over emitted tokens (divide when positive, multiply otherwise), divide by
    the temperature, descending order (ties: lower id first), top-k cut, max-subtracted
    softmax over the cut, top-p smallest prefix with cum >= p, renormalise."""
    p = logits.clone().to(torch.float32)
    if repeat_penalty != 1.0:
        for t in history:
            if 0 <= t < p.shape[0]:
                p[t] = p[t] / repeat_penalty if p[t] > 0 else p[t] * repeat_penalty
    if temperature == 0.0:
        out = torch.zeros_like(p)
        out[argmax_first(p)] = 1.0
        return out
    p = p / np.float32(temperature)
    order = sorted(range(p.shape[0]), key=lambda i: (-float(p[i]), i))
    cut = len(order)
    if top_k > 0:
        cut = min(cut, top_k)
    mx = p[order[0]]
    e = torch.zeros_like(p)
    total = np.float32(0.0)
    for i in order[:cut]:
        e[i] = torch.exp(p[i] - mx)
        total = np.float32(total + np.float32(e[i]))
    if 0.0 < top_p < 1.0:
        cum = np.float32(0.0)
        for j, i in enumerate(order[:cut]):
            cum = np.float32(cum + np.float32(e[i]) / total)
            if cum >= np.float32(top_p):
                cut = j + 1
                break
    keep = order[:cut]
    out = torch.zeros_like(p)
    total2 = sum(float(e[i]) for i in keep)
    for i in keep:
        out[i] = e[i] / total2
    return out


def draw(dist: torch.Tensor, u: float) -> int:
    """First id in descending-probability order with u < cumulative probability, else
    the last survivor (gen/Sampler.cajeta:188-206)."""
    order = sorted((i for i in range(dist.shape[0]) if dist[i] > 0), key=lambda i: (-float(dist[i]), i))
    cum = 0.0
    for i in order:
        cum += float(dist[i])
        if u < cum:
            return i
    return order[-1]
