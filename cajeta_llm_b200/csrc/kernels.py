"""Python face of the CUDA kernels: checks tensors, passes raw pointers through ctypes.

Every function launches on torch's current CUDA stream and raises
:class:`KernelError` when a kernel refuses its arguments or the launch fails.  There is
no fallback: without a CUDA device and the built libraries these functions raise.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from . import build as _build

CJ_F32, CJ_BF16 = 0, 1
_REFUSALS = {-2: "dtype combination not built into this kernel", -3: "a size this kernel does not take",
             -4: "pointer or stride alignment this kernel needs", -5: "null pointer or bad count"}


class KernelError(RuntimeError):
    pass


_libs: Dict[str, ctypes.CDLL] = {}


def library(name: str) -> ctypes.CDLL:
    """The loaded kernel library ``name`` (built first when it has to be)."""
    lib = _libs.get(name)
    if lib is None:
        path = _build.build(name)
        lib = ctypes.CDLL(path)
        _libs[name] = lib
    return lib


def loaded_libraries() -> Dict[str, str]:
    return {n: l._name for n, l in _libs.items()}


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return CJ_F32
    if t.dtype == torch.bfloat16:
        return CJ_BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, found {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


# torch's current stream as a raw handle.  torch.cuda.current_stream() builds a Stream object
# through several layers of Python on every call - a third of the host's time in a step of a few
# hundred launches; the raw getter beneath it costs a fraction of a microsecond.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


launches = 0      # kernels launched through this module since import (each wrapper launches one)
# Measurement: parts name the class of work their next launches belong to (``tag``: "qkv", "expert
# gate/up", ...; costs an assignment); while a trace is open every launch is followed by an event
# on the stream, so that the time between two events is one launch's device time with the launches
# serialised (an event between two kernels keeps them from overlapping).
tag: Optional[str] = None
_trace: Optional[list] = None


def start_trace() -> None:
    global _trace
    _trace = []


def stop_trace() -> list:
    """[(class of work, event recorded after the launch)] since ``start_trace``."""
    global _trace
    out, _trace = _trace or [], None
    return out


_router_tickets: Dict[torch.device, torch.Tensor] = {}      # arrival tickets of the small-batch router (kept zero by the kernel)


def _check(status: int, what: str) -> None:
    global launches
    if status == 0:
        launches += 1
        if _trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _trace.append((tag or what, ev))
        return
    if status in _REFUSALS:
        raise KernelError(f"{what}: refused: {_REFUSALS[status]}")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _need(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; this engine has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")


_i = ctypes.c_int
_ll = ctypes.c_longlong
_f = ctypes.c_float


def embed_gather(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 0.0) -> None:
    """out[t, :] = table[ids[t], :] widened to float32 (times ``scale`` unless that is 0).  out: [T, H] float32."""
    _need(out, "out", torch.float32), _need(table, "table"), _need(ids, "ids", torch.int32)
    T, H = out.shape
    V = table.shape[0]
    st = library("rowwise").cj_embed_gather(_ptr(out), _ptr(table), _i(_code(table)), _ptr(ids), _i(T), _i(H), _i(V), _f(scale),
                                            _stream())
    _check(st, "embed_gather")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            out_f32: Optional[torch.Tensor] = None, row_index: Optional[torch.Tensor] = None,
            partials: Optional[torch.Tensor] = None, out_split: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[row_index[r] or r]) * weight; x, weight float32; out float32 or
    bfloat16; out_f32 an optional float32 copy of the result.  ``partials`` ([S, rows, H]
    float32): x[r] += sum_s partials[s, r] first, and x keeps the sum.  ``out_split``
    (bfloat16 [rows, 3H]): the float32 result as three bfloat16 terms hi | mid | lo."""
    _need(x, "x", torch.float32), _need(weight, "weight", torch.float32), _need(out, "out")
    rows, H = out.shape
    if x.shape[-1] != H or weight.numel() != H:
        raise KernelError(f"rmsnorm: width mismatch x {tuple(x.shape)} weight {tuple(weight.shape)} out {tuple(out.shape)}")
    if out_f32 is not None:
        _need(out_f32, "out_f32", torch.float32)
    if row_index is not None:
        _need(row_index, "row_index", torch.int32)
    if out_split is not None:
        _need(out_split, "out_split", torch.bfloat16)
        if tuple(out_split.shape) != (rows, 3 * H):
            raise KernelError(f"rmsnorm: out_split {tuple(out_split.shape)} is not [{rows}, {3 * H}]")
    n_part, part_stride = 0, 0
    if partials is not None:
        _need(partials, "partials", torch.float32)
        if partials.dim() != 3 or partials.shape[1] != rows or partials.shape[2] != H or row_index is not None:
            raise KernelError(f"rmsnorm: partials {tuple(partials.shape)} do not fit {rows} rows of {H}")
        n_part, part_stride = partials.shape[0], partials.stride(0)
    st = library("rowwise").cj_rmsnorm(_ptr(x), _ptr(weight), _f(eps), _i(rows), _i(H), _ptr(out), _i(_code(out)),
                                       _ptr(out_f32), _ptr(out_split), _ptr(row_index), _ptr(partials), _i(n_part),
                                       _ll(part_stride), _stream())
    _check(st, "rmsnorm")


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
         accumulate: bool = False, w_up: Optional[torch.Tensor] = None, group_offsets: Optional[torch.Tensor] = None,
         a_row_index: Optional[torch.Tensor] = None, rows: Optional[int] = None) -> None:
    """out[M, N] (+)= a[M, K] . w[N, K]^T (+ bias) on the float32 FMA pipe.

    ``w_up`` selects the SwiGLU form silu(a.w^T) * (a.w_up^T).  With ``group_offsets``
    ([G + 1] int32) ``w`` is [G, N, K], output row s belongs to the group whose range
    holds s, and ``a_row_index[s]`` names the row of ``a`` that feeds it.
    """
    _need(a, "a"), _need(w, "w"), _need(out, "out")
    grouped = group_offsets is not None
    N, K = w.shape[-2], w.shape[-1]
    M = rows if rows is not None else out.shape[0]
    if a.shape[-1] != K or out.shape[-1] != N:
        raise KernelError(f"gemm: shapes a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)} do not agree")
    if w_up is not None:
        _need(w_up, "w_up")
        if w_up.shape != w.shape or w_up.dtype != w.dtype:
            raise KernelError("gemm: w_up must match w")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    G = 0
    if grouped:
        _need(group_offsets, "group_offsets", torch.int32)
        G = w.shape[0]
        if group_offsets.numel() != G + 1:
            raise KernelError("gemm: group_offsets must hold one more entry than w has groups")
    if a_row_index is not None:
        _need(a_row_index, "a_row_index", torch.int32)
    st = library("gemm_simt").cj_gemm_simt(
        _ptr(a), _ll(a.stride(0)), _i(_code(a)), _ptr(w), _ptr(w_up), _ll(K), _i(_code(w)), _ptr(bias),
        _ptr(out), _ll(out.stride(0)), _i(_code(out)), _i(M), _i(N), _i(K), _i(1 if accumulate else 0),
        _ptr(group_offsets), _i(G), _ll(N * K), _ptr(a_row_index), _stream())
    _check(st, "gemm")


def rope_kv_write(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor,
                  k_plane: Optional[torch.Tensor], v_plane: Optional[torch.Tensor], positions: torch.Tensor,
                  row_req: Optional[torch.Tensor], table: Optional[torch.Tensor], page_tokens: int, n_heads: int,
                  n_kv: int, head_dim: int, rotary_dim: int, inv_freq: Optional[torch.Tensor], write_kv: bool) -> None:
    """Rotate q and k at each row's position; write q to q_out, rotated k and raw v into
    the cache pages of the row's request.  qkv: float32 [T, ld]."""
    _need(qkv, "qkv", torch.float32), _need(q_out, "q_out"), _need(positions, "positions", torch.int32)
    T = qkv.shape[0]
    cache_dtype = _code(q_out)
    if write_kv:
        _need(k_plane, "k_plane"), _need(v_plane, "v_plane"), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
        cache_dtype = _code(k_plane)
    st = library("rowwise").cj_rope_kv_write(
        _ptr(qkv), _i(qkv.stride(0)), _i(q_off), _i(k_off), _i(v_off), _ptr(q_out), _i(_code(q_out)),
        _ptr(k_plane), _ptr(v_plane), _i(cache_dtype), _ptr(positions), _ptr(row_req), _ptr(table),
        _i(table.stride(0) if table is not None else 0), _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim),
        _i(rotary_dim), _ptr(inv_freq), _i(1 if write_kv else 0), _stream())
    _check(st, "rope_kv_write")


def paged_attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                    positions: torch.Tensor, row_req: torch.Tensor, table: torch.Tensor, page_tokens: int,
                    n_heads: int, n_kv: int, head_dim: int, window: int, scale: float) -> None:
    """Attention of every row over its request's cached keys [from, position]."""
    _need(q, "q"), _need(out, "out"), _need(k_plane, "k_plane"), _need(v_plane, "v_plane")
    _need(positions, "positions", torch.int32), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
    T = q.shape[0]
    if head_dim > 256:
        raise KernelError(f"paged_attention: head_dim {head_dim} is larger than 256")
    st = library("attention_paged").cj_paged_attention(
        _ptr(q), _ptr(out), _i(_code(q)), _ptr(k_plane), _ptr(v_plane), _i(_code(k_plane)), _ptr(positions),
        _ptr(row_req), _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim),
        _i(window), _f(scale), _stream())
    _check(st, "paged_attention")


def _pin_and_gap(pin: Optional[torch.Tensor], gap: Optional[torch.Tensor], T: int, top_k: int) -> None:
    if pin is not None:
        _need(pin, "pin", torch.int32)
        if pin.numel() != T * top_k or gap is not None:
            raise KernelError(f"router: pin must hold {T} x {top_k} experts and excludes gap")
    if gap is not None:
        _need(gap, "gap", torch.float32)
        if gap.numel() != T:
            raise KernelError(f"router: gap must hold {T} margins")


def router_topk(x: torch.Tensor, router_w: torch.Tensor, shared_gate: Optional[torch.Tensor], top_k: int,
                norm_topk: bool, sel: torch.Tensor, weights: torch.Tensor, shared_scale: Optional[torch.Tensor],
                pin: Optional[torch.Tensor] = None, gap: Optional[torch.Tensor] = None) -> None:
    """Router logits, softmax over all experts, top-k and the shared expert's sigmoid gate.
    ``pin`` (int32 [T, k]): the experts are given, not chosen; the weights are still the row's own
    probabilities of them.  ``gap`` (float32 [T], not with ``pin``): each row's routing margin
    (p_k - p_{k+1}) / p_k out."""
    _need(x, "x", torch.float32), _need(router_w, "router_w", torch.float32)
    _need(sel, "sel", torch.int32), _need(weights, "weights", torch.float32)
    T, H = x.shape
    E = router_w.shape[0]
    _pin_and_gap(pin, gap, T, top_k)
    if E > 1024:
        raise KernelError(f"router_topk: {E} experts; this kernel takes at most 1024")
    if shared_gate is not None:
        _need(shared_gate, "shared_gate", torch.float32), _need(shared_scale, "shared_scale", torch.float32)
    logits = torch.empty((T, E + 1), dtype=torch.float32, device=x.device)
    tickets = _router_tickets.get(x.device)
    if tickets is None:
        tickets = _router_tickets[x.device] = torch.zeros((4,), dtype=torch.int32, device=x.device)
    st = library("moe_route").cj_router_topk(_ptr(x), _ptr(router_w), _ptr(shared_gate), _i(T), _i(H), _i(E), _i(top_k),
                                             _i(1 if norm_topk else 0), _ptr(sel), _ptr(weights), _ptr(shared_scale),
                                             _ptr(logits), _ptr(tickets), _ptr(pin), _ptr(gap), _stream())
    _check(st, "router_topk")
    if T > 32:
        global launches
        launches += 1                  # many rows take two kernels: logits, then selection


def router_select(partials: torch.Tensor, num_experts: int, top_k: int, norm_topk: bool, sel: torch.Tensor,
                  weights: torch.Tensor, shared_scale: Optional[torch.Tensor], pin: Optional[torch.Tensor] = None,
                  gap: Optional[torch.Tensor] = None) -> None:
    """Softmax over all experts, top-k and the shared gate's sigmoid from router logits given
    as partial sums ``[S, T, ld]`` (float32; column ``num_experts`` holds the gate's dot when
    ``shared_scale`` is given); the partials of a row are added in order first."""
    _need(partials, "partials", torch.float32), _need(sel, "sel", torch.int32), _need(weights, "weights", torch.float32)
    if partials.dim() != 3:
        raise KernelError(f"router_select: partials {tuple(partials.shape)} are not [S, T, ld]")
    if num_experts > 1024:
        raise KernelError(f"router_select: {num_experts} experts; this kernel takes at most 1024")
    S, T, ld = partials.shape
    _pin_and_gap(pin, gap, T, top_k)
    if shared_scale is not None:
        _need(shared_scale, "shared_scale", torch.float32)
    st = library("moe_route").cj_router_select(_ptr(partials), _i(S), _ll(partials.stride(0)), _i(ld), _i(T), _i(num_experts),
                                               _i(top_k), _i(1 if norm_topk else 0), _ptr(sel), _ptr(weights),
                                               _ptr(shared_scale), _ptr(pin), _ptr(gap), _stream())
    _check(st, "router_select")


def moe_group(sel: torch.Tensor, top_k: int, num_experts: int, offsets: torch.Tensor, slot_token: torch.Tensor,
              slot_of_pick: torch.Tensor, extra_groups: int = 0) -> None:
    """Counting sort of the picks by expert: offsets [E + extra + 1], slot_token, slot_of_pick.
    ``extra_groups`` groups that hold every token follow the routed ones."""
    for n, t in (("sel", sel), ("offsets", offsets), ("slot_token", slot_token), ("slot_of_pick", slot_of_pick)):
        _need(t, n, torch.int32)
    n = sel.numel()
    if offsets.numel() < num_experts + extra_groups + 1 or slot_token.numel() < n + extra_groups * (n // top_k):
        raise KernelError("moe_group: offsets or slot_token too small for the extra groups")
    st = library("moe_route").cj_moe_group(_ptr(sel), _i(n), _i(top_k), _i(num_experts), _i(extra_groups), _ptr(offsets),
                                           _ptr(slot_token), _ptr(slot_of_pick), _stream())
    _check(st, "moe_group")


def moe_combine(hs: torch.Tensor, y: Optional[torch.Tensor], slot_of_pick: Optional[torch.Tensor],
                weights: Optional[torch.Tensor], top_k: int, shared: Optional[torch.Tensor],
                shared_scale: Optional[torch.Tensor]) -> None:
    """hs[t] += sum_j weights[t, j] * y[slot_of_pick[t, j]] (+ shared_scale[t] * sum_c shared[c, t]).
    ``shared`` is [T, H] or, computed in chunks, [chunks, T, H]."""
    _need(hs, "hs", torch.float32)
    T, H = hs.shape
    for n, t in (("y", y), ("weights", weights), ("shared", shared), ("shared_scale", shared_scale)):
        if t is not None:
            _need(t, n, torch.float32)
    if slot_of_pick is not None:
        _need(slot_of_pick, "slot_of_pick", torch.int32)
    chunks, stride = 1, 0
    if shared is not None and shared.dim() == 3:
        chunks, stride = shared.shape[0], shared.stride(0)
    st = library("rowwise").cj_moe_combine(_ptr(hs), _ptr(y), _ptr(slot_of_pick), _ptr(weights), _i(top_k), _ptr(shared),
                                           _i(chunks), _ll(stride), _ptr(shared_scale), _i(T), _i(H), _stream())
    _check(st, "moe_combine")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """First-occurrence argmax of each row of float32 logits into int32 out."""
    _need(logits, "logits", torch.float32), _need(out, "out", torch.int32)
    rows, V = logits.shape
    st = library("sampling").cj_argmax(_ptr(logits), _i(rows), _i(V), _ptr(out), _stream())
    _check(st, "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, scratch: torch.Tensor,
           out: torch.Tensor, top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           repeat_penalty: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None,
           history_offsets: Optional[torch.Tensor] = None) -> None:
    """One token per row by the reference's sampler order; scratch is [rows, V] float32."""
    _need(logits, "logits", torch.float32), _need(temperature, "temperature", torch.float32)
    _need(uniform, "uniform", torch.float32), _need(scratch, "scratch", torch.float32), _need(out, "out", torch.int32)
    rows, V = logits.shape
    if scratch.numel() < rows * V:
        raise KernelError("sample: scratch is smaller than the logits")
    for n, t, d in (("top_k", top_k, torch.int32), ("top_p", top_p, torch.float32),
                    ("repeat_penalty", repeat_penalty, torch.float32), ("history", history, torch.int32),
                    ("history_offsets", history_offsets, torch.int32)):
        if t is not None:
            _need(t, n, d)
    st = library("sampling").cj_sample(_ptr(logits), _i(rows), _i(V), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                       _ptr(repeat_penalty), _ptr(uniform), _ptr(history), _ptr(history_offsets),
                                       _ptr(scratch), _ptr(out), _stream())
    _check(st, "sample")


def random_fill(out: torch.Tensor, key: int, scale: float) -> None:
    """out.flat[i] = float32(n(key, i)) * scale, n a centred sum of eight 16-bit integers hashed
    from (key, i); float32 or bfloat16 (see weights/random_fill.py for the same on the host)."""
    _need(out, "out")
    st = library("random_fill").cj_random_fill(_ptr(out), _i(_code(out)), _ll(out.numel()), ctypes.c_ulonglong(key & (2 ** 64 - 1)),
                                               _f(scale), _stream())
    _check(st, "random_fill")


EPI_STORE_F32, EPI_ACC_F32, EPI_SWIGLU_BF16, EPI_STORE_BF16 = 0, 1, 2, 3


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, swap: bool, n_mma: int,
            bias: Optional[torch.Tensor] = None, w_up: Optional[torch.Tensor] = None,
            group_offsets: Optional[torch.Tensor] = None, tokens: Optional[int] = None, k_splits: int = 1,
            offsets_settled: bool = False) -> None:
    """Tensor-core product out[token, feature] (+)= x[token, :] . w[feature, :] (+ bias) in
    bfloat16 with float32 accumulation (tcgen05, TMA).

    ``swap`` False: tiles of 128 tokens x ``n_mma`` (128 or 256) features; True: tiles of 128
    features x ``n_mma`` (16, 32, 64, 96, 128, 160, 192, 256) tokens.  ``epilogue``: EPI_STORE_F32, EPI_ACC_F32,
    EPI_SWIGLU_BF16 (``w_up`` given), EPI_STORE_BF16.  With ``group_offsets`` the rows of
    ``x`` are sorted by group and ``w`` is [groups, features, K].  ``k_splits`` > 1 (store
    only): ``out`` is [k_splits, tokens, features] of partial sums.  ``offsets_settled``: the
    kernel that wrote ``group_offsets`` is not the one launched just before this product but an
    earlier one; the product then reads them before it waits for the kernel before it.
    """
    _need(x, "x", torch.bfloat16), _need(w, "w", torch.bfloat16), _need(out, "out")
    features, K = w.shape[-2], w.shape[-1]
    T = tokens if tokens is not None else x.shape[0]
    if x.shape[-1] != K or out.shape[-1] != features:
        raise KernelError(f"gemm_tc: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)} do not agree")
    want = torch.bfloat16 if epilogue in (EPI_SWIGLU_BF16, EPI_STORE_BF16) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc: epilogue {epilogue} writes {want}, out is {out.dtype}")
    if w_up is not None:
        _need(w_up, "w_up", torch.bfloat16)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    G = 0
    if group_offsets is not None:
        _need(group_offsets, "group_offsets", torch.int32)
        G = w.shape[0]
    split_stride = out.stride(0) if k_splits > 1 else 0
    ldo = out.stride(-2)
    st = library("gemm_tc").cj_gemm_tc(
        _ptr(x), _ll(x.stride(0)), _ptr(w), _ptr(w_up), _ptr(bias), _ptr(out), _ll(ldo), _i(T), _i(features), _i(K),
        _i(epilogue), _i(1 if swap else 0), _i(n_mma), _ptr(group_offsets), _i(G), _i(k_splits), _ll(split_stride),
        _i(1 if offsets_settled and group_offsets is not None else 0), _stream())
    _check(st, "gemm_tc")


def gemm_tc2(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, n_tok: int,
             bias: Optional[torch.Tensor] = None, w_up: Optional[torch.Tensor] = None,
             group_offsets: Optional[torch.Tensor] = None, tokens: Optional[int] = None) -> None:
    """The same product as ``gemm_tc`` on pairs of SMs (tcgen05 cta_group::2): tiles of 256
    features x ``n_tok`` (128 or 256) tokens, each SM of a pair loading its own 128 weight rows
    and half of the token rows.  For steps with many rows."""
    _need(x, "x", torch.bfloat16), _need(w, "w", torch.bfloat16), _need(out, "out")
    features, K = w.shape[-2], w.shape[-1]
    T = tokens if tokens is not None else x.shape[0]
    if x.shape[-1] != K or out.shape[-1] != features:
        raise KernelError(f"gemm_tc2: shapes x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)} do not agree")
    want = torch.bfloat16 if epilogue in (EPI_SWIGLU_BF16, EPI_STORE_BF16) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc2: epilogue {epilogue} writes {want}, out is {out.dtype}")
    if w_up is not None:
        _need(w_up, "w_up", torch.bfloat16)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    G = 0
    if group_offsets is not None:
        _need(group_offsets, "group_offsets", torch.int32)
        G = w.shape[0]
    st = library("gemm_tc2").cj_gemm_tc2(
        _ptr(x), _ll(x.stride(0)), _ptr(w), _ptr(w_up), _ptr(bias), _ptr(out), _ll(out.stride(-2)), _i(T), _i(features), _i(K),
        _i(epilogue), _i(n_tok), _ptr(group_offsets), _i(G), _stream())
    _check(st, "gemm_tc2")


def gemm_tc_error() -> int:
    """0, or the code of a bounded wait inside a tensor-core kernel that ran out of time."""
    return int(library("gemm_tc").cj_gemm_tc_error())


def gather_rows(x: torch.Tensor, index: torch.Tensor, out: torch.Tensor) -> None:
    """out[s, :] = x[index[s], :]."""
    _need(x, "x"), _need(index, "index", torch.int32), _need(out, "out", x.dtype)
    st = library("rowwise").cj_gather_rows(_ptr(out), _ptr(x), _i(_code(x)), _ptr(index), _i(out.shape[0]), _i(x.shape[-1]), _stream())
    _check(st, "gather_rows")


# CAJETA_B200_DECODE_FMA=1: decode attention on the FMA pipe instead of the tensor cores (for comparison)
DECODE_TENSOR_CORES = os.environ.get("CAJETA_B200_DECODE_FMA", "0") != "1"
# (row, head) pairs from which on the merge of a row's chunks is a kernel of its own: the attention
# blocks then end without a fence and a ticket, and their shared memory is free that much sooner.
# Measured: 64 rows x 16 heads +9 % (576 keys) and +10 % (2,048 keys: 5.1 TB/s); 32 rows the same
# either way; 8 rows of 4,096 keys 7 % slower (few merges, each a long chain, no longer hidden).
# (Rows of many chunks with few rows in the step - 1 or 4 rows of 16,384 keys - were measured too: the merge
# as a kernel of its own is a tail that nothing overlaps, 2.78 -> 3.32 ms and 5.28 -> 6.03 ms a step.)
MERGE_LATER_MIN_ROW_HEADS = 1024


def decode_chunk(span: int) -> int:
    """Keys a block of the split-KV decode kernel takes.  The kernel also takes 64; measured on
    a B200 it gains nothing for a handful of rows and loses 10 % for many, so 128 it is."""
    return 128


def decode_attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                     positions: torch.Tensor, row_req: torch.Tensor, table: torch.Tensor, page_tokens: int,
                     n_heads: int, n_kv: int, head_dim: int, window: int, scale: float, max_context: int,
                     scratch: "DecodeScratch", chunk: int = 0, tensor_cores: Optional[bool] = None,
                     merge_later: Optional[bool] = None) -> None:
    """Split-KV attention of few bfloat16 query rows over their cached keys (head_dim 64 or 128).
    ``tensor_cores``: scores and weighted values of a chunk by mma.sync (the default) or on the
    FMA pipe (``chunk`` 64 or 128 applies to that form only).  ``merge_later``: the chunks of a
    row are merged by a kernel of its own instead of the row's last block (the default for steps
    with many rows; same results to the bit)."""
    for n, t in (("q", q), ("out", out), ("k_plane", k_plane), ("v_plane", v_plane)):
        _need(t, n, torch.bfloat16)
    _need(positions, "positions", torch.int32), _need(row_req, "row_req", torch.int32), _need(table, "table", torch.int32)
    T = q.shape[0]
    span = min(window, max_context) if window > 0 else max_context
    if tensor_cores is None:
        tensor_cores = DECODE_TENSOR_CORES and chunk == 0
    if tensor_cores:
        splits = max(1, -(-span // 128))
        scratch.ensure(T, n_heads, n_kv, head_dim, splits, q.device)
        if merge_later is None:
            merge_later = T * n_heads >= MERGE_LATER_MIN_ROW_HEADS
        st = library("attention_decode").cj_decode_attention_tc(
            _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _ptr(positions), _ptr(row_req), _ptr(table),
            _i(table.stride(0)), _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim), _i(window), _f(scale),
            _i(max_context), _ptr(scratch.acc), _ptr(scratch.ml), _ptr(scratch.counters), _i(scratch.splits),
            _i(1 if merge_later else 0), _stream())
        _check(st, "decode_attention")
        if merge_later and splits > 1:
            global launches
            launches += 1                  # the merge kernel
        return
    chunk = chunk or decode_chunk(span)
    splits = max(1, -(-span // chunk))
    scratch.ensure(T, n_heads, n_kv, head_dim, splits, q.device)
    st = library("attention_decode").cj_decode_attention(
        _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _ptr(positions), _ptr(row_req), _ptr(table), _i(table.stride(0)),
        _i(page_tokens), _i(T), _i(n_heads), _i(n_kv), _i(head_dim), _i(window), _f(scale), _i(max_context),
        _ptr(scratch.acc), _ptr(scratch.ml), _ptr(scratch.counters), _i(scratch.splits), _i(chunk), _stream())
    _check(st, "decode_attention")


class DecodeScratch:
    """Partial results of the split-KV decode kernel and its arrival counters (kept zero
    between launches by the kernel itself)."""

    def __init__(self):
        self.acc = self.ml = self.counters = None
        self.rows = self.heads = self.kv = self.hd = self.splits = 0

    def ensure(self, rows: int, heads: int, kv: int, hd: int, splits: int, device) -> None:
        if (self.acc is None or rows > self.rows or heads != self.heads or kv != self.kv or hd != self.hd
                or splits > self.splits):
            self.rows, self.heads, self.kv, self.hd = max(rows, self.rows), heads, kv, hd
            self.splits = max(splits, self.splits)
            self.acc = torch.empty((self.rows, heads, self.splits, hd), dtype=torch.float32, device=device)
            self.ml = torch.empty((self.rows, heads, self.splits, 2), dtype=torch.float32, device=device)
            self.counters = torch.zeros((self.rows * heads,), dtype=torch.int32, device=device)


def prefill_attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                      req_start: torch.Tensor, req_prior: torch.Tensor, table: torch.Tensor, page_tokens: int,
                      n_heads: int, n_kv: int, head_dim: int, window: int, scale: float, block_rows: int = 0) -> None:
    """Tensor-core attention of a step's rows (request r owns rows req_start[r]..req_start[r+1]
    at positions req_prior[r] + i) over the paged cache; bfloat16, head_dim 64 or 128."""
    for n, t in (("q", q), ("out", out), ("k_plane", k_plane), ("v_plane", v_plane)):
        _need(t, n, torch.bfloat16)
    _need(req_start, "req_start", torch.int32), _need(req_prior, "req_prior", torch.int32), _need(table, "table", torch.int32)
    st = library("attention_prefill").cj_prefill_attention(
        _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _ptr(req_start), _ptr(req_prior), _i(req_prior.numel()),
        _i(q.shape[0]), _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(n_heads), _i(n_kv), _i(head_dim), _i(window),
        _f(scale), _i(block_rows), _stream())
    _check(st, "prefill_attention")


def prefill_attention_tc(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                         req_start: torch.Tensor, req_prior: torch.Tensor, table: torch.Tensor, page_tokens: int,
                         n_heads: int, n_kv: int, head_dim: int, window: int, scale: float, block_rows: int = 0) -> None:
    """The same contract as ``prefill_attention`` on the tcgen05 tensor cores: both products
    from shared memory into tensor memory.  ``block_rows``: 256 query rows a block (two tiles
    taking turns), 128, or 0 = by the size of the launch.  Head size 128 and pages of 16 tokens
    only; anything else is refused."""
    for n, t in (("q", q), ("out", out), ("k_plane", k_plane), ("v_plane", v_plane)):
        _need(t, n, torch.bfloat16)
    _need(req_start, "req_start", torch.int32), _need(req_prior, "req_prior", torch.int32), _need(table, "table", torch.int32)
    if head_dim != 128 or page_tokens != 16:
        raise KernelError(f"prefill_attention_tc takes head size 128 and 16-token pages, not {head_dim} and {page_tokens}")
    st = library("attention_prefill_tc").cj_prefill_attention_tc(
        _ptr(q), _ptr(out), _ptr(k_plane), _ptr(v_plane), _i(k_plane.shape[0]), _ptr(req_start), _ptr(req_prior),
        _i(req_prior.numel()), _i(q.shape[0]), _ptr(table), _i(table.stride(0)), _i(page_tokens), _i(n_heads), _i(n_kv),
        _i(head_dim), _i(window), _f(scale), _i(block_rows), _stream())
    _check(st, "prefill_attention_tc")


def prefill_attention_tc_error() -> int:
    """0, or the code of a bounded wait inside the tensor-core attention that ran out of time."""
    return int(library("attention_prefill_tc").cj_prefill_attention_tc_error())


def wait_errors() -> Dict[str, int]:
    """Codes of bounded waits that ran out inside the tensor-core kernels, by library; empty
    when all is well.  Only libraries that are already loaded are asked."""
    found = {}
    for name, symbol in (("gemm_tc", "cj_gemm_tc_error"), ("gemm_tc2", "cj_gemm_tc2_error"),
                         ("attention_prefill_tc", "cj_prefill_attention_tc_error")):
        lib = _libs.get(name)
        if lib is not None:
            code = int(getattr(lib, symbol)())
            if code != 0:
                found[name] = code
    return found
