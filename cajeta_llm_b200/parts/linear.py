"""One place that decides which matrix-product kernel a part's projection runs on.

``project`` computes ``out[token, feature] (+)= x[token, :] . w[feature, :]`` (+ bias), or
the SwiGLU of two such products, for a dense weight or for the stacked weights of a
mixture of experts.  On the bfloat16 path it runs on the tensor cores (tcgen05 / TMA)
when the shapes allow TMA (K a multiple of 8, 16-byte aligned rows) and are large
enough to fill a tile; otherwise, and always on the float32 path, it runs on the FMA
pipe, whose results do not depend on the batch at all.  Few rows (decode) put the
weights on the rows of the tensor-core product, many rows (prompt portions) the tokens.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import kernels as K

# below these sizes a tensor-core tile would be mostly padding
MIN_K = 128
MIN_FEATURES = 128


def _tc_ok(runtime, x: torch.Tensor, w: torch.Tensor) -> bool:
    if not runtime.fast_kernels or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    Kd, features = w.shape[-1], w.shape[-2]
    return (Kd >= MIN_K and Kd % 8 == 0 and features >= MIN_FEATURES and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.stride(-1) == 1)


TOKEN_TILES = (16, 32, 64, 96, 128, 160, 192, 256)     # token tiles of the weights-on-rows orientation


def _token_tile(rows: int) -> int:
    for n in (16, 32, 64, 128):
        if rows <= n:
            return n
    return 0


def _group_tile(total_rows: int, groups: int) -> int:
    """Token tile for ragged groups: wide enough that a typical group (mean + two standard
    deviations of an even split) is one tile, so its weights are streamed once."""
    mean = total_rows / max(1, groups)
    want = mean + 2.0 * mean ** 0.5
    for n in TOKEN_TILES:
        if want <= n:
            return n
    return TOKEN_TILES[-1]


PAIR_MIN_ROWS = 512          # dense products with at least this many rows run on pairs of SMs
PAIR_MIN_GROUP_ROWS = 96     # grouped products whose groups average at least this many rows do


def _pair_tile(runtime, rows: int, w: torch.Tensor, swiglu: bool, grouped: bool) -> int:
    """Token tile (128 or 256) of the two-SM product when the shape calls for it, else 0."""
    features = w.shape[-2]
    if features < 256:
        return 0
    if swiglu:
        # the two-SM SwiGLU puts 256 tokens on the product's rows: right for a dense layer with
        # many rows, wasteful for ragged groups (an expert with 136 rows pays for 256), which
        # stay on the one-SM kernel with the tokens on the product's N
        return 256 if not grouped and rows >= PAIR_MIN_ROWS else 0
    if grouped:
        mean = rows / max(1, w.shape[0])
        if mean < PAIR_MIN_GROUP_ROWS:
            return 0
        return 256 if mean + 2.0 * mean ** 0.5 > 128 else 128
    if rows < PAIR_MIN_ROWS:
        return 0
    feature_tiles = -(-features // 256)
    # the wider tile only when its tiles still give every pair of SMs one
    return 256 if feature_tiles * -(-rows // 256) >= runtime.sm_count // 2 else 128


def project(runtime, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
            accumulate: bool = False, w_up: Optional[torch.Tensor] = None, group_offsets: Optional[torch.Tensor] = None,
            a_row_index: Optional[torch.Tensor] = None, max_group_rows: Optional[int] = None,
            offsets_settled: bool = False) -> None:
    """``x``: [tokens, K]; ``w``: [features, K] or, with ``group_offsets``, [groups, features, K]
    where output row s belongs to the group whose range holds s and reads row
    ``a_row_index[s]`` of ``x`` (or row s).  ``w_up`` selects the SwiGLU form (``out`` in the
    activation dtype).  ``max_group_rows`` bounds the rows of any one group when known.
    ``offsets_settled``: the kernel that wrote ``group_offsets`` is not the last one launched
    before this call's product (another kernel of this engine ran since, or this call's own
    row gather does); the product may then read the offsets before it waits for that kernel."""
    if not _tc_ok(runtime, x, w):
        K.gemm(x, w, out, bias=bias, accumulate=accumulate, w_up=w_up, group_offsets=group_offsets, a_row_index=a_row_index)
        return
    rows = out.shape[0]
    if w_up is not None:
        epi = K.EPI_SWIGLU_BF16
    elif out.dtype == torch.bfloat16:
        epi = K.EPI_STORE_BF16
    else:
        epi = K.EPI_ACC_F32 if accumulate else K.EPI_STORE_F32
    bound = rows if max_group_rows is None else min(rows, max_group_rows)
    if a_row_index is not None:
        gathered = torch.empty((rows, x.shape[-1]), dtype=x.dtype, device=x.device)
        tag, K.tag = K.tag, "row gather"
        K.gather_rows(x, a_row_index, gathered)
        K.tag = tag
        x = gathered
        offsets_settled = True
    # few rows: weights on the rows of the product; a group of a mixture rarely has more
    # rows than the step has tokens, which bounds the token tile
    tile = _token_tile(bound)
    if not tile and group_offsets is not None:
        # ragged groups: weights on the rows, tokens on the product's N (cut to the tokens a
        # tile really has), the tile wide enough that most groups stream their weights once
        # (the SwiGLU form keeps two accumulators per stage: beyond 128 tokens tensor memory
        # holds one stage only and the epilogue no longer overlaps the next tile: tiles of 160 or 256 tokens
        # measured 131 -> 146 us a layer at 2,048 prompt rows, 198 -> 231 us at 4,096)
        tile = min(128, _group_tile(rows, w.shape[0])) if w_up is not None else _group_tile(rows, w.shape[0])
    pair_tile = 0 if tile and group_offsets is None else _pair_tile(runtime, rows, w, w_up is not None, group_offsets is not None)
    if pair_tile:
        # many rows: tiles of 256 features on pairs of SMs, each loading half of the token rows
        K.gemm_tc2(x, w, out, epi, pair_tile, bias=bias, w_up=w_up, group_offsets=group_offsets, tokens=rows)
    elif tile:
        K.gemm_tc(x, w, out, epi, True, tile, bias=bias, w_up=w_up, group_offsets=group_offsets, tokens=rows,
                  offsets_settled=offsets_settled)
    else:
        n_mma = 256 if (w_up is None and w.shape[-2] >= 512) else 128
        K.gemm_tc(x, w, out, epi, False, n_mma, bias=bias, w_up=w_up, group_offsets=group_offsets, tokens=rows,
                  offsets_settled=offsets_settled)


def project_split(runtime, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """For a few rows and a weight with few output features: the product cut along K into
    enough pieces to occupy the machine.  Returns the partial sums [S, tokens, features]
    (float32; the bias is in the first), to be added by the consumer in order - or None
    when the shapes do not call for it (the caller then uses :func:`project`)."""
    if not _tc_ok(runtime, x, w):
        return None
    rows = x.shape[0]
    tile = _token_tile(rows)
    if not tile:
        return None
    features, Kd = w.shape[-2], w.shape[-1]
    feature_tiles = -(-features // 128) * -(-rows // tile)
    k_blocks = -(-Kd // 64)
    # as many pieces as it takes to give (nearly) every SM a block; 7/8 of them, so that a
    # product of 16 tiles is cut into 8 pieces of equal length rather than 9 ragged ones
    splits = min(8, max(1, (runtime.sm_count * 7 // 8) // feature_tiles), max(1, k_blocks // 4))
    if splits < 2:
        return None
    parts = torch.empty((splits, rows, features), dtype=torch.float32, device=x.device)
    K.gemm_tc(x, w, parts, K.EPI_STORE_F32, True, tile, bias=bias, k_splits=splits)
    return parts
