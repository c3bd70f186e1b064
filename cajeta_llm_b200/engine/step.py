"""The step function: one mixed batch of (request, its next tokens) through the model.

A step holds, for each request in it, the next tokens of that request: a portion of a
prompt of any length, or a single decoded token; portions and single tokens sit side
by side and a prompt may be cut anywhere.  The step runs only these tokens, as one
batch of rows, against what earlier steps left in the cache, and returns the float32
logits at the wanted places.

The reference has three entry points instead (one sequence ``stepSeq``, several prompt
chunks ``stepPrefillBatch``, up to eight decode rows ``stepDecodeBatch``:
model/CausalLM.cajeta:801-878,955-1066,4445-4512) and never mixes chunks with decode
rows in one pass (sched/Scheduler.cajeta:572-573); here one call serves all of them.

Rows are laid out request after request; each row carries its request's index in the
step (``row_req``) and its absolute position, each request its first row, row count and
the length it had before the step.  All of this plus the block-table rows of the
step's requests goes to the device in one pinned buffer and one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from .model import Model


class OutOfPages(RuntimeError):
    """The cache has too few free pages for this step; nothing was changed."""


class StepError(ValueError):
    """A step that cannot run: unknown slot, token id out of range, bad ``want``."""


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class EntryContext:
    """What one schedule entry sees of the cache during a step."""

    index: int
    writes_cache: bool
    k_plane: Optional[torch.Tensor]
    v_plane: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]      # int32 [requests, width] of the entry's group
    page_tokens: int
    state: Optional[torch.Tensor]            # [max_seqs, ...] per-request state of this entry


@dataclass
class StepContext:
    """Metadata of one step, on the device and (``h_`` fields) on the host."""

    n_rows: int
    n_requests: int
    token_ids: torch.Tensor        # int32 [rows]
    positions: torch.Tensor        # int32 [rows] absolute position of each row
    row_req: torch.Tensor          # int32 [rows] index of the row's request within the step
    req_start: torch.Tensor        # int32 [requests + 1] first row of each request
    req_prior: torch.Tensor        # int32 [requests] tokens cached before this step
    req_slot: torch.Tensor         # int32 [requests] cache slot of each request
    want_rows: torch.Tensor        # int32 [wanted] rows whose logits are returned
    tables: List[torch.Tensor]     # per cache group: int32 [requests, width]
    h_req_start: List[int] = field(default_factory=list)
    h_req_prior: List[int] = field(default_factory=list)
    h_req_slot: List[int] = field(default_factory=list)
    max_rows_per_request: int = 0
    max_context: int = 0           # longest prior + new over the step's requests
    all_single: bool = False       # every request brings exactly one token
    decode_scratch: Optional[object] = None    # scratch of the split-KV decode attention for this step (None: the runtime's)
    routing_pin: Optional[Dict[str, torch.Tensor]] = None     # a routed feed-forward's prefix -> int32 [rows, k]: experts given, not chosen
    routing_dump: Optional[Dict[str, tuple]] = None           # filled by routed feed-forwards: prefix -> (experts [rows, k], margins [rows])


@dataclass
class _CapturedStep:
    """A decode step of fixed batch size and context bucket, captured as a CUDA graph."""

    graph: "torch.cuda.CUDAGraph"
    meta: torch.Tensor          # static device metadata the captured kernels read
    logits: torch.Tensor        # static output [batch, vocab]
    launches: int               # kernels the graph replays
    scratch: object             # kernel scratch the graph's kernels point into; lives as long as the graph


GRAPH_CONTEXT_BUCKET = 1024     # captured decode steps are keyed by the context rounded up to this
MIXED_CAPTURE_AFTER = 2         # a step shape (rows, requests, wanted) is captured when it is met this often
MIXED_GRAPHS_MAX = 16           # captured step shapes kept; the one replayed longest ago goes first
WAIT_CHECK_EVERY = 64           # steps between looks at the kernels' wait-error flags


class ModelRunner:
    """Owns a model and its cache; ``step`` is the only way tokens reach the model.

    A step in which every request brings exactly one token (pure decode) is launch-bound:
    hundreds of small kernels.  On the bfloat16 path such a step is captured once per
    (batch size, context bucket) as a CUDA graph and replayed afterwards; the step's
    metadata (tokens, positions, block tables, slots) lives in a static device buffer that is
    refreshed before each replay.  The captured kernels are the same ones an uncaptured
    step launches, so both give the same logits.

    Steps with prompt portions are bound by the host too when they are small (a few hundred
    launches from Python take longer than the device needs for a few hundred rows).  Which
    kernels such a step launches, and with which grids, depends only on its number of rows,
    of requests and of wanted rows - how the rows are shared out among the requests, where
    each request stands and which pages it owns is device metadata - so a shape that comes
    again (the portions of one long prompt beside the same decoding requests, prompts of one
    length) is captured at its second appearance and replayed from then on.
    """

    def __init__(self, model: Model, page_tokens: int = 16, max_seqs: int = 4, max_tokens_per_seq: int = 4096,
                 num_pages: Optional[int] = None, cuda_graphs: bool = True, max_step_tokens: int = 0):
        """``num_pages``: the pool size of every cache group; None sizes each group by its own
        need: ``max_seqs`` requests of ``max_tokens_per_seq`` tokens for a group that keeps every
        key, and for a windowed group ``max_seqs`` times what a window plus one step's tokens of a
        request span (``max_step_tokens``, the most tokens a request brings in one step; 0 = up to
        a whole request, which sizes the windowed group like the others)."""
        self.model = model
        self.runtime = model.runtime
        if num_pages is None:
            whole = -(-max_tokens_per_seq // page_tokens)

            def num_pages(spec):
                if spec.window > 0 and max_step_tokens > 0:
                    return max_seqs * min(whole, -(-(spec.window + max_step_tokens) // page_tokens) + 1)
                return max_seqs * whole
        self.max_step_tokens = max_step_tokens
        self.cache = CacheManager(model.kv_needs(), model.state_needs(), model.cache_from(), page_tokens, max_seqs,
                                  max_tokens_per_seq, num_pages, self.runtime.cache_dtype, self.runtime.device)
        self.page_tokens = page_tokens
        self.max_tokens_per_seq = max_tokens_per_seq
        self.steps_run = 0
        # Steps are captured as CUDA graphs on the bfloat16 path - unless a mixer keeps state and has
        # not said that it is safe to capture.  A mixer with state says so with ``graph_safe = True``:
        # it then finds its requests' slots, rows and positions in the step's DEVICE metadata only
        # (``ctx.req_slot``, ``ctx.req_start``, ``ctx.row_req``, ``ctx.positions``: a captured step is
        # replayed with other values in them), reads nothing back on the host, and leaves alone the
        # requests a step's layout is filled up with (slot -1, no rows).
        mixers = [model.blocks[e.layer].mixer for e in model.plan.schedule]
        graph_safe = all(getattr(m, "graph_safe", m.state_need() is None) for m in mixers)
        self.cuda_graphs = cuda_graphs and graph_safe and self.runtime.fast_kernels and self.runtime.device.type == "cuda"
        # what this model needs is compiled now, side by side (a library not named here is still
        # compiled when it is first wanted)
        if str(self.runtime.device).startswith("cuda"):
            from ..csrc import build as _build
            _build.build_all(sorted(n for n in model.libraries() if n in _build.LIBRARIES))
        self._graphs: Dict[Tuple[int, int], _CapturedStep] = {}
        self._mixed_graphs: Dict[Tuple[int, int, int], _CapturedStep] = {}   # by (rows, wanted rows filled up, requests rounded up), oldest use first
        self._mixed_seen: Dict[Tuple[int, int], int] = {}
        self._graph_pool = None
        self._decode_host: Dict[Tuple[int, int], tuple] = {}   # pinned metadata of decode steps by (rows, width), reused
        self._meta_copied = None                               # event: the last copy out of the buffer in use is over
        self.graph_replays = 0

    # -- requests --------------------------------------------------------------------
    def admit(self) -> Optional[int]:
        return self.cache.admit()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    # -- the step --------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], routing_pin: Optional[Dict[str, torch.Tensor]] = None,
             routing_dump: Optional[Dict[str, tuple]] = None) -> torch.Tensor:
        """Run one batch; returns float32 logits ``[wanted, vocab]`` in the order of the
        entries and of each entry's ``want``.  Raises :class:`OutOfPages` (cache
        unchanged) when the pages for the new tokens are not there.

        ``routing_pin``: for routed feed-forwards, by the part's tensor-name prefix, the experts
        of every row of this step (int32 ``[rows, k]`` on the device, rows in the step's order):
        they are taken as given instead of chosen - the way to replay recorded selections, as
        the reference does (model/MoeFfn.cajeta:626-706).  ``routing_dump``: a dict that receives,
        by prefix, the experts each row picked and its routing margin (p_k - p_{k+1}) / p_k
        (margins are None under a pin).  A step with either is launched kernel by kernel."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return torch.empty((0, self.model.vocab), dtype=torch.float32, device=self.runtime.device)
        self._calls = getattr(self, "_calls", 0) + 1
        if self._calls % WAIT_CHECK_EVERY == 0:
            self.check_waits()
        if routing_pin is not None or routing_dump is not None:
            ctx = self._prepare(entries)
            ctx.routing_pin, ctx.routing_dump = routing_pin, routing_dump
            logits = self._forward(ctx)
        elif self.cuda_graphs and all(len(e.tokens) == 1 for e in entries):
            return self._step_captured(entries)
        elif self.cuda_graphs:
            logits = self._step_mixed(entries)
        else:
            logits = self._forward(self._prepare(entries))
        for e in entries:
            self.cache.commit(e.slot, len(e.tokens))
        self.steps_run += 1
        return logits

    def _step_mixed(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step with prompt portions on the bfloat16 path: uncaptured the first time its shape
        is met, captured the second time, replayed afterwards.  The shape is the number of rows,
        the number of requests rounded up to a power of two (at most ``max_seqs``: the per-request
        arrays are laid out for that many, the others bring no rows) and the number of wanted
        rows, which up to the padded number of requests is filled up to it (the logits of the
        fillers are thrown away; a step that wants nothing stays so) - so that the steps of a
        scheduler that fills a token budget, the same number of rows step after step among a
        changing number of requests of which a changing number ends, replay a few graphs.  (Laid
        out for ``max_seqs`` requests whatever the step has, a lone prompt portion paid for the
        row blocks that sixty-three absent requests could have had: the attention's grid covers
        the most the layout can hold.)"""
        from ..csrc import kernels as K
        rows = sum(len(e.tokens) for e in entries)
        wanted = sum(len(e.want) for e in entries)
        pad_requests = min(self.cache.max_seqs, 1 << max(0, len(entries) - 1).bit_length())
        pad_wanted = 0 if wanted == 0 else max(wanted, min(rows, pad_requests))
        key = (rows, pad_wanted, pad_requests)
        cap = self._mixed_graphs.get(key)
        if cap is None:
            seen = self._mixed_seen[key] = self._mixed_seen.get(key, 0) + 1
            if len(self._mixed_seen) > 4096:
                self._mixed_seen.clear()
            if seen < MIXED_CAPTURE_AFTER:
                return self._forward(self._prepare(entries))
        # block tables as wide as they can ever get: the captured kernels keep the row stride
        host, layout = self._build_meta(entries, self.cache.books.max_pages_per_seq, pad_requests, pad_wanted)
        if cap is None:
            meta = torch.empty(host.shape, dtype=torch.int32, device=self.runtime.device)
            meta.copy_(host, non_blocking=True)
            ctx = self._context(meta, layout, entries)
            logits = self._forward(ctx)                      # this step's result, uncaptured
            torch.cuda.synchronize()
            before = K.launches
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                static_logits = self._forward(ctx)
            while len(self._mixed_graphs) >= MIXED_GRAPHS_MAX:
                self._mixed_graphs.pop(next(iter(self._mixed_graphs)))
            self._mixed_graphs[key] = _CapturedStep(graph, meta, static_logits, K.launches - before, None)
            return logits[:wanted]
        self._mixed_graphs[key] = self._mixed_graphs.pop(key)      # most recently used last
        cap.meta.copy_(host, non_blocking=True)
        cap.graph.replay()
        K.launches += cap.launches
        self.graph_replays += 1
        return cap.logits[:wanted].clone()     # the static buffer is overwritten by the next replay

    def check_waits(self) -> None:
        """Every wait inside the tensor-core kernels is bounded; one that ran out left a code
        behind and its step's result is not to be trusted.  Asked now and then, not every
        step: it reads from the device."""
        from ..csrc import kernels as K
        bad = K.wait_errors()
        if bad:
            raise StepError(f"a bounded wait inside a tensor-core kernel ran out of time: {bad}")

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        """Embedding, every schedule entry, then final norm and head on the wanted rows."""
        hs = self.model.embed(ctx.token_ids)
        for i, e in enumerate(self.model.plan.schedule):
            k_plane, v_plane, group = self.cache.plane(i)
            ectx = EntryContext(index=i, writes_cache=e.cache_from is None, k_plane=k_plane, v_plane=v_plane,
                                block_table=ctx.tables[group] if group is not None else None,
                                page_tokens=self.page_tokens, state=self.cache.state.get(i))
            self.model.blocks[e.layer].forward(hs, ctx, ectx)
        if ctx.want_rows.numel() == 0:
            return torch.empty((0, self.model.vocab), dtype=torch.float32, device=self.runtime.device)
        return self.model.logits(hs, ctx.want_rows)

    def step_chained(self, slots: Sequence[int], device_tokens: torch.Tensor) -> Optional[torch.Tensor]:
        """One decode step for the requests in ``slots`` whose next tokens are still on the
        device (``device_tokens``, int32 [len(slots)], what a sampler left there for the step
        before): the host never sees them before the launch.  Returns the logits of every row,
        or None when this shape has no captured graph yet (the caller then takes the ordinary
        ``step`` once).  Raises :class:`OutOfPages` like ``step``."""
        if not self.cuda_graphs:
            return None
        # chained steps are steps like any other: the kernels' wait flags are looked at as often
        self._calls = getattr(self, "_calls", 0) + 1
        if self._calls % WAIT_CHECK_EVERY == 0:
            self.check_waits()
        entries = [StepEntry(s, [0], [0]) for s in slots]
        return self._step_captured(entries, device_tokens=device_tokens)

    def _step_captured(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None
                       ) -> Optional[torch.Tensor]:
        """Pure decode: logits of every row are computed by a captured graph; the wanted
        ones are returned.  The first step of a (batch, bucket) runs uncaptured and is
        then captured for the steps after it."""
        from ..csrc import kernels as K
        B = len(entries)
        for e in entries:
            if any(w != 0 for w in e.want):
                raise StepError(f"want index {list(e.want)} is outside the 1 tokens of the entry")
        width = self.cache.books.max_pages_per_seq
        host, layout = self._build_meta_decode(entries, width)
        longest = max(layout[5]) + 1
        bucket = min(-(-longest // GRAPH_CONTEXT_BUCKET) * GRAPH_CONTEXT_BUCKET, self.max_tokens_per_seq)
        key = (B, bucket)
        cap = self._graphs.get(key)
        if cap is None and device_tokens is not None:
            # no graph for this shape yet: hand the reserved pages' step back to the ordinary path
            # (the pages stay reserved; the ordinary step finds them there)
            return None
        if cap is None:
            all_rows = [StepEntry(e.slot, e.tokens, [0]) for e in entries]
            meta = torch.empty(host.shape, dtype=torch.int32, device=self.runtime.device)
            meta.copy_(host, non_blocking=True)
            ctx = self._context(meta, layout, all_rows, max_context=bucket)
            # the captured kernels keep raw pointers: their scratch must belong to this graph
            # alone and never be reallocated while the graph lives
            ctx.decode_scratch = K.DecodeScratch()
            logits = self._forward(ctx)                      # this step's result, uncaptured (sizes the scratch)
            torch.cuda.synchronize()
            before = K.launches
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                static_logits = self._forward(ctx)
            self._graphs[key] = _CapturedStep(graph, meta, static_logits, K.launches - before, ctx.decode_scratch)
        else:
            cap.meta.copy_(host, non_blocking=True)
            self._meta_copied.record()         # the pinned buffer may be rewritten once this copy is over
            if device_tokens is not None:
                cap.meta[:B].copy_(device_tokens, non_blocking=True)
            cap.graph.replay()
            K.launches += cap.launches
            self.graph_replays += 1
            logits = cap.logits.clone()        # the static buffer is overwritten by the next replay
        self.cache.books.commit_one_each([e.slot for e in entries])
        self.steps_run += 1
        rows = [i for i, e in enumerate(entries) for _ in e.want]
        if rows == list(range(B)):
            return logits
        if not rows:
            return torch.empty((0, self.model.vocab), dtype=torch.float32, device=self.runtime.device)
        return logits[torch.tensor(rows, device=logits.device)]

    def _prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        host, layout = self._build_meta(entries, None)
        dev = host.to(self.runtime.device, non_blocking=True)
        return self._context(dev, layout, entries)

    def _context(self, dev: torch.Tensor, layout, entries: Sequence[StepEntry], max_context: Optional[int] = None) -> StepContext:
        offs, R, width, G, req_start, req_prior, slots = layout

        def view(i: int) -> torch.Tensor:
            return dev[int(offs[i]): int(offs[i + 1])]

        return StepContext(
            n_rows=req_start[len(entries)], n_requests=R, token_ids=view(0), positions=view(1), row_req=view(2), req_start=view(3),
            req_prior=view(4), req_slot=view(5), want_rows=view(6),
            tables=[view(7 + g).view(R, width) for g in range(G)],
            h_req_start=req_start, h_req_prior=req_prior, h_req_slot=slots,
            max_rows_per_request=max(len(e.tokens) for e in entries),
            max_context=max_context if max_context is not None else max(p + len(e.tokens) for p, e in zip(req_prior, entries)),
            all_single=all(len(e.tokens) == 1 for e in entries))

    def _build_meta_decode(self, entries: Sequence[StepEntry], width: int):
        """``_build_meta`` for a step in which every request brings one token and wants its
        logits: the same checks, the same layout, without a Python loop per row, into a pinned
        buffer that is kept (a decode step is short: what the host spends here the device
        waits for)."""
        cache = self.cache
        R = len(entries)
        slots = [e.slot for e in entries]
        if len(set(slots)) != R:
            raise StepError("a request appears twice in one step")
        toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=R)
        if toks.min() < 0 or toks.max() >= self.model.vocab:
            bad = int(toks[(toks < 0) | (toks >= self.model.vocab)][0])
            raise StepError(f"token id {bad} is outside the vocabulary [0, {self.model.vocab})")
        prior = cache.books.reserve_one_each(slots)
        if prior is None:
            raise OutOfPages(f"step needs a new page for some of its {R} requests; free: {cache.free_pages()}")
        G = cache.num_groups
        kept = self._decode_host.get((R, width))
        if kept is None:
            sizes = [R, R, R, R + 1, R, R, R] + [R * width] * G
            offs = [0]
            for n in sizes:
                offs.append(offs[-1] + n)
            host = torch.empty((offs[-1],), dtype=torch.int32, pin_memory=True)
            h = host.numpy()
            rows = np.arange(R + 1, dtype=np.int32)
            h[offs[2]:offs[3]] = rows[:R]          # row -> request, request starts and wanted rows never change
            h[offs[3]:offs[4]] = rows
            h[offs[6]:offs[7]] = rows[:R]
            kept = self._decode_host[(R, width)] = (host, h, offs, rows.tolist(), torch.cuda.Event())
        else:
            kept[4].synchronize()              # the copy that last read this buffer is over
        host, h, offs, rows, self._meta_copied = kept
        h[offs[0]:offs[1]] = toks
        h[offs[1]:offs[2]] = prior
        h[offs[4]:offs[5]] = prior
        h[offs[5]:offs[6]] = slots
        for g in range(G):
            h[offs[7 + g]:offs[8 + g]] = cache.table_rows(g, slots, width).reshape(-1)
        return host, (offs, R, width, G, rows, prior.tolist(), slots)

    def _build_meta(self, entries: Sequence[StepEntry], width: Optional[int], pad_requests: int = 0, pad_wanted: int = 0):
        """Checks the step, reserves its pages and lays its metadata into one pinned int32
        buffer: tokens | positions | row->request | request starts | prior lengths | slots |
        wanted rows | one block-table slab per cache group.  The reservation (all or nothing
        over the whole step) and the layout are the native books' work.  ``pad_requests`` /
        ``pad_wanted``: the per-request arrays and the wanted rows are laid out for at least that
        many (requests without rows; wanted row 0)."""
        cache = self.cache
        vocab = self.model.vocab
        slots = [e.slot for e in entries]
        if len(set(slots)) != len(slots):
            raise StepError("a request appears twice in one step")
        # every check comes before the first change of the books
        counts = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=len(entries))
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if tokens.min() < 0 or tokens.max() >= vocab:
            bad = int(tokens[(tokens < 0) | (tokens >= vocab)][0])
            raise StepError(f"token id {bad} is outside the vocabulary [0, {vocab})")
        for e in entries:
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"want index {w} is outside the {len(e.tokens)} tokens of the entry")
        n_want = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=len(entries))
        wants = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=int(n_want.sum()))
        slot_arr = np.asarray(slots, dtype=np.int32)
        short = cache.books.reserve_step(slot_arr, counts)        # also refuses a slot that holds no request
        if short is not None:
            raise OutOfPages(f"step needs {short} new pages per group; free: {cache.free_pages()}")
        req_prior = [cache.length(s) for s in slots]

        R = max(len(entries), pad_requests)
        T = int(counts.sum())
        if width is None:
            width = cache.table_width(slots)
        G = cache.num_groups
        sizes = [T, T, T, R + 1, R, R, max(int(n_want.sum()), pad_wanted)] + [R * width] * G
        offs = np.concatenate([[0], np.cumsum(sizes)])
        host = torch.empty((int(offs[-1]),), dtype=torch.int32, pin_memory=True)
        cache.books.layout_step(slot_arr, counts, tokens.astype(np.int32), n_want, wants, width, host.numpy(),
                                pad_requests=pad_requests, pad_wanted=pad_wanted)
        req_start = np.concatenate([[0], np.cumsum(counts)]).tolist()
        return host, (offs, R, width, G, req_start, req_prior, slots)
