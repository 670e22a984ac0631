"""The step function: one batch of (request, its next tokens) through the model.

A step holds portions of prompts beside single decoded tokens, cut anywhere. It runs only the
tokens it is given, against what earlier steps left in the cache, and returns fp32 logits at
the wanted places. The reference's counterpart is ``forward_batch(input_ids, positions,
block_table, caches, logits, need_logits)`` (src/include/model/model.h:173-181); it uploads
one block-table row per *token* (src/source/scheduler/scheduler.cpp:526-551) and computes
logits for all rows, where this one uploads one row per *sequence* and a list of wanted rows.

All integer inputs of a step travel in one pinned buffer and one host-to-device copy.

Pure decode steps can be replayed from CUDA graphs, one per (sequence count rounded up, table
width) as the reference keeps one per batch size (src/source/model/model.cpp:74-254): the step is
laid out with fixed shapes (rows of absent sequences are padding that stores nothing), captured
once, and later steps only refresh the integer inputs and the parts' work lists before the replay.
"""
from __future__ import annotations

import gc

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import CacheLayout, CacheManager, CacheStorage, OutOfPages
from ..csrc import build, ops
from ..csrc.ops import KernelError
from . import tracing

STATUS_TEXT = {
    1: "a token id is outside the vocabulary",
    2: "a block table entry is outside the page pool",
    3: "a row names a sequence outside the batch",
    4: "a bounded wait inside a kernel ran out",
}
GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


@dataclass
class StepEntry:
    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are asked for


class StepError(RuntimeError):
    pass


class StepContext:
    """What every part sees of the running step."""

    def __init__(self, runner: "ModelRunner"):
        self._runner = runner
        self.num_tokens = 0               # rows of the step (with padding rows in a fixed-shape step)
        self.num_seqs = 0                 # sequences of this step (host-side planning loops over them)
        # Rows of the block tables and of ctx_len, q_start, slots: what kernels check a row's sequence number
        # against. In a fixed-shape step it is the shape's capacity, not this step's count: kernel arguments
        # are recorded with the graph, and a later step of the same shape may hold more sequences.
        self.seq_slots = 0
        self.num_logit_rows = 0
        self.status = runner.status
        self.plans: Dict = {}             # per-step host-side plans of parts, cleared each step
        self.seq_cap: Optional[int] = None    # fixed-shape (graph) steps: sequences the shapes are for
        # device int32 views
        self.tokens = self.positions = self.row_seq = None
        self.q_start = self.ctx_len = self.slots = self.logit_rows = None
        # host copies (real sequences only)
        self.h_positions = self.h_q_start = self.h_ctx_len = self.h_slots = None

    def buf(self, key: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """A scratch tensor that lives until the same key is asked for again."""
        return self._runner.workspace(key, shape, dtype)

    def upload_ints(self, key: str, values: np.ndarray, capacity: Optional[int] = None) -> torch.Tensor:
        """Copy a small int32 array to a device buffer that keeps its address from step to step
        (parts send their per-step work lists through this from ``prepare``)."""
        return self._runner.upload_ints(key, values, capacity)


class _PinnedRing:
    """A device int32 buffer fed from four pinned host buffers in turn, so that the host never
    rewrites a buffer whose copy may still be in flight."""

    def __init__(self, cap: int, device):
        self.cap = cap
        self.hosts = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * 4
        self.dev = torch.zeros(cap, dtype=torch.int32, device=device)
        self.turn = 0

    def next_host(self) -> np.ndarray:
        self.turn = (self.turn + 1) % 4
        ev = self.events[self.turn]
        if ev is not None:
            ev.synchronize()
        return self.hosts[self.turn].numpy()

    def send(self, n: int) -> None:
        if n:
            self.dev[:n].copy_(self.hosts[self.turn][:n], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self.events[self.turn] = ev


class ModelRunner:
    """Owns the model's cache (manager + storage), the step's staging buffers and scratch."""

    def __init__(self, model, page_size: int, num_pages: int, max_requests: int,
                 max_step_tokens: int, prefix_reuse: bool = False, max_seq_len: Optional[int] = None):
        if model.device.type != "cuda":
            raise KernelError("the engine runs on a CUDA device only; there is no CPU path")
        self.model = model
        self.device = model.device
        ops.set_device(self.device.index)        # the engine lives on one device: kernels ask for its stream
        build.prebuild(model.kernel_files(page_size))       # together now, not one by one inside the first step
        spec = model.spec
        # Caches and state belong to the places of the run order: a layer that runs twice keeps a
        # cache per run; "cache_from = j" reads the cache of the latest earlier run of layer j.
        order = spec.order
        cache_from = []
        for o, i in enumerate(order):
            src = spec.layers[i].cache_from
            if src is None:
                cache_from.append(None)
                continue
            earlier = [o2 for o2 in range(o) if order[o2] == src]
            if not earlier:
                raise StepError(f"layer {i} reads the cache of layer {src}, which does not run before it")
            cache_from.append(earlier[-1])
        self.layout = CacheLayout([model.blocks[i].mixer.cache_need() for i in order],
                                  [model.blocks[i].mixer.state_need() for i in order], cache_from)
        self.manager = CacheManager(self.layout, page_size, num_pages, max_requests, prefix_reuse)
        self.storage = CacheStorage(self.layout, self.manager, model.dtype, self.device)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_step_tokens = max(max_step_tokens, max_requests)
        self.max_seq_len = int(max_seq_len or num_pages * page_size)
        self.max_width = max(1, min(num_pages, -(-self.max_seq_len // page_size)))
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scratch: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}
        self._uploads: Dict[str, _PinnedRing] = {}
        G = max(1, len(self.manager.groups))
        T, S, W = self.max_step_tokens, max_requests, self.max_width
        self._stage = _PinnedRing(4 * (T + 4) + 3 * (S + 4) + 8 + G * S * W, self.device)
        self._table_arrays: Dict[Tuple[int, Hashable], Tuple[int, np.ndarray]] = {}
        self._graphs: Dict[Tuple[int, int], dict] = {}
        # Shapes whose recording failed: they run directly from then on, as the reference marks a batch size
        # capture_failed and keeps to its direct path (src/source/model/model.cpp:189-227, 251).
        self.capture_failed: Dict[Tuple[int, int], str] = {}
        self.fail_next_capture = False    # host-side fault injection for tests: the next recording raises
        self._generation = 0              # bumped when a captured address may have changed
        self.ctx = StepContext(self)
        self.launches_last_step = 0
        self.h2d_bytes_last_step = 0

    # ---- scratch -----------------------------------------------------------------------
    def workspace(self, key: str, shape, dtype) -> torch.Tensor:
        # the same (key, shape) is asked for at every layer of every step: the views are kept
        shape = tuple(shape)
        view = self._views.get((key, shape, dtype))
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        k = (key, dtype)
        t = self._scratch.get(k)
        if t is None or t.numel() < n:
            if torch.cuda.is_current_stream_capturing():
                raise StepError(f"scratch {key!r} would have to grow during graph capture")
            t = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._scratch[k] = t
            self._views = {vk: v for vk, v in self._views.items() if (vk[0], vk[2]) != k}
            self._drop_graphs()
        view = t[:n].view(*shape)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[(key, shape, dtype)] = view
        return view

    def upload_ints(self, key: str, values: np.ndarray, capacity: Optional[int] = None) -> torch.Tensor:
        values = np.ascontiguousarray(values, dtype=np.int32).reshape(-1)
        n = values.size
        cap = max(capacity or 0, n, 4)
        ring = self._uploads.get(key)
        if ring is None or ring.cap < cap:
            if torch.cuda.is_current_stream_capturing():
                raise StepError(f"upload buffer {key!r} would have to grow during graph capture")
            ring = _PinnedRing(max(cap, 2 * (ring.cap if ring else 0)), self.device)
            self._uploads[key] = ring
            self._drop_graphs()
        ring.next_host()[:n] = values
        ring.send(n)
        self.h2d_bytes_last_step += 4 * n
        return ring.dev[:n]

    def _drop_graphs(self) -> None:
        if self._graphs:
            self._graphs.clear()
        self._generation += 1

    # ---- the step ----------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], feed=None) -> Optional[torch.Tensor]:
        """Run one batch; returns fp32 logits [wanted rows, vocab] (a view into scratch that the
        next step overwrites) or None when nothing is wanted. ``feed = (ids, dst, src)``: token row
        ``dst[i]`` of the batch is not known on the host yet (its entry holds a placeholder) and is
        taken on the device from ``ids[src[i]]`` (int32 tensor, lists)."""
        with tracing.span("prepare"):
            ctx = self._prepare(entries)
            if feed is not None:
                self._feed_tokens(ctx, feed)
            self.storage.zero_new_slots()
            caches = self.storage.layer_views(self._tables)
            before = ops.launch_count()
            self.model.prepare(ctx, caches)
        with tracing.span("forward"):
            logits = self.model.forward(ctx, caches)
        self.launches_last_step = ops.launch_count() - before
        self._commit(entries)
        return logits

    def _feed_tokens(self, ctx, feed) -> None:
        ids, dst, src = feed
        n = len(dst)
        if list(dst) == list(range(n)):                                  # the first n rows: one gather into place
            idx = self.upload_ints("token_feed", np.asarray(src, dtype=np.int32), capacity=self.max_requests)
            torch.index_select(ids, 0, idx, out=ctx.tokens[:n])
            return
        both = self.upload_ints("token_feed_some", np.asarray(list(src) + list(dst), dtype=np.int32),
                                capacity=2 * self.max_requests)
        ctx.tokens.index_copy_(0, both[n:].to(torch.int64), torch.index_select(ids, 0, both[:n]))

    def _commit(self, entries) -> None:
        for e, new_len in zip(entries, self._new_lengths):
            self.manager.commit(e.req, new_len)

    def graphs_available(self) -> bool:
        """Decode steps may be captured only if every part of the model says that it can be."""
        return self.model.capturable()

    def step_decode_graph(self, entries: Sequence[StepEntry], feed=None) -> torch.Tensor:
        """A pure decode step (one token and one wanted row per entry) through a CUDA graph.
        The first step of a shape runs directly and is then captured; later ones are replays.
        Returns logits [len(entries), vocab]. ``feed = (ids, dst, src)`` as in ``step``."""
        S = len(entries)
        if not self.graphs_available():
            raise StepError("a part of this model cannot be captured into a graph; run the step directly")
        if any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries):
            raise StepError("a graph step takes one token and one wanted row per entry")
        cap = next((b for b in GRAPH_BUCKETS if b >= S), None)
        if cap is None or cap > self.max_requests:
            cap = self.max_requests
        if S > cap:
            raise StepError(f"{S} sequences exceed the limit of {self.max_requests}")
        ctx = self._prepare(entries, seq_cap=cap, width_cap=self.max_width)
        if feed is not None:
            self._feed_tokens(ctx, feed)
        self.storage.zero_new_slots()
        caches = self.storage.layer_views(self._tables)
        self.model.prepare(ctx, caches)
        key = (cap, self.max_width)
        g = self._graphs.get(key)
        if g is None:
            before = ops.launch_count()
            logits = self.model.forward(ctx, caches)            # runs this step, allocates all scratch
            launches = ops.launch_count() - before
            self.launches_last_step = launches
            if key not in self.capture_failed:
                with tracing.span("record"):
                    self._record(key, ctx, caches, launches)
        else:
            g["graph"].replay()
            ops.add_launches(g["launches"])
            self.launches_last_step = g["launches"]
            logits = g["logits"]
        self._commit(entries)
        return logits[:S]

    def _record(self, key, ctx, caches, launches: int) -> None:
        """Record the step that has just run into a CUDA graph for later steps of the same shape. A
        recording that fails costs nothing but itself: the step's results are there already, the shape is
        marked and runs directly from then on."""
        gen = self._generation
        graph = torch.cuda.CUDAGraph()
        torch.cuda.current_stream().synchronize()
        # No garbage collection while the stream records: collecting an engine that is no longer
        # used destroys its graphs, a call that is not allowed during capture and spoils it.
        collecting = gc.isenabled()
        gc.collect()
        gc.disable()
        before = ops.launch_count()
        try:
            with torch.cuda.graph(graph):
                if self.fail_next_capture:
                    self.fail_next_capture = False
                    raise StepError("recording failed (injected by fail_next_capture)")
                captured = self.model.forward(ctx, caches)      # recorded, not run
        except Exception as e:                                   # noqa: BLE001 - any failure means: run directly
            self.capture_failed[key] = f"{type(e).__name__}: {e}"
            captured = None
        finally:
            ops.add_launches(before - ops.launch_count())        # recording launched nothing
            if collecting:
                gc.enable()
        if captured is not None and gen == self._generation:      # no buffer moved while recording
            self._graphs[key] = {"graph": graph, "logits": captured, "launches": launches}

    def _prepare(self, entries: Sequence[StepEntry], seq_cap: Optional[int] = None,
                 width_cap: Optional[int] = None) -> StepContext:
        mgr = self.manager
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        T = 0
        for e in entries:
            if e.req in seen:
                raise StepError(f"request {e.req!r} appears twice in one step")
            seen.add(e.req)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.req!r} brings no tokens")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"request {e.req!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
            T += len(e.tokens)
        S = len(entries)
        if T > self.max_step_tokens:
            raise StepError(f"step of {T} tokens exceeds the limit of {self.max_step_tokens}")
        if S > self.max_requests:
            raise StepError(f"step of {S} sequences exceeds the limit of {self.max_requests}")
        for e in entries:
            if not mgr.has(e.req):
                mgr.admit(e.req)
        # all-or-nothing over the whole step
        need = [0] * len(mgr.groups)
        for e in entries:
            for g, m in enumerate(mgr.pages_missing(e.req, mgr.length(e.req) + len(e.tokens))):
                need[g] += m
        for g, n in enumerate(need):
            if n > mgr.free_pages(g):
                raise OutOfPages(f"step needs {n} more pages in group {g}, {mgr.free_pages(g)} are free")
        self._new_lengths = []
        for e in entries:
            new_len = mgr.length(e.req) + len(e.tokens)
            if new_len > self.max_width * self.page_size:
                raise StepError(f"request {e.req!r} would hold {new_len} tokens, above the limit "
                                f"of {self.max_width * self.page_size}")
            mgr.grow(e.req, new_len)
            self._new_lengths.append(new_len)
        self._check_pages_written(entries)

        R = sum(len(e.want) for e in entries)
        G = len(mgr.groups)
        W = max([1] + [len(mgr.table(g, e.req)) for g in range(G) for e in entries])   # pages may be reserved ahead
        fixed = seq_cap is not None
        S_cap = seq_cap or S
        W_cap = width_cap or W
        T_cap = S_cap if fixed else T          # fixed-shape steps: one row per sequence slot
        R_cap = S_cap if fixed else R
        # layout (ints): tokens | positions | row_seq | logit_rows | q_start | ctx_len | slots | tables
        offs = {}
        o = 0
        for name, n in (("tokens", T_cap), ("positions", T_cap), ("row_seq", T_cap), ("logit_rows", max(R_cap, 1)),
                        ("q_start", S_cap + 1), ("ctx_len", S_cap), ("slots", S_cap)):
            offs[name] = o
            o += (n + 3) // 4 * 4                     # 16-byte aligned regions
        table_off = o
        o += G * S_cap * W_cap
        if o > self._stage.cap:
            raise StepError(f"step inputs of {o} integers exceed the staging buffer of {self._stage.cap}")
        h = self._stage.next_host()
        dev = self._stage.dev
        b_tok, b_pos, b_seq = offs["tokens"], offs["positions"], offs["row_seq"]
        b_lr, b_qs, b_cl, b_sl = offs["logit_rows"], offs["q_start"], offs["ctx_len"], offs["slots"]
        if fixed:
            h[b_tok:b_tok + T_cap] = 0
            h[b_pos:b_pos + T_cap] = 0
            h[b_seq:b_seq + T_cap] = -1               # padding rows store nothing
            h[b_lr:b_lr + R_cap] = np.arange(R_cap, dtype=np.int32)
        h[b_qs:b_qs + S_cap + 1] = T
        h[b_cl:b_cl + S_cap] = 0
        h[b_sl:b_sl + S_cap] = 0
        # one assignment a region: the per-entry values are gathered in lists first (a step of 64 decode rows
        # would otherwise pay for several hundred small array writes)
        toks, pos, seqs, qs, cl, sl, lr = [], [], [], [], [], [], []
        row = 0
        for s, e in enumerate(entries):
            n = len(e.tokens)
            start = mgr.length(e.req)
            if n == 1:
                toks.append(e.tokens[0]); pos.append(start); seqs.append(s)
            else:
                toks.extend(e.tokens); pos.extend(range(start, start + n)); seqs.extend([s] * n)
            qs.append(row); cl.append(start + n); sl.append(mgr.slot(e.req))
            for w in e.want:
                lr.append(row + w)
            row += n
        h[b_tok:b_tok + T] = np.asarray(toks, dtype=np.int64).astype(np.int32)   # an id beyond 32 bits wraps and is flagged by the kernel
        h[b_pos:b_pos + T] = pos
        h[b_seq:b_seq + T] = seqs
        h[b_qs:b_qs + S] = qs
        h[b_cl:b_cl + S] = cl
        h[b_sl:b_sl + S] = sl
        if lr:
            h[b_lr:b_lr + len(lr)] = lr
        tabs = h[table_off:table_off + G * S_cap * W_cap].reshape(G, S_cap, W_cap)
        tabs[:] = -1
        for g in range(G):
            for s, e in enumerate(entries):
                t = self._table_array(g, e.req)
                tabs[g, s, :t.size] = t
        self._stage.send(o)
        self.h2d_bytes_last_step = 4 * o       # parts add their uploads in prepare()

        ctx = self.ctx
        ctx.plans.clear()
        ctx.seq_cap = seq_cap
        ctx.num_tokens, ctx.num_seqs, ctx.num_logit_rows = T_cap, S, R_cap
        ctx.seq_slots = S_cap
        ctx.tokens = dev[b_tok:b_tok + T_cap]
        ctx.positions = dev[b_pos:b_pos + T_cap]
        ctx.row_seq = dev[b_seq:b_seq + T_cap]
        ctx.logit_rows = dev[b_lr:b_lr + R_cap]
        ctx.q_start = dev[b_qs:b_qs + S_cap + 1]
        ctx.ctx_len = dev[b_cl:b_cl + S_cap]
        ctx.slots = dev[b_sl:b_sl + S_cap]
        ctx.h_positions = h[b_pos:b_pos + T].copy()
        ctx.h_q_start = h[b_qs:b_qs + S + 1].copy()
        ctx.h_ctx_len = h[b_cl:b_cl + S].copy()
        ctx.h_slots = h[b_sl:b_sl + S].copy()
        dtabs = dev[table_off:table_off + G * S_cap * W_cap].view(G, S_cap, W_cap)
        self._tables = [dtabs[g] for g in range(G)]
        return ctx

    def _check_pages_written(self, entries: Sequence[StepEntry]) -> None:
        """A step may store keys and values only into pages that its request holds alone. A page with more
        than one holder carries a prefix that other requests read (or will read again from the prefix index):
        a store into it is a fault of whoever decided the step, and is refused here, before anything runs.
        (The reference's decode row re-stores the last prompt token's keys into what may be a shared block,
        src/source/scheduler/scheduler.cpp:382-400.)"""
        mgr, ps = self.manager, self.page_size
        for e, new_len in zip(entries, self._new_lengths):
            first = mgr.length(e.req) // ps
            last = (new_len - 1) // ps
            for g, grp in enumerate(mgr.groups):
                t = grp.tables[e.req]
                for b in range(first, min(last + 1, len(t))):
                    page = t[b]
                    if page >= 0 and grp.pool.refcount(page) != 1:
                        raise StepError(
                            f"request {e.req!r} would store positions {max(mgr.length(e.req), b * ps)}.."
                            f"{min(new_len, (b + 1) * ps) - 1} into page {page} of group {g}, which "
                            f"{grp.pool.refcount(page)} holders share; a shared page is never written")

    def _table_array(self, group: int, req) -> np.ndarray:
        """A request's block table as an int32 array, rebuilt only when the table has changed."""
        mgr = self.manager
        version = mgr.versions[req]
        ent = self._table_arrays.get((group, req))
        if ent is None or ent[0] != version:
            ent = (version, np.asarray(mgr.table(group, req), dtype=np.int32))
            if len(self._table_arrays) > 8 * self.max_requests + 64:       # forget requests that have ended
                self._table_arrays = {k: v for k, v in self._table_arrays.items() if mgr.has(k[1])}
            self._table_arrays[(group, req)] = ent
        return ent[1]

    def raise_status(self, code: int) -> None:
        """Turn a non-zero status word (already read) into an error and clear the word."""
        if code:
            self.status.zero_()
            raise StepError(f"a kernel reported status {code}: {STATUS_TEXT.get(code, 'unknown')}")

    def check_status(self) -> None:
        """Synchronise and raise if a kernel reported a fault (it never traps)."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise StepError(f"a kernel reported status {code}: {STATUS_TEXT.get(code, 'unknown')}")

    def finish(self, req: Hashable) -> None:
        """The request has ended; what it holds is given back."""
        self.manager.release(req)
