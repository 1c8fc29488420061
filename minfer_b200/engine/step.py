"""The step function: a batch of sequences, each going on from where its slot stands by one
or more tokens: whole prompts in one step, one token each, a prompt in portions, or a new
prompt beside sequences that decode.

The reference's step is ``forward_cached(tokens, positions, n_out, n_ctx, cache)`` for one
sequence (src/models/qwen2/graph.rs:276-408): it checks ``max(pos) < n_ctx`` (:288-293),
fills ``token_ids``, ``positions`` and ``tail_ids`` as inputs (:352-361) and runs the
graph, in which the KV store of a layer precedes the attention that reads it and only the
last ``n_out`` rows go through the last feed-forward, the final norm and the head
(:126-138).  Positions are data there, not topology; they are here too, so the same code
serves every step.

``Engine.step`` runs only the tokens it is given, as one batch, from the cache that earlier
steps left, and returns float32 logits at the wanted places.  Rows are independent: no
kernel's result for one row depends on what else is in the batch.

Three shapes of a step, told apart on the host: every row starts at position 0 (whole
prompts: attention over the step's own keys), every row brings one token (decoding: replayed
as a CUDA graph), anything else (attention of the step's tokens over the cache, which holds
their keys by then).  A cache group that keeps a ring of positions can take only so many new
positions of a sequence in a step of the third shape; longer rows are run in portions.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.paged import PAGE, Cache, CacheError, GroupKey
from ..kernels import api as K
from ..model import Model
from ..parts.base import CacheView, CallBinding, StepContext, settle_pending


class StepError(RuntimeError):
    pass


def _int_array(values, what: str) -> np.ndarray:
    """A row's integers (token ids, wanted places) as an int64 array; refuses what is no integer."""
    if isinstance(values, torch.Tensor):
        values = values.detach().cpu().numpy()
    try:
        a = np.asarray(values)
    except (TypeError, ValueError) as e:
        raise StepError(f"{what} of a row must be a flat sequence of integers") from e
    if a.ndim != 1:
        a = a.reshape(-1) if a.size == 0 else a
    if a.ndim != 1:
        raise StepError(f"{what} of a row must be a flat sequence of integers")
    if a.size == 0:
        return np.zeros(0, dtype=np.int64)
    if a.dtype.kind not in "iu":
        as_int = a.astype(np.int64, copy=True) if a.dtype.kind in "fb" else None
        if as_int is None or not np.array_equal(as_int, a):
            raise StepError(f"{what} must be integers")
        return as_int
    return a.astype(np.int64, copy=False)


def padded_rows(n_rows: int) -> int:
    """The batch size a decode graph is captured for: the next power of two (a padding row
    costs little beside the weights, but not nothing: one sequence alone stays alone)."""
    size = 1
    while size < n_rows:
        size *= 2
    return size


class Engine:
    """A model plus its cache.  ``max_tokens`` is the most tokens live sequences hold at any
    time, each sequence's count rounded up to a multiple of 64; it sizes the cache.
    ``ring_step_tokens``: how many tokens a sequence that goes on may bring in one pass over
    layers with a window (their rings are that much longer than the window; longer rows are
    run in portions of at least that many tokens)."""

    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None,
                 cuda_graphs: bool = True, ring_step_tokens: int = 256):
        if model.device is None or model.device.type != "cuda":
            raise StepError("the model's weights must be on a CUDA device (there is no CPU path)")
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        plan = model.plan
        max_tokens = ((int(max_tokens) + PAGE - 1) // PAGE) * PAGE
        if max_seqs is None:
            max_seqs = max(1, min(max_tokens // PAGE, 256))
        self.max_seqs = int(max_seqs)
        self.cuda_graphs = bool(cuda_graphs)

        # which call writes which cache entry, and what that entry has to hold
        requests: Dict[int, GroupKey] = {}
        readers: Dict[int, int] = {}
        for call in plan.schedule:
            req = model.blocks[call.layer].mixer.cache_request()
            if req is None:
                continue
            key = GroupKey(req.n_kv_heads, req.head_dim, req.window, req.value_dim)
            if call.writes_cache:
                requests[call.cache] = key
            else:
                readers[call.cache] = readers.get(call.cache, 0) + 1
        for call in plan.schedule:
            req = model.blocks[call.layer].mixer.cache_request()
            if req is not None and not call.writes_cache:
                want = GroupKey(req.n_kv_heads, req.head_dim, req.window, req.value_dim)
                if requests.get(call.cache) != want:
                    raise StepError(
                        f"a call reads cache entry {call.cache} with {want}, but it is written "
                        f"with {requests.get(call.cache)}")
        self._readers = readers
        self.cache = Cache(requests, max_tokens, self.max_seqs, self.dtype, self.device,
                           step_tokens=ring_step_tokens)
        # per-sequence state of fixed size, per call
        self._call_state: List[Dict[str, torch.Tensor]] = []
        for i, call in enumerate(plan.schedule):
            tensors = {}
            for req in model.blocks[call.layer].mixer.state_request():
                tensors[req.name] = self.cache.state.add(f"call{i}.{req.name}", req.shape, req.dtype)
            self._call_state.append(tensors)
        from ..kernels import build
        # every part of the model, asked of the blocks themselves
        parts = [model.final_norm] + model.model_parts()
        for block in model.blocks:
            parts.append(block)
            parts.extend(block.parts())
        # what this model's steps will load, compiled side by side if it is not built yet: the
        # engine's own kernels (embedding, row selection, the head's product) and the parts'
        libs = ["ops", "gemm_tc" if self.dtype == torch.bfloat16 else "gemm_simt"]
        for p in parts:
            for name in p.libraries(self.dtype):
                if name not in libs:
                    libs.append(name)
        build.prebuild(libs)
        # one word for the error bits of this engine's kernels, read back without waiting: after
        # every step it is copied to pinned host memory, and the next step (or check_status)
        # raises if a copy that has arrived shows a bit
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_event = torch.cuda.Event()
        self._status_in_flight = False
        self._graphs: Dict[tuple, dict] = {}
        self._seen_shapes: set = set()
        # a part that reads device memory on the host, or changes state outside its kernels,
        # cannot be captured: every part has to declare itself capturable
        if not all(getattr(p, "capturable", False) for p in parts):
            self.cuda_graphs = False
        self._graph_pool = None
        self.steps_run = 0
        self.h2d_bytes = 0          # bytes of step inputs copied to the device so far
        self.d2h_bytes = 0          # bytes of results read back so far

    # ---- slots --------------------------------------------------------------------------
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- one step -----------------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """``tokens[b]`` are the next tokens of the sequence in ``slots[b]``; ``want[b]`` the
        places among them whose logits are asked for (default: the last).  Returns float32
        logits ``[wanted, vocab]`` in the order of the rows and of ``want``."""
        plan = self.model.plan
        self._raise_if_flagged()
        n_rows = len(slots)
        if n_rows == 0:
            raise StepError("a step needs at least one sequence")
        if len(tokens) != n_rows or (want is not None and len(want) != n_rows):
            raise StepError("slots, tokens and want must have one entry per sequence")
        if len(set(slots)) != n_rows:
            raise StepError("a slot appears twice in one step")
        counts = [len(t) for t in tokens]
        if min(counts) < 1:
            raise StepError("every sequence of a step brings at least one token")
        starts = [self.cache.length(s) for s in slots]
        # the rows' tokens as integer arrays from here on (a prompt of thousands of tokens is
        # checked and laid out without a Python loop over its tokens)
        tokens = [_int_array(t, "token ids") for t in tokens]
        for b in range(n_rows):
            if starts[b] + counts[b] > plan.max_positions:
                raise StepError(
                    f"sequence in slot {slots[b]} would reach position "
                    f"{starts[b] + counts[b] - 1}, beyond max_position_embeddings "
                    f"{plan.max_positions}")
            bad = (tokens[b] < 0) | (tokens[b] >= plan.vocab_size)
            if bad.any():
                t = int(tokens[b][int(np.argmax(bad))])
                raise StepError(f"token id {t} is outside the vocabulary of {plan.vocab_size}")
        if want is None:
            want = [[c - 1] for c in counts]
        want = [_int_array(w, "wanted places") for w in want]
        for b in range(n_rows):
            bad = (want[b] < 0) | (want[b] >= counts[b])
            if bad.any():
                w = int(want[b][int(np.argmax(bad))])
                raise StepError(f"wanted place {w} is outside the {counts[b]} tokens given")
        for b in range(n_rows):
            self.cache.reserve(slots[b], starts[b] + counts[b])
        from_start = all(s == 0 for s in starts)
        limit = self.cache.max_new_positions()
        if not from_start and limit is not None and max(counts) > limit:
            logits = self._step_in_portions(slots, tokens, want, counts, limit)
        else:
            logits = self._step_once(slots, tokens, want, counts, starts)
        self.steps_run += 1
        self._post_status()
        return logits

    def _step_once(self, slots, tokens, want, counts, starts) -> torch.Tensor:
        """One pass of the model over the rows' tokens (pages are reserved already)."""
        n_rows = len(slots)
        from_start = all(s == 0 for s in starts)
        single = all(c == 1 for c in counts)
        logits = None
        if (self.cuda_graphs and single and not from_start
                and all(list(w) == [0] for w in want)):
            logits = self._graph_step(slots, tokens, starts, None)
            if logits is not None:
                logits = logits.clone()
        if logits is None:
            ctx, want_rows = self._context(slots, tokens, counts, starts, want, from_start, single)
            logits = self._run(ctx, want_rows)
        for b in range(n_rows):
            self.cache.set_length(slots[b], starts[b] + counts[b])
        return logits

    def _step_in_portions(self, slots, tokens, want, counts, limit: int) -> torch.Tensor:
        """A step some of whose rows bring more tokens than a ring of the cache can take at
        once: pass ``i`` runs tokens ``[i * limit, (i + 1) * limit)`` of every row that has
        them.  The wanted logits come back in the order of the rows and of ``want``."""
        n_rows = len(slots)
        # where each wanted place goes in the result
        first = [0] * n_rows
        for b in range(1, n_rows):
            first[b] = first[b - 1] + len(want[b - 1])
        n_want = first[-1] + len(want[-1])
        out = torch.empty((n_want, self.model.plan.vocab_size), dtype=torch.float32,
                          device=self.device)
        for lo in range(0, max(counts), limit):
            rows = [b for b in range(n_rows) if counts[b] > lo]
            sub_tokens = [tokens[b][lo:lo + limit] for b in rows]
            sub_want, dest = [], []
            for b in rows:
                hi = min(lo + limit, counts[b])
                picked = [(i, int(w)) for i, w in enumerate(want[b]) if lo <= int(w) < hi]
                sub_want.append([w - lo for _, w in picked])
                dest.extend(first[b] + i for i, _ in picked)
            sub_slots = [slots[b] for b in rows]
            sub_counts = [len(t) for t in sub_tokens]
            sub_starts = [self.cache.length(s) for s in sub_slots]
            got = self._step_once(sub_slots, sub_tokens, sub_want, sub_counts, sub_starts)
            if dest:
                out[torch.tensor(dest, dtype=torch.long, device=self.device)] = got
        return out

    def decode_on_device(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One token per sequence, the token ids already on the device (int32 [rows], for
        instance the sampler's output): nothing is read back, so steps can follow one
        another without the host waiting.  Out-of-range ids set the status word.  With CUDA
        graphs the returned logits live in the graph's own memory and are overwritten by the
        next step of the same shape."""
        self._raise_if_flagged()
        n_rows = len(slots)
        if tokens.dtype != torch.int32 or tokens.numel() != n_rows or not tokens.is_cuda:
            raise StepError("decode_on_device takes int32 token ids on the device, one per row")
        if len(set(slots)) != n_rows:
            raise StepError("a slot appears twice in one step")
        starts = [self.cache.length(s) for s in slots]
        for b in range(n_rows):
            if starts[b] < 1:
                raise StepError("decode_on_device goes on from a prompt; this slot is empty")
            if starts[b] + 1 > self.model.plan.max_positions:
                raise StepError(f"sequence in slot {slots[b]} is at the model's last position")
            self.cache.reserve(slots[b], starts[b] + 1)
        counts = [1] * n_rows
        logits = self._graph_step(slots, [[0]] * n_rows, starts, tokens) if self.cuda_graphs \
            else None
        if logits is None:
            ctx, want_rows = self._context(slots, [[0]] * n_rows, counts, starts, [[0]] * n_rows,
                                           False, True)
            ctx.token_ids = tokens
            logits = self._run(ctx, want_rows)
        for b in range(n_rows):
            self.cache.set_length(slots[b], starts[b] + 1)
        self.steps_run += 1
        self._post_status()
        return logits

    # ---- metadata -----------------------------------------------------------------------
    def _host_fields(self, slots, tokens, counts, starts, want, widths, order=None):
        """The step's integers, field by field: tokens, positions, batch row of each token,
        cu_seqlens, lengths after the step, slots, wanted rows, then one page table per cache
        group (``widths[g]`` entries a row, -1 where a sequence has no page).  ``order``: the
        rows are given in another order than the caller's; ``order[i]`` is the row here that
        was the caller's row ``i``, and the wanted rows are listed in the caller's order."""
        n_rows = len(slots)
        if all(c == 1 for c in counts) and all(len(w) == 1 and w[0] == 0 for w in want):
            # one token a row, each row's logits wanted (decoding): no loop over the rows' tokens
            rows = list(range(n_rows))
            fields = [[int(t[0]) for t in tokens], list(starts), rows, list(range(n_rows + 1)),
                      [p + 1 for p in starts], list(slots), rows]
            for g, width in zip(self.cache.groups, widths):
                fields.append(g.table_flat(slots, width))
            return fields
        counts_a = np.asarray(counts, dtype=np.int64)
        starts_a = np.asarray(starts, dtype=np.int64)
        cu = np.zeros(n_rows + 1, dtype=np.int64)           # (rows may have been reordered by the caller)
        np.cumsum(counts_a, out=cu[1:])
        flat_tokens = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens])
        token_row = np.repeat(np.arange(n_rows, dtype=np.int64), counts_a)
        # position of a token = its row's start + its place in the row
        positions = np.arange(int(cu[-1]), dtype=np.int64) - np.repeat(cu[:-1] - starts_a, counts_a)
        rows = order if order is not None else range(n_rows)
        want_rows = [cu[b] + np.asarray(want[b], dtype=np.int64) for b in rows]
        want_rows = np.concatenate(want_rows) if want_rows else np.zeros(0, dtype=np.int64)
        fields = [flat_tokens, positions, token_row, cu, starts_a + counts_a,
                  np.asarray(slots, dtype=np.int64), want_rows]
        for g, width in zip(self.cache.groups, widths):
            fields.append(g.table_flat(slots, width))
        return fields

    def _views(self, dev: torch.Tensor, sizes) -> List[torch.Tensor]:
        views, at = [], 0
        for n in sizes:
            views.append(dev[at:at + n])
            at += n
        return views

    def _make_ctx(self, views, widths, n_tokens, slots, from_start, single, max_row_tokens,
                  max_end) -> StepContext:
        tables = {id(g): (views[7 + gi], widths[gi]) for gi, g in enumerate(self.cache.groups)}
        ctx = StepContext(
            device=self.device, act_dtype=self.dtype, n_tokens=n_tokens, n_rows=len(slots),
            token_ids=views[0], positions=views[1], token_row=views[2], cu_seqlens=views[3],
            seq_end=views[4], slots=views[5], from_start=from_start, single_token=single,
            max_row_tokens=max_row_tokens, max_end=max_end, status=self.status,
            host_slots=list(slots))
        ctx.extras["page_tables"] = tables
        return ctx

    def _context(self, slots, tokens, counts, starts, want, from_start, single):
        # A step in which some rows bring one token and others more: the one-token rows go first,
        # so that a mixer can hand them to its decode kernel as one contiguous stretch of tokens
        # and the others to its kernel for portions.  Rows are independent, so their order in
        # the step is the engine's to choose; the logits still come back in the caller's order.
        order, n_single = None, 0
        if not from_start and not single:
            n_single = sum(1 for c in counts if c == 1)
            if 0 < n_single < len(slots):
                perm = sorted(range(len(slots)), key=lambda b: counts[b] != 1)      # stable
                order = [0] * len(slots)
                for here, b in enumerate(perm):
                    order[b] = here
                slots, tokens, counts, starts, want = ([x[b] for b in perm] for x in
                                                       (slots, tokens, counts, starts, want))
            else:
                n_single = 0
        widths = [max(1, g.max_pages_of(slots)) for g in self.cache.groups]
        fields = self._host_fields(slots, tokens, counts, starts, want, widths, order)
        sizes = [len(f) for f in fields]
        host = torch.from_numpy(np.concatenate(
            [np.asarray(f, dtype=np.int32) for f in fields])).pin_memory()
        dev = host.to(self.device, non_blocking=True)
        self.h2d_bytes += host.numel() * 4
        views = self._views(dev, sizes)
        ctx = self._make_ctx(views, widths, sum(counts), slots, from_start, single, max(counts),
                             max(starts[b] + counts[b] for b in range(len(slots))))
        # every row wanted, in order (decoding): the last layer needs no row selection
        n_tokens = sum(counts)
        ctx.extras["want_is_identity"] = (len(fields[6]) == n_tokens and
                                          bool(np.array_equal(fields[6], np.arange(n_tokens))))
        ctx.extras["single_rows"] = n_single          # rows of one token, first in the batch
        return ctx, (views[6] if sizes[6] else None)

    # ---- decode steps replayed as CUDA graphs -------------------------------------------------
    def _graph_step(self, slots, tokens, starts, device_tokens: Optional[torch.Tensor]):
        """A one-token-per-sequence step through a captured graph.  The graph is keyed by the
        number of rows and by a coarse bound on the sequences' lengths (which fixes the
        page tables' width and the number of key chunks); positions, slots, tokens and page
        tables are data in a buffer the graph reads, as positions are in the reference
        (src/graph/params.rs:10-60: the reuse identity has no n_past)."""
        n_live = len(slots)
        # fill the batch up to a size that has (or gets) a graph: rows that point at the spare
        # slot, bring token 0 at position 0 and whose logits nobody reads.  Sequences that end
        # at different steps then keep one graph instead of capturing one for every size.
        n_rows = padded_rows(n_live)
        if n_rows > n_live:
            pad = n_rows - n_live
            slots = list(slots) + [self.cache.spare_slot] * pad
            tokens = list(tokens) + [[0]] * pad
            starts = list(starts) + [0] * pad
        max_end = max(starts) + 1
        # a bound on the lengths: 256, 512, 1024, then multiples of 512 (a new graph every 512
        # positions; a key chunk beyond a sequence's end costs a CTA that leaves at once:
        # 2 % of a step at batch 64 with multiples of 1024)
        cap = 256
        while cap < max_end and cap < 1024:
            cap *= 2
        if cap < max_end:
            cap = ((max_end + 511) // 512) * 512
        key = (n_rows, cap)
        entry = self._graphs.get(key)
        if entry is None and key not in self._seen_shapes:
            # the first step of a shape runs kernel by kernel (it also builds libraries and sets
            # kernel attributes, which capture does not allow); the second one is captured
            self._seen_shapes.add(key)
            return None
        widths = [(g.ring // PAGE) if g.ring else cap // PAGE for g in self.cache.groups]
        counts = [1] * n_rows
        want = [[0]] * n_rows
        fields = self._host_fields(slots, tokens, counts, starts, want, widths)
        sizes = [len(f) for f in fields]
        flat = [x for f in fields for x in f]
        if entry is None:
            entry = self._capture(key, sizes, widths, flat, slots, cap)
        ring = entry["ring"]
        slot_i = entry["next"] % len(ring)
        entry["next"] += 1
        host, event = ring[slot_i]
        event.synchronize()                         # the copy that last used this buffer is done
        host.numpy()[:] = flat
        entry["dev"].copy_(host, non_blocking=True)
        event.record()
        self.h2d_bytes += host.numel() * 4
        if device_tokens is not None:
            entry["dev"][:n_live].copy_(device_tokens)
        entry["graph"].replay()
        K.launches += entry["kernels"]
        return entry["logits"][:n_live]

    def _capture(self, key, sizes, widths, flat, slots, cap):
        n_rows = key[0]
        total = sum(sizes)
        dev = torch.zeros(total, dtype=torch.int32, device=self.device)
        dev.copy_(torch.tensor(flat, dtype=torch.int32))
        views = self._views(dev, sizes)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        ctx = self._make_ctx(views, widths, n_rows, slots, False, True, 1, cap)
        ctx.extras["want_is_identity"] = True       # one token a row, each row's logits wanted
        before = K.launches
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self._run(ctx, views[6])
        captured = K.launches - before
        K.launches = before                         # nothing ran yet; replays are counted
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        ring = []
        for _ in range(4):
            host = torch.empty(total, dtype=torch.int32).pin_memory()
            ring.append((host, torch.cuda.Event()))
        entry = {"graph": graph, "dev": dev, "logits": logits, "ring": ring, "next": 0,
                 "kernels": captured}
        self._graphs[key] = entry
        return entry

    def _bindings(self, ctx: StepContext) -> List[CallBinding]:
        plan = self.model.plan
        tables = ctx.extras["page_tables"]
        out = []
        for i, call in enumerate(plan.schedule):
            view = None
            g = self.cache.group_of.get(call.cache)
            if g is not None and self.model.blocks[call.layer].mixer.cache_request() is not None:
                k, v = g.entry_tensors(call.cache)
                table, width = tables[id(g)]
                view = CacheView(k=k, v=v, page_table=table, table_stride=width, ring=g.ring)
            out.append(CallBinding(
                cache=view, writes_cache=call.writes_cache, entry=call.cache,
                has_readers=call.writes_cache and self._readers.get(call.cache, 0) > 0,
                state=self._call_state[i]))
        return out

    # ---- the model ------------------------------------------------------------------------
    def _run(self, ctx: StepContext, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        from ..kernels import gemm
        model, plan = self.model, self.model.plan
        gemm.use_status_word(self.status)           # this engine's products report into its word
        h = torch.empty((ctx.n_tokens, plan.hidden_size), dtype=torch.float32, device=self.device)
        K.embed(model.embedding, ctx.token_ids, h, self.status, plan.embedding_scale)
        if model.after_embedding is not None:
            model.after_embedding.forward_inplace(h, ctx)
        bindings = self._bindings(ctx)
        last = len(plan.schedule) - 1
        n_want = 0 if want_rows is None else want_rows.numel()
        all_rows = n_want == ctx.n_tokens and bool(ctx.extras.get("want_is_identity"))
        for i, call in enumerate(plan.schedule):
            block = model.blocks[call.layer]
            takes_pending = getattr(block, "accepts_pending", False)
            if not takes_pending:
                settle_pending(ctx, h)
                ctx.extras.pop("prepared", None)     # h is complete: the block norms it itself
            # rows of h are dropped between the last mixer and its feed-forward unless all are wanted
            ctx.extras["rows_stay"] = i != last or all_rows
            block.mix(h, ctx, bindings[i])
            if not takes_pending or (i == last and not all_rows):
                settle_pending(ctx, h)
            if i == last:
                if n_want == 0:
                    return torch.empty((0, plan.vocab_size), dtype=torch.float32,
                                       device=self.device)
                if not all_rows:
                    ctx.extras.pop("prepared", None)
                    picked = torch.empty((n_want, plan.hidden_size), dtype=torch.float32,
                                         device=self.device)
                    K.gather_rows(h, want_rows, picked)
                    h = picked
            # the norm that reads h after this block's feed-forward: the next block's first, if
            # it can take its input prepared, or the model's last (the head applies the scale)
            if i < last:
                ctx.extras["next_norm"] = model.blocks[plan.schedule[i + 1].layer].entry_norm()
            else:
                ctx.extras["next_norm"] = (model.final_norm if model.head.takes_row_scale()
                                           and model.final_norm.foldable() is not None else None)
            block.feed(h, ctx)
        prepared = ctx.extras.pop("prepared", None)
        if prepared is not None and prepared.norm is model.final_norm:
            logits = model.head.forward(prepared.x, torch.float32, row_scale=prepared.scale)
        else:
            pending = ctx.extras.pop("pending", None)
            if pending is not None:
                x = model.final_norm.forward_settling(h, pending, self.dtype)
            else:
                x = model.final_norm.forward(h, self.dtype)
            logits = model.head.forward(x, torch.float32)
        if model.on_logits is not None:
            model.on_logits.forward_inplace(logits, ctx)
        return logits

    # ---- marks on the stream, for device times -------------------------------------------------
    def time_mark(self) -> torch.cuda.Event:
        """An event recorded now on the current stream."""
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def seconds_between(self, first: torch.cuda.Event, second: torch.cuda.Event) -> float:
        """Device time between two marks (waits for the second to have happened)."""
        second.synchronize()
        return first.elapsed_time(second) * 1e-3

    # ---- the status word ----------------------------------------------------------------------
    def _post_status(self) -> None:
        """Sends the status word on its way to the host behind the step just launched."""
        if self._status_in_flight and not self._status_event.query():
            return                                   # the last copy is still under way
        self._status_host.copy_(self.status, non_blocking=True)
        self._status_event.record()
        self._status_in_flight = True

    def _raise_if_flagged(self) -> None:
        """Raises if a copy of the status word that has arrived shows an error bit (no wait)."""
        if self._status_in_flight and self._status_event.query():
            self._status_in_flight = False
            if int(self._status_host[0]) != 0:
                self.check_status()

    def check_status(self) -> None:
        """Raises if a kernel of this engine flagged a bad token or position or gave up a
        bounded wait (reads the device: a sync).  ``step`` and ``decode_on_device`` look at
        the word themselves without waiting, so an error surfaces at the latest one call after
        the step it belongs to has finished; callers that must know now call this."""
        bits = int(self.status.item())
        self._status_in_flight = False
        if bits:
            self.status.zero_()
            raise StepError("a kernel reported: " + ", ".join(status_bits(bits)))


def status_bits(bits: int) -> List[str]:
    """What the bits of a status word say (the meanings of ``MF_STATUS_*`` in csrc/common.cuh)."""
    what = []
    if bits & 1:
        what.append("a token id outside the vocabulary")
    if bits & 2:
        what.append("a position outside its sequence's pages")
    if bits & 4:
        what.append("a bounded wait on a barrier ran out")
    return what or [f"status {bits}"]
