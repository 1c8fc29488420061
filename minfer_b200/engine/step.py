"""The step function: a batch of sequences that start together, with unequal lengths; their
whole prompts in one step, then one token each.

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
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.paged import PAGE, Cache, CacheError, GroupKey
from ..kernels import api as K
from ..model import Model
from ..parts.base import CacheView, CallBinding, StepContext


class StepError(RuntimeError):
    pass


@dataclass
class StepResult:
    logits: torch.Tensor            # float32 [n_wanted, vocab] on the device


class Engine:
    """A model plus its cache.  ``max_tokens`` is the most tokens live sequences hold at any
    time, each sequence's count rounded up to a multiple of 64; it sizes the cache."""

    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None,
                 cuda_graphs: bool = True):
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
            key = GroupKey(req.n_kv_heads, req.head_dim, req.window)
            if call.writes_cache:
                requests[call.cache] = key
            else:
                readers[call.cache] = readers.get(call.cache, 0) + 1
        for call in plan.schedule:
            req = model.blocks[call.layer].mixer.cache_request()
            if req is not None and not call.writes_cache:
                want = GroupKey(req.n_kv_heads, req.head_dim, req.window)
                if requests.get(call.cache) != want:
                    raise StepError(
                        f"a call reads cache entry {call.cache} with {want}, but it is written "
                        f"with {requests.get(call.cache)}")
        self._readers = readers
        self.cache = Cache(requests, max_tokens, self.max_seqs, self.dtype, self.device)
        # per-sequence state of fixed size, per call
        self._call_state: List[Dict[str, torch.Tensor]] = []
        for i, call in enumerate(plan.schedule):
            tensors = {}
            for req in model.blocks[call.layer].mixer.state_request():
                tensors[req.name] = self.cache.state.add(f"call{i}.{req.name}", req.shape, req.dtype)
            self._call_state.append(tensors)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
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
        from_start = all(s == 0 for s in starts)
        single = all(c == 1 for c in counts)
        if not from_start and not single:
            raise StepError(
                "the sequences of a step either all start at their first token or all go on "
                "by one token")
        for b in range(n_rows):
            if starts[b] + counts[b] > plan.max_positions:
                raise StepError(
                    f"sequence in slot {slots[b]} would reach position "
                    f"{starts[b] + counts[b] - 1}, beyond max_position_embeddings "
                    f"{plan.max_positions}")
            for t in tokens[b]:
                if not 0 <= int(t) < plan.vocab_size:
                    raise StepError(f"token id {t} is outside the vocabulary of {plan.vocab_size}")
        if want is None:
            want = [[c - 1] for c in counts]
        for b in range(n_rows):
            for w in want[b]:
                if not 0 <= int(w) < counts[b]:
                    raise StepError(f"wanted place {w} is outside the {counts[b]} tokens given")
        for b in range(n_rows):
            self.cache.reserve(slots[b], starts[b] + counts[b])

        ctx, want_rows = self._context(slots, tokens, counts, starts, want, from_start, single)
        logits = self._run(ctx, want_rows)
        for b in range(n_rows):
            self.cache.set_length(slots[b], starts[b] + counts[b])
        self.steps_run += 1
        return logits

    def decode_on_device(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One token per sequence, the token ids already on the device (int32 [rows], for
        instance the sampler's output): nothing is read back, so steps can follow one
        another without the host waiting.  Out-of-range ids set the status word."""
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
        ctx, want_rows = self._context(slots, [[0]] * n_rows, counts, starts, [[0]] * n_rows,
                                       False, True)
        ctx.token_ids = tokens
        logits = self._run(ctx, want_rows)
        for b in range(n_rows):
            self.cache.set_length(slots[b], starts[b] + 1)
        self.steps_run += 1
        return logits

    def assume_filled(self, slot: int, length: int) -> None:
        """Benchmarks only: gives the sequence ``length`` positions of cache without running
        the model; whatever the pages hold stands in for keys and values."""
        self.cache.reserve(slot, length)
        self.cache.set_length(slot, length)

    # ---- metadata -----------------------------------------------------------------------
    def _context(self, slots, tokens, counts, starts, want, from_start, single):
        n_rows = len(slots)
        n_tokens = sum(counts)
        flat_tokens, positions, token_row, cu, want_rows = [], [], [], [0], []
        for b in range(n_rows):
            base = cu[-1]
            flat_tokens.extend(int(t) for t in tokens[b])
            positions.extend(range(starts[b], starts[b] + counts[b]))
            token_row.extend([b] * counts[b])
            cu.append(base + counts[b])
            want_rows.extend(base + int(w) for w in want[b])
        seq_end = [starts[b] + counts[b] for b in range(n_rows)]
        fields = [flat_tokens, positions, token_row, cu, seq_end, list(slots), want_rows]
        widths = []
        for g in self.cache.groups:
            width = max(1, g.max_pages_of(slots))
            widths.append(width)
            rows = g.table_rows(slots, width)
            fields.append([p for row in rows for p in row])
        sizes = [len(f) for f in fields]
        host = torch.tensor([x for f in fields for x in f], dtype=torch.int32).pin_memory()
        dev = host.to(self.device, non_blocking=True)
        self.h2d_bytes += host.numel() * 4
        views, at = [], 0
        for n in sizes:
            views.append(dev[at:at + n])
            at += n
        tables = {}
        for gi, g in enumerate(self.cache.groups):
            tables[id(g)] = (views[7 + gi], widths[gi])
        ctx = StepContext(
            device=self.device, act_dtype=self.dtype, n_tokens=n_tokens, n_rows=n_rows,
            token_ids=views[0], positions=views[1], token_row=views[2], cu_seqlens=views[3],
            seq_end=views[4], slots=views[5], from_start=from_start, single_token=single,
            max_row_tokens=max(counts), max_end=max(seq_end), status=self.status,
            host_slots=list(slots))
        ctx.extras["page_tables"] = tables
        return ctx, (views[6] if want_rows else None)

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
        model, plan = self.model, self.model.plan
        h = torch.empty((ctx.n_tokens, plan.hidden_size), dtype=torch.float32, device=self.device)
        K.embed(model.embedding, ctx.token_ids, h, self.status)
        bindings = self._bindings(ctx)
        last = len(plan.schedule) - 1
        n_want = 0 if want_rows is None else want_rows.numel()
        for i, call in enumerate(plan.schedule):
            block = model.blocks[call.layer]
            block.mix(h, ctx, bindings[i])
            if i == last:
                if n_want == 0:
                    return torch.empty((0, plan.vocab_size), dtype=torch.float32,
                                       device=self.device)
                if not (n_want == ctx.n_tokens and ctx.extras.get("want_is_identity")):
                    picked = torch.empty((n_want, plan.hidden_size), dtype=torch.float32,
                                         device=self.device)
                    K.gather_rows(h, want_rows, picked)
                    h = picked
            block.feed(h, ctx)
        x = model.final_norm.forward(h, self.dtype)
        return model.head.forward(x, torch.float32)

    def check_status(self) -> None:
        """Raises if a kernel flagged a bad token or position (reads the device: a sync)."""
        bits = int(self.status.item())
        if bits:
            self.status.zero_()
            what = []
            if bits & 1:
                what.append("a token id outside the vocabulary")
            if bits & 2:
                what.append("a position outside its sequence's pages")
            if bits & 4:
                what.append("a bounded wait on a barrier ran out")
            raise StepError("a kernel reported: " + ", ".join(what or [f"status {bits}"]))
