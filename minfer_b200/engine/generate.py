"""The generation loop above the step function.

The reference's loop (src/main.rs:528-598): sample from the last logits; a stop token
(``eos`` or ``<|im_end|>``, src/main.rs:626-628) ends the sequence and is neither emitted
nor fed; otherwise the token is appended and fed as a one-token step; the loop ends after
``n_predict`` tokens.  It serves one sequence.  Here a batch of unequal prompts starts
together (all prompts in one step), every following step carries one token of each
sequence that is still running, sequences that end earlier leave the batch, slots go back
when the batch ends, and as many batches run one after another as there are requests.

The loop is written against two small interfaces so that its decisions can be tested
without a GPU: an *engine* (``acquire``, ``release``, ``step(slots, tokens) -> logits``,
``max_positions``) and a *sampler* (``begin(slots, prompts)``,
``sample(logits, slots, streams) -> list[int]``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence

from ..sampling.params import SamplingParams

PAGE = 64


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str              # "stop": a stop token was drawn; "length": a limit was hit
    prompt_tokens: int


@dataclass
class GenerationStats:
    """Counts and times of ``generate`` calls.  ``*_seconds`` is the host's clock around each
    step (what a caller waits for); ``*_device_seconds`` is the time between events recorded
    on the device's stream (before the prompts' step, after the first tokens are sampled, after
    the batch's last step), where the engine offers such marks.  The reference prints the same
    two calibres from host timers (src/main.rs:552-609)."""

    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_seconds: float = 0.0
    batches: int = 0
    steps: int = 0
    prefill_device_seconds: float = 0.0
    decode_device_seconds: float = 0.0


class _DeviceClock:
    """Three marks on the engine's stream per batch, if the engine has ``time_mark`` and
    ``seconds_between`` (the mock engines of the loop's tests have not)."""

    def __init__(self, engine: Any):
        self.mark = getattr(engine, "time_mark", None)
        self.between = getattr(engine, "seconds_between", None)
        self.marks: List[Any] = []

    def tick(self) -> None:
        if self.mark is not None and self.between is not None:
            self.marks.append(self.mark())

    def add_to(self, stats: GenerationStats) -> None:
        if len(self.marks) == 3:
            stats.prefill_device_seconds += self.between(self.marks[0], self.marks[1])
            stats.decode_device_seconds += self.between(self.marks[1], self.marks[2])


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, max_batch: int,
                 max_tokens: int) -> List[List[int]]:
    """Splits requests, in order, into batches that fit: at most ``max_batch`` sequences and
    at most ``max_tokens`` cached tokens when every sequence has grown to its limit (each
    sequence's count rounded up to a multiple of 64)."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lengths):
        need = ((n + max_new_tokens + PAGE - 1) // PAGE) * PAGE
        if need > max_tokens:
            raise ValueError(
                f"request {i} needs room for {need} tokens but the cache holds {max_tokens}")
        if cur and (len(cur) >= max_batch or used + need > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def run_batch(engine: Any, sampler: Any, prompts: Sequence[Sequence[int]], streams: Sequence[int],
              max_new_tokens: int, stop_token_ids: Sequence[int], max_positions: int,
              stats: Optional[GenerationStats] = None, sync: Any = None) -> List[GenerationResult]:
    """One batch from its prompts to its last token."""
    stats = stats if stats is not None else GenerationStats()
    stop = set(int(t) for t in stop_token_ids)
    n = len(prompts)
    results = [GenerationResult([], "length", len(p)) for p in prompts]
    if max_new_tokens <= 0:
        return results
    slots = [engine.acquire() for _ in range(n)]
    try:
        sampler.begin(slots, prompts)
        live = list(range(n))
        clock = _DeviceClock(engine)
        clock.tick()
        t0 = time.perf_counter()
        logits = engine.step([slots[i] for i in live], [list(prompts[i]) for i in live])
        first = True
        while live:
            tokens = sampler.sample(logits, [slots[i] for i in live], [streams[i] for i in live])
            now = time.perf_counter()
            if first:
                clock.tick()
                stats.prefill_tokens += sum(len(prompts[i]) for i in live)
                stats.prefill_seconds += now - t0
                first = False
            else:
                stats.decode_tokens += len(live)
                stats.decode_seconds += now - t0
            t0 = now
            stats.steps += 1
            still, feed = [], []
            for i, tok in zip(live, tokens):
                tok = int(tok)
                r = results[i]
                if tok in stop:
                    r.finish_reason = "stop"        # neither emitted nor fed
                    continue
                r.tokens.append(tok)
                if len(r.tokens) >= max_new_tokens:
                    r.finish_reason = "length"
                    continue
                if r.prompt_tokens + len(r.tokens) > max_positions:
                    r.finish_reason = "length"      # no position left to feed this token at
                    continue
                still.append(i)
                feed.append([tok])
            live = still
            if live:
                logits = engine.step([slots[i] for i in live], feed)
        clock.tick()
        clock.add_to(stats)
    finally:
        for s in slots:
            engine.release(s)
    stats.batches += 1
    return results


def run_batch_pipelined(engine: Any, sampler: Any, prompts: Sequence[Sequence[int]],
                        streams: Sequence[int], max_new_tokens: int,
                        stop_token_ids: Sequence[int], max_positions: int,
                        stats: Optional[GenerationStats] = None) -> List[GenerationResult]:
    """The same decisions as ``run_batch`` with the host one step behind the device: the next
    decode step is launched from the sampled tokens while they are still on the device, and
    only then are the previous step's tokens read.  Ends by length are known in advance from
    the counts; an end by a stop token is seen one step late, and the step that sequence ran
    in the meantime is dropped (a row's result never depends on the other rows, so the tokens
    are those of ``run_batch``).

    Needs ``engine.decode_on_device(slots, tokens)`` and ``sampler.sample_on_device`` /
    ``sampler.fetch``."""
    import torch
    stats = stats if stats is not None else GenerationStats()
    stop = set(int(t) for t in stop_token_ids)
    n = len(prompts)
    results = [GenerationResult([], "length", len(p)) for p in prompts]
    if max_new_tokens <= 0:
        return results
    slots = [engine.acquire() for _ in range(n)]
    try:
        sampler.begin(slots, prompts)
        clock = _DeviceClock(engine)
        clock.tick()
        t0 = time.perf_counter()
        logits = engine.step(list(slots), [list(p) for p in prompts])
        cur = list(range(n))                       # sequences in the order of `tokens`
        tokens = sampler.sample_on_device(logits, slots, list(streams))
        clock.tick()
        fetch = sampler.fetch(tokens)
        drawn = [1] * n                            # tokens drawn so far (the last may be unread)
        stopped = [False] * n
        first = True
        while cur:
            # who goes on is known from the counts alone: a token is fed if it is not the last
            # one allowed and there is a position left for it
            nxt = [i for i in cur if not stopped[i] and drawn[i] < max_new_tokens
                   and len(prompts[i]) + drawn[i] <= max_positions]
            next_tokens = next_fetch = None
            if nxt:
                feed = tokens
                if nxt != cur:
                    where = {i: k for k, i in enumerate(cur)}
                    index = torch.tensor([where[i] for i in nxt], dtype=torch.long,
                                         device=tokens.device)
                    feed = tokens.index_select(0, index)
                logits = engine.decode_on_device([slots[i] for i in nxt], feed)
                next_tokens = sampler.sample_on_device(logits, [slots[i] for i in nxt],
                                                       [streams[i] for i in nxt])
                next_fetch = sampler.fetch(next_tokens)
            host = fetch.get()                     # the step before the one just launched
            now = time.perf_counter()
            if first:
                stats.prefill_tokens += sum(len(p) for p in prompts)
                stats.prefill_seconds += now - t0
                first = False
            else:
                stats.decode_tokens += len(cur)
                stats.decode_seconds += now - t0
            t0 = now
            stats.steps += 1
            for i, tok in zip(cur, host):
                if stopped[i]:
                    continue                       # the extra step of a sequence that had stopped
                tok = int(tok)
                if tok in stop:
                    results[i].finish_reason = "stop"
                    stopped[i] = True
                    continue
                results[i].tokens.append(tok)
            for i in nxt:
                drawn[i] += 1
            cur, tokens, fetch = nxt, next_tokens, next_fetch
        clock.tick()
        clock.add_to(stats)
    finally:
        for s in slots:
            engine.release(s)
    stats.batches += 1
    return results


class Generator:
    """A model with its cache, ready to generate.

        gen = Generator(Model.from_folder(folder, "bfloat16"), max_tokens=8 * 4096)
        results = gen.generate([[1, 2, 3], [4, 5]], max_new_tokens=32,
                               sampling=SamplingParams.greedy())
    """

    def __init__(self, model, max_tokens: int = 16384, max_batch: int = 64,
                 cuda_graphs: bool = True, pipelined: bool = True):
        from .step import Engine
        self.model = model
        self.max_batch = int(max_batch)
        self.engine = Engine(model, max_tokens=max_tokens, max_seqs=max(self.max_batch, 1),
                             cuda_graphs=cuda_graphs)
        self.max_tokens = self.engine.cache.max_tokens
        self.stats = GenerationStats()
        self.pipelined = bool(pipelined)    # host one step behind the device (same tokens)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 512,
                 sampling: Optional[SamplingParams] = None,
                 stop_token_ids: Optional[Sequence[int]] = None) -> List[GenerationResult]:
        from ..sampling.device import DeviceSampler
        sampling = sampling if sampling is not None else SamplingParams()
        plan = self.model.plan
        if stop_token_ids is None:
            stop_token_ids = plan.stop_token_ids
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError(f"prompt {i} is empty")
            if len(p) > plan.max_positions:
                raise ValueError(f"prompt {i} has {len(p)} tokens, more than the model's "
                                 f"{plan.max_positions} positions")
        room = [min(max_new_tokens, plan.max_positions - len(p)) for p in prompts]
        batches = plan_batches([len(p) for p in prompts], max(room, default=0), self.max_batch,
                               self.max_tokens)
        sampler = DeviceSampler(self.engine, sampling)
        results: List[Optional[GenerationResult]] = [None] * len(prompts)
        loop = run_batch_pipelined if self.pipelined else run_batch
        for batch in batches:
            out = loop(self.engine, sampler, [prompts[i] for i in batch], batch,
                       max_new_tokens, stop_token_ids, plan.max_positions, self.stats)
            for i, r in zip(batch, out):
                results[i] = r
        self.engine.check_status()
        return results  # type: ignore[return-value]


def generate(model_or_folder: Any, prompts: Sequence[Sequence[int]], max_new_tokens: int = 512,
             sampling: Optional[SamplingParams] = None,
             stop_token_ids: Optional[Sequence[int]] = None, dtype: str = "bfloat16",
             max_tokens: Optional[int] = None) -> List[GenerationResult]:
    """The Python entry point: token ids in, token ids out.

    ``model_or_folder`` is a ``Model`` or a folder with config.json and model.safetensors.
    """
    from ..model import Model
    model = model_or_folder if isinstance(model_or_folder, Model) \
        else Model.from_folder(model_or_folder, dtype)
    if max_tokens is None:
        per = max(len(p) for p in prompts) + max_new_tokens
        max_tokens = min(len(prompts), 64) * (((per + PAGE - 1) // PAGE) * PAGE)
    gen = Generator(model, max_tokens=max_tokens, max_batch=min(max(len(prompts), 1), 64))
    return gen.generate(prompts, max_new_tokens, sampling, stop_token_ids)
