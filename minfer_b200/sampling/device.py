"""The sampler that generation uses: one kernel launch per step for the whole batch.

Per sequence it keeps, in the cache's fixed-size state area, the window of the last 64
tokens the penalties look at and the number of draws made, so that a sequence's draws do
not depend on the rest of the batch: draw n of stream s is Philox(seed; n, s).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..kernels import api as K
from .params import RECENT_WINDOW, SamplingParams

STATE_NAME = "sampler"


class DeviceSampler:
    RING = 8        # pinned token buffers in rotation

    def __init__(self, engine, params: SamplingParams):
        params.validate()
        self.engine = engine
        self.params = params
        self.device = engine.device
        pool = engine.cache.state
        self.width = 2 + RECENT_WINDOW
        if STATE_NAME not in pool.tensors:
            pool.add(STATE_NAME, (self.width,), torch.int32)
        self.state = pool.tensors[STATE_NAME]
        if K.sampler_state_ints() != self.width:
            raise K.KernelError("the sampler kernel and its state layout disagree")
        self._meta_key = None
        self._meta_dev = None
        self._meta_host = None
        self._copy_stream = torch.cuda.Stream(device=self.device)
        self._pinned: list = []
        self._next_pinned = 0

    def begin(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> None:
        """Seeds each sequence's window with the tail of its prompt (src/main.rs:537-540) and
        sets its draw counter to zero."""
        rows = torch.zeros((len(slots), self.width), dtype=torch.int32)
        for b, prompt in enumerate(prompts):
            tail = list(prompt[-RECENT_WINDOW:])
            rows[b, 0] = len(tail)
            rows[b, 2:2 + len(tail)] = torch.tensor(tail, dtype=torch.int32)
        index = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        self.state.index_copy_(0, index, rows.to(self.device))

    def _meta(self, slots: Sequence[int], streams: Sequence[int]) -> torch.Tensor:
        """Slots and RNG streams of the rows on the device; kept while the rows stay the same."""
        key = (tuple(slots), tuple(streams))
        if self._meta_key != key:
            host = torch.tensor(list(slots) + list(streams), dtype=torch.int32).pin_memory()
            self._meta_dev = host.to(self.device, non_blocking=True)
            self._meta_host = host                      # keep the pinned buffer alive
            self._meta_key = key
            self.engine.h2d_bytes += host.numel() * 4
        return self._meta_dev

    def sample_on_device(self, logits: torch.Tensor, slots: Sequence[int],
                         streams: Sequence[int]) -> torch.Tensor:
        """One token per row of ``logits`` (changed in place); the tokens stay on the device
        (int32 [rows]), so that the next step can be launched without waiting for them."""
        p = self.params
        n = logits.shape[0]
        meta = self._meta(slots, streams)
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        K.sample(logits, out, temperature=p.temperature, top_k=p.top_k, top_p=p.top_p,
                 repeat_penalty=p.repeat_penalty, frequency_penalty=p.frequency_penalty,
                 presence_penalty=p.presence_penalty, seed=p.seed, slots=meta[:n],
                 state=self.state, stream_ids=meta[n:], update_state=True)
        return out

    def fetch(self, tokens: torch.Tensor) -> "TokenFetch":
        """Starts copying ``tokens`` to the host on a side stream; ``.get()`` waits for that
        copy only, not for whatever was launched after it."""
        self.engine.d2h_bytes += tokens.numel() * 4
        # pinned buffers are made once and reused in turn (allocating pinned memory is slow and
        # synchronises with the device); a buffer comes around again after RING fetches, long
        # after its tokens were read
        n = tokens.numel()
        if not self._pinned or self._pinned[0].numel() < n:
            self._pinned = [torch.empty(max(n, 64), dtype=torch.int32).pin_memory()
                            for _ in range(self.RING)]
        host = self._pinned[self._next_pinned % self.RING][:n]
        self._next_pinned += 1
        return TokenFetch(tokens, self._copy_stream, host)

    def sample(self, logits: torch.Tensor, slots: Sequence[int],
               streams: Sequence[int]) -> List[int]:
        """One token per row of ``logits`` (changed in place); returns them on the host."""
        return self.fetch(self.sample_on_device(logits, slots, streams)).get()


class TokenFetch:
    """A device-to-host copy of a few token ids that does not wait for later work."""

    def __init__(self, tokens: torch.Tensor, copy_stream: torch.cuda.Stream, host: torch.Tensor):
        self.host = host
        self.done = torch.cuda.Event()
        ready = torch.cuda.Event()
        ready.record()                                  # after the sampling kernel
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ready)
            self.host.copy_(tokens, non_blocking=True)
            self.done.record()
        self._keep = tokens                             # not freed before the copy has run

    def get(self) -> List[int]:
        self.done.synchronize()
        return self.host.tolist()
