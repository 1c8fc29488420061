"""The generation loop's decisions with a mock engine and a scripted sampler (no GPU): the
idea of the reference's MockEngine (src/conversation.rs:583-613)."""
import pytest

from minfer_b200.engine.generate import GenerationStats, plan_batches, run_batch


class MockEngine:
    def __init__(self, n_slots=8):
        self.free = list(range(n_slots))
        self.lengths = {}
        self.steps = []
        self.released = []

    def acquire(self):
        s = self.free.pop(0)
        self.lengths[s] = 0
        return s

    def release(self, s):
        assert s in self.lengths, "released twice"
        del self.lengths[s]
        self.released.append(s)
        self.free.append(s)

    def step(self, slots, tokens):
        self.steps.append((list(slots), [list(t) for t in tokens]))
        for s, t in zip(slots, tokens):
            self.lengths[s] += len(t)
        return [(s, self.lengths[s]) for s in slots]       # stands in for logits


class ScriptedSampler:
    """Sequence i emits script[i][n] as its n-th token."""

    def __init__(self, script):
        self.script = script
        self.count = {}
        self.begun = None

    def begin(self, slots, prompts):
        self.begun = (list(slots), [list(p) for p in prompts])

    def sample(self, logits, slots, streams):
        out = []
        for st in streams:
            n = self.count.get(st, 0)
            self.count[st] = n + 1
            out.append(self.script[st][n])
        return out


def test_unequal_prompts_then_one_token_each_and_early_ends():
    eng = MockEngine()
    script = {0: [10, 11, 99], 1: [20, 99], 2: [30, 31, 32, 33, 34]}
    prompts = [[1, 2, 3], [4], [5, 6]]
    stats = GenerationStats()
    res = run_batch(eng, ScriptedSampler(script), prompts, [0, 1, 2], 4, [99], 1000, stats)
    assert [r.tokens for r in res] == [[10, 11], [20], [30, 31, 32, 33]]
    assert [r.finish_reason for r in res] == ["stop", "stop", "length"]
    # the whole prompts in one step, then one token per live sequence
    assert eng.steps[0] == ([0, 1, 2], prompts)
    assert eng.steps[1] == ([0, 1, 2], [[10], [20], [30]])
    assert eng.steps[2] == ([0, 2], [[11], [31]])          # sequence 1 ended
    assert eng.steps[3] == ([2], [[32]])                   # sequence 0 ended
    assert len(eng.steps) == 4                             # the last token is not fed
    assert sorted(eng.released) == [0, 1, 2] and eng.lengths == {}
    assert stats.prefill_tokens == 6 and stats.decode_tokens == 3 + 2 + 1 and stats.batches == 1


def test_stop_token_is_neither_emitted_nor_fed():
    eng = MockEngine()
    res = run_batch(eng, ScriptedSampler({0: [99]}), [[1, 2]], [0], 5, [99], 1000)
    assert res[0].tokens == [] and res[0].finish_reason == "stop" and len(eng.steps) == 1


def test_the_model_s_last_position_ends_a_sequence():
    eng = MockEngine()
    res = run_batch(eng, ScriptedSampler({0: [7] * 10}), [[1, 2, 3]], [0], 10, [], 5)
    # positions 0..4 exist: two fed tokens, and the token drawn after the last position
    assert res[0].tokens == [7, 7, 7] and res[0].finish_reason == "length"
    assert eng.lengths == {} and max(sum(len(t) for t in s[1]) for s in eng.steps) <= 3


def test_slots_go_back_even_if_a_step_fails():
    class Failing(MockEngine):
        def step(self, slots, tokens):
            if len(self.steps) == 1:
                raise RuntimeError("boom")
            return super().step(slots, tokens)
    eng = Failing()
    with pytest.raises(RuntimeError):
        run_batch(eng, ScriptedSampler({0: [1, 2, 3], 1: [1, 2, 3]}), [[1], [2]], [0, 1], 3, [], 100)
    assert eng.lengths == {} and sorted(eng.released) == [0, 1]


def test_batches_one_after_another_fit_the_cache():
    assert plan_batches([10, 10, 10, 10, 10], 20, 2, 10000) == [[0, 1], [2, 3], [4]]
    # 100+28 -> 128 tokens each; 300 tokens of cache hold two at a time
    assert plan_batches([100, 100, 100], 28, 8, 300) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="request 1"):
        plan_batches([10, 500], 20, 4, 256)
    assert plan_batches([], 5, 4, 256) == []


class TensorSampler(ScriptedSampler):
    """The scripted sampler with the interface of the pipelined loop (tokens as tensors)."""

    def sample_on_device(self, logits, slots, streams):
        import torch
        return torch.tensor(self.sample(logits, slots, streams), dtype=torch.int32)

    def fetch(self, tokens):
        class Fetch:
            def get(self_inner):
                return tokens.tolist()
        return Fetch()


class TensorEngine(MockEngine):
    def __init__(self):
        super().__init__()
        self.device_steps = []

    def decode_on_device(self, slots, tokens):
        self.device_steps.append((list(slots), tokens.tolist()))
        return self.step(slots, [[int(t)] for t in tokens.tolist()])


@pytest.mark.parametrize("max_new,max_pos", [(4, 1000), (1, 1000), (6, 6), (3, 4)])
def test_pipelined_loop_makes_the_same_decisions(max_new, max_pos):
    from minfer_b200.engine.generate import run_batch_pipelined
    script = {0: [10, 11, 99, 12, 13, 14, 15], 1: [20, 99, 21, 22, 23, 24, 25],
              2: [30, 31, 32, 33, 34, 35, 36], 3: [99, 1, 2, 3, 4, 5, 6]}
    prompts = [[1, 2, 3], [4], [5, 6], [7, 8]]
    want = run_batch(MockEngine(), ScriptedSampler(script), prompts, [0, 1, 2, 3], max_new, [99],
                     max_pos)
    eng = TensorEngine()
    stats = GenerationStats()
    got = run_batch_pipelined(eng, TensorSampler(script), prompts, [0, 1, 2, 3], max_new, [99],
                              max_pos, stats)
    assert [r.tokens for r in got] == [r.tokens for r in want]
    assert [r.finish_reason for r in got] == [r.finish_reason for r in want]
    assert eng.lengths == {} and sorted(eng.released) == [0, 1, 2, 3]
    # no sequence ever runs past the model's last position, and a stopped sequence runs at most
    # one step more than in the plain loop
    for slots, _ in eng.device_steps:
        assert len(slots) == len(set(slots))
    assert stats.batches == 1
