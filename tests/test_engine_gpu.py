"""The engine against the plain implementation, in float32 and in bfloat16: each request
alone and whole; with the last 32 tokens one by one; in batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again."""
import pytest
import torch

import plain_qwen2 as P
from helpers import TINY, TOL, make_folder, random_ids, rel_err

pytestmark = pytest.mark.gpu

LENGTHS = [37, 5, 90, 64, 1, 65, 130]


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E", "F"])
def tiny(request):
    folder = make_folder(request.param)
    cfg, w = P.load_folder(folder)
    prompts = [random_ids(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS)]
    plain = [P.forward(cfg, w, ids) for ids in prompts]
    return {"name": request.param, "folder": folder, "cfg": cfg, "prompts": prompts, "plain": plain}


def _engine(folder, dtype, max_tokens=2048):
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    return Engine(Model.from_folder(folder, dtype, "cuda:0"), max_tokens=max_tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_requests(tiny, dtype):
    eng = _engine(tiny["folder"], dtype)
    for ids, want in zip(tiny["prompts"], tiny["plain"]):
        s = eng.acquire()
        got = eng.step([s], [ids], [list(range(len(ids)))])
        eng.release(s)
        assert got.shape == want.shape
        assert rel_err(got, want) < TOL[dtype]
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(tiny, dtype):
    eng = _engine(tiny["folder"], dtype)
    for ids, want in zip(tiny["prompts"], tiny["plain"]):
        n = len(ids)
        head = max(1, n - 32)
        s = eng.acquire()
        rows = [eng.step([s], [ids[:head]], [list(range(head))])]
        for t in range(head, n):
            rows.append(eng.step([s], [[ids[t]]], [[0]]))
        eng.release(s)
        got = torch.cat(rows)
        assert rel_err(got, want) < TOL[dtype]
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_slots_reused(tiny, dtype):
    """Batches of unequal lengths: the prompts' first parts in one step, then one token
    each; a request that runs out of tokens leaves the batch; the next batch starts in the
    slots the first one gave back."""
    eng = _engine(tiny["folder"], dtype, max_tokens=1024)
    prompts, plain = tiny["prompts"], tiny["plain"]
    batches = [[0, 1, 2], [3, 4, 5, 6], [2, 0]]
    seen_slots = []
    for batch in batches:
        slots = [eng.acquire() for _ in batch]
        seen_slots.append(list(slots))
        # every request decodes its last min(8, n-1) tokens one by one
        heads = {r: max(1, len(prompts[r]) - 8) for r in batch}
        got = {r: [] for r in batch}
        live = list(batch)
        out = eng.step([slots[batch.index(r)] for r in live], [prompts[r][:heads[r]] for r in live],
                       [list(range(heads[r])) for r in live])
        at = 0
        for r in live:
            got[r].append(out[at:at + heads[r]])
            at += heads[r]
        pos = dict(heads)
        while True:
            live = [r for r in live if pos[r] < len(prompts[r])]
            if not live:
                break
            out = eng.step([slots[batch.index(r)] for r in live], [[prompts[r][pos[r]]] for r in live])
            for i, r in enumerate(live):
                got[r].append(out[i:i + 1])
                pos[r] += 1
        for s in slots:
            eng.release(s)
        for r in batch:
            assert rel_err(torch.cat(got[r]), plain[r]) < TOL[dtype], (tiny["name"], r)
    assert set(seen_slots[1]) & set(seen_slots[0]), "the second batch did not reuse a slot"
    assert all(n == eng.cache.groups[i].n_pages for i, n in enumerate(eng.cache.free_pages()))
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_through_cuda_graphs_equals_kernel_by_kernel(tiny, dtype):
    """Long decoding (300 steps across page and chunk boundaries), a batch of three whose
    shortest prompt is one token, replayed as CUDA graphs and launched kernel by kernel:
    the same bits."""
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    model = Model.from_folder(tiny["folder"], dtype, "cuda:0")
    V = tiny["cfg"]["vocab_size"]
    prompts = [random_ids(n, V, 900 + n) for n in (1, 50, 200)]
    feed = [random_ids(300, V, 950 + i) for i in range(3)]
    outs = []
    for graphs in (True, False):
        eng = Engine(model, max_tokens=2048, cuda_graphs=graphs)
        assert eng.cuda_graphs == graphs
        slots = [eng.acquire() for _ in prompts]
        rows = [eng.step(slots, prompts)]
        for t in range(300):
            rows.append(eng.step(slots, [[f[t]] for f in feed]))
        outs.append(torch.stack(rows))
        if graphs:
            assert len(eng._graphs) >= 2          # the length bound was crossed at least once
        eng.check_status()
    assert torch.equal(outs[0], outs[1])
    # and the last logits of the longest request agree with the plain implementation
    ids = prompts[2] + feed[2]
    want = P.forward(tiny["cfg"], P.load_folder(tiny["folder"])[1], ids)
    assert rel_err(outs[0][-1, 2], want[-1]) < TOL[dtype]
    assert rel_err(outs[0][150, 2], want[200 + 149]) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_sequence_many_tiles_and_chunks(dtype):
    """2,100 tokens (33 query tiles, 9 key chunks, a window edge far from the start) whole,
    then 40 more tokens one by one, with a second, short sequence beside it; against the
    plain implementation at the places asked for."""
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    folder = make_folder("D")
    cfg, w = P.load_folder(folder)
    V = cfg["vocab_size"]
    long_ids = random_ids(2140, V, 4242)
    short_ids = random_ids(47, V, 4243)
    want_long = P.forward(cfg, w, long_ids)
    want_short = P.forward(cfg, w, short_ids)
    eng = Engine(Model.from_folder(folder, dtype, "cuda:0"), max_tokens=2304 + 128)
    a, b = eng.acquire(), eng.acquire()
    places = [0, 63, 64, 1000, 2047, 2099]
    out = eng.step([a, b], [long_ids[:2100], short_ids[:7]], [places, [6]])
    assert rel_err(out[:6], want_long[places]) < TOL[dtype]
    assert rel_err(out[6:], want_short[6:7]) < TOL[dtype]
    for t in range(40):
        out = eng.step([a, b], [[long_ids[2100 + t]], [short_ids[7 + t]]])
        assert rel_err(out[0], want_long[2100 + t]) < TOL[dtype], t
        assert rel_err(out[1], want_short[7 + t]) < TOL[dtype], t
    eng.check_status()


def test_batches_that_shrink_share_graphs_and_padding_changes_nothing():
    """Decode graphs are captured for batch sizes that are powers of two; a batch of 5, then 3
    (two sequences ended) is filled up with rows on the spare slot.  The live rows' logits are
    those of the same sequences decoded alone, and only the padded sizes get graphs."""
    folder = make_folder("D")
    cfg, w = P.load_folder(folder)
    eng = _engine(folder, "float32")
    prompts = [random_ids(n, cfg["vocab_size"], 300 + n) for n in (9, 4, 17, 1, 30)]
    nxt = [random_ids(12, cfg["vocab_size"], 400 + i) for i in range(5)]
    alone = []
    for p, t in zip(prompts, nxt):
        s = eng.acquire()
        eng.step([s], [p])
        alone.append(torch.cat([eng.step([s], [[tok]]) for tok in t]))
        eng.release(s)
    graphs_before = set(eng._graphs)
    slots = [eng.acquire() for _ in prompts]
    eng.step(slots, prompts)
    got = [[] for _ in prompts]
    live = list(range(5))
    for step in range(12):
        if step == 6:
            live = [0, 2, 4]                          # two sequences end here
        out = eng.step([slots[b] for b in live], [[nxt[b][step]] for b in live])
        for i, b in enumerate(live):
            got[b].append(out[i:i + 1])
    for b in range(5):
        have = torch.cat(got[b])
        assert torch.equal(have, alone[b][:have.shape[0]]), b      # float32: the same bits
    sizes = {k[0] for k in set(eng._graphs) - graphs_before}
    assert sizes <= {4, 8}, sizes
    for s in slots:
        eng.release(s)
    eng.check_status()
