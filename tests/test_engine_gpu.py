"""The engine against the plain implementation, in float32 and in bfloat16: each request
alone and whole; with the last 32 tokens one by one; in batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots are used again."""
import pytest
import torch

import plain_qwen2 as P
from helpers import TINY, TOL, logits_err, make_folder, random_ids, rel_err

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
    eng.cache.check_canaries()


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


# ---- any cut: prompts in portions, several tokens onto a sequence, starting beside decoding ----
CUT_LENGTHS = [130, 300, 66]


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E", "F"])
def tiny_cuts(request):
    folder = make_folder(request.param)
    cfg, w = P.load_folder(folder)
    prompts = [random_ids(n, cfg["vocab_size"], 720 + i) for i, n in enumerate(CUT_LENGTHS)]
    plain = [P.forward(cfg, w, ids) for ids in prompts]
    return {"name": request.param, "folder": folder, "cfg": cfg, "prompts": prompts, "plain": plain}


def _close(got, want, dtype):
    err, bound = logits_err(got, want, dtype)
    return err < bound


def _in_portions(eng, ids, sizes):
    """Feeds ``ids`` into a fresh slot in portions of the given sizes (the last size repeats),
    asking for every place; returns the logits [len(ids), vocab]."""
    s = eng.acquire()
    rows, at, i = [], 0, 0
    while at < len(ids):
        n = sizes[min(i, len(sizes) - 1)]
        part = ids[at:at + n]
        rows.append(eng.step([s], [part], [list(range(len(part)))]))
        at += len(part)
        i += 1
    eng.release(s)
    return torch.cat(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [[7], [64], [65], [200], [1, 2, 63, 64, 65], [2]])
def test_prompt_in_portions(tiny_cuts, dtype, sizes):
    """A prompt cut into portions of 7, 64, 65, 200, two tokens, or at 1, 3, 66, 130, 195: the
    logits at every place are those of the whole sequence."""
    eng = _engine(tiny_cuts["folder"], dtype)
    for ids, want in zip(tiny_cuts["prompts"], tiny_cuts["plain"]):
        if sizes == [2] and len(ids) > 140:
            continue
        got = _in_portions(eng, ids, sizes)
        assert got.shape == want.shape
        assert _close(got, want, dtype), (tiny_cuts["name"], len(ids), sizes)
    eng.check_status()


@pytest.mark.parametrize("min_tokens", [1, 10 ** 9])
def test_portions_through_either_attention_kernel(tiny_cuts, min_tokens, monkeypatch):
    """A bfloat16 step over the cache runs the tcgen05 kernel over pages from some number of
    tokens on and the decode kernel (a row per token) below; here each of them takes all
    portions, small and large, and the mixed step."""
    import minfer_b200.parts.attention as attention_part
    monkeypatch.setattr(attention_part, "PAGED_PROMPT_MIN_TOKENS", min_tokens)
    eng = _engine(tiny_cuts["folder"], "bfloat16")
    for ids, want in zip(tiny_cuts["prompts"], tiny_cuts["plain"]):
        for sizes in ([7], [100, 3, 64]):
            got = _in_portions(eng, ids, sizes)
            assert _close(got, want, "bfloat16"), (tiny_cuts["name"], len(ids), sizes, min_tokens)
    p, plain = tiny_cuts["prompts"], tiny_cuts["plain"]
    a, b = eng.acquire(), eng.acquire()
    eng.step([a], [p[1][:200]])
    out = eng.step([a, b], [[p[1][200]], p[0][:90]], [[0], [89, 5]])
    assert _close(out, torch.stack([plain[1][200], plain[0][89], plain[0][5]]), "bfloat16")
    out = eng.step([b, a], [p[0][90:130], p[1][201:204]], [[39], [2]])
    assert _close(out, torch.stack([plain[0][129], plain[1][203]]), "bfloat16")
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_rings_run_long_portions_in_passes(tiny_cuts, dtype):
    """Rings no longer than the window's pages: a portion longer than a ring takes is run in
    several passes by the engine, with the same logits; the last 32 tokens in portions of 4."""
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    eng = Engine(Model.from_folder(tiny_cuts["folder"], dtype, "cuda:0"), max_tokens=2048,
                 ring_step_tokens=1)
    limit = eng.cache.max_new_positions()
    windowed = bool(tiny_cuts["cfg"].get("use_sliding_window"))
    assert (limit is not None) == windowed
    for ids, want in zip(tiny_cuts["prompts"], tiny_cuts["plain"]):
        got = _in_portions(eng, ids, [50, 200])
        assert _close(got, want, dtype), (tiny_cuts["name"], len(ids))
        got = _in_portions(eng, ids, [len(ids) - 32, 4])
        assert _close(got, want, dtype), (tiny_cuts["name"], len(ids))
    assert all(n == eng.cache.groups[i].n_pages for i, n in enumerate(eng.cache.free_pages()))
    eng.check_status()
    eng.cache.check_canaries()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rows_that_start_beside_rows_that_go_on(tiny_cuts, dtype):
    """One step holds a whole new prompt, two sequences that go on by one token and one that
    goes on by five; the next one a second portion beside decoding rows; wanted places in
    another order than the tokens'."""
    eng = _engine(tiny_cuts["folder"], dtype)
    p, plain = tiny_cuts["prompts"], tiny_cuts["plain"]
    a, b, c, d = (eng.acquire() for _ in range(4))
    ids_d = p[0][:47]                                   # a fourth request: the start of the first
    out = eng.step([a, b, c], [p[0][:100], p[1][:250], p[2][:30]])
    assert _close(out, torch.stack([plain[0][99], plain[1][249], plain[2][29]]), dtype)
    out = eng.step([a, d, b, c], [[p[0][100]], ids_d[:40], [p[1][250]], p[2][30:35]],
                   [[0], [39, 0, 17], [0], [4, 0]])
    want = torch.stack([plain[0][100], plain[0][39], plain[0][0], plain[0][17], plain[1][250],
                        plain[2][34], plain[2][30]])
    assert _close(out, want, dtype), tiny_cuts["name"]
    out = eng.step([d, a, c], [ids_d[40:47], [p[0][101]], [p[2][35]]], [[6, 5], [0], [0]])
    want = torch.stack([plain[0][46], plain[0][45], plain[0][101], plain[2][35]])
    assert _close(out, want, dtype), tiny_cuts["name"]
    # and decoding goes on from there (through the graph path, if any)
    for t in range(3):
        out = eng.step([a, b, c, d], [[p[0][102 + t]], [p[1][251 + t]], [p[2][36 + t]], [p[0][47 + t]]])
        want = torch.stack([plain[0][102 + t], plain[1][251 + t], plain[2][36 + t], plain[0][47 + t]])
        assert _close(out, want, dtype), (tiny_cuts["name"], t)
    for s in (a, b, c, d):
        eng.release(s)
    eng.check_status()
    eng.cache.check_canaries()


# ---- what a step refuses ---------------------------------------------------------------------
def test_step_refusals():
    """Every refusal of ``Engine.step`` and ``decode_on_device`` is an error before anything is
    launched or written: the slot's length, its pages and the status word stay as they were."""
    from minfer_b200.cache.paged import CacheError, OutOfPages
    from minfer_b200.engine.step import Engine, StepError
    from minfer_b200.model import Model
    folder = make_folder("B")
    cfg = TINY["B"][0]
    eng = Engine(Model.from_folder(folder, "float32", "cuda:0"), max_tokens=256, max_seqs=3)
    a, b = eng.acquire(), eng.acquire()
    free_before = eng.cache.free_pages()
    with pytest.raises(StepError, match="at least one sequence"):
        eng.step([], [])
    with pytest.raises(StepError, match="one entry per sequence"):
        eng.step([a, b], [[1, 2]])
    with pytest.raises(StepError, match="one entry per sequence"):
        eng.step([a], [[1, 2]], [[0], [1]])
    with pytest.raises(StepError, match="appears twice"):
        eng.step([a, a], [[1], [2]])
    with pytest.raises(StepError, match="at least one token"):
        eng.step([a, b], [[1], []])
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([a], [[1, cfg["vocab_size"]]])
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([a], [[-1]])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([a], [[1, 2, 3]], [[3]])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([a], [[1, 2, 3]], [[-1]])
    with pytest.raises(StepError, match="max_position_embeddings"):
        eng.step([a], [[1] * (cfg["max_position_embeddings"] + 1)])
    with pytest.raises(CacheError, match="not held"):
        eng.step([2], [[1]])                                  # a slot nobody acquired
    with pytest.raises(CacheError, match="out of range"):
        eng.step([7], [[1]])
    assert eng.length(a) == 0 and eng.length(b) == 0 and eng.steps_run == 0
    assert eng.cache.free_pages() == free_before
    with pytest.raises(OutOfPages):                           # 300 tokens into a cache of 256
        eng.step([a], [[1] * 300])
    assert eng.length(a) == 0
    # decode_on_device: int32 device tokens, one per row, onto sequences that have a prompt
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(StepError, match="this slot is empty"):
        eng.decode_on_device([b], tok)
    with pytest.raises(StepError, match="int32 token ids"):
        eng.decode_on_device([b], tok.long())
    with pytest.raises(StepError, match="int32 token ids"):
        eng.decode_on_device([b], torch.zeros(2, dtype=torch.int32, device="cuda"))
    eng.release(a)
    a = eng.acquire()
    eng.step([a], [[5, 6, 7]])
    with pytest.raises(StepError, match="appears twice"):
        eng.decode_on_device([a, a], torch.zeros(2, dtype=torch.int32, device="cuda"))
    eng.check_status()
    # a token id that only the device sees (the sampler's output fed back) is outside the
    # vocabulary: the embedding kernel writes zeros for it and sets bit 1 of the status word;
    # nothing faults, and check_status raises and clears the word
    eng.decode_on_device([a], torch.tensor([cfg["vocab_size"] + 3], dtype=torch.int32, device="cuda"))
    with pytest.raises(StepError, match="token id outside the vocabulary"):
        eng.check_status()
    eng.check_status()
    with pytest.raises(CacheError, match="not held"):
        eng.release(b), eng.release(b)


def test_whole_prompts_through_the_mma_twin_of_the_prompt_kernel(monkeypatch):
    """``MINFER_B200_PROMPT_ATTENTION=mma`` puts whole prompts on the mma.sync kernel instead of
    the tcgen05 one (both are held to float64 kernel by kernel); here the engine runs with it:
    the same logits within bfloat16's tolerance, window and unequal batch included."""
    import minfer_b200.parts.attention as attention_part
    folder = make_folder("D")
    cfg, w = P.load_folder(folder)
    prompts = [random_ids(n, cfg["vocab_size"], 50 + n) for n in (300, 65, 1)]
    want = torch.cat([P.forward(cfg, w, ids) for ids in prompts])
    outs = {}
    for kind in ("tcgen05", "mma"):
        monkeypatch.setattr(attention_part, "PROMPT_ATTENTION", kind)
        eng = _engine(folder, "bfloat16")
        slots = [eng.acquire() for _ in prompts]
        outs[kind] = eng.step(slots, prompts, [list(range(len(p))) for p in prompts])
        eng.check_status()
    for kind, got in outs.items():
        err, bound = logits_err(got, want, "bfloat16")
        assert err < bound, (kind, err)
    if not attention_part.FORCE_GENERIC_ATTENTION:
        assert not torch.equal(outs["mma"], outs["tcgen05"])   # two kernels really ran


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed", [("B", 1), ("D", 2), ("C", 3), ("F", 4)])
def test_random_schedules_of_any_cut(name, seed, dtype):
    """Seeded random schedules: up to five requests live at once, each fed in random portions
    (1 to 90 tokens, often 1), requests starting in steps where others go on, ending at different
    steps, their slots and pages taken by later ones; every step's wanted places (a random
    subset, in random order) against the plain implementation.  Rings of the windowed
    configurations are short here (one page of slack), so long portions also run in passes."""
    import random
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    rng = random.Random(seed)
    folder = make_folder(name)
    cfg, w = P.load_folder(folder)
    V = cfg["vocab_size"]
    eng = Engine(Model.from_folder(folder, dtype, "cuda:0"), max_tokens=2048, max_seqs=5,
                 ring_step_tokens=40)
    requests = []
    for i in range(9):
        ids = random_ids(rng.choice([1, 3, 40, 64, 65, 130, 200, 257]), V, 1000 * seed + i)
        requests.append({"ids": ids, "plain": P.forward(cfg, w, ids), "at": 0, "slot": None})
    waiting, live, worst = list(range(len(requests))), [], 0.0
    while waiting or live:
        while waiting and len(live) < 5 and (not live or rng.random() < 0.5):
            r = waiting.pop(0)
            requests[r]["slot"] = eng.acquire()
            live.append(r)
        rows = [r for r in live if rng.random() < 0.8] or live[:1]
        rng.shuffle(rows)
        tokens, want, expect = [], [], []
        for r in rows:
            q = requests[r]
            left = len(q["ids"]) - q["at"]
            n = min(left, 1 if rng.random() < 0.4 else rng.randint(1, 90))
            tokens.append(q["ids"][q["at"]:q["at"] + n])
            places = rng.sample(range(n), rng.randint(0, min(n, 4)))
            want.append(places)
            expect += [q["plain"][q["at"] + p] for p in places]
            q["at"] += n
        out = eng.step([requests[r]["slot"] for r in rows], tokens, want)
        assert out.shape[0] == len(expect)
        if expect:
            err, bound = logits_err(out, torch.stack(expect), dtype)
            assert err < bound, (name, dtype, err, [len(t) for t in tokens])
            worst = max(worst, err)
        for r in list(live):
            if requests[r]["at"] == len(requests[r]["ids"]):
                eng.release(requests[r]["slot"])
                live.remove(r)
    assert all(n == g.n_pages for n, g in zip(eng.cache.free_pages(), eng.cache.groups))
    assert eng.cache.slots.n_free() == 5
    eng.check_status()
    eng.cache.check_canaries()


def test_matrices_stored_in_32_bit_stay_so_in_the_bfloat16_engine(capfd):
    """A folder whose matrices are stored in float32: the bfloat16 engine keeps them as stored
    (their products then run on the FP32 pipe with bfloat16 activations), says so once when it
    loads them, and still gives the plain implementation's logits, whole and in portions."""
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    folder = make_folder("D", store_dtype="float32")
    cfg, w = P.load_folder(folder)
    model = Model.from_folder(folder, "bfloat16", "cuda:0")
    err = capfd.readouterr().err
    assert "stored in 32-bit" in err and "FP32 pipe" in err
    assert model.blocks[0].mixer.qkv.weight.dtype == torch.float32
    assert model.blocks[0].mixer.accepts_row_scale is False        # no tensor-core product to fold into
    eng = Engine(model, max_tokens=1024)
    ids = random_ids(150, cfg["vocab_size"], 77)
    want = P.forward(cfg, w, ids)
    s = eng.acquire()
    got = torch.cat([eng.step([s], [ids[:100]], [list(range(100))]),
                     eng.step([s], [ids[100:140]], [list(range(40))])] +
                    [eng.step([s], [[t]]) for t in ids[140:]])
    assert _close(got, want, "bfloat16")
    eng.check_status()
