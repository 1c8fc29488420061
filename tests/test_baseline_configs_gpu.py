"""The two tiny configurations exactly as the headline's record states them, with their stated
workloads: A (2 layers, width 64, 4 heads on 1 key/value head of 16, feed-forward 128,
vocabulary 256, tied, theta 1e4, eps 1e-6, 128 positions, weights N(0, 0.02), norm weights 1):
three prompts of 5/9/13 tokens, then 8 greedy tokens; B (3 layers, width 192, 6 heads on 2 of
32, feed-forward 320, vocabulary 384, untied, theta 1e6, eps 1e-5, window 16 from layer 1, 256
positions, norm weights 1 + N(0, 0.01)): four prompts of 1/7/20/33 tokens, then 12 tokens at
temperature 0.8, sampler seed 7.  And the three schedules at lengths these models allow."""
import pytest
import torch

import plain_qwen2 as P
from helpers import TINY, TOL, follows_plain, logits_err, make_folder, random_ids

pytestmark = pytest.mark.gpu

WORKLOAD = {"A0": dict(lengths=(5, 9, 13), new=8, temp=0.0, seed=0),
            "B0": dict(lengths=(1, 7, 20, 33), new=12, temp=0.8, seed=7)}


@pytest.fixture(scope="module", params=["A0", "B0"])
def stated(request):
    name = request.param
    folders = {"float32": make_folder(name, store_dtype="float32"),
               "bfloat16": make_folder(name, store_dtype="bfloat16")}
    loaded = {d: P.load_folder(f) for d, f in folders.items()}
    return {"name": name, "folders": folders, "loaded": loaded}


def test_weights_are_as_stated(stated):
    cfg, w = stated["loaded"]["float32"]
    for key, value in TINY[stated["name"]][0].items():
        assert cfg[key] == value, key
    big = torch.cat([t.flatten() for n, t in w.items() if "norm" not in n])
    assert abs(float(big.std()) - 0.02) < 1e-3 and abs(float(big.mean())) < 1e-3
    norms = torch.cat([t.flatten() for n, t in w.items() if "norm" in n])
    if stated["name"] == "A0":
        assert torch.equal(norms, torch.ones_like(norms))
    else:
        assert abs(float(norms.mean()) - 1.0) < 3e-3 and 0.005 < float(norms.std()) < 0.015


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stated_workload(stated, dtype):
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    cfg, w = stated["loaded"][dtype]
    work = WORKLOAD[stated["name"]]
    prompts = [random_ids(n, cfg["vocab_size"], 10 + n) for n in work["lengths"]]
    sp = SamplingParams(temperature=work["temp"], top_k=0, top_p=1.0, repeat_penalty=1.0,
                        seed=work["seed"])
    gen = Generator(Model.from_folder(stated["folders"][dtype], dtype, "cuda:0"),
                    max_tokens=len(prompts) * 64, max_batch=len(prompts))
    got = gen.generate(prompts, work["new"], sp, stop_token_ids=[])
    assert gen.stats.batches == 1
    for i, (p, r) in enumerate(zip(prompts, got)):
        assert len(r.tokens) == work["new"] and r.finish_reason == "length"
        follows_plain(P, cfg, w, p, r.tokens, dtype, temp=work["temp"], seed=work["seed"], stream=i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_three_schedules_and_portions(stated, dtype):
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    cfg, w = stated["loaded"][dtype]
    top = cfg["max_position_embeddings"]
    lens = [top, 45, 1, 64, 65, top - 1]
    prompts = [random_ids(n, cfg["vocab_size"], 200 + i) for i, n in enumerate(lens)]
    plain = [P.forward(cfg, w, ids) for ids in prompts]
    eng = Engine(Model.from_folder(stated["folders"][dtype], dtype, "cuda:0"), max_tokens=1024)

    def check(got, want, what):
        err, bound = logits_err(got, want, dtype)
        assert err < bound, (stated["name"], what, err)

    for i, ids in enumerate(prompts):
        s = eng.acquire()                               # alone and whole
        check(eng.step([s], [ids], [list(range(len(ids)))]), plain[i], ("whole", i))
        eng.release(s)
        head = max(1, len(ids) - 32)                    # the last 32 one by one
        s = eng.acquire()
        rows = [eng.step([s], [ids[:head]], [list(range(head))])]
        rows += [eng.step([s], [[t]]) for t in ids[head:]]
        check(torch.cat(rows), plain[i], ("one by one", i))
        eng.release(s)
        s = eng.acquire()                               # in portions of 7
        rows = [eng.step([s], [ids[a:a + 7]], [list(range(len(ids[a:a + 7])))]) for a in range(0, len(ids), 7)]
        check(torch.cat(rows), plain[i], ("portions", i))
        eng.release(s)
    for batch in ([0, 1, 2], [3, 4, 5, 2]):             # unequal batches, slots used again
        slots = [eng.acquire() for _ in batch]
        heads = {r: max(1, lens[r] - 5) for r in batch}
        out = eng.step(slots, [prompts[r][:heads[r]] for r in batch])
        check(out, torch.stack([plain[r][heads[r] - 1] for r in batch]), ("batch", batch))
        pos = dict(heads)
        live = list(batch)
        while True:
            live = [r for r in live if pos[r] < lens[r]]
            if not live:
                break
            out = eng.step([slots[batch.index(r)] for r in live], [[prompts[r][pos[r]]] for r in live])
            check(out, torch.stack([plain[r][pos[r]] for r in live]), ("batch", batch, pos))
            for r in live:
                pos[r] += 1
        for s in slots:
            eng.release(s)
    # one position past the model's last is refused, and nothing was written for it
    from minfer_b200.engine.step import StepError
    s = eng.acquire()
    with pytest.raises(StepError, match="max_position_embeddings"):
        eng.step([s], [random_ids(top + 1, cfg["vocab_size"], 1)])
    assert eng.length(s) == 0
    eng.release(s)
    eng.check_status()
