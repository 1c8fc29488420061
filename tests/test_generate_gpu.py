"""Generation through the entry point against the plain implementation: greedy tokens,
sampled tokens with the same seed, stop tokens, batches one after another, and the
sampling kernel alone."""
import math

import pytest
import torch

import plain_qwen2 as P
from helpers import TINY, follows_plain, make_folder, random_ids

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request):
    folder = make_folder(request.param)
    cfg, w = P.load_folder(folder)
    return {"name": request.param, "folder": folder, "cfg": cfg, "w": w}


def _generator(folder, dtype="float32", max_batch=4, max_tokens=2048):
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    return Generator(Model.from_folder(folder, dtype, "cuda:0"), max_tokens=max_tokens,
                     max_batch=max_batch)


def test_greedy_equals_plain(tiny):
    from minfer_b200.sampling.params import SamplingParams
    cfg, w = tiny["cfg"], tiny["w"]
    prompts = [random_ids(n, cfg["vocab_size"], 40 + n) for n in (5, 9, 13, 1, 33)]
    want = [P.generate(cfg, w, p, 8) for p in prompts]
    gen = _generator(tiny["folder"], max_batch=3)          # 5 requests -> two batches
    got = gen.generate(prompts, 8, SamplingParams.greedy(), stop_token_ids=[])
    assert [r.tokens for r in got] == want
    assert gen.stats.batches == 2
    assert all(r.finish_reason == "length" for r in got)


def test_stop_token_ends_a_sequence_early(tiny):
    from minfer_b200.sampling.params import SamplingParams
    cfg, w = tiny["cfg"], tiny["w"]
    prompts = [random_ids(n, cfg["vocab_size"], 70 + n) for n in (6, 11, 3)]
    free = [P.generate(cfg, w, p, 10) for p in prompts]
    stop = free[1][4]                     # the fifth token of the second request stops it
    want = [P.generate(cfg, w, p, 10, stop_ids=[stop]) for p in prompts]
    gen = _generator(tiny["folder"])
    got = gen.generate(prompts, 10, SamplingParams.greedy(), stop_token_ids=[stop])
    assert [r.tokens for r in got] == want
    assert got[1].finish_reason == "stop" and len(got[1].tokens) <= 4
    assert stop not in got[1].tokens
    # every slot and page went back
    assert gen.engine.cache.slots.n_free() == gen.engine.max_seqs
    assert all(n == g.n_pages for n, g in zip(gen.engine.cache.free_pages(), gen.engine.cache.groups))


@pytest.mark.parametrize("params", [
    dict(temperature=0.8, top_k=0, top_p=1.0, repeat_penalty=1.0),
    dict(temperature=0.8, top_k=40, top_p=0.95, repeat_penalty=1.1),
    dict(temperature=1.3, top_k=5, top_p=0.5, repeat_penalty=1.3, frequency_penalty=0.2,
         presence_penalty=0.1),
    dict(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.5, presence_penalty=0.4),
])
def test_sampled_generation_equals_plain_and_ignores_the_batch(tiny, params):
    from minfer_b200.sampling.params import SamplingParams
    cfg, w = tiny["cfg"], tiny["w"]
    prompts = [random_ids(n, cfg["vocab_size"], 90 + n) for n in (1, 7, 20, 33)]
    sp = SamplingParams(seed=7, **params)
    gen = _generator(tiny["folder"])
    got = [r.tokens for r in gen.generate(prompts, 12, sp, stop_token_ids=[])]
    for i, p in enumerate(prompts):
        want = P.generate(cfg, w, p, 12, temp=sp.temperature, top_k=sp.top_k, top_p=sp.top_p,
                          repeat=sp.repeat_penalty, frequency=sp.frequency_penalty,
                          presence=sp.presence_penalty, seed=7, stream=i)
        assert got[i] == want, (i, params)
    # the same requests in another batch composition give the same tokens
    gen2 = _generator(tiny["folder"], max_batch=2)
    again = [r.tokens for r in gen2.generate(prompts, 12, sp, stop_token_ids=[])]
    assert again == got


@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("params", [
    dict(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0),
    dict(temperature=0.8, top_k=40, top_p=0.95, repeat_penalty=1.1),
])
def test_bfloat16_generation_follows_plain(name, params):
    """The bfloat16 engine (tensor-core products and attention, graphs, the pipelined loop)
    generates what the plain implementation generates, token by token on the engine's own
    prefix, up to what bfloat16 rounding can tip (``helpers.follows_plain``); and the same
    requests in another batch composition follow it too.  In bfloat16 the two compositions
    need not give the same bits: the tensor-core product picks its token tile and its K
    splits from the number of rows, which changes the order of the sums."""
    from minfer_b200.sampling.params import SamplingParams
    folder = make_folder(name)
    cfg, w = P.load_folder(folder)
    prompts = [random_ids(n, cfg["vocab_size"], 60 + n) for n in (1, 7, 20, 33, 70)]
    sp = SamplingParams(seed=11, **params)
    for max_batch in (5, 2):
        gen = _generator(folder, "bfloat16", max_batch=max_batch)
        got = gen.generate(prompts, 10, sp, stop_token_ids=[])
        for i, (p, r) in enumerate(zip(prompts, got)):
            assert len(r.tokens) == 10
            follows_plain(P, cfg, w, p, r.tokens, "bfloat16", temp=sp.temperature, top_k=sp.top_k,
                          top_p=sp.top_p, repeat=sp.repeat_penalty, seed=11, stream=i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_loop_with_the_host_in_step_equals_the_pipelined_loop(tiny, dtype):
    """``Generator(pipelined=False)`` reads every step's tokens before it launches the next
    (``run_batch``); the default keeps the host one step behind (``run_batch_pipelined``).
    The same tokens and finish reasons, stop tokens and early ends included."""
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    cfg, w = tiny["cfg"], tiny["w"]
    prompts = [random_ids(n, cfg["vocab_size"], 20 + n) for n in (3, 12, 1, 40, 9)]
    model = Model.from_folder(tiny["folder"], dtype, "cuda:0")
    sp = SamplingParams(seed=3, temperature=0.9, top_k=20, top_p=0.9, repeat_penalty=1.2)
    free = Generator(model, max_tokens=2048, max_batch=3).generate(prompts, 14, sp, stop_token_ids=[])
    stop = [free[1].tokens[5], free[3].tokens[2]]
    outs = []
    for pipelined in (True, False):
        gen = Generator(model, max_tokens=2048, max_batch=3, pipelined=pipelined)
        outs.append([(r.tokens, r.finish_reason) for r in gen.generate(prompts, 14, sp, stop_token_ids=stop)])
        assert gen.engine.cache.slots.n_free() == gen.engine.max_seqs
    assert outs[0] == outs[1]
    assert any(reason == "stop" for _, reason in outs[0])


def test_sampling_kernel_alone():
    """The kernel against the plain sampler on logits made so that ties, the top-k edge and
    the top-p edge all occur; a vocabulary that is no power of two."""
    from minfer_b200.kernels import api as K
    V, rows = 1531, 6
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(rows, V, generator=g) * 3.0
    logits[0, 100] = logits[0, 7] = logits[0].max() + 1.0           # tie: lowest index wins
    logits[1, :50] = 2.5                                            # many ties at the top-k edge
    logits[2, 5] = 30.0                                             # one dominant token
    cases = [dict(temp=0.0, top_k=0, top_p=1.0), dict(temp=0.7, top_k=40, top_p=0.95),
             dict(temp=1.0, top_k=0, top_p=0.9), dict(temp=1.0, top_k=0, top_p=1.0),
             dict(temp=2.0, top_k=3, top_p=1.0)]
    for case in cases:
        for seed in (1, 2):
            dev = logits.clone().cuda()
            out = torch.empty(rows, dtype=torch.int32, device="cuda")
            K.sample(dev, out, temperature=case["temp"], top_k=case["top_k"], top_p=case["top_p"],
                     repeat_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0, seed=seed)
            got = out.cpu().tolist()
            for r in range(rows):
                u = P.philox_uniform(seed, 0, r)
                want = P.sample(logits[r].double(), case["temp"], case["top_k"], case["top_p"],
                                1.0, 0.0, 0.0, [], u)
                assert got[r] == want, (case, seed, r)


def test_cli_generates(tiny, capsys):
    from minfer_b200 import cli
    rc = cli.main([tiny["folder"], "5,17,3", "--greedy", "--repeat-penalty", "1.0", "-n", "6",
                   "--dtype", "float32", "--stop", "100000"])
    out = capsys.readouterr().out
    assert rc == 0
    want = P.generate(tiny["cfg"], tiny["w"], [5, 17, 3], 6)
    assert " ".join(str(t) for t in want) in out
    assert "Prefill: 3 tokens" in out and "Generated: 6 tokens" in out


def test_cli_as_a_process(tiny):
    """``bin/minfer-b200`` as a user starts it: its own process, killed if it hangs.  The
    reference prints usage and fails on an unknown flag (src/main.rs:280-286); so does this."""
    import os
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    exe = os.path.join(root, "bin", "minfer-b200")
    run = subprocess.run([sys.executable, exe, tiny["folder"], "5,17,3", "--greedy",
                          "--repeat-penalty", "1.0", "-n", "4", "--dtype", "bfloat16"],
                         capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr[-2000:]
    assert "Prefill: 3 tokens" in run.stdout and "Generated:" in run.stdout
    bad = subprocess.run([sys.executable, exe, tiny["folder"], "--no-such-flag"],
                         capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0
    assert "usage" in (bad.stderr + bad.stdout).lower()


def test_model_conveniences(tiny):
    """``from_pretrained``, ``new_session`` and ``Model.generate`` are the loader, the engine
    and the generator under other names: the same logits and tokens."""
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    model = Model.from_pretrained(tiny["folder"], "float32")
    ids = [5, 17, 3, 9]
    session = model.new_session(max_seqs=2, max_positions=128)
    s = session.acquire()
    logits = session.step([s], [ids], [list(range(len(ids)))])
    session.release(s)
    want = P.forward(tiny["cfg"], tiny["w"], ids)
    assert float((logits.double().cpu() - want).abs().max() / want.abs().max()) < 2e-5
    out = model.generate([ids], 5, SamplingParams.greedy(), stop_token_ids=[], max_batch=1,
                         max_positions=128)
    assert out[0].tokens == P.generate(tiny["cfg"], tiny["w"], ids, 5)


def test_sampling_kernel_at_a_large_vocabulary():
    """The same comparison at a vocabulary of 50,021 (no multiple of anything): the short-list
    path of top-k (k = 40 and k = 1000), top-k beyond the list's reach (k = 3000: radix selection
    over the row, then top-p over more than 1,024 survivors), plain temperature, and logits
    whose scale puts thousands of values into one binary order of magnitude."""
    from minfer_b200.kernels import api as K
    V, rows = 50021, 3
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(rows, V, generator=g)
    logits[0] *= 0.3                                               # the top 40 share one exponent
    logits[1] *= 4.0
    logits[2, 123] = 9.0                                           # one token far ahead
    cases = [dict(temp=0.8, top_k=40, top_p=0.95), dict(temp=1.0, top_k=1000, top_p=0.9),
             dict(temp=1.2, top_k=3000, top_p=0.8), dict(temp=0.9, top_k=0, top_p=1.0),
             dict(temp=0.0, top_k=0, top_p=1.0)]
    for case in cases:
        dev = logits.clone().cuda()
        out = torch.empty(rows, dtype=torch.int32, device="cuda")
        K.sample(dev, out, temperature=case["temp"], top_k=case["top_k"], top_p=case["top_p"],
                 repeat_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0, seed=5)
        got = out.cpu().tolist()
        for r in range(rows):
            u = P.philox_uniform(5, 0, r)
            want = P.sample(logits[r].double(), case["temp"], case["top_k"], case["top_p"],
                            1.0, 0.0, 0.0, [], u)
            assert got[r] == want, (case, r)
