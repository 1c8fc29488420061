"""bin/trace_run as a user runs it: a process fed JSON lines, writing <step>.f32 files.
Whole requests, the last tokens one by one (long decoding included), batches of unequal
lengths one after another, and a request in portions beside others that decode or start, in
float32 and bfloat16, against the plain implementation."""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

import plain_qwen2 as P
from helpers import TOL, make_folder, random_ids, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(folder, dtype, steps, max_tokens):
    out = tempfile.mkdtemp(prefix="minfer_b200_trace_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", dtype, "--out", out, "--max-tokens", str(max_tokens)],
                          input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    return out


def read_logits(out, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, vocab))


@pytest.fixture(scope="module")
def tiny():
    folder = make_folder("B")
    cfg, w = P.load_folder(folder)
    lens = [150, 33, 64, 1, 257]
    prompts = {f"r{i}": random_ids(n, cfg["vocab_size"], 500 + i) for i, n in enumerate(lens)}
    plain = {k: P.forward(cfg, w, v) for k, v in prompts.items()}
    return folder, cfg, prompts, plain


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_three_ways(tiny, dtype):
    folder, cfg, prompts, plain = tiny
    V = cfg["vocab_size"]
    steps, expect = [], []          # expect: (step, [(request, places)])
    n = 0
    # 1. each request alone and whole
    for rid, ids in prompts.items():
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}],
                      "end": [rid]})
        expect.append((n, [(rid, list(range(len(ids))))]))
        n += 1
    # 2. the last 32 tokens one by one (r4: 225 whole then 32 decoded; wants only some places)
    for rid in ("r0", "r4"):
        ids = prompts[rid]
        head = len(ids) - 32
        steps.append({"step": n, "entries": [{"id": rid + "x", "tokens": ids[:head], "want": [0, head - 1]}],
                      "end": []})
        expect.append((n, [(rid, [0, head - 1])]))
        n += 1
        for t in range(head, len(ids)):
            last = t == len(ids) - 1
            steps.append({"step": n, "entries": [{"id": rid + "x", "tokens": [ids[t]], "want": [0]}],
                          "end": [rid + "x"] if last else []})
            expect.append((n, [(rid, [t])]))
            n += 1
    # 3. batches of unequal lengths, one after another (slots and pages are used again)
    for batch in (["r0", "r1", "r2", "r3"], ["r4", "r3", "r1"]):
        heads = {r: max(1, len(prompts[r]) - 6) for r in batch}
        steps.append({"step": n, "entries": [{"id": r + "b", "tokens": prompts[r][:heads[r]],
                                              "want": [heads[r] - 1]} for r in batch], "end": []})
        expect.append((n, [(r, [heads[r] - 1]) for r in batch]))
        n += 1
        pos = dict(heads)
        live = list(batch)
        while True:
            live = [r for r in live if pos[r] < len(prompts[r])]
            if not live:
                break
            ending = [r + "b" for r in live if pos[r] == len(prompts[r]) - 1]
            steps.append({"step": n, "entries": [{"id": r + "b", "tokens": [prompts[r][pos[r]]],
                                                  "want": [0]} for r in live], "end": ending})
            expect.append((n, [(r, [pos[r]]) for r in live]))
            for r in live:
                pos[r] += 1
            n += 1
        # requests of one token never decoded: end them with an empty step
        rest = [r + "b" for r in batch if len(prompts[r]) == 1]
        steps.append({"step": n, "entries": [], "end": rest})
        n += 1
    # 4. a request fed in portions (7 tokens, then 64, then the rest) while another decodes beside it,
    #    joined by a third that starts later
    ids0, ids4, ids1 = prompts["r0"], prompts["r4"], prompts["r1"]
    steps.append({"step": n, "entries": [{"id": "c4", "tokens": ids4[:200], "want": [199]},
                                         {"id": "c0", "tokens": ids0[:7], "want": [6, 0]}], "end": []})
    expect.append((n, [("r4", [199]), ("r0", [6, 0])]))
    n += 1
    steps.append({"step": n, "entries": [{"id": "c4", "tokens": [ids4[200]], "want": [0]},
                                         {"id": "c0", "tokens": ids0[7:71], "want": [63, 1]}], "end": []})
    expect.append((n, [("r4", [200]), ("r0", [70, 8])]))
    n += 1
    steps.append({"step": n, "entries": [{"id": "c1", "tokens": ids1, "want": [len(ids1) - 1]},
                                         {"id": "c4", "tokens": ids4[201:203], "want": [0, 1]},
                                         {"id": "c0", "tokens": ids0[71:], "want": list(range(len(ids0) - 71))}],
                  "end": ["c0", "c1", "c4"]})
    expect.append((n, [("r1", [len(ids1) - 1]), ("r4", [201, 202]), ("r0", list(range(71, len(ids0))))]))
    n += 1
    steps.append({"step": n, "entries": [], "end": []})
    n += 1
    # the cache is sized for what is live at once: the largest batch, each rounded up to 64
    live_max = max(sum(-(-len(prompts[r]) // 64) * 64 for r in b)
                   for b in (["r0", "r1", "r2", "r3"], ["r4", "r3", "r1"], ["r4", "r0", "r1"]))
    out = run_trace(folder, dtype, steps, live_max)
    for step, wants in expect:
        got = read_logits(out, step, V)
        want = torch.cat([plain[r][places] for r, places in wants])
        assert got.shape == want.shape, step
        assert rel_err(got, want) < TOL[dtype], step
    assert not os.path.exists(os.path.join(out, f"{n - 1}.f32"))      # nothing wanted: no file


def test_replay_refuses_what_the_cache_cannot_hold(tiny):
    folder, cfg, prompts, plain = tiny
    out = tempfile.mkdtemp()
    step = {"step": 0, "entries": [{"id": "a", "tokens": prompts["r0"], "want": []}], "end": []}
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                          input=json.dumps(step) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "no free page" in proc.stderr
