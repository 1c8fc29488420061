"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
``Model.from_folder`` and ``Engine.step``, the ones generation uses.  The reference's
nearest tool is the dump that ``MINFER_GRAPH_DUMP`` switches on inside its forward
(src/models/qwen2/graph.rs:362-399), which writes ``logits_<prefill|decode>.f32``; here the
steps come from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at the
wanted places, in the order of the entries and of ``want``, as little-endian float32
``[wanted, vocab]``.  After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    args = ap.parse_args(argv)

    print("[trace_run] loading torch and the model ...", file=sys.stderr, flush=True)
    import torch
    from .engine.step import Engine
    from .model import Model

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is available; there is no CPU path", file=sys.stderr)
        return 2
    os.makedirs(args.out, exist_ok=True)
    model = Model.from_folder(args.model, args.dtype, "cuda:0")
    engine = Engine(model, max_tokens=args.max_tokens)
    slot_of: Dict[str, int] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = rec.get("entries", [])
        if entries:
            slots, tokens, want = [], [], []
            for e in entries:
                rid = str(e["id"])
                if rid not in slot_of:
                    slot_of[rid] = engine.acquire()
                slots.append(slot_of[rid])
                tokens.append([int(t) for t in e["tokens"]])
                want.append([int(x) for x in e.get("want", [])])
            logits = engine.step(slots, tokens, want)
            if logits.shape[0] > 0:
                data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4")
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                data.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
            engine.check_status()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slot_of:
                engine.release(slot_of.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
