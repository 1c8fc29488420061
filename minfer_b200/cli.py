"""Command line in the reference's manner (src/main.rs:72-118, flags parsed by hand at
:147-291): ``<model> [prompt] [OPTIONS]`` plus the ``info`` subcommand; the same option
names, meanings and defaults where the reference has them.  Text is out of scope (no
tokenizer), so the prompt is a list of token ids and ``--stop`` takes a token id.

    minfer-b200 <model> "1,2,3" [OPTIONS]
    minfer-b200 <model> --prompt-file ids.txt [OPTIONS]      one sequence per line
    minfer-b200 info <model>
    minfer-b200 random <config.json> <folder> [--seed N] [--store-dtype bfloat16|float32]
"""
from __future__ import annotations

import json
import sys
import time
from typing import List, Optional

from . import __version__

USAGE = """minfer-b200 - a small B200-native LLM generation library in minfer's manner

USAGE:
  {prog} <model> [prompt] [OPTIONS]
  {prog} info <model>                      (also: {prog} --info <model>)
  {prog} random <config.json> <folder> [--seed N] [--store-dtype bfloat16|float32]

MODEL - a folder with config.json and model.safetensors
PROMPT - token ids separated by commas or spaces, e.g. "151644,872,198"

OPTIONS:
  --meta                  print the configuration and key tensors
  --prompt-ids <IDS>      the prompt as an option instead of the second argument
  --prompt-file <FILE>    one prompt per line (token ids); all lines run as batches
  --max-seqs <N>          sequences per batch (default: all prompts, at most 64)
  --temp <T>              sampling temperature (default 0.8; 0 = greedy)
  --greedy                greedy decoding (--temp 0)
  --top-k <K>             top-K sampling (default 40)
  --top-p <P>             top-P nucleus sampling (default 0.95)
  --repeat-penalty <N>    penalize repeated tokens (default 1.1; 1.0 = off)
  --frequency-penalty <N> penalize by token count in the window (default 0.0)
  --presence-penalty <N>  penalize any token present in the window (default 0.0)
  --stop <ID>             stop generation at this token id (repeatable; also --stop-id;
                          default: the model's eos_token_id)
  -n, --n-predict <N>     max tokens to generate (default 512)
  --seed <N>              RNG seed for sampling (default 42)
  --n-ctx <N>             context per sequence (default 4096); sizes the cache
  --dtype <D>             bfloat16 (default) or float32 (true 32-bit everywhere)
  --no-cuda-graph         launch decode steps kernel by kernel
  -h, --help              show this help
  -V, --version           print version and exit
"""


def usage(prog: str = "minfer-b200") -> str:
    return USAGE.format(prog=prog)


class CliError(Exception):
    pass


def parse_ids(text: str) -> List[int]:
    parts = text.replace(",", " ").split()
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise CliError(f"a prompt is a list of token ids, got {text!r}") from None


def parse_args(argv: List[str]) -> dict:
    opts = {"model": None, "prompt": None, "prompt_file": None, "meta": False, "temp": 0.8,
            "top_k": 40, "top_p": 0.95, "repeat_penalty": 1.1, "frequency_penalty": 0.0,
            "presence_penalty": 0.0, "stop": [], "n_predict": 512, "seed": 42, "n_ctx": 4096,
            "dtype": "bfloat16", "cuda_graph": True, "command": "run", "store_dtype": "bfloat16",
            "positional": []}
    i = 0

    def value(flag: str) -> str:
        nonlocal i
        i += 1
        if i >= len(argv):
            raise CliError(f"{flag} needs a value")
        return argv[i]

    def number(flag: str, kind):
        v = value(flag)
        try:
            return kind(v)
        except ValueError:
            raise CliError(f"{flag} needs a number, got {v!r}") from None

    while i < len(argv):
        a = argv[i]
        if a in ("-h", "--help"):
            opts["command"] = "help"
        elif a in ("-V", "--version"):
            opts["command"] = "version"
        elif a == "--meta":
            opts["meta"] = True
        elif a == "--prompt-file":
            opts["prompt_file"] = value(a)
        elif a == "--prompt-ids":
            opts["prompt"] = parse_ids(value(a))
        elif a == "--info":
            opts["command"] = "info"
        elif a == "--max-seqs":
            opts["max_seqs"] = number(a, int)
        elif a in ("--temp", "-t"):
            opts["temp"] = number(a, float)
        elif a == "--greedy":
            opts["temp"] = 0.0
        elif a == "--top-k":
            opts["top_k"] = number(a, int)
        elif a == "--top-p":
            opts["top_p"] = number(a, float)
        elif a == "--repeat-penalty":
            opts["repeat_penalty"] = number(a, float)
        elif a == "--frequency-penalty":
            opts["frequency_penalty"] = number(a, float)
        elif a == "--presence-penalty":
            opts["presence_penalty"] = number(a, float)
        elif a in ("--stop", "--stop-id"):
            opts["stop"].append(number(a, int))
        elif a in ("-n", "--n-predict"):
            opts["n_predict"] = number(a, int)
        elif a == "--seed":
            opts["seed"] = number(a, int)
        elif a == "--n-ctx":
            opts["n_ctx"] = number(a, int)
        elif a == "--dtype":
            opts["dtype"] = value(a)
            if opts["dtype"] not in ("bfloat16", "float32", "bf16", "fp32"):
                raise CliError("--dtype is bfloat16 or float32")
        elif a == "--store-dtype":
            opts["store_dtype"] = value(a)
        elif a == "--no-cuda-graph":
            opts["cuda_graph"] = False
        elif a.startswith("-") and len(a) > 1 and not a[1:].replace(",", "").isdigit():
            raise CliError(f"unknown option {a}")
        else:
            opts["positional"].append(a)
        i += 1
    pos = opts["positional"]
    if opts["command"] in ("help", "version"):
        return opts
    if opts["command"] == "info":                        # --info <model>
        if len(pos) != 1:
            raise CliError("usage: --info <model>")
        opts["model"] = pos[0]
    elif pos and pos[0] == "info":
        if len(pos) != 2:
            raise CliError("usage: info <model>")
        opts["command"], opts["model"] = "info", pos[1]
    elif pos and pos[0] == "random":
        if len(pos) != 3:
            raise CliError("usage: random <config.json> <folder>")
        opts["command"], opts["config"], opts["model"] = "random", pos[1], pos[2]
    else:
        if not pos:
            raise CliError("no model given")
        if len(pos) > 2:
            raise CliError(f"unexpected argument {pos[2]!r}")
        opts["model"] = pos[0]
        if len(pos) == 2:
            if opts["prompt"] is not None:
                raise CliError("a prompt was given twice (positional and --prompt-ids)")
            opts["prompt"] = parse_ids(pos[1])
    return opts


def print_info(folder: str, out=sys.stdout) -> None:
    from .model import Model
    from .registry import read_config
    from .weights.safetensors_io import Checkpoint
    import os
    with open(os.path.join(folder, "config.json")) as f:
        raw = json.load(f)
    cfg = read_config(raw, os.path.join(folder, "config.json"))
    model = Model(cfg.plan(), "float32", cfg)
    print(f"architecture: {model.plan.architecture}", file=out)
    for k, v in sorted(vars(cfg).items()):
        if k != "extra":
            print(f"  {k}: {v}", file=out)
    ck = Checkpoint(folder)
    total = 0
    for spec in model.tensor_specs():
        if spec.name in ck.where:
            e = ck.entry(spec.name)
            n = 1
            for s in e.shape:
                n *= s
            total += n
    print(f"tensors: {len(ck.names())} in the checkpoint, {len(model.tensor_specs())} expected, "
          f"{total / 1e6:.1f} M parameters", file=out)
    for name in list(ck.names())[:8]:
        e = ck.entry(name)
        print(f"  {name}: {list(e.shape)} {e.dtype_name}", file=out)
    ck.close()


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        opts = parse_args(argv)
    except CliError as e:
        print(f"error: {e}\n", file=sys.stderr)
        print(usage(), file=sys.stderr)
        return 2
    if opts["command"] == "help":
        print(usage())
        return 0
    if opts["command"] == "version":
        print(f"minfer-b200 {__version__}")
        return 0
    if opts["command"] == "info":
        print_info(opts["model"])
        return 0
    if opts["command"] == "random":
        from .model import write_random_model
        with open(opts["config"]) as f:
            cfg = json.load(f)
        write_random_model(opts["model"], cfg, opts["seed"], opts["store_dtype"])
        print(f"wrote {opts['model']}/config.json and model.safetensors (seed {opts['seed']})")
        return 0

    prompts: List[List[int]] = []
    if opts["prompt_file"]:
        with open(opts["prompt_file"]) as f:
            prompts = [parse_ids(line) for line in f if line.strip()]
    if opts["prompt"] is not None:
        prompts.insert(0, opts["prompt"])
    if opts["meta"]:
        print_info(opts["model"])
    if not prompts:
        if opts["meta"]:
            return 0
        print("error: no prompt given\n", file=sys.stderr)
        print(usage(), file=sys.stderr)
        return 2

    from .engine.generate import Generator
    from .model import Model
    from .sampling.params import SamplingParams
    model = Model.from_folder(opts["model"], opts["dtype"], "cuda:0")
    per_seq = ((min(opts["n_ctx"], model.plan.max_positions) + 63) // 64) * 64
    batch = min(len(prompts), 64)
    if opts.get("max_seqs"):
        batch = max(1, min(batch, opts["max_seqs"]))
    gen = Generator(model, max_tokens=per_seq * batch, max_batch=batch,
                    cuda_graphs=opts["cuda_graph"])
    sampling = SamplingParams(opts["temp"], opts["top_k"], opts["top_p"], opts["repeat_penalty"],
                              opts["frequency_penalty"], opts["presence_penalty"], opts["seed"])
    n_prompt = sum(len(p) for p in prompts)
    print(f"Prompt: {n_prompt} tokens" + (f" in {len(prompts)} sequences" if len(prompts) > 1 else ""))
    room = max(1, per_seq - max(len(p) for p in prompts))
    t0 = time.perf_counter()
    results = gen.generate(prompts, min(opts["n_predict"], room), sampling, opts["stop"] or None)
    total = time.perf_counter() - t0
    st = gen.stats
    print(f"Prefill: {st.prefill_tokens} tokens in {st.prefill_seconds:.2f}s "
          f"({st.prefill_tokens / max(st.prefill_seconds, 1e-9):.1f} tok/s)")
    for r in results:
        print(" ".join(str(t) for t in r.tokens) + f"  [{r.finish_reason}]")
    n_gen = sum(len(r.tokens) for r in results)
    print("\n---")
    print(f"Generated: {n_gen} tokens in {st.decode_seconds:.2f}s "
          f"({st.decode_tokens / max(st.decode_seconds, 1e-9):.1f} tok/s)")
    print(f"Total:     {n_prompt + n_gen} tokens in {total:.2f}s "
          f"({(n_prompt + n_gen) / max(total, 1e-9):.1f} tok/s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
