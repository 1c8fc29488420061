"""Benchmark of the flagship serving step: decoding with the Qwen2.5-7B shape in bfloat16,
random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 from 2,048-token
contexts, timed on the device with CUDA events over K decode steps (model step + greedy
sampling, token ids staying on the device).  ``e2e`` is the same through the Python entry
point (``Generator.generate``): host token ids in, host token ids out, every step.
``prefill`` is one 2,048-token prompt; ``roofline`` is the decode step's bytes (every
weight it uses once, plus the cache of the live requests) over its time, against the
measured copy bandwidth; ``points`` are decoding at batch 1 and 64.

The reference (yusiwen/minfer) is a Rust program; there is no Rust toolchain here, so
``--impl reference`` prints its ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the headline configuration (Qwen2.5-7B shape)
CONFIG_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 152064, "hidden_size": 3584, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "use_sliding_window": False, "max_position_embeddings": 32768,
}
CONTEXT = 4096          # positions per sequence the cache is sized for
PROMPT = 2048           # tokens each sequence holds when decoding starts
BATCH = 8
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            found = 0

            def look(node):                       # the keys may sit at the top or one level down
                nonlocal found
                if isinstance(node, dict):
                    for k, v in node.items():
                        if k in out and isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
                            out[k] = float(v)
                            found += 1
                        elif k in out and isinstance(v, dict) and isinstance(v.get("value"), (int, float)):
                            out[k] = float(v["value"])
                            found += 1
                        else:
                            look(v)
            look(d)
            if found:
                return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, window=None):
        """Summary of the samples; with ``window`` (host times of the timed region's start and
        end) only of those taken inside it, if there are any."""
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = [line for _, line in self.samples]
        if window is not None:
            inside = [line for t, line in self.samples if window[0] <= t <= window[1]]
            if inside:
                lines = inside
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_bytes(model, batch, context_tokens):
    """Bytes one decode step has to read: every weight it uses once (the embedding table is
    only touched at `batch` rows) and the cache of the live requests."""
    plan = model.plan
    weights = model.parameter_bytes()
    esz = 2 if str(model.dtype).endswith("bfloat16") else 4
    if model.head.weight.data_ptr() != model.embedding.data_ptr():
        weights -= model.embedding.numel() * model.embedding.element_size()
    kv = 0
    for call in plan.schedule:
        req = model.blocks[call.layer].mixer.cache_request()
        if req is not None and call.writes_cache:
            kv += 2 * req.n_kv_heads * req.head_dim * esz * context_tokens
    return weights + batch * kv


def prefill_flops(cfg, tokens):
    """Matrix-product flops of one whole prompt (head on the last row only) plus causal
    attention."""
    ne, nh, nk = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, nf, L, V = ne // nh, cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    per_token = 2 * ne * (nh + 2 * nk) * hd + 2 * ne * nh * hd + 2 * ne * 2 * nf + 2 * nf * ne
    linear = L * per_token * tokens + 2 * ne * V
    attention = L * nh * 4 * hd * tokens * (tokens + 1) / 2
    return linear + attention


SETTLE_S = 1.0


def time_decode(engine, torch, K, batch, steps, warmup, prompt_len, seed=0):
    """CUDA-event time of `steps` decode steps at `batch`, after `warmup` untimed ones.  The
    sequences' caches come from a real prefill of `batch` random prompts of `prompt_len`
    tokens in one step."""
    from minfer_b200.kernels import api
    plan = engine.model.plan
    slots = [engine.acquire() for _ in range(batch)]
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, plan.vocab_size, (prompt_len,), generator=g).tolist()
               for _ in range(batch)]
    logits = engine.step(slots, prompts)
    out = torch.empty(batch, dtype=torch.int32, device="cuda")
    K.sample(logits, out, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
             frequency_penalty=0.0, presence_penalty=0.0, seed=0)
    tokens = out.clone()
    del logits, prompts
    # the prefill that built the caches is a burst at over 1 PFLOP/s; for some twenty steps
    # after it the GPU's power management holds the clocks down (3.9 ms, then 3.5, then the
    # steady 3.26 ms a step).  That belongs to the prefill, not to a decode step: let it pass.
    torch.cuda.synchronize()
    time.sleep(SETTLE_S)

    def one_step(tok):
        logits = engine.decode_on_device(slots, tok)
        K.sample(logits, out, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                 frequency_penalty=0.0, presence_penalty=0.0, seed=0)
        return out

    for _ in range(warmup):
        tokens = one_step(tokens).clone()
    torch.cuda.synchronize()
    before = api.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    start.record()
    for _ in range(steps):
        tokens = one_step(tokens)
    end.record()
    torch.cuda.synchronize()
    time_decode.window = (t0, time.time())
    ms = start.elapsed_time(end)
    launched = api.launches - before
    engine.check_status()
    for s in slots:
        engine.release(s)
    return ms / steps, launched


CONFIG_05B = dict(CONFIG_7B, vocab_size=151936, hidden_size=896, num_hidden_layers=24,
                  num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864,
                  tie_word_embeddings=True)
CONFIG_14B = dict(CONFIG_7B, hidden_size=5120, num_hidden_layers=48, num_attention_heads=40,
                  num_key_value_heads=8, intermediate_size=13824, rms_norm_eps=1e-5)


def other_workload(name: str, steps: int) -> int:
    """The two side workloads of the baseline: not the contract line, one JSON line of their own.
    0.5b: 64 sequences with prompt lengths uniform in [16, 1024], 256 decoded tokens each,
          through Generator.generate (host ids in and out).
    14b:  prefill of one 8,192-token prompt, then decode at batch 8 from 8,192-token contexts."""
    import torch
    from minfer_b200.engine.generate import Generator
    from minfer_b200.kernels import api as K
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    pk, pk_kind = peaks()
    torch.cuda.set_device(0)
    if name == "0.5b":
        cfg = dict(CONFIG_05B)
        model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
        g = torch.Generator().manual_seed(3)
        lens = torch.randint(16, 1025, (64,), generator=g).tolist()
        prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
        gen = Generator(model, max_tokens=64 * 1280, max_batch=64)
        gen.generate(prompts, 8, SamplingParams.greedy(), stop_token_ids=[])      # warm-up
        gen.stats.__init__()
        t0 = time.perf_counter()
        out = gen.generate(prompts, 256, SamplingParams.greedy(), stop_token_ids=[])
        wall = time.perf_counter() - t0
        st = gen.stats
        ms_step = st.decode_seconds / max(st.steps - 1, 1) * 1e3
        mean_ctx = sum(lens) / 64 + 128
        step_bytes = decode_bytes(model, 64, mean_ctx)
        print(json.dumps({
            "workload": "Qwen2.5-0.5B shape, 64 ragged prompts [16,1024], 256 new tokens each",
            "decode_tokens_per_s": round(st.decode_tokens / st.decode_seconds, 1),
            "ms_per_step": round(ms_step, 3), "prefill_tokens": st.prefill_tokens,
            "prefill_tokens_per_s": round(st.prefill_tokens / st.prefill_seconds, 1),
            "generated": sum(len(r.tokens) for r in out), "wall_s": round(wall, 3),
            "roofline_frac": round(step_bytes / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
            "of": pk_kind}))
        return 0
    cfg = dict(CONFIG_14B)
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
    steps = min(steps, 240)
    gen = Generator(model, max_tokens=8 * (8192 + 256), max_batch=8)
    engine = gen.engine
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg["vocab_size"], (8192,), generator=g).tolist()
    times = []
    for _ in range(3):
        s = engine.acquire()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([s], [ids])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.release(s)
    ms_prefill = min(times[1:])
    ms_step, _ = time_decode(engine, torch, K, 8, steps, 3, 8192)
    step_bytes = decode_bytes(model, 8, 8192 + 3 + steps / 2)
    print(json.dumps({
        "workload": "Qwen2.5-14B shape, prefill 1 x 8192, decode batch 8 at 8192-token contexts",
        "prefill_ms": round(ms_prefill, 2), "prefill_tokens_per_s": round(8192e3 / ms_prefill, 1),
        "prefill_frac": round(prefill_flops(cfg, 8192) / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
        "decode_tokens_per_s": round(8e3 / ms_step, 1), "ms_per_step": round(ms_step, 3),
        "roofline_frac": round(step_bytes / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"], 4), "of": pk_kind}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="7b", choices=["7b", "0.5b", "14b"],
                    help="7b: the contract line; 0.5b and 14b: the baseline's side workloads")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--skip-points", action="store_true", help="no batch-1/64 and prefill extras")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "yusiwen/minfer is a Rust program that loads GGUF files; there is no "
                          "Rust toolchain (cargo/rustc) in this image, pip cannot build it, and "
                          "its CUDA forward path is dead code at this commit"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload != "7b":
        return other_workload(args.workload, max(1, args.steps))

    import torch
    from minfer_b200.engine.generate import Generator
    from minfer_b200.engine.step import Engine
    from minfer_b200.kernels import api as K
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams

    warmup = max(3, args.warmup)
    steps = max(1, min(args.steps, CONTEXT - PROMPT - warmup - 2))     # the context is 4,096
    cfg = dict(CONFIG_7B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk, pk_kind = peaks()

    torch.cuda.set_device(0)
    t_build = time.time()
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.time() - t_build:.1f} s, "
          f"{model.parameter_bytes() / 1e9:.2f} GB of weights", file=sys.stderr, flush=True)

    max_batch = BATCH if args.skip_points else 64
    gen = Generator(model, max_tokens=max_batch * CONTEXT, max_batch=max_batch)
    engine = gen.engine
    clocks = ClockSampler()
    clocks.start()
    ms_step, launched = time_decode(engine, torch, K, BATCH, steps, warmup, PROMPT)
    clock_summary = clocks.stop(time_decode.window)
    value = BATCH * 1000.0 / ms_step

    # roofline of the decode step, mean context over the timed steps
    ctx_tokens = PROMPT + warmup + steps / 2
    step_bytes = decode_bytes(model, BATCH, ctx_tokens)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_kind}

    # end to end through the Python entry point: host ids in, host ids out every step
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg["vocab_size"], (PROMPT,), generator=g).tolist()
               for _ in range(BATCH)]
    # long enough that the clock dip which follows the prompt's burst (about 30 steps: 3.9 ms,
    # then 3.5 ms, then the steady 3.3 ms a step) does not dominate
    e2e_new = max(steps, 128) + 1
    gen.stats.__init__()
    engine.h2d_bytes = engine.d2h_bytes = 0
    gen.generate(prompts, e2e_new, SamplingParams.greedy(), stop_token_ids=[])
    st = gen.stats
    e2e_value = st.decode_tokens / max(st.decode_seconds, 1e-9)
    prompt_bytes = 4 * BATCH * PROMPT
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int((engine.h2d_bytes - prompt_bytes) / max(st.steps, 1)),
           "d2h_bytes_per_step": int(engine.d2h_bytes / max(st.steps, 1)), "steps": st.steps - 1}

    out = {
        "metric": "decode tokens/s, Qwen2.5-7B shape, batch 8, 2048-token contexts",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": "Qwen2.5-7B shape, random weights", "global_batch": BATCH,
            "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single GPU",
            "layers": cfg["num_hidden_layers"], "layers_of_config": full_layers,
            "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"],
            "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"],
            "l2": "inputs larger than L2 (weights read every step)",
            "cache": "decode starts from a real prefill of batch x 2048 random tokens",
            "settle_s": SETTLE_S,
        },
        "clocks": clock_summary, "e2e": e2e, "gpu_launches": launched, "roofline": roofline,
    }

    if not args.skip_points:
        # prefill of one 2,048-token prompt
        ids = torch.randint(0, cfg["vocab_size"], (PROMPT,), generator=g).tolist()
        times = []
        for i in range(3):
            s = engine.acquire()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            engine.step([s], [ids])
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
            engine.release(s)
        ms_prefill = min(times[1:])
        flops = prefill_flops(cfg, PROMPT)
        out["prefill"] = {"value": round(PROMPT * 1000.0 / ms_prefill, 1), "tokens": PROMPT,
                          "ms": round(ms_prefill, 3),
                          "frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "of": pk_kind}
        points = {}
        for b in (1, 64):
            ms_b, _ = time_decode(engine, torch, K, b, max(4, steps // 2), 3, PROMPT)
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
