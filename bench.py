"""Benchmark of the flagship serving step: decoding with the Qwen2.5-7B shape in bfloat16,
random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 from 2,048-token
contexts, timed on the device with CUDA events over K decode steps (model step + greedy
sampling, token ids staying on the device).  ``e2e`` is the same through the Python entry
point (``Generator.generate``): host token ids in, host token ids out, every step.
``prefill`` is one 2,048-token prompt (median of 20); ``roofline`` is the decode step's bytes
(every weight it uses once, plus the cache of the live requests) over its time, against the
measured copy bandwidth; ``points`` are medians of per-step device times of the other
workloads: decoding at batch 1 and 64, the 0.5B shape with 64 ragged prompts, the 14B shape
at 8,192 positions, one sequence at 32,000 positions, each with its fraction of the roofline,
and the host's share of a step where the host could show.  ``points_clocks`` gives the median
SM clock inside each figure's own window.  ``reference_kernels`` times the reference's own
float32 CUDA kernels, compiled unchanged, beside this library's kernels for the same op.

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
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def summary(self, window=None):
        """Summary of the samples; with ``window`` (host times of the timed region's start and
        end) only of those taken inside it, if there are any."""
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        samples = list(self.samples)
        lines = [line for _, line in samples]
        if window is not None:
            inside = [line for t, line in samples if window[0] <= t <= window[1]]
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
    """CUDA-event times of `steps` decode steps at `batch`, after `warmup` untimed ones: the
    mean (all steps between two events, the contract's figure), the median of the per-step
    times (an event after every step), and the kernels launched.  The sequences' caches come
    from a real prefill of `batch` random prompts of `prompt_len` tokens (one number, or a
    length for each row) in one step."""
    from minfer_b200.kernels import api
    plan = engine.model.plan
    slots = [engine.acquire() for _ in range(batch)]
    g = torch.Generator().manual_seed(seed)
    lens = list(prompt_len) if isinstance(prompt_len, (list, tuple)) else [prompt_len] * batch
    prompts = [torch.randint(0, plan.vocab_size, (n,), generator=g).tolist() for n in lens]
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
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    t0 = time.time()
    marks[0].record()
    for i in range(steps):
        tokens = one_step(tokens)
        marks[i + 1].record()
    torch.cuda.synchronize()
    time_decode.window = (t0, time.time())
    ms = marks[0].elapsed_time(marks[steps])
    per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    time_decode.median_ms = statistics.median(per_step)
    launched = api.launches - before
    engine.check_status()
    for s in slots:
        engine.release(s)
    return ms / steps, launched


def time_prefill(engine, torch, ids, reps):
    """Median device time of `reps` whole-prompt steps of `ids` (one warm-up first), in ms."""
    times = []
    t0 = None
    for i in range(reps + 1):
        s = engine.acquire()
        torch.cuda.synchronize()
        if i == 1:
            t0 = time.time()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([s], [ids])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.release(s)
    time_prefill.window = (t0, time.time())
    time_prefill.times = times[1:]
    return statistics.median(times[1:])


CONFIG_05B = dict(CONFIG_7B, vocab_size=151936, hidden_size=896, num_hidden_layers=24,
                  num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864,
                  tie_word_embeddings=True)
CONFIG_14B = dict(CONFIG_7B, hidden_size=5120, num_hidden_layers=48, num_attention_heads=40,
                  num_key_value_heads=8, intermediate_size=13824, rms_norm_eps=1e-5)


def _frac(step_bytes, ms, pk):
    return round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)


def point_05b(torch, K, pk, new_tokens=256):
    """Qwen2.5-0.5B shape, 64 sequences with prompt lengths uniform in [16, 1024], `new_tokens`
    decoded tokens each: the device's time of a step (graph replays fed from the device, an
    event after every step), and the same through Generator.generate (host ids in and out every
    step, the host's clock).  Their difference is what the Python host adds to a step."""
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    cfg = dict(CONFIG_05B)
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(16, 1025, (64,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    gen = Generator(model, max_tokens=64 * 1280, max_batch=64)
    time_decode(gen.engine, torch, K, 64, new_tokens, 3, lens, seed=3)
    ms_dev, window = time_decode.median_ms, time_decode.window
    gen.generate(prompts, 8, SamplingParams.greedy(), stop_token_ids=[])      # warm-up
    gen.stats.__init__()
    gen.generate(prompts, new_tokens, SamplingParams.greedy(), stop_token_ids=[])
    st = gen.stats
    ms_host = st.decode_seconds / max(st.steps - 1, 1) * 1e3
    step_bytes = decode_bytes(model, 64, sum(lens) / 64 + new_tokens / 2)
    out = {"decode_05b_ragged64_ms": round(ms_dev, 4),
           "decode_05b_ragged64_frac": _frac(step_bytes, ms_dev, pk),
           "decode_05b_ragged64_e2e_ms": round(ms_host, 4),
           "host_share_05b_ragged64": round(max(0.0, ms_host - ms_dev) / ms_host, 4)}
    return out, {"decode_05b_ragged64": (window, ms_dev)}


def point_14b(torch, K, pk, steps=96):
    """Qwen2.5-14B shape: prefill of one 8,192-token prompt, decode at batch 8 from 8,192-token
    contexts."""
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    cfg = dict(CONFIG_14B)
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
    gen = Generator(model, max_tokens=8 * (8192 + 256), max_batch=8)
    engine = gen.engine
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg["vocab_size"], (8192,), generator=g).tolist()
    ms_prefill = time_prefill(engine, torch, ids, 5)
    w_prefill = time_prefill.window
    time_decode(engine, torch, K, 8, steps, 3, 8192)
    ms_step = time_decode.median_ms
    step_bytes = decode_bytes(model, 8, 8192 + 3 + steps / 2)
    out = {"prefill_14b_8192_ms": round(ms_prefill, 2),
           "prefill_14b_8192_frac": round(prefill_flops(cfg, 8192) / (ms_prefill * 1e-3) /
                                          (pk["bf16_tflops"] * 1e12), 4),
           "decode_14b_b8_ctx8192_ms": round(ms_step, 4),
           "decode_14b_b8_ctx8192_frac": _frac(step_bytes, ms_step, pk)}
    return out, {"prefill_14b_8192": (w_prefill, ms_prefill),
                 "decode_14b_b8_ctx8192": (time_decode.window, ms_step)}


def point_long(engine, torch, K, pk, cfg, context=32000, steps=32):
    """The headline shape with one sequence at 32,000 positions: its prefill, then decoding."""
    g = torch.Generator().manual_seed(6)
    ids = torch.randint(0, cfg["vocab_size"], (context,), generator=g).tolist()
    ms_prefill = time_prefill(engine, torch, ids, 2)
    w_prefill = time_prefill.window
    time_decode(engine, torch, K, 1, steps, 3, context, seed=6)
    ms_step = time_decode.median_ms
    step_bytes = decode_bytes(engine.model, 1, context + 3 + steps / 2)
    out = {"prefill_7b_32000_ms": round(ms_prefill, 2),
           "prefill_7b_32000_frac": round(prefill_flops(cfg, context) / (ms_prefill * 1e-3) /
                                          (pk["bf16_tflops"] * 1e12), 4),
           "decode_7b_b1_ctx32000_ms": round(ms_step, 4),
           "decode_7b_b1_ctx32000_frac": _frac(step_bytes, ms_step, pk)}
    return out, {"prefill_7b_32000": (w_prefill, ms_prefill),
                 "decode_7b_b1_ctx32000": (time_decode.window, ms_step)}


REF_KERNELS = os.path.join(ROOT, "baseline", "_ref", "libref_kernels.so")
# the reference's checkout, if it sits beside this repository (or where MINFER_REFERENCE_DIR says)
REF_SOURCE = os.path.join(os.environ.get("MINFER_REFERENCE_DIR",
                                         os.path.join(os.path.dirname(ROOT), "reference")),
                          "src", "cuda_kernels.cu")


def reference_kernel_times(torch, K):
    """The reference's own float32 CUDA kernels (src/cuda_kernels.cu of yusiwen/minfer, compiled
    as they are into baseline/_ref/, driven through its stock launchers at its stock launch
    shapes) timed beside this library's kernels for the same op and sizes: median of 10 runs,
    CUDA events, L2 flushed between runs.  A kernel-level comparison, not a model-level one:
    the reference's model path cannot be built here."""
    import ctypes
    import math
    if not os.path.exists(REF_KERNELS) and os.path.exists(REF_SOURCE):
        os.makedirs(os.path.dirname(REF_KERNELS), exist_ok=True)
        subprocess.run(["nvcc", "-shared", "-Xcompiler", "-fPIC", "-gencode",
                        "arch=compute_100a,code=sm_100a", "-O2", "-o", REF_KERNELS, REF_SOURCE],
                       check=False, capture_output=True)
    if not os.path.exists(REF_KERNELS):
        return {"unavailable": "baseline/_ref/libref_kernels.so is not there and the reference's "
                               "source is not on this machine"}
    lib = ctypes.CDLL(REF_KERNELS)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.launch_rms_norm_f32.argtypes = [vp, vp, vp, ci, cf, ci, vp]
    lib.launch_rope_f32.argtypes = [vp, ci, ci, ci, cf, cf, vp, vp]
    lib.launch_swiglu_f32.argtypes = [vp, vp, vp, ci, vp]
    lib.launch_store_kv_f32.argtypes = [vp, vp, ci, ci, vp, vp]
    lib.launch_gqa_attn_f32.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, cf, ci, vp]
    dev = "cuda:0"
    stream = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def med_us(fn, reps=10):
        fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        return round(statistics.median(times), 1)

    nh, nk, hd, ne, nf, T, ctx = 28, 4, 128, 3584, 18944, 2048, 2048
    scale = 1.0 / math.sqrt(hd)
    g = torch.Generator(device=dev).manual_seed(1)
    out = {}
    st = torch.zeros(1, dtype=torch.int32, device=dev)

    def rnd(*shape):
        return torch.randn(*shape, generator=g, device=dev)

    # ---- attention, one new token over 2,048 cached positions --------------------------------
    kc, vc = rnd(ctx, nk * hd), rnd(ctx, nk * hd)
    q1, o1 = rnd(1, nh, hd), torch.empty(1, nh, hd, device=dev)
    pos1 = torch.tensor([ctx - 1], dtype=torch.int32, device=dev)
    out["attn_decode_ctx2048_ref_us"] = med_us(lambda: lib.launch_gqa_attn_f32(
        q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), o1.data_ptr(), pos1.data_ptr(), nh, nk, hd,
        scale, 1, stream))
    pages = ctx // 64
    table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
    row0 = torch.zeros(1, dtype=torch.int32, device=dev)
    for name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        kp = kc.view(pages, 64, nk, hd).transpose(1, 2).contiguous().to(dt)
        vp_ = vc.view(pages, 64, nk, hd).transpose(1, 2).contiguous().to(dt)
        qd = q1.to(dt)
        od = torch.empty(1, nh * hd, dtype=dt, device=dev)
        n_chunks = ctx // 256
        part = torch.empty(nh * n_chunks * (hd + 2), device=dev)
        out[f"attn_decode_ctx2048_ours_{name}_us"] = med_us(lambda: K.attention_paged(
            qd, kp, vp_, row0, pos1, table, pages, 0, od, part, nh, nk, hd, 0, 256, n_chunks, scale,
            status=st, old_keys_final=True))
    # ---- attention, a whole prompt of 2,048 tokens --------------------------------------------
    qT, kT, vT = rnd(T, nh, hd), rnd(T, nk, hd), rnd(T, nk, hd)
    oT = torch.empty(T, nh, hd, device=dev)
    posT = torch.arange(T, dtype=torch.int32, device=dev)
    kT2, vT2 = kT.reshape(T, nk * hd), vT.reshape(T, nk * hd)
    out["attn_prefill_2048_ref_us"] = med_us(lambda: lib.launch_gqa_attn_f32(
        qT.data_ptr(), kT2.data_ptr(), vT2.data_ptr(), oT.data_ptr(), posT.data_ptr(), nh, nk, hd,
        scale, T, stream), reps=3)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    rowT = torch.zeros(T, dtype=torch.int32, device=dev)
    of = torch.empty(T, nh * hd, device=dev)
    out["attn_prefill_2048_ours_f32_us"] = med_us(lambda: K.attention_packed(
        qT, kT, vT, rowT, posT, cu, of, nh, nk, hd, 0, scale), reps=3)
    qb, kb, vb = qT.bfloat16(), kT.bfloat16(), vT.bfloat16()
    ob = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=dev)
    out["attn_prefill_2048_ours_bf16_us"] = med_us(lambda: K.attention_prefill_tc(
        qb, kb, vb, cu, ob, 1, T, nh, nk, hd, 0, scale, st))
    # ---- RMSNorm of 2,048 rows of 3,584 ----------------------------------------------------------
    x, w = rnd(T, ne), rnd(ne)
    y = torch.empty(T, ne, device=dev)
    out["rmsnorm_2048x3584_ref_us"] = med_us(lambda: lib.launch_rms_norm_f32(
        x.data_ptr(), w.data_ptr(), y.data_ptr(), ne, 1e-6, T, stream))
    out["rmsnorm_2048x3584_ours_f32_us"] = med_us(lambda: K.rmsnorm(x, w, 1e-6, y))
    yb = torch.empty(T, ne, dtype=torch.bfloat16, device=dev)
    out["rmsnorm_2048x3584_ours_bf16_us"] = med_us(lambda: K.rmsnorm(x, w, 1e-6, yb))
    # ---- rotation of q and k plus the cache write, 2,048 tokens ----------------------------------
    qkv = rnd(T, (nh + 2 * nk) * hd)
    qr, kr = rnd(T, nh, hd), rnd(T, nk, hd)
    vr = rnd(T, nk * hd)
    kcache, vcache = torch.zeros(T, nk * hd, device=dev), torch.zeros(T, nk * hd, device=dev)

    def ref_rope_store():
        lib.launch_rope_f32(qr.data_ptr(), nh, hd, T, 1e6, 1.0, posT.data_ptr(), stream)
        lib.launch_rope_f32(kr.data_ptr(), nk, hd, T, 1e6, 1.0, posT.data_ptr(), stream)
        lib.launch_store_kv_f32(kr.data_ptr(), kcache.data_ptr(), nk * hd, T, posT.data_ptr(), stream)
        lib.launch_store_kv_f32(vr.data_ptr(), vcache.data_ptr(), nk * hd, T, posT.data_ptr(), stream)
    out["rope_store_2048_ref_us"] = med_us(ref_rope_store)
    inv = (1e6 ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd)).to(dev)
    seq_end = torch.tensor([T], dtype=torch.int32, device=dev)
    tableT = torch.arange(T // 64, dtype=torch.int32, device=dev).reshape(1, T // 64)
    for name, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        qo = torch.empty(T, nh, hd, dtype=dt, device=dev)
        ko, vo = torch.empty(T, nk, hd, dtype=dt, device=dev), torch.empty(T, nk, hd, dtype=dt, device=dev)
        kpg = torch.zeros(T // 64, nk, 64, hd, dtype=dt, device=dev)
        vpg = torch.zeros_like(kpg)
        out[f"rope_store_2048_ours_{name}_us"] = med_us(lambda: K.rope_kvstore(
            qkv, posT, rowT, seq_end, inv, qo, ko, vo, kpg, vpg, tableT, T // 64, 0, nh, nk, hd, hd, 0, st))
    # ---- SwiGLU, 2,048 rows of 18,944 -------------------------------------------------------------
    gate, up = rnd(T, nf), rnd(T, nf)
    dst = torch.empty(T, nf, device=dev)
    out["swiglu_2048x18944_ref_us"] = med_us(lambda: lib.launch_swiglu_f32(
        gate.data_ptr(), up.data_ptr(), dst.data_ptr(), T * nf, stream))
    gu = torch.cat([gate, up], dim=1).contiguous()
    out["swiglu_2048x18944_ours_f32_us"] = med_us(lambda: K.swiglu(gu, dst))
    gub, dstb = gu.bfloat16(), torch.empty(T, nf, dtype=torch.bfloat16, device=dev)
    out["swiglu_2048x18944_ours_bf16_us"] = med_us(lambda: K.swiglu(gub, dstb))
    torch.cuda.synchronize()
    if int(st.item()) != 0:
        out["status"] = int(st.item())
    # reference time over ours, per op: float32 against float32, and against the bfloat16 kernel
    # that the product path runs
    for op in ("attn_decode_ctx2048", "attn_prefill_2048", "rmsnorm_2048x3584", "rope_store_2048",
               "swiglu_2048x18944"):
        for name in ("f32", "bf16"):
            out[f"{op}_ref_over_ours_{name}"] = round(out[f"{op}_ref_us"] / out[f"{op}_ours_{name}_us"], 2)
    out["note"] = ("the reference's float32 kernels, unchanged, through its own launchers; in the "
                   "bfloat16 engine SwiGLU runs inside the product's epilogue, not as this kernel")
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--skip-points", action="store_true",
                    help="only the headline figure and its end-to-end twin")
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

    import torch
    from minfer_b200.engine.generate import Generator
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
    clock_summary = clocks.summary(time_decode.window)
    value = BATCH * 1000.0 / ms_step

    # roofline of the decode step, mean context over the timed steps
    ctx_tokens = PROMPT + warmup + steps / 2
    step_bytes = decode_bytes(model, BATCH, ctx_tokens)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_kind}

    # end to end through the Python entry point: host ids in, host ids out every step
    def end_to_end(batch, new_tokens):
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg["vocab_size"], (PROMPT,), generator=g).tolist()
                   for _ in range(batch)]
        gen.stats.__init__()
        engine.h2d_bytes = engine.d2h_bytes = 0
        gen.generate(prompts, new_tokens, SamplingParams.greedy(), stop_token_ids=[])
        return gen.stats

    # long enough that the clock dip which follows the prompt's burst (about 30 steps: 3.9 ms,
    # then 3.5 ms, then the steady 3.3 ms a step) does not dominate
    st = end_to_end(BATCH, max(steps, 128) + 1)
    e2e_value = st.decode_tokens / max(st.decode_seconds, 1e-9)
    prompt_bytes = 4 * BATCH * PROMPT
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int((engine.h2d_bytes - prompt_bytes) / max(st.steps, 1)),
           "d2h_bytes_per_step": int(engine.d2h_bytes / max(st.steps, 1)), "steps": st.steps - 1,
           "device_value": round(st.decode_tokens / max(st.decode_device_seconds, 1e-9), 1)}

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
        "ms_per_step_median": round(time_decode.median_ms, 4),
    }

    if not args.skip_points:
        points, windows = {}, {}
        # prefill of one 2,048-token prompt: median of 20
        g = torch.Generator().manual_seed(2)
        ids = torch.randint(0, cfg["vocab_size"], (PROMPT,), generator=g).tolist()
        ms_prefill = time_prefill(engine, torch, ids, 20)
        windows["prefill"] = (time_prefill.window, ms_prefill)
        flops = prefill_flops(cfg, PROMPT)
        out["prefill"] = {"value": round(PROMPT * 1000.0 / ms_prefill, 1), "tokens": PROMPT,
                          "ms": round(ms_prefill, 3),
                          "frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "of": pk_kind, "runs": 20, "statistic": "median",
                          # the first timed prompt runs before the power cap pulls the clock down,
                          # as one prompt that arrives alone does: its time against the burst peak
                          "ms_first": round(time_prefill.times[0], 3),
                          "frac_first": round(flops / (time_prefill.times[0] * 1e-3) /
                                              (pk["bf16_tflops"] * 1e12), 4),
                          # twenty prompts back to back run under the power cap, as the
                          # library's seconds-long product does: the fraction of that peak too
                          "frac_sustained": round(flops / (ms_prefill * 1e-3) /
                                                  (pk["bf16_tflops_sustained"] * 1e12), 4)}
        n_point = max(64, min(steps, 128))
        for b in (1, 64):
            time_decode(engine, torch, K, b, n_point, 3, PROMPT)
            ms_b = time_decode.median_ms
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
            points[f"decode_b{b}_frac"] = _frac(decode_bytes(model, b, PROMPT + 3 + n_point / 2), ms_b, pk)
            windows[f"decode_b{b}"] = (time_decode.window, ms_b)
        # the host's share at batch 64: the same loop the user calls, device marks beside the host's clock
        st64 = end_to_end(64, 129)
        host_ms = st64.decode_seconds / max(st64.steps - 1, 1) * 1e3
        dev_ms = windows["decode_b64"][1]
        points["decode_b64_e2e"] = round(64e3 / host_ms, 1)
        points["host_share_7b_b64"] = round(max(0.0, host_ms - dev_ms) / host_ms, 4)
        more, win = point_long(engine, torch, K, pk, cfg)
        points.update(more)
        windows.update(win)
        out["reference_kernels"] = reference_kernel_times(torch, K)
        # the other shapes need the memory: the headline model goes first
        del gen, engine, model
        torch.cuda.empty_cache()
        for fn, fn_args in ((point_05b, (torch, K, pk)), (point_14b, (torch, K, pk))):
            more, win = fn(*fn_args)
            points.update(more)
            windows.update(win)
            torch.cuda.empty_cache()
        out["points"] = points
        out["points_note"] = ("medians of per-step device times (CUDA events); *_frac is the step's "
                              "bytes or flops over its time over the measured peak")
        pc = {}
        for name, (window, ms) in windows.items():
            c = clocks.summary(window)
            pc[name] = {"sm_mhz": c["sm_mhz"], "reasons": c["reasons"], "samples": c["samples"],
                        "ms_x_mhz": round(ms * c["sm_mhz"], 1) if c["sm_mhz"] else None}
        out["points_clocks"] = pc
    clocks.stop()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
