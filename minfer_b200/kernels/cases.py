"""Small, named workloads of single kernels and of short model steps, for timing and for
profilers:

    python -m minfer_b200.kernels.cases LIST
    python -m minfer_b200.kernels.cases <case> [--reps N]

Each case builds inputs larger than L2 but at most a few GB, runs its kernel a few times
and prints the mean CUDA-event time with the bytes or flops it stands for.  The sizes are
those of the Qwen2.5-7B shape (hidden 3584, 28 heads / 4 KV heads of 128, intermediate
18944).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import api as K

NE, NH, NK, HD, NF, VOCAB = 3584, 28, 4, 128, 18944, 152064


def _time(fn, reps, graph=True):
    """Mean device time of one call in microseconds.  With ``graph`` the calls are captured
    into one CUDA graph and replayed, so that host launch overhead is not in the number."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        g.replay()
        torch.cuda.synchronize()
        a.record()
        g.replay()
        b.record()
    else:
        a.record()
        for _ in range(reps):
            fn()
        b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3


def _gemm(m, n, k, epi, reps):
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    n_w = max(2, min(8, int(1.2e9 // (n * k * 2))))         # rotate weights: no L2 reuse
    ws = [(torch.randn(n, k, device="cuda") * 0.05).bfloat16() for _ in range(n_w)]
    out = (torch.zeros(m, n // 2, dtype=torch.bfloat16, device="cuda") if epi == K.EPI_SWIGLU
           else torch.zeros(m, n, device="cuda"))
    state = {"i": 0}

    def run():
        K.gemm_tc(x, ws[state["i"] % n_w], None, out, epi, st)
        state["i"] += 1
    us = _time(run, reps)
    print(f"gemm_tc m={m} n={n} k={k} epi={epi} plan={K.gemm_tc_plan(m, n, k, epi)}: {us:.1f} us, "
          f"{2.0 * m * n * k / us / 1e6:.1f} TFLOP/s, {n * k * 2 / us / 1e3:.1f} GB/s of weights")


def gemm_decode(reps):
    """The gate|up projection with fused SwiGLU for 8 tokens: streams 271.6 MB of weights."""
    _gemm(8, 2 * NF, NE, K.EPI_SWIGLU, reps)


def gemm_decode_split(reps):
    """The down projection for 8 tokens (split along K, partial sums reduced)."""
    _gemm(8, NE, NF, K.EPI_ACCUM, reps)


def gemm_decode_m64(reps):
    """The gate|up projection with fused SwiGLU for 64 tokens."""
    _gemm(64, 2 * NF, NE, K.EPI_SWIGLU, reps)


def gemm_decode_split_m64(reps):
    """The down projection for 64 tokens (split along K, partial sums reduced)."""
    _gemm(64, NE, NF, K.EPI_ACCUM, reps)


def gemm_prefill(reps):
    """The gate|up projection with fused SwiGLU for 2,048 tokens: 556 GFLOP."""
    _gemm(2048, 2 * NF, NE, K.EPI_SWIGLU, reps)


def gemm_prefill_down(reps):
    """The down projection for 2,048 tokens, accumulated into the residual: 278 GFLOP."""
    _gemm(2048, NE, NF, K.EPI_ACCUM, reps)


def _gemm_cluster(m, n, k, reps):
    """A product that completes the residual and prepares the next norm (K split over a
    cluster), then the product that applies the norm's 1/rms, as a decode step chains them."""
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    n_w = max(2, min(8, int(1.2e9 // (n * k * 2))))
    ws = [(torch.randn(n, k, device="cuda") * 0.05).bfloat16() for _ in range(n_w)]
    h = torch.zeros(m, n, device="cuda")
    g = torch.ones(n, device="cuda")
    parts = K.gemm_tc_prep_parts(m, n, k)
    xp = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ssq = torch.empty(max(parts, 1), m, device="cuda")
    state = {"i": 0}

    def run():
        K.gemm_tc_fused(x, ws[state["i"] % n_w], None, h, K.EPI_ACCUM, st, prep_x=xp, prep_weight=g,
                        prep_ssq=ssq)
        state["i"] += 1
    us = _time(run, reps)
    print(f"gemm_tc cluster m={m} n={n} k={k} parts={parts}: {us:.1f} us, "
          f"{n * k * 2 / us / 1e3:.1f} GB/s of weights")


def gemm_decode_cluster(reps):
    """The down projection for 8 tokens, K split over clusters of 8 CTAs that add their tiles
    through distributed shared memory, residual and next norm's input in the epilogue."""
    _gemm_cluster(8, NE, NF, reps)


def gemm_decode_cluster_o(reps):
    """The output projection for 8 tokens in the same form (25.7 MB of weights)."""
    _gemm_cluster(8, NE, NE, reps)


def gemm_decode_cluster_m64(reps):
    """The down projection for 64 tokens in the same form."""
    _gemm_cluster(64, NE, NF, reps)


def attention_portion(reps, old=2048, new=2048, heads=NH, kv=NK):
    """Attention of a 2,048-token portion that goes on from 2,048 cached positions, on tcgen05
    over the cache's pages (key tiles of two pages by TMA): 90 GFLOP."""
    end = old + new
    pages = (end + 63) // 64
    kc = torch.randn(pages, kv, 64, HD, device="cuda").bfloat16()
    vc = torch.randn(pages, kv, 64, HD, device="cuda").bfloat16()
    table = torch.randperm(pages, device="cuda").to(torch.int32).reshape(1, pages)
    q = torch.randn(new, heads, HD, device="cuda").bfloat16()
    cu = torch.tensor([0, new], dtype=torch.int32, device="cuda")
    seq_end = torch.tensor([end], dtype=torch.int32, device="cuda")
    out = torch.empty(new, heads * HD, dtype=torch.bfloat16, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    us = _time(lambda: K.attention_prefill_tc_paged(q, kc, vc, cu, seq_end, table, pages, 0, out, 1, new,
                                                    heads, kv, HD, 0, 1 / math.sqrt(HD), st), reps)
    flops = heads * 4 * HD * (new * old + new * (new + 1) / 2)
    print(f"attention of a portion (tcgen05, paged) old={old} new={new} heads={heads}: {us:.1f} us, "
          f"{flops / us / 1e6:.1f} TFLOP/s")


def attention_portion_512_on_8k(reps):
    """A 512-token portion onto 8,192 cached positions, 40 heads / 8 KV heads (the 14B shape)."""
    attention_portion(reps, old=8192, new=512, heads=40, kv=8)


def attention_decode(reps, batch=64, ctx=2048):
    """Decode attention of 64 sequences at 2,048 cached positions: reads 268 MB of K and V."""
    pos = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    rows = torch.arange(batch, dtype=torch.int32, device="cuda")
    q = torch.randn(batch, NH, HD, device="cuda").bfloat16()
    pages_per = (ctx + 64) // 64
    n_pages = batch * pages_per
    kc = torch.randn(n_pages, NK, 64, HD, device="cuda").bfloat16()
    vc = torch.randn(n_pages, NK, 64, HD, device="cuda").bfloat16()
    table = torch.arange(n_pages, dtype=torch.int32, device="cuda").reshape(batch, pages_per)
    out = torch.empty(batch, NH * HD, dtype=torch.bfloat16, device="cuda")
    from ..parts.attention import decode_chunks
    chunk, n_chunks = decode_chunks(batch * NK, ctx + 1)          # as the attention part cuts them
    partial = torch.empty(batch * NH * n_chunks * (HD + 2), device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    us = _time(lambda: K.attention_paged(q, kc, vc, rows, pos, table, pages_per, 0, out, partial,
                                         NH, NK, HD, 0, chunk, n_chunks, 1 / math.sqrt(HD),
                                         status=st, old_keys_final=True), reps)
    nbytes = batch * (ctx + 1) * NK * HD * 2 * 2
    print(f"attention decode batch={batch} ctx={ctx}, {n_chunks} chunks of {chunk} keys: {us:.1f} us "
          f"(kernel + merge), {nbytes / us / 1e3:.1f} GB/s of cache")


def attention_decode_b8(reps):
    """Decode attention of 8 sequences at 2,048 cached positions (latency-bound)."""
    attention_decode(reps, batch=8)


def attention_decode_long(reps):
    """Decode attention of 8 sequences at 8,192 cached positions: reads 537 MB of K and V."""
    attention_decode(reps, batch=8, ctx=8192)


def attention_prefill(reps, tokens=2048):
    """Causal attention of one 2,048-token prompt, 28 heads: 30 GFLOP."""
    q = torch.randn(tokens, NH, HD, device="cuda").bfloat16()
    k = torch.randn(tokens, NK, HD, device="cuda").bfloat16()
    v = torch.randn(tokens, NK, HD, device="cuda").bfloat16()
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    out = torch.empty(tokens, NH * HD, dtype=torch.bfloat16, device="cuda")
    us = _time(lambda: K.attention_prefill(q, k, v, cu, out, 1, tokens, NH, NK, HD, 0,
                                           1 / math.sqrt(HD)), reps)
    flops = NH * 4 * HD * tokens * (tokens + 1) / 2
    print(f"attention prefill tokens={tokens}: {us:.1f} us, {flops / us / 1e6:.1f} TFLOP/s (causal)")


def attention_prefill_tc(reps, tokens=2048, heads=NH, kv=NK):
    """The same prompt attention on tcgen05 (S and O in tensor memory)."""
    q = torch.randn(tokens, heads, HD, device="cuda").bfloat16()
    k = torch.randn(tokens, kv, HD, device="cuda").bfloat16()
    v = torch.randn(tokens, kv, HD, device="cuda").bfloat16()
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    out = torch.empty(tokens, heads * HD, dtype=torch.bfloat16, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    us = _time(lambda: K.attention_prefill_tc(q, k, v, cu, out, 1, tokens, heads, kv, HD, 0,
                                              1 / math.sqrt(HD), st), reps)
    flops = heads * 4 * HD * tokens * (tokens + 1) / 2
    print(f"attention prefill (tcgen05) tokens={tokens} heads={heads}: {us:.1f} us, "
          f"{flops / us / 1e6:.1f} TFLOP/s (causal)")


def attention_prefill_tc_8k(reps):
    """Prompt attention on tcgen05 at 8,192 tokens, 40 heads / 8 KV heads (the 14B shape)."""
    attention_prefill_tc(reps, tokens=8192, heads=40, kv=8)


def attention_prefill_8k(reps):
    """Prompt attention on mma.sync at 8,192 tokens, 40 heads / 8 KV heads (the 14B shape)."""
    tokens, heads, kv = 8192, 40, 8
    q = torch.randn(tokens, heads, HD, device="cuda").bfloat16()
    k = torch.randn(tokens, kv, HD, device="cuda").bfloat16()
    v = torch.randn(tokens, kv, HD, device="cuda").bfloat16()
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    out = torch.empty(tokens, heads * HD, dtype=torch.bfloat16, device="cuda")
    us = _time(lambda: K.attention_prefill(q, k, v, cu, out, 1, tokens, heads, kv, HD, 0,
                                           1 / math.sqrt(HD)), reps)
    flops = heads * 4 * HD * tokens * (tokens + 1) / 2
    print(f"attention prefill (mma.sync) tokens={tokens} heads={heads}: {us:.1f} us, "
          f"{flops / us / 1e6:.1f} TFLOP/s (causal)")


def _engine(layers, max_tokens=8 * 4096, max_seqs=8, **sizes):
    from ..engine.step import Engine
    from ..model import Model
    cfg = {"architectures": ["Qwen2ForCausalLM"], "vocab_size": VOCAB, "hidden_size": NE,
           "num_hidden_layers": layers, "num_attention_heads": NH, "num_key_value_heads": NK,
           "intermediate_size": NF, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
           "tie_word_embeddings": False, "max_position_embeddings": 32768}
    cfg.update(sizes)
    model = Model.from_config(cfg, seed=0, dtype="bfloat16", device="cuda:0", make_on="device")
    return Engine(model, max_tokens=max_tokens, max_seqs=max_seqs), cfg


def step_prefill(reps, layers=4):
    """One 2,048-token prompt through 4 layers of the 7B shape plus the head."""
    eng, cfg = _engine(layers)
    ids = torch.randint(0, VOCAB, (2048,)).tolist()

    def run():
        s = eng.acquire()
        eng.step([s], [ids])
        eng.release(s)
    us = _time(run, reps, graph=False)
    print(f"prefill step, {layers} layers, 2048 tokens: {us / 1e3:.2f} ms")


def step_prefill_timeline(reps, layers=4):
    """The kernels of one 2,048-token prompt step through 4 layers with their start and end
    times, from CUPTI activity records."""
    from torch.profiler import ProfilerActivity, profile
    eng, cfg = _engine(layers)
    ids = torch.randint(0, VOCAB, (2048,)).tolist()

    def run():
        s = eng.acquire()
        eng.step([s], [ids])
        eng.release(s)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    t0, prev = evs[0].time_range.start, evs[0].time_range.start
    print(f"{'kernel':46s} {'start':>8s} {'end':>8s} {'after the one before':>21s}")
    for e in evs:
        print(f"{e.name[:46]:46s} {e.time_range.start - t0:8.1f} {e.time_range.end - t0:8.1f} "
              f"{e.time_range.end - max(prev, t0):21.1f}")
        prev = max(prev, e.time_range.end)
    print(f"step: {prev - t0:.1f} us")


def step_portions(reps, layers=4):
    """A 4,096-token prompt in two portions of 2,048 through 4 layers plus the head: the second
    portion attends over the cache (tcgen05 over pages) where the first attends over itself."""
    eng, cfg = _engine(layers)
    ids = torch.randint(0, VOCAB, (4096,)).tolist()
    times = {}
    for name, cuts in (("whole", [4096]), ("two portions", [2048, 2048])):
        def run():
            s = eng.acquire()
            at = 0
            for n in cuts:
                eng.step([s], [ids[at:at + n]])
                at += n
            eng.release(s)
        times[name] = _time(run, reps, graph=False)
    print(f"4,096-token prompt, {layers} layers: whole {times['whole'] / 1e3:.2f} ms, "
          f"in two portions {times['two portions'] / 1e3:.2f} ms")


def step_decode(reps, layers=4, batch=8):
    """Decode steps of 8 sequences at 2,048 positions through 4 layers plus the head."""
    eng, cfg = _engine(layers, max_tokens=batch * 2304, max_seqs=batch)
    slots = [eng.acquire() for _ in range(batch)]
    for i in range(0, batch, 8):            # prompts of 8 sequences at a time
        eng.step(slots[i:i + 8], [torch.randint(0, VOCAB, (2048,)).tolist() for _ in range(8)])
    tokens = torch.randint(0, VOCAB, (batch,), dtype=torch.int32, device="cuda")
    us = _time(lambda: eng.decode_on_device(slots, tokens), reps, graph=False)
    print(f"decode step, {layers} layers, batch {batch}: {us:.1f} us")


def step_decode_sweep(reps, layers=28):
    """Decode steps of the whole Qwen2.5-7B shape (28 layers) over batch sizes 1 to 128 and
    contexts of 512 to 8,192 cached positions: time of a replayed step (median of `reps`, CUDA
    events) and the bytes it has to read (weights once, the cache of the live rows) over that
    time."""
    import statistics
    eng, cfg = _engine(layers, max_tokens=128 * 8192 + 128 * 512, max_seqs=128)
    weights = eng.model.parameter_bytes() - eng.model.embedding.numel() * 2
    kv_per_pos = layers * 2 * NK * HD * 2
    print(f"{'batch':>6s} {'context':>8s} {'ms/step':>9s} {'tokens/s':>10s} {'GB/s':>8s}")
    for ctx_len in (512, 2048, 8192):
        for batch in (1, 4, 8, 16, 32, 64, 128):
            slots = [eng.acquire() for _ in range(batch)]
            for i in range(0, batch, 8):        # prompts of 8 sequences at a time
                part = slots[i:i + 8]
                eng.step(part, [torch.randint(0, VOCAB, (ctx_len,)).tolist() for _ in part])
            tokens = torch.randint(0, VOCAB, (batch,), dtype=torch.int32, device="cuda")
            for _ in range(4):
                eng.decode_on_device(slots, tokens)
            torch.cuda.synchronize()
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
            marks[0].record()
            for i in range(reps):
                eng.decode_on_device(slots, tokens)
                marks[i + 1].record()
            torch.cuda.synchronize()
            ms = statistics.median(marks[i].elapsed_time(marks[i + 1]) for i in range(reps))
            nbytes = weights + batch * (ctx_len + 4 + reps / 2) * kv_per_pos
            print(f"{batch:6d} {ctx_len:8d} {ms:9.3f} {batch / ms * 1e3:10.0f} {nbytes / ms / 1e6:8.0f}")
            for s_ in slots:
                eng.release(s_)
    eng.check_status()


def step_prefill_sweep(reps, layers=28):
    """Whole-prompt steps of the whole Qwen2.5-7B shape (28 layers) over prompt lengths of 256 to
    32,000 tokens and batches of 2,048-token prompts: the first prompt's time after a pause (the
    clock of an idle GPU) and the median of `reps` back to back (the clock under the power cap),
    with the step's flops (products, causal attention, the head on the wanted row) over them,
    and the time the host needs to issue the step's launches (a whole-prompt step is not a
    graph: below about 512 tokens the device waits for the host)."""
    import statistics
    import time
    eng, cfg = _engine(layers, max_tokens=8 * 4096 + 64, max_seqs=8)
    matrix_flops = 2.0 * layers * (NE * (NH + 2 * NK) * HD + NH * HD * NE + 3 * NE * NF)

    def flops(lens):
        attn = sum(4.0 * layers * NH * HD * (n * (n + 1) / 2) for n in lens)
        return sum(lens) * matrix_flops + attn + 2.0 * len(lens) * NE * VOCAB

    print(f"{'prompts':>8s} {'tokens':>7s} {'first ms':>9s} {'PFLOP/s':>8s} {'median ms':>10s} {'PFLOP/s':>8s} {'tokens/s':>10s} {'host ms':>8s}")
    for lens in ([256], [512], [1024], [2048], [4096], [8192], [16384], [32000], [2048] * 4, [2048] * 8,
                 [300, 700, 1500, 2048, 40, 1000, 1900, 64]):
        ids = [torch.randint(0, VOCAB, (n,)).tolist() for n in lens]
        times, host = [], []
        for i in range(reps + 2):
            slots = [eng.acquire() for _ in lens]
            if i == 1:
                torch.cuda.synchronize()
                time.sleep(1.0)                       # the first timed step starts from an idle clock
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            h0 = time.perf_counter()
            a.record()
            eng.step(slots, ids)
            b.record()
            host.append((time.perf_counter() - h0) * 1e3)     # until the host has issued the step
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
            for s_ in slots:
                eng.release(s_)
        first, med = times[1], statistics.median(times[2:])
        f = flops(lens)
        print(f"{len(lens):8d} {sum(lens):7d} {first:9.2f} {f / first / 1e12:8.3f} {med:10.2f} "
              f"{f / med / 1e12:8.3f} {sum(lens) / med * 1e3:10.0f} {statistics.median(host[2:]):8.2f}")
    eng.check_status()


def step_decode_timeline(reps, layers=4, batch=8):
    """The kernels of one replayed decode step (8 sequences at 2,048 positions, 4 layers) with
    their start and end times inside the graph, from CUPTI activity records."""
    from torch.profiler import ProfilerActivity, profile
    eng, cfg = _engine(layers, max_tokens=batch * 2304, max_seqs=batch)
    slots = [eng.acquire() for _ in range(batch)]
    for i in range(0, batch, 8):
        eng.step(slots[i:i + 8], [torch.randint(0, VOCAB, (2048,)).tolist() for _ in range(8)])
    tokens = torch.randint(0, VOCAB, (batch,), dtype=torch.int32, device="cuda")
    for _ in range(5):
        eng.decode_on_device(slots, tokens)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(max(1, reps)):
            eng.decode_on_device(slots, tokens)
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(evs) if "embed_kernel" in e.name][-1]
    step = evs[first:]
    t0 = step[0].time_range.start
    # a kernel starts early (its CTAs wait for the kernel before it): what it costs the step is
    # the time from the end of the kernel before it to its own end
    print(f"{'kernel':46s} {'start':>8s} {'end':>8s} {'after the one before':>21s}")
    prev_end = t0
    for e in step:
        start, end = e.time_range.start - t0, e.time_range.end - t0
        print(f"{e.name[:46]:46s} {start:8.1f} {end:8.1f} {end - max(prev_end - t0, 0.0):21.1f}")
        prev_end = max(prev_end, e.time_range.end)
    print(f"step: {step[-1].time_range.end - t0:.1f} us")


def step_decode_timeline_b64(reps):
    """The same timeline for 64 sequences at 2,048 positions."""
    step_decode_timeline(reps, batch=64)


def step_decode_b64(reps):
    """Decode steps of 64 sequences at 2,048 positions through 4 layers plus the head."""
    step_decode(reps, batch=64)


def step_decode_small(reps, layers=24):
    """Decode steps of 64 sequences at 16 to 1,024 positions, Qwen2.5-0.5B shape (hidden 896,
    14 heads / 2 KV heads of 64, intermediate 4864, tied head), all 24 layers."""
    eng, cfg = _engine(layers, max_tokens=64 * 1280, max_seqs=64, vocab_size=151936,
                       hidden_size=896, num_attention_heads=14, num_key_value_heads=2,
                       intermediate_size=4864, tie_word_embeddings=True)
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(16, 1025, (64,), generator=g).tolist()
    slots = [eng.acquire() for _ in range(64)]
    eng.step(slots, [torch.randint(0, 151936, (n,), generator=g).tolist() for n in lens])
    tokens = torch.randint(0, 151936, (64,), dtype=torch.int32, device="cuda")
    us = _time(lambda: eng.decode_on_device(slots, tokens), reps, graph=False)
    print(f"decode step, small shape, {layers} layers, batch 64 ragged: {us:.1f} us")


CASES = {f.__name__: f for f in (gemm_decode, gemm_decode_split, gemm_decode_m64, gemm_decode_split_m64, gemm_prefill, gemm_prefill_down,
                                 gemm_decode_cluster, gemm_decode_cluster_o, gemm_decode_cluster_m64,
                                 attention_decode, attention_decode_b8, attention_decode_long, attention_prefill,
                                 attention_prefill_tc, attention_prefill_tc_8k, attention_prefill_8k,
                                 attention_portion, attention_portion_512_on_8k,
                                 step_prefill, step_prefill_timeline, step_portions, step_decode, step_decode_sweep, step_prefill_sweep, step_decode_timeline,
                                 step_decode_timeline_b64, step_decode_b64, step_decode_small)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m minfer_b200.kernels.cases")
    ap.add_argument("case", help="a case name, or LIST")
    ap.add_argument("--reps", type=int, default=10)
    args = ap.parse_args(argv)
    if args.case == "LIST":
        for name, fn in CASES.items():
            print(f"{name:22s} {fn.__doc__.strip()}")
        return 0
    if args.case not in CASES:
        print(f"unknown case {args.case!r}; try LIST", file=sys.stderr)
        return 2
    CASES[args.case](args.reps)
    return 0


if __name__ == "__main__":
    sys.exit(main())
