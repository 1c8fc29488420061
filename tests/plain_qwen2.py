"""A plain, slow implementation of the Qwen2 dense decoder and of the sampler: whole
sequences, no cache, one function per part, float64 by default.  It shares no code with
``minfer_b200``: it reads ``config.json`` as a dictionary and the weights with the
``safetensors`` package.

It rests on the reference's formulas, not on running the reference's model: yusiwen/minfer is
Rust, there is no Rust toolchain here, and it reads GGUF files only, so its model code can be
neither imported nor compiled in this environment.  Each function cites the lines of the
reference (paths within that project) that it restates.  What of the reference does compile
are its float32 CUDA kernels (src/cuda_kernels.cu, plain C): their outputs for RMSNorm, the
NeoX rotation, SwiGLU and grouped-query attention on seeded inputs lie under tests/golden/
with the script that made them, and tests/test_plain.py holds this file's functions to them.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

DT = torch.float64


# ---------------------------------------------------------------------------------------
# loading
# ---------------------------------------------------------------------------------------
def load_folder(folder: str, dtype: torch.dtype = DT) -> Tuple[dict, Dict[str, torch.Tensor]]:
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


# ---------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------
def embed(ids: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """h[t] = E[ids[t]]  (src/graph/cpu_backend.rs:249-291, src/models/qwen2/graph.rs:54)."""
    return table[torch.tensor(list(ids), dtype=torch.long, device=table.device)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * 1/sqrt(mean(x^2) + eps) * w; the weight multiplies after the scale
    (src/vec_ops.rs:500-522)."""
    mean = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(mean + eps)) * w


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t][o] = dot(w[o], x[t]) (+ bias[o]); weights are [out][in]
    (src/graph/cpu_backend.rs:214-247)."""
    y = x @ w.t()
    return y if b is None else y + b


def rope_neox(x: torch.Tensor, positions: Sequence[int], theta: float,
              freq_scale: float = 1.0) -> torch.Tensor:
    """x: [tokens, heads, hd].  freq_i = scale / theta^(2i/hd); pairs (i, i + hd/2):
    x0' = x0 cos - x1 sin, x1' = x0 sin + x1 cos  (src/graph/cpu_backend.rs:403-434,
    NonInterleaved style)."""
    hd = x.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=DT)
    freqs = freq_scale / torch.pow(torch.tensor(theta, dtype=DT), 2.0 * i / hd)
    ang = torch.tensor(list(positions), dtype=DT)[:, None] * freqs[None, :]     # [T, half]
    cos = torch.cos(ang)[:, None, :].to(device=x.device, dtype=x.dtype)
    sin = torch.sin(ang)[:, None, :].to(device=x.device, dtype=x.dtype)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: int = 0) -> torch.Tensor:
    """q [T, nh, hd], k/v [T, nk, hd] of ONE sequence at positions 0..T-1.  Head h uses KV
    head h // (nh / nk); key j is visible to the query at p iff j <= p (and p - j < window
    in a windowed layer); scores * scale, softmax, weighted sum of values
    (src/graph/cpu_backend.rs:437-494).  The window has no counterpart in the reference; its
    convention is: the query itself and the window-1 positions before it."""
    T, nh, hd = q.shape
    nk = k.shape[1]
    g = nh // nk
    out = torch.zeros_like(q)
    for h in range(nh):
        hk = h // g
        for t in range(T):
            lo = max(0, t - window + 1) if window > 0 else 0
            s = (k[lo:t + 1, hk, :] @ q[t, h, :]) * scale
            s = s - s.max()
            p = torch.exp(s)
            p = p / p.sum()
            out[t, h, :] = p @ v[lo:t + 1, hk, :]
    return out


def swiglu_mlp(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """down( silu(gate x) * (up x) ), silu(z) = z / (1 + exp(-z))
    (src/models/qwen2/graph.rs:154-175, src/vec_ops.rs:131-146)."""
    g = linear(x, wg)
    u = linear(x, wu)
    return linear(g / (1.0 + torch.exp(-g)) * u, wd)


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------
def layer_window(cfg: dict, layer: int) -> int:
    if cfg.get("use_sliding_window", False) and layer >= cfg["max_window_layers"]:
        return int(cfg["sliding_window"])
    return 0


def attention_block(cfg: dict, w: Dict[str, torch.Tensor], layer: int, x: torch.Tensor,
                    shared_kv: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """Projections with bias, rotary on q and k after the bias, attention, output projection
    (src/models/qwen2/graph.rs:100-125).  Returns (output, (k, v)) so that a call that reads
    another call's keys and values can be expressed."""
    nh = cfg["num_attention_heads"]
    nk = cfg.get("num_key_value_heads", nh)
    hd = cfg["hidden_size"] // nh
    p = f"model.layers.{layer}.self_attn."
    T = x.shape[0]
    pos = list(range(T))
    theta = cfg.get("rope_theta", 10000.0)
    q = linear(x, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).reshape(T, nh, hd)
    q = rope_neox(q, pos, theta)
    if shared_kv is None:
        k = linear(x, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).reshape(T, nk, hd)
        v = linear(x, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).reshape(T, nk, hd)
        k = rope_neox(k, pos, theta)
    else:
        k, v = shared_kv
    o = attention(q, k, v, 1.0 / math.sqrt(hd), layer_window(cfg, layer))
    return linear(o.reshape(T, nh * hd), w[p + "o_proj.weight"]), (k, v)


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int],
            schedule: Optional[Sequence[Tuple[int, int, bool]]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  Per layer: norm, attention, residual, norm,
    feed-forward, residual; then the final norm and the head, which is the embedding table
    when the embeddings are tied (src/models/qwen2/graph.rs:59-182,
    src/models/qwen2/loader.rs:256-263).  ``schedule`` lists (layer, cache entry, writes) in
    run order; by default every layer once with an entry of its own."""
    eps = cfg.get("rms_norm_eps", 1e-6)
    L = cfg["num_hidden_layers"]
    if schedule is None:
        schedule = [(l, l, True) for l in range(L)]
    h = embed(ids, w["model.embed_tokens.weight"])
    kv_of: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    for layer, entry, writes in schedule:
        p = f"model.layers.{layer}."
        x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        a, kv = attention_block(cfg, w, layer, x, None if writes else kv_of[entry])
        if writes:
            kv_of[entry] = kv
        h = h + a
        x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])
    x = rms_norm(h, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return linear(x, head)


# ---------------------------------------------------------------------------------------
# sampling (src/sampler.rs)
# ---------------------------------------------------------------------------------------
def greedy(logits: torch.Tensor) -> int:
    """The first maximum wins (src/sampler.rs:16-26)."""
    best, best_i = logits[0].item(), 0
    for i, v in enumerate(logits.tolist()):
        if v > best:
            best, best_i = v, i
    return best_i


def apply_penalties(logits: torch.Tensor, recent: Sequence[int], repeat: float, frequency: float,
                    presence: float) -> torch.Tensor:
    """Per distinct token of the window: minus count*frequency, minus presence, then the
    repeat penalty (<= 0 multiplied, else divided)  (src/sampler.rs:44-76)."""
    out = logits.clone()
    if abs(repeat - 1.0) < 1e-6 and abs(frequency) < 1e-6 and abs(presence) < 1e-6:
        return out
    counts: Dict[int, int] = {}
    for t in recent:
        counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        if t >= out.numel():
            continue
        nv = out[t].item()
        if abs(frequency) >= 1e-6 or abs(presence) >= 1e-6:
            nv -= c * frequency
            nv -= presence
        if abs(repeat - 1.0) >= 1e-6 and repeat >= 1.0:
            nv = nv * repeat if nv <= 0.0 else nv / repeat
        out[t] = nv
    return out


def apply_top_k(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Everything below the k-th largest value becomes -inf; ties stay
    (src/sampler.rs:125-137)."""
    out = logits.clone()
    if k == 0 or k >= out.numel():
        return out
    threshold = torch.sort(out, descending=True).values[k - 1]
    out[out < threshold] = -math.inf
    return out


def apply_top_p(logits: torch.Tensor, p: float) -> torch.Tensor:
    """Softmax of the survivors, sorted by descending probability (ties in index order),
    keep up to and including the first whose running sum exceeds p
    (src/sampler.rs:149-196)."""
    out = logits.clone()
    if p <= 0.0 or p >= 1.0:
        return out
    idx = [i for i, v in enumerate(out.tolist()) if v > -math.inf]
    if not idx:
        return out
    vals = out[idx]
    probs = torch.exp(vals - vals.max())
    probs = probs / probs.sum()
    order = sorted(range(len(idx)), key=lambda j: (-probs[j].item(), idx[j]))
    cum, keep = 0.0, len(order)
    for n, j in enumerate(order):
        cum += probs[j].item()
        if cum > p:
            keep = n + 1
            break
    for j in order[keep:]:
        out[idx[j]] = -math.inf
    return out


def sample_temperature(logits: torch.Tensor, temp: float, r: float) -> int:
    """logits / temp, softmax, the first index (ascending, zero probabilities skipped) whose
    running sum reaches r; the last index otherwise  (src/sampler.rs:224-267)."""
    if temp < 1e-6:
        return greedy(logits)
    x = logits * (1.0 / temp)
    probs = torch.exp(x - x.max())
    probs[x == -math.inf] = 0.0
    probs = probs / probs.sum()
    cum = 0.0
    for i, pv in enumerate(probs.tolist()):
        if pv <= 0.0:
            continue
        cum += pv
        if r <= cum:
            return i
    return probs.numel() - 1


def sample(logits: torch.Tensor, temp: float, top_k: int, top_p: float, repeat: float,
           frequency: float, presence: float, recent: Sequence[int], r: float) -> int:
    """penalties -> greedy | top-k -> top-p -> temperature  (src/sampler.rs:272-290)."""
    x = apply_penalties(logits, recent, repeat, frequency, presence)
    if temp < 1e-6:
        return greedy(x)
    x = apply_top_k(x, top_k)
    x = apply_top_p(x, top_p)
    return sample_temperature(x, temp, r)


# ---------------------------------------------------------------------------------------
# Philox4x32-10: the uniform number a (seed, draw, stream) triple gives.  Written from the
# published algorithm (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
# ---------------------------------------------------------------------------------------
def philox_uniform(seed: int, draw: int, stream: int) -> float:
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    mask = 0xFFFFFFFF
    k0, k1 = seed & mask, (seed >> 32) & mask
    x = [draw & mask, stream & mask, 0, 0]
    for _ in range(10):
        p0, p1 = M0 * x[0], M1 * x[2]
        x = [((p1 >> 32) ^ x[1] ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ x[3] ^ k1) & mask, p0 & mask]
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return (x[0] >> 8) / 16777216.0


def generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], max_new: int,
             stop_ids: Sequence[int] = (), temp: float = 0.0, top_k: int = 0, top_p: float = 1.0,
             repeat: float = 1.0, frequency: float = 0.0, presence: float = 0.0, seed: int = 0,
             stream: int = 0) -> List[int]:
    """Sample from the last logits; a stop token ends the sequence and is neither emitted
    nor fed; otherwise append and run the whole sequence again  (src/main.rs:559-598).  The
    penalty window is the last 64 tokens, seeded with the prompt's tail (src/main.rs:537-540)."""
    ids = list(prompt)
    out: List[int] = []
    recent = list(prompt[-64:])
    for n in range(max_new):
        logits = forward(cfg, w, ids)[-1]
        tok = sample(logits, temp, top_k, top_p, repeat, frequency, presence, recent,
                     philox_uniform(seed, n, stream))
        if tok in stop_ids:
            break
        out.append(tok)
        ids.append(tok)
        recent = (recent + [tok])[-64:]
    return out
