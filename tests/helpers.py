"""Tiny configurations and shared helpers of the tests."""
from __future__ import annotations

import os
import tempfile
from typing import Dict, List, Sequence

import torch

# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 1, "intermediate_size": 128,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "use_sliding_window": False, "max_position_embeddings": 512, "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 389, "hidden_size": 192, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "intermediate_size": 328,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 16, "max_window_layers": 1,
    "max_position_embeddings": 1024, "eos_token_id": [3, 5],
}
# head size 48 (a multiple of 16 that is no power of two), 3:1 groups, window wider than a page
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 131, "hidden_size": 144, "num_hidden_layers": 2,
    "num_attention_heads": 3, "num_key_value_heads": 3, "intermediate_size": 200,
    "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 70, "max_window_layers": 0,
    "max_position_embeddings": 1024,
}
# head sizes 64 and 128: the sizes the tensor-core attention kernels take, so that the
# bfloat16 engine runs its product kernels in the whole-model comparisons
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 300, "hidden_size": 256, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 384,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1,
    "max_position_embeddings": 4096,
}
TINY_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 211, "hidden_size": 384, "num_hidden_layers": 2,
    "num_attention_heads": 3, "num_key_value_heads": 1, "intermediate_size": 264,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "use_sliding_window": False, "max_position_embeddings": 2048,
}
# a group of 20 query heads on one key/value head: more than the 16 rows of the decode
# kernel's MMA tile, so decoding takes the generic kernel while prompts take the tcgen05 one
TINY_F = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 151, "hidden_size": 1280, "num_hidden_layers": 1,
    "num_attention_heads": 20, "num_key_value_heads": 1, "intermediate_size": 136,
    "rope_theta": 500000.0, "rms_norm_eps": 2e-6, "tie_word_embeddings": True,
    "use_sliding_window": False, "max_position_embeddings": 512,
}
# The two tiny configurations exactly as the headline's record states them (sizes, options,
# weights N(0, 0.02), norm weights 1 and 1 + N(0, 0.01)); A-F above are louder variants of
# them (other vocabulary and widths that are no multiples of anything, weights N(0, 0.08)).
TINY_A0 = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 1, "intermediate_size": 128,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "use_sliding_window": False, "max_position_embeddings": 128,
}
TINY_B0 = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 384, "hidden_size": 192, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "intermediate_size": 320,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "use_sliding_window": True, "sliding_window": 16, "max_window_layers": 1,
    "max_position_embeddings": 256,
}
TINY = {"A0": (TINY_A0, 0, 0.0, 0.02), "B0": (TINY_B0, 1, 0.01, 0.02), "A": (TINY_A, 0, 0.0), "B": (TINY_B, 1, 0.01), "C": (TINY_C, 2, 0.02),
        "D": (TINY_D, 3, 0.01), "E": (TINY_E, 4, 0.0), "F": (TINY_F, 5, 0.01)}

# Tolerances, as a fraction of the largest logit magnitude of the comparison.  float32
# differs from the float64 plain implementation by summation order only; bfloat16 rounds
# weights-times-activations products' inputs to 8 bits of mantissa at every layer.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


def make_folder(name: str, weight_std: float = None, store_dtype: str = "bfloat16") -> str:
    """A random model folder for a tiny configuration, in a fresh temporary folder.  Unless
    the configuration states its own, the weights are N(0, 0.08): larger than N(0, 0.02), so
    that logits differ visibly between tokens."""
    from minfer_b200.model import write_random_model
    cfg, seed, norm_std, *own_std = TINY[name]
    if weight_std is None:
        weight_std = own_std[0] if own_std else 0.08
    folder = tempfile.mkdtemp(prefix=f"minfer_b200_tiny{name}_")
    write_random_model(folder, cfg, seed, store_dtype, norm_std=norm_std, weight_std=weight_std)
    return folder


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got = got.detach().to(torch.float64).cpu()
    want = want.detach().to(torch.float64).cpu()
    return float((got - want).abs().max() / max(1e-30, float(want.abs().max())))


# bfloat16, row by row: the root mean square error of a row of logits as a fraction of the
# largest logit of the comparison.  The largest single error of a bfloat16 run has a long tail
# (one logit in 14,000 of configuration E is 3.2 % off on the whole-prompt path itself), while a
# fault of the cache or of the batch (a key missing, a stale page, a neighbour's row) moves a
# whole row by tens of per cent; measured over all six configurations the worst row stays
# below 0.9 %.
ROW_RMS_TOL = 1.25e-2


def row_rms_err(got: torch.Tensor, want: torch.Tensor) -> float:
    got = got.detach().to(torch.float64).cpu()
    want = want.detach().to(torch.float64).cpu()
    rms = (got - want).pow(2).mean(dim=-1).sqrt().max()
    return float(rms / max(1e-30, float(want.abs().max())))


def logits_err(got: torch.Tensor, want: torch.Tensor, dtype: str) -> tuple:
    """(error, bound): float32 by the largest single error, bfloat16 by the worst row."""
    if dtype == "float32":
        return rel_err(got, want), TOL["float32"]
    return row_rms_err(got, want), ROW_RMS_TOL


def _draw_interval(P, logits, temp, top_k, top_p, tok):
    """[lo, hi) of the uniform numbers for which the plain sampler draws ``tok`` from these
    (penalised) logits, or None if it never does."""
    import math
    x = P.apply_top_p(P.apply_top_k(logits, top_k), top_p) * (1.0 / temp)
    probs = torch.exp(x - x.max())
    probs[x == -math.inf] = 0.0
    probs = probs / probs.sum()
    if float(probs[tok]) <= 0.0:
        return None
    lo = float(probs[:tok].sum())
    return lo, lo + float(probs[tok])


def follows_plain(P, cfg, w, prompt, tokens, dtype, *, temp=0.0, top_k=0, top_p=1.0, repeat=1.0,
                  frequency=0.0, presence=0.0, seed=0, stream=0) -> None:
    """Holds generated ``tokens`` to the plain implementation token by token, each on the
    prefix the engine itself produced (so one rounding difference does not fail all later
    tokens).  float32: the token is the plain sampler's.  bfloat16: logits are off by up to
    TOL of the largest one, so the token must be the plain sampler's for the same uniform
    number, or one that rounding can tip the choice to: greedy, a token within twice the
    tolerance of the maximum; sampled, a token whose range of uniform numbers in the plain
    cumulative distribution (with or without the top-k/top-p cut, which rounding can move by
    one token) comes within 0.05 of the number drawn."""
    ids = list(prompt)
    recent = list(prompt[-64:])
    for n, tok in enumerate(tokens):
        logits = P.forward(cfg, w, ids)[-1]
        r = P.philox_uniform(seed, n, stream)
        want = P.sample(logits, temp, top_k, top_p, repeat, frequency, presence, recent, r)
        if tok != want:
            assert dtype == "bfloat16", (n, tok, want)
            x = P.apply_penalties(logits, recent, repeat, frequency, presence)
            if temp < 1e-6:
                slack = 2 * TOL["bfloat16"] * float(logits.abs().max())
                assert float(x[tok]) >= float(x.max()) - slack, (n, tok, want)
            else:
                spans = [_draw_interval(P, x, temp, top_k, top_p, tok),
                         _draw_interval(P, x, temp, 0, 1.0, tok)]
                assert any(sp is not None and sp[0] - 0.05 <= r <= sp[1] + 0.05 for sp in spans), \
                    (n, tok, want, r, spans)
        ids.append(tok)
        recent = (recent + [tok])[-64:]
