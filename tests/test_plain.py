"""The plain implementation itself: hand-computed cases, among them the reference's own
unit-test vectors (src/graph/cpu_backend.rs:568-594 rms_norm, :639-682 one key: softmax of
one score is 1, so the output is the value) (no GPU)."""
import math

import torch

import plain_qwen2 as P
from helpers import TINY_A, make_folder


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = P.rms_norm(x, w, 0.0)                       # mean square 12.5
    s = 1 / math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3 * s * 2, 4 * s * 0.5]], dtype=torch.float64))


def test_rope_rotates_pairs_i_and_i_plus_half():
    x = torch.zeros(2, 1, 4, dtype=torch.float64)
    x[:, 0, 0] = 1.0                                # pair (0, 2) with frequency 1
    y = P.rope_neox(x, [0, 1], theta=10000.0)
    assert torch.allclose(y[0, 0], x[0, 0])
    assert abs(y[1, 0, 0] - math.cos(1.0)) < 1e-12 and abs(y[1, 0, 2] - math.sin(1.0)) < 1e-12
    assert y[1, 0, 1] == 0 and y[1, 0, 3] == 0
    x2 = torch.zeros(1, 1, 4, dtype=torch.float64)
    x2[0, 0, 1] = 1.0                               # pair (1, 3) with frequency 1/100
    y2 = P.rope_neox(x2, [50], theta=10000.0)
    assert abs(y2[0, 0, 1] - math.cos(0.5)) < 1e-12 and abs(y2[0, 0, 3] - math.sin(0.5)) < 1e-12


def test_attention_one_key_returns_the_value_and_groups_share_heads():
    q = torch.randn(1, 4, 8, dtype=torch.float64)
    k = torch.randn(1, 2, 8, dtype=torch.float64)
    v = torch.randn(1, 2, 8, dtype=torch.float64)
    o = P.attention(q, k, v, 0.3)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 1], v[0, 0])
    assert torch.allclose(o[0, 2], v[0, 1]) and torch.allclose(o[0, 3], v[0, 1])


def test_attention_is_causal_and_windowed():
    T = 6
    q = torch.zeros(T, 1, 2, dtype=torch.float64)          # all scores 0: uniform weights
    k = torch.zeros(T, 1, 2, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64)[:, None, None].repeat(1, 1, 2)
    full = P.attention(q, k, v, 1.0)
    assert torch.allclose(full[:, 0, 0], torch.tensor([0, 0.5, 1, 1.5, 2, 2.5], dtype=torch.float64))
    win = P.attention(q, k, v, 1.0, window=2)              # itself and one before
    assert torch.allclose(win[:, 0, 0], torch.tensor([0, 0.5, 1.5, 2.5, 3.5, 4.5], dtype=torch.float64))


def test_swiglu_by_hand():
    x = torch.tensor([[1.0, 2.0]], dtype=torch.float64)
    wg = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    wu = torch.tensor([[0.0, 1.0]], dtype=torch.float64)
    wd = torch.tensor([[3.0]], dtype=torch.float64)
    y = P.swiglu_mlp(x, wg, wu, wd)
    assert abs(y.item() - (1 / (1 + math.exp(-1))) * 2 * 3) < 1e-12


def test_sampler_rules():
    lg = torch.tensor([1.0, 5.0, 5.0, -2.0], dtype=torch.float64)
    assert P.greedy(lg) == 1                                            # first maximum
    pen = P.apply_penalties(lg, [1, 1, 3], 2.0, 0.5, 0.25)
    assert pen[1] == (5.0 - 2 * 0.5 - 0.25) / 2.0 and pen[3] == (-2.0 - 0.5 - 0.25) * 2.0
    assert pen[0] == 1.0 and pen[2] == 5.0
    k = P.apply_top_k(torch.tensor([1.0, 3.0, 3.0, 2.0, 0.0], dtype=torch.float64), 2)
    assert k.tolist() == [-math.inf, 3.0, 3.0, -math.inf, -math.inf]
    k3 = P.apply_top_k(torch.tensor([1.0, 3.0, 2.0, 2.0], dtype=torch.float64), 2)
    assert k3.tolist() == [-math.inf, 3.0, 2.0, 2.0]                   # ties at the edge stay
    p = P.apply_top_p(torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05], dtype=torch.float64)), 0.7)
    assert [v > -math.inf for v in p.tolist()] == [True, True, False, False]
    probs = torch.log(torch.tensor([0.2, 0.5, 0.3], dtype=torch.float64))
    assert P.sample_temperature(probs, 1.0, 0.1) == 0
    assert P.sample_temperature(probs, 1.0, 0.2000001) == 1
    assert P.sample_temperature(probs, 1.0, 0.95) == 2
    assert P.sample_temperature(probs, 0.0, 0.95) == 1


def test_philox_is_a_pure_function_in_the_unit_interval():
    a = P.philox_uniform(7, 0, 0)
    assert a == P.philox_uniform(7, 0, 0) and 0.0 <= a < 1.0
    vals = {P.philox_uniform(7, n, s) for n in range(20) for s in range(5)}
    assert len(vals) == 100 and abs(sum(vals) / 100 - 0.5) < 0.1
    # known answer of Philox4x32-10 for an all-zero counter and key (first output word)
    assert int(P.philox_uniform(0, 0, 0) * 16777216) == 0x6627e8d5 >> 8


def test_decoding_a_prefix_matches_the_whole_sequence_and_schedule_repeats_layers():
    folder = make_folder("A")
    cfg, w = P.load_folder(folder)
    ids = [5, 17, 3, 99, 201, 7, 7, 30]
    whole = P.forward(cfg, w, ids)
    part = P.forward(cfg, w, ids[:5])
    assert torch.allclose(whole[:5], part, atol=1e-12)                  # causal
    twice = P.forward(cfg, w, ids, schedule=[(0, 0, True), (1, 1, True), (0, 2, True)])
    assert twice.shape == whole.shape and not torch.allclose(twice, whole)
    shared = P.forward(cfg, w, ids, schedule=[(0, 0, True), (1, 0, False)])
    assert not torch.allclose(shared, whole)


def test_parts_agree_with_the_references_own_cuda_kernels():
    """RMSNorm, NeoX rotation (at positions up to 4095 and both frequency bases), SwiGLU and
    grouped-query attention over a cache: the plain implementation in float64 against what the
    reference's float32 CUDA kernels (src/cuda_kernels.cu, compiled unchanged) gave on the
    same seeded inputs; tests/golden/make_reference_kernel_vectors.py made the file."""
    import importlib.util
    import os

    import numpy as np
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location(
        "make_reference_kernel_vectors", os.path.join(here, "golden", "make_reference_kernel_vectors.py"))
    maker = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(maker)
    cases = maker.inputs()
    gold = np.load(os.path.join(here, "golden", "reference_kernels.npz"))

    def err(got, name):
        want = torch.from_numpy(gold[name]).double()
        assert got.shape == want.shape
        return float((got.double() - want).abs().max() / want.abs().max())

    c = cases["rms_norm"]
    assert err(P.rms_norm(c["x"].double(), c["w"].double(), c["eps"]), "rms_norm") < 1e-6
    # the reference forms the angle in float32 (pos * freq): 1e-4 rad off at position 4095
    for name, tol in (("rope", 3e-4), ("rope_base_10000", 3e-4)):
        c = cases[name]
        assert err(P.rope_neox(c["x"].double(), c["positions"], c["theta"], c["scale"]), name) < tol
    early = cases["rope"]["x"][:4].double()          # positions 0, 1, 2, 7: float32 angles are exact enough
    got = P.rope_neox(early, cases["rope"]["positions"][:4], cases["rope"]["theta"])
    assert float((got - torch.from_numpy(gold["rope"][:4]).double()).abs().max()) < 2e-6
    c = cases["swiglu"]
    g, u = c["gate"].double(), c["up"].double()
    assert err(g / (1.0 + torch.exp(-g)) * u, "swiglu") < 1e-6
    c = cases["attention"]
    assert err(P.attention(c["q"].double(), c["k"].double(), c["v"].double(), c["scale"]), "attention") < 2e-6


def test_a_whole_layer_agrees_with_the_references_kernels_chained_in_its_order():
    """The plain model's composition (bias before the rotation, q and k rotated but not v, keys
    and values read back by position, attention, output projection added to the layer's input,
    second norm, SwiGLU, second residual, final norm) against the reference's own CUDA kernels
    launched in the order of its graph (src/models/qwen2/graph.rs:63-176) on one seeded layer.
    The plain side sees the layer as a one-layer model whose embedding rows are the layer's
    input rows and whose head is the identity, so its logits are the normed output rows."""
    import importlib.util
    import os

    import numpy as np
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location(
        "make_reference_kernel_vectors", os.path.join(here, "golden", "make_reference_kernel_vectors.py"))
    maker = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(maker)
    c = {k: v.double() for k, v in maker.inputs()["layer"].items()}
    gold = np.load(os.path.join(here, "golden", "reference_kernels.npz"))
    L = maker.LAYER
    T, ne = L["tokens"], L["hidden"]
    cfg = {"num_hidden_layers": 1, "hidden_size": ne, "num_attention_heads": L["heads"],
           "num_key_value_heads": L["kv_heads"], "intermediate_size": L["ffn"], "vocab_size": T,
           "rope_theta": L["theta"], "rms_norm_eps": L["eps"], "tie_word_embeddings": False}
    p = "model.layers.0."
    w = {"model.embed_tokens.weight": c["h0"], "lm_head.weight": torch.eye(ne, dtype=torch.float64),
         "model.norm.weight": c["final"], p + "input_layernorm.weight": c["ln1"],
         p + "post_attention_layernorm.weight": c["ln2"],
         p + "self_attn.q_proj.weight": c["wq"], p + "self_attn.q_proj.bias": c["bq"],
         p + "self_attn.k_proj.weight": c["wk"], p + "self_attn.k_proj.bias": c["bk"],
         p + "self_attn.v_proj.weight": c["wv"], p + "self_attn.v_proj.bias": c["bv"],
         p + "self_attn.o_proj.weight": c["wo"], p + "mlp.gate_proj.weight": c["wg"],
         p + "mlp.up_proj.weight": c["wu"], p + "mlp.down_proj.weight": c["wd"]}
    got = P.forward(cfg, w, list(range(T)))
    want = torch.from_numpy(gold["layer_normed"]).double()
    assert got.shape == want.shape
    assert float((got - want).abs().max() / want.abs().max()) < 5e-6
    # and the attention output alone (before the output projection)
    x = P.rms_norm(c["h0"], c["ln1"], L["eps"])
    hd = L["head_dim"]
    q = P.rope_neox(P.linear(x, c["wq"], c["bq"]).reshape(T, L["heads"], hd), range(T), L["theta"])
    k = P.rope_neox(P.linear(x, c["wk"], c["bk"]).reshape(T, L["kv_heads"], hd), range(T), L["theta"])
    v = P.linear(x, c["wv"], c["bv"]).reshape(T, L["kv_heads"], hd)
    o = P.attention(q, k, v, 1.0 / hd ** 0.5).reshape(T, -1)
    want_o = torch.from_numpy(gold["layer_attention"]).double()
    assert float((o - want_o).abs().max() / want_o.abs().max()) < 5e-6
