"""A toy mixer with state of its own, a toy feed-forward and a toy position encoding, all
defined here, are registered, built and stepped without a change to the framework's files.
They are not models of anyone's: they only show that the interfaces carry other parts.

The toy mixer keeps, per sequence, a decaying sum of its projected inputs:
    s_t = decay * s_{t-1} + W_in x_t ;  y_t = W_out s_t
Its state has a fixed size, whatever the sequence's length, and must give the same result
for a whole prompt and token by token, and be zero again when a slot is reused."""
import json
import os
import tempfile

import pytest
import torch

from helpers import random_ids, rel_err

pytestmark = pytest.mark.gpu

VOCAB, WIDTH, INNER = 97, 48, 24
SOFT_CAP = 4.0


def _register():
    from minfer_b200 import registry
    from minfer_b200.config.base import (ConfigReader, LayerSpec, ModelPlan, PartSpec,
                                         default_schedule)
    from minfer_b200.kernels import api as K
    from minfer_b200.parts.base import (FeedForward, Mixer, ModelPart, PositionEncoding,
                                        StateRequest)
    from minfer_b200.weights.spec import MATRIX, Init, TensorSpec

    class DecayMixer(Mixer):
        def __init__(self, width, inner, decay):
            self.width, self.inner, self.decay = width, inner, decay

        def tensor_specs(self, prefix):
            return [TensorSpec(f"{prefix}mix.in.weight", (self.inner, self.width), MATRIX, Init(0, 0.2)),
                    TensorSpec(f"{prefix}mix.out.weight", (self.width, self.inner), MATRIX, Init(0, 0.2))]

        def load(self, prefix, weights):
            self.w_in = weights[f"{prefix}mix.in.weight"]
            self.w_out = weights[f"{prefix}mix.out.weight"]

        def state_request(self):
            return [StateRequest("sum", (self.inner,), torch.float32)]

        def forward_add(self, x, ctx, binding, residual):
            # the toy's own arithmetic is plain tensor code; a real part would be a kernel
            state = binding.state["sum"]                       # [max_slots, inner]
            u = torch.empty((x.shape[0], self.inner), dtype=torch.float32, device=x.device)
            K.gemm_simt(x, self.w_in, None, u)
            s_all = torch.empty_like(u)
            cu = ctx.cu_seqlens.tolist()
            for b, slot in enumerate(ctx.host_slots):
                s = state[slot].clone()
                for t in range(cu[b], cu[b + 1]):
                    s = self.decay * s + u[t]
                    s_all[t] = s
                state[slot] = s
            K.gemm_simt(s_all.to(x.dtype), self.w_out, None, residual, accumulate=True)

    class SquareFeedForward(FeedForward):
        """y = W2 (W1 x)^2: another feed-forward than the gated one."""
        def __init__(self, width, inner):
            self.width, self.inner = width, inner

        def tensor_specs(self, prefix):
            return [TensorSpec(f"{prefix}ff.w1", (self.inner, self.width), MATRIX, Init(0, 0.2)),
                    TensorSpec(f"{prefix}ff.w2", (self.width, self.inner), MATRIX, Init(0, 0.2))]

        def load(self, prefix, weights):
            self.w1, self.w2 = weights[f"{prefix}ff.w1"], weights[f"{prefix}ff.w2"]

        def forward_add(self, x, ctx, residual):
            u = torch.empty((x.shape[0], self.inner), dtype=torch.float32, device=x.device)
            K.gemm_simt(x, self.w1, None, u)
            K.gemm_simt((u * u).to(x.dtype), self.w2, None, residual, accumulate=True)

    class ShiftPosition(PositionEncoding):
        """Adds 0.01 * position to every dimension of q and k: not a rotation, so it goes
        through ``apply`` instead of the fused rotary kernel."""
        def apply(self, qkv32, ctx, n_heads, n_kv_heads, head_dim):
            n_rot = (n_heads + n_kv_heads) * head_dim
            qkv32[:, :n_rot] += 0.01 * ctx.positions.to(torch.float32)[:, None]

    class LearnedPositions(ModelPart):
        """A vector per absolute position, added to the residual stream after the embedding."""
        capturable = True

        def __init__(self, width, positions):
            self.width, self.positions = width, positions

        def tensor_specs(self, prefix):
            return [TensorSpec(f"{prefix}positions", (self.positions, self.width), MATRIX, Init(0.0, 0.1))]

        def load(self, prefix, weights):
            self.table = weights[f"{prefix}positions"]

        def forward_inplace(self, h, ctx):
            h += self.table[ctx.positions.long()].to(h.dtype)

    class SoftCap(ModelPart):
        """logits <- cap * tanh(logits / cap)."""
        capturable = True

        def __init__(self, cap):
            self.cap = float(cap)

        def forward_inplace(self, logits, ctx):
            logits.div_(self.cap).tanh_().mul_(self.cap)

    class ToyConfig:
        def __init__(self, d):
            r = ConfigReader(d)
            self.vocab, self.width, self.inner = r.integer("vocab"), r.integer("width"), r.integer("inner")
            self.layers, self.decay = r.integer("layers"), r.number("decay")

        def plan(self):
            norm = PartSpec("rms_norm", {"size": self.width, "eps": 1e-5})
            layers = []
            for l in range(self.layers):
                if l % 2 == 0:      # layers differ: the state mixer here, attention there
                    mixer = PartSpec("toy_decay", dict(width=self.width, inner=self.inner, decay=self.decay))
                else:
                    mixer = PartSpec("attention", dict(
                        hidden_size=self.width, n_heads=3, n_kv_heads=1, head_dim=16, scale=0.25,
                        window=0, qkv_bias=False, position=PartSpec("toy_shift", {})))
                ffn = (PartSpec("toy_square", dict(width=self.width, inner=self.inner)) if l % 2 == 0
                       else PartSpec("gated_mlp", dict(hidden_size=self.width, intermediate_size=40)))
                layers.append(LayerSpec(f"toy.{l}.", PartSpec("pre_norm", {}), mixer,
                                        norm.with_params(name="n1"), ffn, norm.with_params(name="n2")))
            # the embedding rows are multiplied by 3 on their way in and the logits get a bias;
            # a vector per position is added after the embedding and the logits are soft-capped:
            # hooks of the plan that the shipped architecture leaves at their defaults
            return ModelPlan("ToyStateLM", self.vocab, self.width, "toy.embed", None,
                             norm.with_params(name="final"), "toy.", layers,
                             default_schedule(self.layers), 128, (), embedding_scale=3.0,
                             head_bias_name="toy.head_bias",
                             after_embedding=PartSpec("toy_learned_positions",
                                                      dict(width=self.width, positions=128)),
                             on_logits=PartSpec("toy_soft_cap", dict(cap=SOFT_CAP)),
                             model_part_prefix="toy.")

    registry.register_part("mixer", "toy_decay", DecayMixer, replace=True)
    registry.register_part("feed_forward", "toy_square", SquareFeedForward, replace=True)
    registry.register_part("position", "toy_shift", ShiftPosition, replace=True)
    registry.register_part("model", "toy_learned_positions", LearnedPositions, replace=True)
    registry.register_part("model", "toy_soft_cap", SoftCap, replace=True)
    registry.register_architecture("ToyStateLM", lambda d, where: ToyConfig(d), replace=True)


CONFIG = {"architectures": ["ToyStateLM"], "vocab": VOCAB, "width": WIDTH, "inner": INNER,
          "layers": 3, "decay": 0.9}


def _reference(w, ids):
    """The toy model in float64, whole sequence."""
    def norm(x, wt):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * wt
    T = len(ids)
    h = w["toy.embed"][torch.tensor(ids)] * 3.0 + w["toy.positions"][:T]
    for l in range(3):
        p = f"toy.{l}."
        x = norm(h, w[p + "n1.weight"])
        if l % 2 == 0:
            u = x @ w[p + "mix.in.weight"].t()
            s, out = torch.zeros(INNER, dtype=torch.float64), []
            for t in range(T):
                s = 0.9 * s + u[t]
                out.append(s)
            h = h + torch.stack(out) @ w[p + "mix.out.weight"].t()
        else:
            a = p + "self_attn."
            pos = torch.arange(T, dtype=torch.float64)[:, None]
            q = (x @ w[a + "q_proj.weight"].t() + 0.01 * pos).reshape(T, 3, 16)
            k = (x @ w[a + "k_proj.weight"].t() + 0.01 * pos).reshape(T, 1, 16)
            v = (x @ w[a + "v_proj.weight"].t()).reshape(T, 1, 16)
            o = torch.zeros(T, 3, 16, dtype=torch.float64)
            for hh in range(3):
                sc = (q[:, hh] @ k[:, 0].t()) * 0.25
                sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
                o[:, hh] = torch.softmax(sc, -1) @ v[:, 0]
            h = h + o.reshape(T, 48) @ w[a + "o_proj.weight"].t()
        x = norm(h, w[p + "n2.weight"])
        if l % 2 == 0:
            h = h + ((x @ w[p + "ff.w1"].t()) ** 2) @ w[p + "ff.w2"].t()
        else:
            g, u = x @ w[p + "mlp.gate_proj.weight"].t(), x @ w[p + "mlp.up_proj.weight"].t()
            h = h + (torch.nn.functional.silu(g) * u) @ w[p + "mlp.down_proj.weight"].t()
    logits = norm(h, w["toy.final.weight"]) @ w["toy.embed"].t() + w["toy.head_bias"]
    return SOFT_CAP * torch.tanh(logits / SOFT_CAP)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(dtype):
    _register()
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model, write_random_model
    from minfer_b200.weights.safetensors_io import load_all
    with tempfile.TemporaryDirectory() as folder:
        json.dump(CONFIG, open(os.path.join(folder, "config.json"), "w"))
        from minfer_b200.registry import read_config
        cfg = read_config(CONFIG)
        from minfer_b200.weights.random_init import write_model_folder
        write_model_folder(folder, CONFIG, Model(cfg.plan(), "float32", cfg).tensor_specs(), 5, "bfloat16")
        w = {k: v.double() for k, v in load_all(folder).items()}
        model = Model.from_folder(folder, dtype, "cuda:0")
    eng = Engine(model, 1024, max_seqs=3)
    assert eng.cache.state.bytes_per_slot() == 2 * INNER * 4          # two state layers
    assert len(eng.cache.groups) == 1                                 # one attention layer
    tol = 2e-5 if dtype == "float32" else 3e-2
    prompts = [random_ids(n, VOCAB, n) for n in (30, 7, 70)]
    want = [_reference(w, p) for p in prompts]
    # batch of unequal lengths: heads in one step, then one token each, shorter ones ending
    for round_ in range(2):                                           # second round reuses slots
        slots = [eng.acquire() for _ in prompts]
        heads = [len(p) - 5 for p in prompts]
        out = eng.step(slots, [p[:h] for p, h in zip(prompts, heads)],
                       [list(range(h)) for h in heads])
        got = [[o] for o in torch.split(out, heads)]
        for t in range(5):
            o = eng.step(slots, [[p[h + t]] for p, h in zip(prompts, heads)])
            for b in range(3):
                got[b].append(o[b:b + 1])
        for s in slots:
            eng.release(s)
        for b in range(3):
            assert rel_err(torch.cat(got[b]), want[b]) < tol, (round_, b)
    eng.check_status()


# ---------------------------------------------------------------------------------------------
# A toy feed-forward with routing: each token goes to the one of three small experts whose
# router logit is largest (router in float32), y = W2_e (W1_e x)^2 * gate.  Layers alternate
# between it and the gated MLP, and the run order names layer 0 twice.
# ---------------------------------------------------------------------------------------------
N_EXPERTS, EXPERT_INNER = 3, 16


def _register_routed():
    from minfer_b200 import registry
    from minfer_b200.config.base import ConfigReader, LayerCall, LayerSpec, ModelPlan, PartSpec
    from minfer_b200.kernels import api as K
    from minfer_b200.parts.base import FeedForward
    from minfer_b200.weights.spec import MATRIX, Init, TensorSpec

    class RoutedSquare(FeedForward):
        def __init__(self, width, inner, experts):
            self.width, self.inner, self.experts = width, inner, experts

        def tensor_specs(self, prefix):
            specs = [TensorSpec(f"{prefix}moe.router", (self.experts, self.width), MATRIX, Init(0, 0.5))]
            for e in range(self.experts):
                specs.append(TensorSpec(f"{prefix}moe.{e}.w1", (self.inner, self.width), MATRIX, Init(0, 0.2)))
                specs.append(TensorSpec(f"{prefix}moe.{e}.w2", (self.width, self.inner), MATRIX, Init(0, 0.2)))
            return specs

        def load(self, prefix, weights):
            self.router = weights[f"{prefix}moe.router"]
            self.w1 = [weights[f"{prefix}moe.{e}.w1"] for e in range(self.experts)]
            self.w2 = [weights[f"{prefix}moe.{e}.w2"] for e in range(self.experts)]

        def forward_add(self, x, ctx, residual):
            n = x.shape[0]
            logits = torch.empty((n, self.experts), dtype=torch.float32, device=x.device)
            K.gemm_simt(x, self.router, None, logits)              # router logits in float32
            gate = torch.softmax(logits, -1)
            choice = logits.argmax(-1)
            for e in range(self.experts):                          # each expert takes its own rows
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows].contiguous()
                u = torch.empty((rows.numel(), self.inner), dtype=torch.float32, device=x.device)
                K.gemm_simt(xe, self.w1[e], None, u)
                y = torch.empty((rows.numel(), self.width), dtype=torch.float32, device=x.device)
                K.gemm_simt((u * u).to(x.dtype), self.w2[e], None, y)
                residual[rows] += y * gate[rows, e][:, None]

    class RoutedConfig:
        def __init__(self, d):
            r = ConfigReader(d)
            self.vocab, self.width, self.layers = r.integer("vocab"), r.integer("width"), r.integer("layers")

        def plan(self):
            norm = PartSpec("rms_norm", {"size": self.width, "eps": 1e-5})
            layers = []
            for l in range(self.layers):
                mixer = PartSpec("attention", dict(
                    hidden_size=self.width, n_heads=2, n_kv_heads=2, head_dim=16, scale=0.25, window=0,
                    qkv_bias=True, position=PartSpec("rotary", dict(head_dim=16, rotary_dim=16, theta=100.0))))
                ffn = (PartSpec("toy_routed", dict(width=self.width, inner=EXPERT_INNER, experts=N_EXPERTS))
                       if l % 2 == 0 else
                       PartSpec("gated_mlp", dict(hidden_size=self.width, intermediate_size=24)))
                layers.append(LayerSpec(f"r.{l}.", PartSpec("pre_norm", {}), mixer,
                                        norm.with_params(name="n1"), ffn, norm.with_params(name="n2")))
            # layer 0 runs twice: its second run has a cache entry of its own
            order = [LayerCall(0, 0, True), LayerCall(1, 1, True), LayerCall(0, 2, True)]
            return ModelPlan("ToyRoutedLM", self.vocab, self.width, "r.embed", None,
                             norm.with_params(name="final"), "r.", layers, order, 4096, ())

    registry.register_part("feed_forward", "toy_routed", RoutedSquare, replace=True)
    registry.register_architecture("ToyRoutedLM", lambda d, where: RoutedConfig(d), replace=True)


ROUTED_CONFIG = {"architectures": ["ToyRoutedLM"], "vocab": 61, "width": 32, "layers": 2}


def _routed_reference(w, ids):
    def norm(x, wt):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * wt
    T = len(ids)
    h = w["r.embed"][torch.tensor(ids)]
    pos = torch.arange(T, dtype=torch.float64)
    inv = 100.0 ** (-torch.arange(0, 16, 2, dtype=torch.float64) / 16)
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rope(x):
        a, b = x[..., :8], x[..., 8:]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], -1)
    for l in (0, 1, 0):
        p = f"r.{l}."
        a = p + "self_attn."
        x = norm(h, w[p + "n1.weight"])
        q = rope((x @ w[a + "q_proj.weight"].t() + w[a + "q_proj.bias"]).reshape(T, 2, 16))
        k = rope((x @ w[a + "k_proj.weight"].t() + w[a + "k_proj.bias"]).reshape(T, 2, 16))
        v = (x @ w[a + "v_proj.weight"].t() + w[a + "v_proj.bias"]).reshape(T, 2, 16)
        o = torch.zeros(T, 2, 16, dtype=torch.float64)
        for hh in range(2):
            sc = (q[:, hh] @ k[:, hh].t()) * 0.25
            sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            o[:, hh] = torch.softmax(sc, -1) @ v[:, hh]
        h = h + o.reshape(T, 32) @ w[a + "o_proj.weight"].t()
        x = norm(h, w[p + "n2.weight"])
        if l == 0:
            logits = x @ w[p + "moe.router"].t()
            gate, choice = torch.softmax(logits, -1), logits.argmax(-1)
            y = torch.zeros_like(h)
            for t in range(T):
                e = int(choice[t])
                y[t] = ((w[p + f"moe.{e}.w1"] @ x[t]) ** 2) @ w[p + f"moe.{e}.w2"].t() * gate[t, e]
            h = h + y
        else:
            g, u = x @ w[p + "mlp.gate_proj.weight"].t(), x @ w[p + "mlp.up_proj.weight"].t()
            h = h + (torch.nn.functional.silu(g) * u) @ w[p + "mlp.down_proj.weight"].t()
    return norm(h, w["r.final.weight"]) @ w["r.embed"].t()


def test_toy_routed_feed_forward_and_a_layer_that_runs_twice():
    """float32 only: a routing decision is a comparison, so a bfloat16 rounding could flip it
    against the float64 reference; the part itself works in either engine."""
    _register_routed()
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    from minfer_b200.registry import read_config
    from minfer_b200.weights.random_init import write_model_folder
    from minfer_b200.weights.safetensors_io import load_all
    with tempfile.TemporaryDirectory() as folder:
        json.dump(ROUTED_CONFIG, open(os.path.join(folder, "config.json"), "w"))
        cfg = read_config(ROUTED_CONFIG)
        write_model_folder(folder, ROUTED_CONFIG, Model(cfg.plan(), "float32", cfg).tensor_specs(), 9, "float32")
        w = {k: v.double() for k, v in load_all(folder).items()}
        model = Model.from_folder(folder, "float32", "cuda:0")
    eng = Engine(model, 512, max_seqs=2)
    assert sum(len(g.entries) for g in eng.cache.groups) == 3         # three calls, three entries
    prompts = [random_ids(n, 61, 40 + n) for n in (21, 50)]
    want = [_routed_reference(w, p) for p in prompts]
    slots = [eng.acquire() for _ in prompts]
    heads = [len(p) - 4 for p in prompts]
    out = eng.step(slots, [p[:h] for p, h in zip(prompts, heads)], [list(range(h)) for h in heads])
    got = [[o] for o in torch.split(out, heads)]
    for t in range(4):
        o = eng.step(slots, [[p[h + t]] for p, h in zip(prompts, heads)])
        for b in range(2):
            got[b].append(o[b:b + 1])
    for b in range(2):
        assert rel_err(torch.cat(got[b]), want[b]) < 2e-5, b
    eng.check_status()


# ---------------------------------------------------------------------------------------------
# A toy block kind with members of other names than the shipped block's: ONE norm used before
# the mixer and again before the feed-forward.  The engine learns its parts from ``parts()``:
# decode steps are replayed as graphs only if every one of them says it can be captured, and
# the libraries to build come from the parts too.
# ---------------------------------------------------------------------------------------------
def _register_shared_norm_block():
    from minfer_b200 import registry
    from minfer_b200.config.base import ConfigReader, LayerSpec, ModelPlan, PartSpec, default_schedule
    from minfer_b200.parts.base import Block
    from minfer_b200.registry import build_part

    class SharedNormBlock(Block):
        capturable = True

        def __init__(self, layer):
            self.prefix = layer.prefix
            self.pre = build_part("norm", layer.mixer_norm)
            self.mixer = build_part("mixer", layer.mixer)
            self.ff = build_part("feed_forward", layer.feed_forward)

        def parts(self):
            return (self.pre, self.mixer, self.ff)

        def tensor_specs(self, prefix=""):
            return [s for part in self.parts() for s in part.tensor_specs(self.prefix)]

        def load(self, prefix, weights):
            for part in self.parts():
                part.load(self.prefix, weights)

        def mix(self, h, ctx, binding):
            self.mixer.forward_add(self.pre.forward(h, ctx.act_dtype), ctx, binding, h)

        def feed(self, h, ctx):
            self.ff.forward_add(self.pre.forward(h, ctx.act_dtype), ctx, h)

    class SharedNormConfig:
        def __init__(self, d):
            r = ConfigReader(d)
            self.vocab, self.width, self.layers = r.integer("vocab"), r.integer("width"), r.integer("layers")
            self.ff = r.string("ff")

        def plan(self):
            norm = PartSpec("rms_norm", {"size": self.width, "eps": 1e-5, "name": "n"})
            mixer = PartSpec("attention", dict(
                hidden_size=self.width, n_heads=2, n_kv_heads=1, head_dim=16, scale=0.25, window=0,
                qkv_bias=True, position=PartSpec("rotary", dict(head_dim=16, rotary_dim=16, theta=100.0))))
            ffn = (PartSpec("gated_mlp", dict(hidden_size=self.width, intermediate_size=24))
                   if self.ff == "gated" else PartSpec("toy_square", dict(width=self.width, inner=24)))
            layers = [LayerSpec(f"s.{l}.", PartSpec("toy_shared_norm", {}), mixer, norm, ffn, norm)
                      for l in range(self.layers)]
            return ModelPlan("ToySharedNormLM", self.vocab, self.width, "s.embed", None,
                             norm.with_params(name="final"), "s.", layers,
                             default_schedule(self.layers), 512, ())

    _register()                                                       # toy_square
    registry.register_part("block", "toy_shared_norm", SharedNormBlock, replace=True)
    registry.register_architecture("ToySharedNormLM", lambda d, where: SharedNormConfig(d), replace=True)


def _shared_norm_reference(w, ids):
    def norm(x, wt):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * wt
    T = len(ids)
    h = w["s.embed"][torch.tensor(ids)]
    ang = torch.arange(T, dtype=torch.float64)[:, None] * (100.0 ** (-torch.arange(0, 16, 2, dtype=torch.float64) / 16))[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rope(x):
        a, b = x[..., :8], x[..., 8:]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], -1)
    for l in range(2):
        p, a = f"s.{l}.", f"s.{l}.self_attn."
        x = norm(h, w[p + "n.weight"])
        q = rope((x @ w[a + "q_proj.weight"].t() + w[a + "q_proj.bias"]).reshape(T, 2, 16))
        k = rope((x @ w[a + "k_proj.weight"].t() + w[a + "k_proj.bias"]).reshape(T, 1, 16))
        v = (x @ w[a + "v_proj.weight"].t() + w[a + "v_proj.bias"]).reshape(T, 1, 16)
        o = torch.zeros(T, 2, 16, dtype=torch.float64)
        for hh in range(2):
            sc = (q[:, hh] @ k[:, 0].t()) * 0.25
            sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            o[:, hh] = torch.softmax(sc, -1) @ v[:, 0]
        h = h + o.reshape(T, 32) @ w[a + "o_proj.weight"].t()
        x = norm(h, w[p + "n.weight"])
        g, u = x @ w[p + "mlp.gate_proj.weight"].t(), x @ w[p + "mlp.up_proj.weight"].t()
        h = h + (torch.nn.functional.silu(g) * u) @ w[p + "mlp.down_proj.weight"].t()
    return norm(h, w["s.final.weight"]) @ w["s.embed"].t()


def test_toy_block_with_other_member_names_gets_the_capture_check():
    _register_shared_norm_block()
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    from minfer_b200.registry import read_config
    from minfer_b200.weights.random_init import write_model_folder
    from minfer_b200.weights.safetensors_io import load_all
    engines = {}
    for ff in ("gated", "square"):
        config = {"architectures": ["ToySharedNormLM"], "vocab": 53, "width": 32, "layers": 2, "ff": ff}
        with tempfile.TemporaryDirectory() as folder:
            json.dump(config, open(os.path.join(folder, "config.json"), "w"))
            cfg = read_config(config)
            write_model_folder(folder, config, Model(cfg.plan(), "float32", cfg).tensor_specs(), 3, "float32")
            w = {k: v.double() for k, v in load_all(folder).items()}
            engines[ff] = (Engine(Model.from_folder(folder, "float32", "cuda:0"), 512, max_seqs=2), w)
    # every part of the first model launches kernels only: graphs; the second one's feed-forward
    # (plain tensor code, ``capturable`` left False) switches them off for its engine
    assert engines["gated"][0].cuda_graphs is True
    assert engines["square"][0].cuda_graphs is False
    eng, w = engines["gated"]
    ids = random_ids(60, 53, 8)
    want = _shared_norm_reference(w, ids)
    s = eng.acquire()
    rows = [eng.step([s], [ids[:20]], [list(range(20))]),             # whole, a portion, then one by one
            eng.step([s], [ids[20:45]], [list(range(25))])]
    rows += [eng.step([s], [[t]]) for t in ids[45:]]
    assert len(eng._graphs) >= 1
    assert rel_err(torch.cat(rows), want) < 2e-5
    eng.check_status()


# ---------------------------------------------------------------------------------------------
# A toy mixer whose values are wider than its keys (keys of 16, values of 40, one head): it asks
# the cache for both widths, writes its own keys and values into the pages it is given and
# reads them back by page table.  Plain tensor code on purpose: only the cache's interface is
# under test here (slots, pages, page tables, reuse), not a kernel.
# ---------------------------------------------------------------------------------------------
KEY_DIM, VALUE_DIM = 16, 40


def _register_wide_values():
    from minfer_b200 import registry
    from minfer_b200.config.base import ConfigReader, LayerSpec, ModelPlan, PartSpec, default_schedule
    from minfer_b200.parts.base import CacheRequest, Mixer
    from minfer_b200.weights.spec import MATRIX, Init, TensorSpec

    class WideValueMixer(Mixer):
        def __init__(self, width):
            self.width = width

        def tensor_specs(self, prefix):
            shapes = {"q": (KEY_DIM, self.width), "k": (KEY_DIM, self.width),
                      "v": (VALUE_DIM, self.width), "o": (self.width, VALUE_DIM)}
            return [TensorSpec(f"{prefix}wide.{n}", shape, MATRIX, Init(0.0, 0.2))
                    for n, shape in shapes.items()]

        def load(self, prefix, weights):
            self.w = {n: weights[f"{prefix}wide.{n}"].float() for n in "qkvo"}

        def cache_request(self):
            return CacheRequest(1, KEY_DIM, 0, value_dim=VALUE_DIM)

        def forward_add(self, x, ctx, binding, residual):
            x = x.float()
            q, k, v = (x @ self.w[n].t() for n in "qkv")
            cache = binding.cache
            assert cache.k.shape[-1] == KEY_DIM and cache.v.shape[-1] == VALUE_DIM
            rows, positions = ctx.token_row.tolist(), ctx.positions.tolist()
            table = cache.page_table.view(-1, cache.table_stride).tolist()
            for t, (b, pos) in enumerate(zip(rows, positions)):        # write, then read: the step's
                page = table[b][pos // 64]                             # own keys are in the cache
                cache.k[page, 0, pos % 64] = k[t].to(cache.k.dtype)
                cache.v[page, 0, pos % 64] = v[t].to(cache.v.dtype)
            out = torch.zeros_like(v)
            for t, (b, pos) in enumerate(zip(rows, positions)):
                pages = torch.tensor(table[b][:pos // 64 + 1], device=x.device)
                keys = cache.k[pages, 0].reshape(-1, KEY_DIM)[:pos + 1].float()
                values = cache.v[pages, 0].reshape(-1, VALUE_DIM)[:pos + 1].float()
                out[t] = torch.softmax(keys @ q[t] * 0.25, 0) @ values
            residual += out @ self.w["o"].t()

    class WideConfig:
        def __init__(self, d):
            r = ConfigReader(d)
            self.vocab, self.width, self.layers = r.integer("vocab"), r.integer("width"), r.integer("layers")

        def plan(self):
            norm = PartSpec("rms_norm", {"size": self.width, "eps": 1e-5})
            layers = [LayerSpec(f"w.{l}.", PartSpec("pre_norm", {}),
                                PartSpec("toy_wide_value", dict(width=self.width)),
                                norm.with_params(name="n1"),
                                PartSpec("gated_mlp", dict(hidden_size=self.width, intermediate_size=24)),
                                norm.with_params(name="n2")) for l in range(self.layers)]
            return ModelPlan("ToyWideValueLM", self.vocab, self.width, "w.embed", None,
                             norm.with_params(name="final"), "w.", layers,
                             default_schedule(self.layers), 512, ())

    registry.register_part("mixer", "toy_wide_value", WideValueMixer, replace=True)
    registry.register_architecture("ToyWideValueLM", lambda d, where: WideConfig(d), replace=True)


def _wide_reference(w, ids, layers):
    def norm(x, wt):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * wt
    h = w["w.embed"][torch.tensor(ids)]
    T = len(ids)
    mask = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
    for l in range(layers):
        p = f"w.{l}."
        x = norm(h, w[p + "n1.weight"])
        q, k, v = (x @ w[p + f"wide.{n}"].t() for n in "qkv")
        sc = (q @ k.t() * 0.25).masked_fill(mask, float("-inf"))
        h = h + (torch.softmax(sc, -1) @ v) @ w[p + "wide.o"].t()
        x = norm(h, w[p + "n2.weight"])
        g, u = x @ w[p + "mlp.gate_proj.weight"].t(), x @ w[p + "mlp.up_proj.weight"].t()
        h = h + (torch.nn.functional.silu(g) * u) @ w[p + "mlp.down_proj.weight"].t()
    return norm(h, w["w.final.weight"]) @ w["w.embed"].t()


def test_toy_mixer_with_values_wider_than_keys_uses_the_cache():
    _register_wide_values()
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    from minfer_b200.registry import read_config
    from minfer_b200.weights.random_init import write_model_folder
    from minfer_b200.weights.safetensors_io import load_all
    config = {"architectures": ["ToyWideValueLM"], "vocab": 61, "width": 32, "layers": 2}
    with tempfile.TemporaryDirectory() as folder:
        json.dump(config, open(os.path.join(folder, "config.json"), "w"))
        cfg = read_config(config)
        write_model_folder(folder, config, Model(cfg.plan(), "float32", cfg).tensor_specs(), 4, "float32")
        w = {k: v.double() for k, v in load_all(folder).items()}
        eng = Engine(Model.from_folder(folder, "float32", "cuda:0"), 512, max_seqs=2)
    group = eng.cache.groups[0]
    assert group.k.shape[-1] == KEY_DIM and group.v.shape[-1] == VALUE_DIM
    assert eng.cuda_graphs is False                                   # the mixer reads on the host
    prompts = [random_ids(n, 61, 40 + n) for n in (150, 70, 90)]
    want = [_wide_reference(w, p, 2) for p in prompts]
    # two sequences at a time, the third in the slot and pages the first gives back
    a, b = eng.acquire(), eng.acquire()
    got_a = [eng.step([a], [prompts[0][:100]], [list(range(100))])]
    out = eng.step([a, b], [prompts[0][100:140], prompts[1][:60]], [list(range(40)), list(range(60))])
    got_a.append(out[:40]); got_b = [out[40:]]
    for t in range(10):
        out = eng.step([a, b], [[prompts[0][140 + t]], [prompts[1][60 + t]]])
        got_a.append(out[0:1]); got_b.append(out[1:2])
    eng.release(a)
    c = eng.acquire()
    assert c == a
    got_c = [eng.step([c], [prompts[2]], [list(range(90))])]
    eng.release(b); eng.release(c)
    for got, ref in ((got_a, want[0]), (got_b, want[1]), (got_c, want[2])):
        assert rel_err(torch.cat(got), ref) < 2e-5
    assert all(n == g.n_pages for n, g in zip(eng.cache.free_pages(), eng.cache.groups))
    eng.check_status()
    eng.cache.check_canaries()
