"""Each part alone (norm, position encoding, mixer, feed-forward, block) against the plain
implementation's function for it, and models whose run order names a layer twice or lets a
layer read another layer's cache."""
import math

import pytest
import torch

import plain_qwen2 as P
from helpers import TINY_B, TOL, make_folder, random_ids, rel_err
from minfer_b200.parts.base import settle_pending

pytestmark = pytest.mark.gpu


def _ctx(n, dtype, positions=None):
    from minfer_b200.parts.base import StepContext
    dev = torch.device("cuda")
    pos = torch.arange(n, dtype=torch.int32, device=dev) if positions is None else positions
    return StepContext(
        device=dev, act_dtype=dtype, n_tokens=n, n_rows=1,
        token_ids=torch.zeros(n, dtype=torch.int32, device=dev), positions=pos,
        token_row=torch.zeros(n, dtype=torch.int32, device=dev),
        cu_seqlens=torch.tensor([0, n], dtype=torch.int32, device=dev),
        seq_end=torch.tensor([n], dtype=torch.int32, device=dev),
        slots=torch.zeros(1, dtype=torch.int32, device=dev), from_start=True, single_token=n == 1,
        max_row_tokens=n, max_end=n, status=torch.zeros(1, dtype=torch.int32, device=dev))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from minfer_b200.parts.norm import RmsNorm
    part = RmsNorm(size=200, eps=3e-6, name="ln")
    assert [s.name for s in part.tensor_specs("a.")] == ["a.ln.weight"]
    w = 1 + 0.1 * torch.randn(200)
    part.load("a.", {"a.ln.weight": w.cuda()})
    x = torch.randn(9, 200).cuda()
    got = part.forward(x, dtype)
    assert got.dtype == dtype
    assert rel_err(got, P.rms_norm(x.double().cpu(), w.double(), 3e-6)) < (2e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part_adds_into_the_residual(dtype):
    from minfer_b200.parts.mlp import GatedMlp
    part = GatedMlp(hidden_size=72, intermediate_size=200)
    names = [s.name for s in part.tensor_specs("L.")]
    assert names == ["L.mlp.gate_proj.weight", "L.mlp.up_proj.weight", "L.mlp.down_proj.weight"]
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.randn(s.shape, generator=g) * 0.1).to(dtype) for n, s in
         zip(names, part.tensor_specs("L."))}
    part.load("L.", {k: v.cuda() for k, v in w.items()})
    x = torch.randn(11, 72, generator=g).to(dtype)
    h = torch.randn(11, 72, generator=g)
    res = h.clone().cuda()
    ctx = _ctx(11, dtype)
    part.forward_add(x.cuda(), ctx, res)
    settle_pending(ctx, res)            # a split projection may leave its sums for the next norm
    want = h.double() + P.swiglu_mlp(x.double(), *(w[n].double() for n in names))
    assert rel_err(res, want) < (2e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_whole_then_one_token(dtype):
    """The mixer with a cache of its own: a whole prompt, then one more token from the
    cache; both against the plain attention block."""
    from minfer_b200.cache.paged import Cache, GroupKey
    from minfer_b200.config.base import PartSpec
    from minfer_b200.parts.attention import Attention
    from minfer_b200.parts.base import CacheView, CallBinding
    nh, nk, hd, ne, window = 6, 2, 32, 192, 16
    part = Attention(hidden_size=ne, n_heads=nh, n_kv_heads=nk, head_dim=hd, scale=hd ** -0.5,
                     window=window, position=PartSpec("rotary", dict(head_dim=hd, rotary_dim=hd,
                                                                     theta=1e6)))
    specs = part.tensor_specs("model.layers.0.")
    g = torch.Generator().manual_seed(1)
    w = {s.name: (torch.randn(s.shape, generator=g) * 0.08).to(dtype) for s in specs}
    part.load("model.layers.0.", {k: (v.float() if v.dim() == 1 else v).cuda() for k, v in w.items()})
    cfg = dict(TINY_B, num_hidden_layers=1, max_window_layers=0)
    T = 41
    x = torch.randn(T + 1, ne, generator=g).to(dtype)
    want, _ = P.attention_block(cfg, {k: v.double() for k, v in w.items()}, 0, x.double())

    req = part.cache_request()
    cache = Cache({0: GroupKey(req.n_kv_heads, req.head_dim, req.window)}, 256, 2, dtype, "cuda")
    slot = cache.acquire()
    cache.reserve(slot, T + 1)
    grp = cache.groups[0]
    k, v = grp.entry_tensors(0)
    table = torch.tensor(grp.table_rows([slot], 2), dtype=torch.int32, device="cuda")
    view = CacheView(k=k, v=v, page_table=table, table_stride=2, ring=grp.ring)
    res = torch.zeros(T, ne, device="cuda")
    ctx0 = _ctx(T, dtype)
    part.forward_add(x[:T].cuda(), ctx0, CallBinding(cache=view, entry=0), res)
    settle_pending(ctx0, res)
    tolr = 2e-5 if dtype == torch.float32 else 2e-2
    assert rel_err(res, want[:T]) < tolr
    ctx = _ctx(1, dtype, torch.tensor([T], dtype=torch.int32, device="cuda"))
    ctx.from_start = False
    ctx.seq_end = torch.tensor([T + 1], dtype=torch.int32, device="cuda")
    ctx.max_end = T + 1
    res1 = torch.zeros(1, ne, device="cuda")
    part.forward_add(x[T:].cuda(), ctx, CallBinding(cache=view, entry=0), res1)
    settle_pending(ctx, res1)
    assert rel_err(res1, want[T:]) < tolr


def _plain_vs_engine(folder, plan_edit, schedule, dtype, ids):
    from minfer_b200.config.base import ModelPlan
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    from minfer_b200.registry import read_config
    from minfer_b200.weights.loader import load_weights
    import json, os
    raw = json.load(open(os.path.join(folder, "config.json")))
    cfg = read_config(raw)
    plan = plan_edit(cfg.plan())
    model = Model(plan, dtype, cfg)
    w = load_weights(folder, model.tensor_specs(), model.dtype, "cuda:0", model.ignorable_tensors())
    model.bind(w, "cuda:0")
    eng = Engine(model, 1024)
    pcfg, pw = P.load_folder(folder)
    want = P.forward(pcfg, pw, ids, schedule=schedule)
    s = eng.acquire()
    n = len(ids)
    head = n - 20
    rows = [eng.step([s], [ids[:head]], [list(range(head))])]
    rows += [eng.step([s], [[t]]) for t in ids[head:]]
    eng.release(s)
    eng.check_status()
    return rel_err(torch.cat(rows), want)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_names_a_layer_twice(dtype):
    from minfer_b200.config.base import LayerCall, ModelPlan
    folder = make_folder("A")
    sched = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2)]
    err = _plain_vs_engine(folder, lambda p: ModelPlan(**{**p.__dict__, "schedule": sched}),
                           [(0, 0, True), (1, 1, True), (0, 2, True)], dtype,
                           random_ids(90, 256, 3))
    assert err < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_a_layer_reads_another_layer_s_cache(dtype, name):
    """Layer 1 keeps no keys of its own: it attends over what layer 0 wrote (in "C" through
    a windowed ring, with a prompt longer than the ring)."""
    from minfer_b200.config.base import LayerCall, ModelPlan
    folder = make_folder(name)
    sched = [LayerCall(0, 0), LayerCall(1, 0, writes_cache=False)]
    vocab = 256 if name == "A" else 131
    err = _plain_vs_engine(folder, lambda p: ModelPlan(**{**p.__dict__, "schedule": sched}),
                           [(0, 0, True), (1, 0, False)], dtype, random_ids(170, vocab, 4))
    assert err < TOL[dtype]
