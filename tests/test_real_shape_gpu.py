"""The product kernels at the layer sizes of the headline configuration (Qwen2.5-7B shape:
hidden 3584, 28 heads / 4 KV heads of 128, intermediate 18944, vocabulary 152064), all 28
layers deep, random weights N(0, 0.02) rounded to bfloat16:

* the plain implementation (float64, run on the GPU as an oracle only) for a short prompt,
  against the float32 engine and the bfloat16 engine;
* the float32 engine (FP32-pipe kernels only) under the three schedules: whole, the last
  tokens one by one, an unequal batch whose rows end at different steps, and a prompt in
  portions;
* the bfloat16 engine (tcgen05 GEMMs, tensor-core attention, CUDA graphs) under the same
  schedules against the float32 engine on the same weights, for a prompt long enough to take
  the CTA-pair GEMM, and for a 2,048-token prompt (the sizes at which that kernel takes two
  token tiles a pair).
"""
import pytest
import torch

import plain_qwen2 as P
from helpers import ROW_RMS_TOL, random_ids, rel_err, row_rms_err

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 152064, "hidden_size": 3584,
    "num_hidden_layers": 28, "num_attention_heads": 28, "num_key_value_heads": 4,
    "intermediate_size": 18944, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 32768,
}
LENS = (300, 1, 70)
DECODE = 12
# float32 against float64 at this depth: 28 layers of sums of up to 18,944 float32 terms, where
# the tiny models' 2e-5 stands for 2-3 layers of sums of a few hundred terms (measured 2.5e-5)
TOL32 = 1e-4


class _AsFloat64(dict):
    """The engine's weights by checkpoint name, widened to float64 one tensor at a time."""

    def __getitem__(self, name):
        return dict.__getitem__(self, name).to(torch.float64)


def _schedules(eng, prompts, feed):
    """Logits of the three schedules and of a prompt in portions, in one fixed order."""
    rows = []
    slots = [eng.acquire() for _ in prompts]
    rows.append(eng.step(slots, prompts, [[0, len(p) - 1] for p in prompts]))      # unequal batch
    for t in range(DECODE):
        live = [b for b in range(len(prompts)) if t < (DECODE if b != 1 else 5)]   # row 1 ends earlier
        rows.append(eng.step([slots[b] for b in live], [[feed[b][t]] for b in live]))
    for s in slots:
        eng.release(s)
    ids = prompts[2] + feed[2]                          # alone: whole, then the last 32 one by one
    s = eng.acquire()
    rows.append(eng.step([s], [ids], [[len(ids) - 33, len(ids) - 1]]))
    eng.release(s)
    s = eng.acquire()
    rows.append(eng.step([s], [ids[:-32]]))
    rows += [eng.step([s], [[t]]) for t in ids[-32:]]
    eng.release(s)
    s = eng.acquire()                                   # in portions of 50 beside a row that decodes
    other = eng.acquire()
    eng.step([other], [prompts[0][:40]])
    for a in range(0, len(ids), 50):
        part = ids[a:a + 50]
        rows.append(eng.step([s, other], [part, [prompts[0][40 + a // 50]]], [[len(part) - 1], [0]]))
    eng.release(s)
    eng.release(other)
    eng.check_status()
    return torch.cat(rows).float().cpu()


def test_all_layers_at_real_sizes():
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    V = CONFIG["vocab_size"]
    prompts = [random_ids(n, V, 31 + n) for n in LENS]
    feed = [random_ids(DECODE, V, 77 + i) for i in range(3)]
    short = random_ids(48, V, 5)
    long_prompt = random_ids(2048, V, 9)                # products with two token tiles a CTA pair
    long_want = [0, 255, 256, 1000, 2047]
    outs, short_out, long_out = {}, {}, {}
    oracle = None
    for dtype in ("float32", "bfloat16"):
        # the same bfloat16-rounded weights in both engines (float32 holds them exactly)
        model = Model.from_config(CONFIG, seed=5, dtype=dtype, device="cuda:0",
                                  store_dtype="bfloat16", make_on="device")
        eng = Engine(model, max_tokens=3072, max_seqs=4)
        if dtype == "float32":
            with torch.no_grad():
                oracle = P.forward(CONFIG, _AsFloat64(model.export_state_dict()), short).cpu()
        s = eng.acquire()
        short_out[dtype] = eng.step([s], [short], [list(range(len(short)))]).cpu()
        eng.release(s)
        outs[dtype] = _schedules(eng, prompts, feed)
        s = eng.acquire()
        long_out[dtype] = eng.step([s], [long_prompt], [long_want]).cpu()
        eng.release(s)
        eng.check_status()
        del eng, model
        torch.cuda.empty_cache()
    # against the plain implementation
    assert rel_err(short_out["float32"], oracle) < TOL32
    assert row_rms_err(short_out["bfloat16"], oracle) < ROW_RMS_TOL
    # the schedules agree with one another in float32 (same sequence, other cuts)
    f32 = outs["float32"]
    n_batch = 2 * len(LENS) + sum(3 if t < 5 else 2 for t in range(DECODE))
    whole = f32[n_batch:n_batch + 2]
    one_by_one = f32[n_batch + 2:n_batch + 2 + 33]
    assert rel_err(one_by_one[[0, 32]], whole) < TOL32
    batch_last = f32[n_batch - 1]                       # row 2 of the last decode step of the batch
    assert rel_err(batch_last, whole[1]) < TOL32
    portions = f32[n_batch + 2 + 33:]
    assert rel_err(portions[-2], whole[1]) < TOL32
    # bfloat16 against float32, every row of every schedule
    assert outs["bfloat16"].shape == f32.shape
    assert torch.isfinite(outs["bfloat16"]).all()
    assert row_rms_err(outs["bfloat16"], f32) < ROW_RMS_TOL
    # a 2,048-token prompt: the bfloat16 engine's products run two token tiles a CTA pair (O,
    # down) and 256-token tiles (q|k|v, gate|up), its attention on tcgen05
    assert row_rms_err(long_out["bfloat16"], long_out["float32"]) < ROW_RMS_TOL
    # the argmax agrees wherever the float32 margin is larger than the tolerance
    top2 = f32.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.05 * f32.abs().max()
    assert torch.equal(outs["bfloat16"].argmax(-1)[clear], f32.argmax(-1)[clear])
