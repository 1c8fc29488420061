"""The product kernels at the layer sizes of the headline configuration (Qwen2.5-7B shape:
hidden 3584, 28 heads / 4 KV heads of 128, intermediate 18944, vocabulary 152064), two
layers deep: the bfloat16 engine (tcgen05 GEMMs, tensor-core attention, CUDA graphs) against
the float32 engine (FP32-pipe kernels only) on the same weights, for a prompt long enough to
take the CTA-pair GEMM, then decoding in a batch of unequal lengths."""
import pytest
import torch

from helpers import random_ids, rel_err

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "vocab_size": 152064, "hidden_size": 3584,
    "num_hidden_layers": 2, "num_attention_heads": 28, "num_key_value_heads": 4,
    "intermediate_size": 18944, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 32768,
}


def test_bfloat16_engine_matches_float32_engine_at_real_sizes():
    from minfer_b200.engine.step import Engine
    from minfer_b200.model import Model
    lens = (300, 1, 70)
    prompts = [random_ids(n, CONFIG["vocab_size"], 31 + n) for n in lens]
    feed = [random_ids(12, CONFIG["vocab_size"], 77 + i) for i in range(3)]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        # the same bfloat16-rounded weights in both engines (float32 holds them exactly)
        model = Model.from_config(CONFIG, seed=5, dtype=dtype, device="cuda:0",
                                  store_dtype="bfloat16", make_on="device")
        eng = Engine(model, max_tokens=1024, max_seqs=4)
        slots = [eng.acquire() for _ in prompts]
        rows = [eng.step(slots, prompts, [[0, n - 1] for n in lens])]
        for t in range(12):
            live = [b for b in range(3) if t < (12 if b != 1 else 5)]    # row 1 ends earlier
            rows.append(eng.step([slots[b] for b in live], [[feed[b][t]] for b in live]))
        eng.check_status()
        outs[dtype] = torch.cat(rows).float().cpu()
        del eng, model
        torch.cuda.empty_cache()
    assert outs["bfloat16"].shape == outs["float32"].shape
    assert torch.isfinite(outs["bfloat16"]).all()
    assert rel_err(outs["bfloat16"], outs["float32"]) < 2.5e-2
    # the argmax agrees wherever the float32 margin is larger than the tolerance
    top2 = outs["float32"].topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.05 * outs["float32"].abs().max()
    assert torch.equal(outs["bfloat16"].argmax(-1)[clear], outs["float32"].argmax(-1)[clear])
