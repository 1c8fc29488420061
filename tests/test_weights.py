"""Weights: the safetensors container, loading by name with one error for everything that
is wrong, and the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, make_folder
from minfer_b200.model import Model, write_random_model
from minfer_b200.registry import read_config
from minfer_b200.weights.loader import WeightError, held_dtype, load_weights
from minfer_b200.weights.safetensors_io import Checkpoint, SafetensorsError, load_all, save_file
from minfer_b200.weights.spec import INT_TABLE, MATRIX, VECTOR, TensorSpec


def _model(cfg, dtype="bfloat16"):
    c = read_config(cfg)
    return Model(c.plan(), dtype, c)


def test_container_round_trip_and_agrees_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file as st_save
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "e": torch.zeros(0, 4)}
    path = str(tmp_path / "model.safetensors")
    save_file(tensors, path)
    theirs = load_file(path)                      # their reader, our writer
    for k, v in tensors.items():
        assert theirs[k].dtype == v.dtype and torch.equal(theirs[k], v)
    st_save(tensors, path)                        # their writer, our reader
    ours = load_all(str(tmp_path))
    for k, v in tensors.items():
        assert ours[k].dtype == v.dtype and torch.equal(ours[k], v)


def test_truncated_and_malformed_files_are_refused(tmp_path):
    path = str(tmp_path / "model.safetensors")
    save_file({"a": torch.randn(64, 64)}, path)
    blob = open(path, "rb").read()
    open(path, "wb").write(blob[:len(blob) // 2])
    with pytest.raises(SafetensorsError, match="truncated"):
        Checkpoint(str(tmp_path))
    open(path, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        Checkpoint(str(tmp_path))
    open(path, "wb").write(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="JSON"):
        Checkpoint(str(tmp_path))
    os.remove(path)
    with pytest.raises(SafetensorsError, match="neither"):
        Checkpoint(str(tmp_path))


def test_sharded_checkpoint(tmp_path):
    save_file({"a": torch.ones(2)}, str(tmp_path / "m-1.safetensors"))
    save_file({"b": torch.zeros(3)}, str(tmp_path / "m-2.safetensors"))
    json.dump({"weight_map": {"a": "m-1.safetensors", "b": "m-2.safetensors"}},
              open(tmp_path / "model.safetensors.index.json", "w"))
    got = load_all(str(tmp_path))
    assert sorted(got) == ["a", "b"] and got["b"].shape == (3,)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder("A")
    tensors = load_all(folder)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16)
    tensors["model.layers.0.self_attn.k_proj.bias"] = torch.ones(17)
    tensors["model.embed_tokens.weight"] = torch.ones(256, 64, dtype=torch.int32)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    m = _model(TINY_A)
    with pytest.raises(WeightError) as e:
        load_weights(folder, m.tensor_specs(), torch.bfloat16, "cpu", m.ignorable_tensors())
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.k_proj.bias"]
    assert [w[0] for w in err.wrong_type] == ["model.embed_tokens.weight"]
    text = str(err)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)",
                 "is [17], expected [16]", "wrong types (1)"):
        assert word in text


def test_tied_model_ignores_a_separate_head_and_untied_needs_one():
    folder = make_folder("A")                       # tied
    tensors = load_all(folder)
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    m = _model(TINY_A)
    load_weights(folder, m.tensor_specs(), torch.float32, "cpu", m.ignorable_tensors())
    folder_b = make_folder("B")                     # untied
    tensors = load_all(folder_b)
    del tensors["lm_head.weight"]
    save_file(tensors, os.path.join(folder_b, "model.safetensors"))
    mb = _model(TINY_B)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(folder_b, mb.tensor_specs(), torch.float32, "cpu", mb.ignorable_tensors())


def test_held_precision():
    mat, vec, tab = (TensorSpec("m", (2, 2), MATRIX), TensorSpec("v", (2,), VECTOR),
                     TensorSpec("t", (2,), INT_TABLE))
    bf, f32 = torch.bfloat16, torch.float32
    assert held_dtype(mat, bf, bf) == bf and held_dtype(mat, torch.float16, bf) == bf
    assert held_dtype(mat, f32, bf) == f32          # stored in 32-bit stays so
    assert held_dtype(mat, bf, f32) == f32
    assert held_dtype(vec, bf, bf) == f32 and held_dtype(tab, torch.int64, bf) == torch.int32


def test_random_mode_is_a_function_of_seed_and_name_only(tmp_path):
    a, b, c = str(tmp_path / "a"), str(tmp_path / "b"), str(tmp_path / "c")
    write_random_model(a, TINY_B, 11, "bfloat16")
    write_random_model(b, TINY_B, 11, "bfloat16")
    write_random_model(c, TINY_B, 12, "bfloat16")
    ta, tb, tc = load_all(a), load_all(b), load_all(c)
    assert sorted(ta) == sorted(tb) and all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"])
    # a tensor's values do not depend on what else is made: a model with fewer layers shares them
    small = dict(TINY_B, num_hidden_layers=1)
    d = str(tmp_path / "d")
    write_random_model(d, small, 11, "bfloat16")
    td = load_all(d)
    assert all(torch.equal(td[k], ta[k]) for k in td)
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["architectures"] == ["Qwen2ForCausalLM"] and cfg["sliding_window"] == 16
    assert ta["model.norm.weight"].dtype == torch.bfloat16
    assert abs(float(ta["lm_head.weight"].float().std()) - 0.02) < 0.002
    # in-place random weights equal the folder's
    m = Model.from_config(TINY_B, seed=11, dtype="bfloat16", device="cpu")
    assert torch.equal(m.embedding, ta["model.embed_tokens.weight"])


def test_export_state_dict_returns_what_was_loaded():
    """Packed projections come back under their checkpoint names with the loaded values, in
    both engines (rows alternate gate/up in the bfloat16 one)."""
    import tempfile

    import torch
    from helpers import TINY_B
    from minfer_b200.model import Model, write_random_model
    from minfer_b200.weights.safetensors_io import load_all
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, TINY_B, 3, "bfloat16")
        stored = load_all(folder)
        for dtype in ("bfloat16", "float32"):
            model = Model.from_pretrained(folder, dtype, "cpu")
            got = model.export_state_dict()
            assert set(got) == set(stored)
            for name, t in stored.items():
                assert got[name].shape == t.shape
                assert torch.equal(got[name].float(), t.float()), name
