"""Configuration and registry (no GPU)."""
import copy

import pytest

from helpers import TINY_A, TINY_B
from minfer_b200.config.base import ConfigError, LayerCall, ModelPlan, PartSpec
from minfer_b200.config.qwen2 import Qwen2Config
from minfer_b200 import registry
import minfer_b200.models  # noqa: F401  (registers the shipped architecture)


def test_reads_every_key():
    c = Qwen2Config.from_dict(TINY_B)
    assert (c.vocab_size, c.hidden_size, c.num_hidden_layers) == (389, 192, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 2, 32)
    assert c.intermediate_size == 328 and c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5
    assert not c.tie_word_embeddings and c.use_sliding_window
    assert c.eos_token_ids == (3, 5)
    assert [c.layer_window(l) for l in range(3)] == [0, 16, 16]
    assert abs(c.attention_scale - 32 ** -0.5) < 1e-12


def test_defaults_follow_the_reference():
    d = {k: TINY_A[k] for k in ("architectures", "vocab_size", "hidden_size", "num_hidden_layers",
                                "num_attention_heads", "intermediate_size")}
    c = Qwen2Config.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.max_position_embeddings == 32768 and not c.tie_word_embeddings
    assert c.eos_token_ids == ()


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers",
                                 "num_attention_heads", "intermediate_size"])
def test_missing_required_key_is_named(key):
    d = copy.deepcopy(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


@pytest.mark.parametrize("patch, word", [
    ({"hidden_size": 66}, "multiple"), ({"num_key_value_heads": 3}, "multiple"),
    ({"vocab_size": "many"}, "integer"), ({"rms_norm_eps": 0}, "> 0"),
    ({"use_sliding_window": True}, "sliding_window"), ({"hidden_act": "gelu"}, "silu"),
    ({"tie_word_embeddings": "yes"}, "true or false"), ({"head_dim": 8}, "head_dim"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"), ({"eos_token_id": 100000}, "vocabulary"),
])
def test_bad_values_are_refused(patch, word):
    d = copy.deepcopy(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(d)


def test_plan_names_parts_and_sizes_per_layer():
    plan = Qwen2Config.from_dict(TINY_B).plan()
    assert len(plan.layers) == 3 and [c.layer for c in plan.schedule] == [0, 1, 2]
    assert [l.mixer.params["window"] for l in plan.layers] == [0, 16, 16]
    m = plan.layers[0].mixer
    assert m.kind == "attention" and m.params["n_heads"] == 6 and m.params["n_kv_heads"] == 2
    assert m.params["position"].params["theta"] == 1e6
    assert plan.layers[2].feed_forward.params["intermediate_size"] == 328
    assert plan.head_name == "lm_head.weight"
    assert Qwen2Config.from_dict(TINY_A).plan().head_name is None
    assert plan.stop_token_ids == (3, 5)


def test_round_trip_through_to_dict():
    c = Qwen2Config.from_dict(TINY_B)
    again = Qwen2Config.from_dict(c.to_dict())
    assert again == c


def test_registry_picks_the_architecture_and_refuses_unknown_ones():
    cfg = registry.read_config(TINY_A)
    assert isinstance(cfg, Qwen2Config)
    d = dict(TINY_A, architectures=["LlamaForCausalLM"])
    with pytest.raises(registry.UnsupportedArchitecture, match="LlamaForCausalLM.*known.*Qwen2ForCausalLM"):
        registry.read_config(d)
    with pytest.raises(ConfigError, match="architectures"):
        registry.read_config({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_unknown_part_kind_is_refused():
    with pytest.raises(ConfigError, match="no mixer of kind 'hyena'"):
        registry.build_part("mixer", PartSpec("hyena", {}))


def test_schedule_is_checked():
    plan = Qwen2Config.from_dict(TINY_A).plan()

    def with_schedule(s):
        return ModelPlan(**{**plan.__dict__, "schedule": s})

    with_schedule([LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2)]).validate()     # a layer twice
    with_schedule([LayerCall(0, 0), LayerCall(1, 0, writes_cache=False)]).validate()  # shared cache
    with pytest.raises(ConfigError, match="names layer 5"):
        with_schedule([LayerCall(5, 0)]).validate()
    with pytest.raises(ConfigError, match="both write"):
        with_schedule([LayerCall(0, 0), LayerCall(1, 0)]).validate()
    with pytest.raises(ConfigError, match="before"):
        with_schedule([LayerCall(0, 1, writes_cache=False), LayerCall(1, 1)]).validate()
    with pytest.raises(ConfigError, match="no call writes"):
        with_schedule([LayerCall(0, 0), LayerCall(1, 3, writes_cache=False)]).validate()


def test_builder_removes_only_a_librarys_own_old_versions(tmp_path):
    from minfer_b200.kernels.build import remove_old_versions
    names = ["libmf_attention_0123456789abcdef.so", "libmf_attention_fedcba9876543210.so",
             "libmf_attention_prefill_tc_0123456789abcdef.so", "libmf_attention_prefill_0123456789abcdef.so",
             "libmf_attention_0123456789abcdef.so.123.tmp", "notes.txt"]
    for n in names:
        (tmp_path / n).write_bytes(b"")
    remove_old_versions("attention", str(tmp_path / names[0]))
    left = sorted(p.name for p in tmp_path.iterdir())
    assert left == sorted(n for n in names if n != "libmf_attention_fedcba9876543210.so")
