"""Configuration and registry: typed reading of config.json keys, defaults, errors that name the key."""
import copy
import json

import pytest

from burn_lm_b200 import ConfigError, LlamaConfig, architecture, architecture_of, list_architectures, plan_of
from burn_lm_b200.config import read_config_json
from tiny import CONFIGS, TINY_A, TINY_B


def test_reads_every_key():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 192, 6, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 512, 384)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-6 and not c.tie_word_embeddings
    s = c.rope_scaling
    assert (s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings) == (8.0, 1.0, 4.0, 64)
    assert c.eos_token_ids == (7, 11) and c.max_position_embeddings == 256


def test_defaults_follow_the_reference():
    d = {"hidden_size": 64, "intermediate_size": 100, "num_hidden_layers": 1, "num_attention_heads": 4, "vocab_size": 10}
    c = LlamaConfig.from_dict(d)
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.rope_scaling is None
    assert not c.tie_word_embeddings


def test_round_trip():
    for cfg in CONFIGS.values():
        c = LlamaConfig.from_dict(cfg)
        assert LlamaConfig.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("key,value,word", [
    ("hidden_size", None, "required"), ("vocab_size", "big", "integer"), ("num_hidden_layers", 0, "at least"),
    ("num_key_value_heads", 3, "divide"), ("rms_norm_eps", -1.0, "positive"), ("hidden_act", "gelu", "silu"),
    ("attention_bias", True, "attention_bias"), ("mlp_bias", True, "mlp_bias"),
    ("tie_word_embeddings", "yes", "true or false"), ("head_dim", 15, "even"),
])
def test_errors_name_the_key(key, value, word):
    d = copy.deepcopy(TINY_A)
    if value is None:
        del d[key]
    else:
        d[key] = value
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(d)
    assert key in str(e.value) and word in str(e.value)


def test_rope_scaling_errors():
    d = copy.deepcopy(TINY_B)
    d["rope_scaling"]["rope_type"] = "yarn"
    with pytest.raises(ConfigError, match="rope_scaling.rope_type"):
        LlamaConfig.from_dict(d)
    d = copy.deepcopy(TINY_B)
    del d["rope_scaling"]["factor"]
    with pytest.raises(ConfigError, match="rope_scaling.factor"):
        LlamaConfig.from_dict(d)


def test_registry_by_name_and_alias():
    assert architecture("LlamaForCausalLM") is architecture("llama")
    assert architecture_of({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert architecture_of({"model_type": "llama"}).name == "LlamaForCausalLM"
    assert any(a.name == "LlamaForCausalLM" for a in list_architectures())
    with pytest.raises(ConfigError, match="registered"):
        architecture("MambaForCausalLM")
    with pytest.raises(ConfigError, match="names no architecture"):
        architecture_of({})


def test_plan_takes_every_size_from_the_configuration():
    _, cfg, plan = plan_of(TINY_B)
    assert len(plan.layers) == 3 and [e.layer for e in plan.schedule] == [0, 1, 2]
    a = plan.layers[1].part("mixer").spec
    assert (a.n_heads, a.n_kv_heads, a.head_dim, a.hidden_size) == (6, 1, 32, 192)
    assert a.position.spec.theta == 500000.0 and a.position.spec.scaling.factor == 8.0
    assert plan.layers[0].part("feed_forward").spec.intermediate_size == 512
    assert plan.final_norm.spec.eps == 1e-6
    assert plan.head.tensors["weight"] == "lm_head.weight"
    _, _, plan_a = plan_of(TINY_A)
    assert plan_a.head.tensors["weight"] == "model.embed_tokens.weight"      # tied
    assert plan_a.layers[0].part("mixer").spec.position.spec.scaling is None


def test_read_config_json_errors(tmp_path):
    with pytest.raises(ConfigError, match="no such file"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert read_config_json(str(tmp_path))["hidden_size"] == 64


def test_schedule_is_checked():
    from burn_lm_b200.plan import ModelPlan, ScheduleEntry
    _, _, plan = plan_of(TINY_A)
    import dataclasses
    with pytest.raises(ValueError, match="names layer"):
        dataclasses.replace(plan, schedule=(ScheduleEntry(5),))
    with pytest.raises(ValueError, match="does not run before"):
        dataclasses.replace(plan, schedule=(ScheduleEntry(0, cache_of=0),))
    ok = dataclasses.replace(plan, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1)))
    assert len(ok.schedule) == 4


def test_presets_are_the_reference_sizes():
    """crates/burn-lm-llama/src/nn/llama/base.rs:75-123 and the benchmark configurations."""
    from burn_lm_b200.config import LlamaConfig, preset, preset_names, ConfigError
    assert {"llama3_2_1b", "llama3_2_3b", "llama3_1_8b", "tiny_a", "tiny_b"} <= set(preset_names())
    one = LlamaConfig.from_dict(preset("llama3_2_1b"))
    assert (one.num_hidden_layers, one.hidden_size, one.num_attention_heads, one.num_key_value_heads, one.head_dim,
            one.intermediate_size, one.vocab_size, one.tie_word_embeddings) == (16, 2048, 32, 8, 64, 8192, 128256, True)
    assert one.rope_theta == 500000.0 and one.rope_scaling.factor == 32.0 and one.rope_scaling.original_max_position_embeddings == 8192
    assert one.eos_token_ids == (128001, 128008, 128009)
    three = LlamaConfig.from_dict(preset("Llama3.2-3B"))
    assert (three.num_hidden_layers, three.hidden_size, three.num_attention_heads, three.head_dim) == (28, 3072, 24, 128)
    eight = LlamaConfig.from_dict(preset("llama3_1_8b"))
    assert (eight.num_hidden_layers, eight.hidden_size, eight.intermediate_size, eight.rope_scaling.factor,
            eight.tie_word_embeddings) == (32, 4096, 14336, 8.0, False)
    p = preset("tiny_a")
    p["hidden_size"] = 1
    assert preset("tiny_a")["hidden_size"] == 64         # a fresh copy every time
    with pytest.raises(ConfigError, match="no preset"):
        preset("llama9")


def test_a_position_encoding_that_wants_a_score_bias_is_refused():
    """The attention kernels compute q.k * scale and the mask; an encoding that biases the scores per head cannot
    be given to the attention mixer and says so when the model is built."""
    import dataclasses
    import torch
    from burn_lm_b200 import register_part
    from burn_lm_b200.parts import AttentionSpec, Part
    from burn_lm_b200.parts.attention import Attention
    from burn_lm_b200.parts.base import Runtime
    from burn_lm_b200.plan import PartPlan
    from burn_lm_b200 import registry

    @register_part("position", "toy_slopes", replace=True)
    class Slopes(Part):
        family = "position"

        def rotation(self):
            return None, 0, False

        def score_bias(self):
            return [2.0 ** -(h + 1) for h in range(4)]

    try:
        spec = AttentionSpec(64, 4, 2, 16, PartPlan("toy_slopes", None))
        with pytest.raises(ValueError, match="bias on the attention scores"):
            Attention(spec, {"q": "q", "k": "k", "v": "v", "o": "o"}, Runtime(torch.float32, torch.device("cpu")))
    finally:
        registry.unregister_part("position", "toy_slopes")
