"""Configuration and registry (no GPU)."""
import json

import pytest

from helpers import TINY_A, TINY_B, TINY_C
from titan_b200.config import (ConfigError, Qwen3Config, config_from_dict, known_architectures,
                               load_config, register_architecture)


def test_reads_every_size_from_config_json():
    for d in (TINY_A, TINY_B, TINY_C):
        c = config_from_dict(d)
        assert isinstance(c, Qwen3Config)
        assert (c.num_hidden_layers, c.hidden_size, c.intermediate_size) == (d["num_hidden_layers"], d["hidden_size"], d["intermediate_size"])
        assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (d["num_attention_heads"], d["num_key_value_heads"], d["head_dim"])
        assert (c.vocab_size, c.rms_norm_eps, c.rope_theta) == (d["vocab_size"], d["rms_norm_eps"], d["rope_theta"])
        assert c.tie_word_embeddings == d["tie_word_embeddings"]
        assert config_from_dict(c.to_dict()) == c            # round trip


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "num_key_value_heads", "rms_norm_eps", "rope_theta", "max_position_embeddings")}
    c = config_from_dict(d)
    assert c.head_dim == 64 // 4 and c.num_key_value_heads == 4
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0 and c.max_position_embeddings == 4096


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads", "vocab_size"])
def test_missing_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"hidden_act": "gelu"}, "gelu"),
    ({"attention_bias": True}, "attention_bias"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"hidden_size": 2.5}, "integer"), ({"vocab_size": 0}, "positive"), ({"eos_token_id": 999}, "vocabulary"),
    ({"layer_types": ["full_attention"]}, "layer_types"), ({"architectures": ["NopeForCausalLM"]}, "Qwen3ForCausalLM"),
    ({"rope_parameters": {"rope_type": "yarn", "factor": 4.0, "rope_theta": 1e6}}, "rope_parameters"),
    ({"rope_parameters": {"rope_type": "default", "rope_theta": 5.0}}, "disagree"),
    ({"mlp_bias": True}, "mlp_bias"), ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict({**TINY_A, **patch})


def test_frequency_base_in_either_key():
    """Newer files carry the frequency base inside rope_parameters; it is never silently defaulted."""
    d = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    assert config_from_dict({**d, "rope_parameters": {"rope_type": "default", "rope_theta": 123456.0}}).rope_theta == 123456.0
    assert config_from_dict({**d, "rope_theta": 777.0, "rope_scaling": None, "rope_parameters": None}).rope_theta == 777.0
    assert config_from_dict({**d, "rope_theta": 777.0, "rope_scaling": {"rope_type": "default"}}).rope_theta == 777.0
    assert config_from_dict({**TINY_A, "rope_parameters": {"rope_theta": TINY_A["rope_theta"]}}).rope_theta == TINY_A["rope_theta"]


def test_windows_per_layer():
    c = config_from_dict(TINY_C)
    assert c.layer_windows == (20, None, 20, 20)
    d = {**TINY_A, "use_sliding_window": True, "sliding_window": 8, "max_window_layers": 1}
    assert config_from_dict(d).layer_windows == (None, 8)
    assert config_from_dict({**TINY_A, "sliding_window": 8}).layer_windows == (None, None)   # not switched on


def test_model_spec_is_data():
    spec = config_from_dict(TINY_C).to_model_spec()
    assert spec.order == (0, 1, 2, 3) and len(spec.layers) == 4
    assert [l.mixer.window for l in spec.layers] == [20, None, 20, 20]
    assert spec.layers[0].mixer.kind == "attention" and spec.layers[0].feed_forward.kind == "gated_mlp"
    assert spec.layers[0].mixer.position.theta == 500000.0 and spec.layers[0].mixer.qk_norm.eps == 3e-6
    assert spec.lm_head == "lm_head.weight" and config_from_dict(TINY_A).to_model_spec().lm_head is None


def test_order_and_cache_sharing_are_checked():
    import dataclasses
    spec = config_from_dict(TINY_A).to_model_spec()
    with pytest.raises(ConfigError, match="order"):
        dataclasses.replace(spec, order=(0, 5)).validate()
    shared = dataclasses.replace(spec.layers[0], mixer=dataclasses.replace(spec.layers[0].mixer, cache_from=1))
    with pytest.raises(ConfigError, match="before it is written"):
        dataclasses.replace(spec, layers=(shared, spec.layers[1])).validate()
    dataclasses.replace(spec, order=(0, 1, 1, 0)).validate()      # a layer may run twice


def test_a_reader_must_fit_the_cache_it_reads():
    """A layer that reads another layer's cache must see exactly what the owner keeps: same kind of mixer, same
    window (a full-attention reader over a ring would read rows that were overwritten), same head size, a
    number of query heads that the owner's kv heads divide; and it must run, after its owner."""
    import dataclasses
    spec = config_from_dict(TINY_A).to_model_spec()
    l0, l1 = spec.layers
    reader = lambda **kw: dataclasses.replace(l1, mixer=dataclasses.replace(l1.mixer, cache_from=0, **kw))
    dataclasses.replace(spec, layers=(l0, reader())).validate()
    windowed = dataclasses.replace(l0, mixer=dataclasses.replace(l0.mixer, window=8))
    with pytest.raises(ConfigError, match="window"):
        dataclasses.replace(spec, layers=(windowed, reader())).validate()
    with pytest.raises(ConfigError, match="heads of"):
        dataclasses.replace(spec, layers=(l0, reader(head_dim=32))).validate()
    with pytest.raises(ConfigError, match="query heads"):
        dataclasses.replace(spec, layers=(l0, reader(num_heads=3))).validate()
    with pytest.raises(ConfigError, match="another kind"):
        dataclasses.replace(spec, layers=(dataclasses.replace(l0, mixer=dataclasses.replace(l0.mixer, kind="something_else")), reader())).validate()
    with pytest.raises(ConfigError, match="never runs"):
        dataclasses.replace(spec, layers=(l0, reader()), order=(0,)).validate()
    with pytest.raises(ConfigError, match="owns none"):
        dataclasses.replace(spec, layers=(dataclasses.replace(l0, mixer=dataclasses.replace(l0.mixer, cache_from=1)), reader())).validate()


def test_tensor_names_come_from_the_spec():
    """Which tensors a part binds is its spec's business: the defaults are this architecture's names, another
    checkpoint layout (a fused q|k|v tensor, a fused gate|up tensor, other names) is a matter of the spec."""
    import dataclasses
    from titan_b200.parts import declare_weights
    spec = config_from_dict(TINY_A).to_model_spec()
    names = [w.name for w in declare_weights(spec)]
    assert "model.layers.0.self_attn.q_proj.weight" in names and "model.layers.1.mlp.gate_proj.weight" in names
    l0 = spec.layers[0]
    fused = dataclasses.replace(l0, mixer=dataclasses.replace(l0.mixer, names=(("qkv", "wqkv.weight"), ("o", "wo.weight"))),
                                feed_forward=dataclasses.replace(l0.feed_forward, names=(("gate_up", "w13.weight"), ("down", "w2.weight"))))
    by_name = {w.name: w.shape for w in declare_weights(dataclasses.replace(spec, layers=(fused, spec.layers[1])))}
    assert by_name["model.layers.0.self_attn.wqkv.weight"] == ((4 + 2 * 2) * 16, 64)
    assert by_name["model.layers.0.self_attn.wo.weight"] == (64, 64)
    assert by_name["model.layers.0.mlp.w13.weight"] == (256, 64) and by_name["model.layers.0.mlp.w2.weight"] == (64, 128)
    assert not any("layers.0.self_attn.q_proj" in n or "layers.0.mlp.up_proj" in n for n in by_name)


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(str(tmp_path)).vocab_size == 509
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))


def test_registering_another_architecture():
    class Other:
        @classmethod
        def from_dict(cls, d):
            return cls()

        def to_model_spec(self):
            return None
    register_architecture("OtherForCausalLM", Other)
    assert "OtherForCausalLM" in known_architectures()
    assert isinstance(config_from_dict({"architectures": ["OtherForCausalLM"]}), Other)
