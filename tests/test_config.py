"""Configuration: keys, defaults, refusals and the architecture registry."""
import json

import pytest

import kllm_b200.models  # noqa: F401
from kllm_b200.config import (ConfigError, LlamaConfig, build_model_spec, known_architectures, load_config,
                              parse_config, register_architecture)
from helpers import TINY_A, TINY_B


def test_reads_every_key():
    c = parse_config(TINY_B)
    assert isinstance(c, LlamaConfig)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size, c.rope_theta, c.rms_norm_eps, c.max_position_embeddings,
            c.tie_word_embeddings, c.eos_token_ids) == (3, 96, 3, 1, 32, 256, 512, 500000.0, 1e-6, 256, True, (511,))


def test_defaults_follow_the_reference():
    d = {"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 1,
         "num_attention_heads": 4, "vocab_size": 10, "intermediate_size": 8, "max_position_embeddings": 32}
    c = parse_config(d)
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6 and c.eos_token_ids == ()
    assert c.num_key_value_heads == 4 and c.head_dim == 16 and c.tie_word_embeddings is False


def test_rope_parameters_block_and_eos_list():
    d = dict(TINY_A, rope_parameters={"rope_theta": 12345.0, "rope_type": "default"}, eos_token_id=[2, 7])
    c = parse_config(d)
    assert c.rope_theta == 12345.0 and c.eos_token_ids == (2, 7)
    assert parse_config(c.to_dict()) == c


@pytest.mark.parametrize("patch,needle", [
    ({"hidden_size": 0}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8}}, "rope_scaling"),
    ({"rope_parameters": {"rope_theta": 1e4, "rope_type": "yarn"}}, "rope_type"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "bias"),
    ({"intermediate_size": None}, "intermediate_size"),
    ({"vocab_size": 2.5}, "integer"),
    ({"architectures": ["NoSuchModel"]}, "unknown architecture"),
    ({"architectures": []}, "architectures"),
])
def test_refusals(patch, needle):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError) as e:
        parse_config(d)
    assert needle in str(e.value)


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError) as e:
        parse_config({"architectures": ["Foo"]})
    assert "LlamaForCausalLM" in str(e.value)
    assert "LlamaForCausalLM" in known_architectures()


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert load_config(str(tmp_path)).hidden_size == 64
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_spec_carries_every_size_and_the_schedule():
    spec = build_model_spec(parse_config(TINY_B))
    assert len(spec.blocks) == 3 and [c.block for c in spec.schedule] == [0, 1, 2]
    m = spec.blocks[1].mixer
    assert m.kind == "paged_attention" and m.params["n_heads"] == 3 and m.params["n_kv_heads"] == 1
    assert m.params["head_dim"] == 32 and m.params["position"].params["theta"] == 500000.0
    assert spec.blocks[2].feed_forward.params["intermediate"] == 256
    assert spec.final_norm.params["eps"] == 1e-6 and spec.head.params["tied_to"] == "model.embed_tokens.weight"
    assert build_model_spec(parse_config(TINY_A)).head.params["tied_to"] is None


def test_registering_another_architecture():
    from dataclasses import dataclass
    from kllm_b200.config import ModelConfig

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int = 8

        @classmethod
        def from_dict(cls, d):
            return cls(architecture=d["architectures"][0], width=d["width"])

    register_architecture("ToyTestModel", ToyConfig, lambda c: ("spec of", c.width))
    c = parse_config({"architectures": ["ToyTestModel"], "width": 24})
    assert build_model_spec(c) == ("spec of", 24)


def test_bench_shapes_are_configurations_of_the_architecture():
    """The layer sizes that bench.py offers parse as configurations and build a spec."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "kllm_bench", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    from kllm_b200.config.base import build_model_spec, parse_config
    assert "tinyllama-1.1b" in bench.SHAPES and len(bench.SHAPES) >= 3
    for name, d in bench.SHAPES.items():
        cfg = parse_config(dict(d))
        model = build_model_spec(cfg)
        assert len(model.blocks) == len(model.schedule) == d["num_hidden_layers"], name
