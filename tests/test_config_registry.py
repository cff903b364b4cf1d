"""Typed configuration and the architecture registry (no GPU)."""
import copy

import pytest

import tiny_configs
from easy_gpt.cpp_b200 import model_spec_from_config, resolve_architecture
from easy_gpt.cpp_b200.config.qwen2 import ConfigError, Qwen2Config
from easy_gpt.cpp_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def test_reads_every_key():
    c = Qwen2Config.from_dict(tiny_configs.CONFIG_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 80, 6, 2)
    assert c.head_dim == 32 and c.intermediate_size == 208 and c.vocab_size == 391
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings
    assert c.eos_token_id == 7 and c.bos_token_id == -1
    assert [c.layer_window(i) for i in range(3)] == [None, 24, 24]


def test_defaults_follow_the_reference():
    # head size = hidden / heads (src/models/self_attn.cpp:169-174), eps 1e-6 (src/models/norm.cpp:41),
    # bos/eos -1 (include/config.hpp:22-23)
    d = {k: v for k, v in tiny_configs.CONFIG_A.items() if k not in ("rms_norm_eps", "bos_token_id", "eos_token_id")}
    c = Qwen2Config.from_dict(d)
    assert c.head_dim == 16 and c.rms_norm_eps == 1e-6 and c.eos_token_id == -1 and c.bos_token_id == -1
    assert c.attention_bias and not c.attention_out_bias and not c.mlp_bias


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "rope_theta", "max_position_embeddings"])
def test_missing_key_is_an_error(key):
    d = copy.deepcopy(tiny_configs.CONFIG_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


@pytest.mark.parametrize("patch, text", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_size": 66}, "divisible"),
    ({"head_dim": 15}, "even"),
    ({"rope_theta": 0.0}, "rope_theta"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"vocab_size": 2.5}, "integer"),
])
def test_bad_values_are_refused(patch, text):
    d = copy.deepcopy(tiny_configs.CONFIG_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=text):
        Qwen2Config.from_dict(d)


def test_registry_rule():
    # src/models/layer_key_prefix.cpp:24-28: substring of architectures[0], or model_type equal, case-insensitive
    assert resolve_architecture({"architectures": ["Qwen2ForCausalLM"]}).key == "qwen2"
    assert resolve_architecture({"architectures": ["x"], "model_type": "QWEN2"}).key == "qwen2"
    with pytest.raises(ValueError, match="architecture='LlamaForCausalLM', model_type='llama'"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_spec_is_built_from_parts():
    spec = model_spec_from_config(tiny_configs.CONFIG_B)
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    l1 = spec.layers[1]
    assert l1.mixer.kind == "attention" and l1.mixer.params["window"] == 24 and l1.mixer.params["head_dim"] == 32
    assert l1.mixer.prefix == "model.layers.1.self_attn"          # src/models/layer_key_prefix.cpp:77-87
    assert l1.feed_forward.kind == "swiglu" and l1.feed_forward.params["intermediate_size"] == 208
    assert l1.mixer_norm.params["eps"] == 1e-5 and l1.position.params["theta"] == 1e6
    assert spec.lm_head.params["tied_to"] is None
    assert model_spec_from_config(tiny_configs.CONFIG_A).lm_head.params["tied_to"] == "model.embed_tokens"


def test_run_order_is_checked():
    spec = model_spec_from_config(tiny_configs.CONFIG_A)
    kw = dict(architecture="t", vocab_size=8, hidden_size=8, max_positions=8, layers=spec.layers,
              embedding=spec.embedding, final_norm=spec.final_norm, lm_head=spec.lm_head)
    ModelSpec(run_order=(RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2), RunEntry(1, 0, writes_cache=False)), **kw)
    with pytest.raises(ValueError, match="names layer 5"):
        ModelSpec(run_order=(RunEntry(5, 0),), **kw)
    with pytest.raises(ValueError, match="written by run entries"):
        ModelSpec(run_order=(RunEntry(0, 0), RunEntry(1, 0)), **kw)
    with pytest.raises(ValueError, match="no entry writes"):
        ModelSpec(run_order=(RunEntry(0, 0), RunEntry(1, 3, writes_cache=False)), **kw)
    with pytest.raises(ValueError, match="before entry"):
        ModelSpec(run_order=(RunEntry(0, 1, writes_cache=False), RunEntry(1, 1)), **kw)


def test_a_head_size_beyond_the_kernels_is_refused_when_the_model_is_built():
    import torch

    from easy_gpt.cpp_b200.engine.model import Model

    config = dict(tiny_configs.CONFIG_A, head_dim=272)
    with pytest.raises(ValueError, match="head_dim 272 is outside what the attention kernels take"):
        Model(model_spec_from_config(config), "cpu", torch.float32)
    Model(model_spec_from_config(dict(tiny_configs.CONFIG_A, head_dim=256)), "cpu", torch.float32)
