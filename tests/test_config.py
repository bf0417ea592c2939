"""Configuration and registry (no GPU)."""
import json

import pytest

from lgml_b200.config import (ConfigError, LlamaConfig, ModelConfig, architectures, config_from_dict, load_config,
                              lookup_architecture, register_architecture)
from tests import helpers as H


def test_llama_defaults_follow_the_reference():
    d = {"architectures": ["LlamaForCausalLM"], "vocab_size": 100, "hidden_size": 96, "intermediate_size": 50,
         "num_hidden_layers": 1, "num_attention_heads": 6, "rms_norm_eps": 1e-5, "max_position_embeddings": 64}
    c = config_from_dict(d)
    assert c.num_key_value_heads == 6            # defaults to the heads
    assert c.head_dim == 16                      # hidden // heads
    assert c.rope_theta == 10000.0
    assert c.rope_scaling is None and not c.tie_word_embeddings and not c.attention_bias and not c.mlp_bias


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_round_trip(which):
    cfg, _ = H.TINY[which]
    c = config_from_dict(cfg)
    again = config_from_dict(json.loads(json.dumps(c.to_dict())))
    assert again == c
    assert c.head_dim == cfg["head_dim"] and c.vocab_size == cfg["vocab_size"]


def test_head_width_may_differ_from_hidden():
    c = config_from_dict(H.TINY_B)
    assert c.num_attention_heads * c.head_dim == 192 != c.hidden_size


def test_rope_parameters_style():
    d = dict(H.TINY_B)
    rs = d.pop("rope_scaling")
    theta = d.pop("rope_theta")
    d["rope_parameters"] = dict(rs, rope_theta=theta)
    assert config_from_dict(d) == config_from_dict(H.TINY_B)
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": 1234.0}
    c = config_from_dict(d)
    assert c.rope_theta == 1234.0 and c.rope_scaling is None


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "rms_norm_eps", "max_position_embeddings"])
def test_missing_key_is_named(key):
    d = dict(H.TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"vocab_size": 0}, "vocab_size"),
])
def test_bad_values_are_refused(change, match):
    with pytest.raises(ConfigError, match=match):
        config_from_dict({**H.TINY_A, **change})


def test_unknown_architecture_is_named():
    with pytest.raises(ConfigError, match="MambaForCausalLM"):
        config_from_dict({**H.TINY_A, "architectures": ["MambaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in H.TINY_A.items() if k != "architectures"})
    assert "LlamaForCausalLM" in architectures()


def test_load_config_errors(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(H.TINY_B))
    assert isinstance(load_config(tmp_path), LlamaConfig)


def test_eos_forms():
    assert config_from_dict({**H.TINY_A, "eos_token_id": 7}).eos_token_ids == [7]
    assert config_from_dict({**H.TINY_A, "eos_token_id": [7, 9]}).eos_token_ids == [7, 9]


def test_registry_takes_a_new_architecture():
    class Toy(ModelConfig):
        @classmethod
        def from_dict(cls, d):
            return cls(architecture="ToyForTest")

        def validate(self):
            pass

    register_architecture("ToyForTest", Toy, lambda cfg: "model")
    cls, builder = lookup_architecture("ToyForTest")
    assert cls is Toy and builder(None) == "model"
    assert config_from_dict({"architectures": ["ToyForTest"]}).architecture == "ToyForTest"


def test_k_ranges_of_a_small_product_are_never_empty():
    """The number of K ranges a product is cut into: every range gets at least one block (9 ranges
    of 8 blocks would leave the ninth of 64 blocks empty).  A block is 64 elements up to 64 tokens
    and a stage of 128 from 65 tokens on, where the product runs on pairs of CTAs; many tokens
    and many tiles leave K whole."""
    from lgml_b200.ops import tcgen05_splits

    for M in (1, 8, 16, 17, 64, 65, 128, 200, 256, 300, 2048):
        for N in (1024, 3072, 4096, 5120, 6144, 9216, 14336, 28672, 128256):
            for K in (64, 512, 3072, 4096, 5120, 8192, 13824, 14336):
                s = tcgen05_splits(M, N, K)
                blocks = -(-K // (64 if M <= 64 else 128))
                per = -(-blocks // s)
                assert 1 <= s <= (16 if M <= 64 else 8) and (s - 1) * per < blocks, (M, N, K, s)
                if M > 64 and s > 1:
                    assert per >= 4                         # no range shorter than four stages
                if M >= 2048 and N >= 3072:
                    assert s == 1


def test_key_ranges_of_the_decode_attention_stay_within_their_bounds():
    """The rule that cuts a token's keys into ranges: at least one range, never more than the
    merge kernel takes, no range shorter than four pages, never more CTAs than fill the SMs twice
    (once for one or two short requests), and one range from 37 requests on 8 KV heads up."""
    from lgml_b200.ops import decode_splits, sm_count

    for n in (1, 2, 3, 4, 8, 16, 37, 64, 256):
        for kv, group in ((8, 4), (40, 1), (1, 12), (5, 9)):
            for ctx in (1, 64, 65, 1024, 4096, 16384, 32768, 131072, 1 << 20):
                s = decode_splits(n, kv, group, ctx)
                pages = -(-ctx // 64)
                ctas = n * kv * ((group + 7) // 8)
                assert 1 <= s <= 512
                assert s == 1 or -(-pages // s) >= 4 or s * 4 <= pages + 3, (n, kv, group, ctx, s)
                assert s == 1 or s * ctas <= 2 * sm_count(), (n, kv, group, ctx, s)
    assert decode_splits(37, 8, 4, 4096) == 1 and decode_splits(1, 8, 4, 4096) == 16 and decode_splits(2, 8, 4, 4096) == 9


def test_end_tokens_of_generation_config_join_those_of_config(tmp_path):
    import json

    from lgml_b200.config import ConfigError, load_config
    from tests import helpers as H

    d = dict(H.TINY_B, eos_token_id=7)
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert load_config(tmp_path).eos_token_ids == [7]
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [9, 7, 11], "temperature": 0.6}))
    assert load_config(tmp_path).eos_token_ids == [7, 9, 11]
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 3}))
    assert load_config(tmp_path).eos_token_ids == [7, 3]
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": "x"}))
    with pytest.raises(ConfigError, match="eos_token_id"):
        load_config(tmp_path)
