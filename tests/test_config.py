"""Configuration and registry (no GPU)."""
import copy

import pytest

from conftest import TINY_A, TINY_B, TINY_C
from sharpinference_b200.config import ConfigError, Llama4TextConfig
from sharpinference_b200.registry import (get_architecture, known_architectures, register_architecture, resolve,
                                           unregister_architecture)


def test_tiny_a_fields():
    c = Llama4TextConfig.from_dict(TINY_A)
    assert (c.vocab_size, c.hidden_size, c.num_hidden_layers) == (256, 64, 4)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (4, 2, 16)
    assert c.no_rope_layers == (3,) and c.moe_layers == (0, 1, 2, 3)
    assert c.rope_scaling is None and c.attention_chunk_size == 16
    assert c.use_qk_norm and c.qk_norm_eps == 1e-6 and c.attn_temperature_tuning
    assert c.floor_scale == 8.0 and c.attn_scale == 0.1 and c.rms_norm_eps == 1e-5
    assert [c.layer_uses_rope(i) for i in range(4)] == [True, True, True, False]


def test_tiny_b_fields():
    c = Llama4TextConfig.from_dict(TINY_B)
    assert c.moe_layers == (1, 3, 5) and c.no_rope_layers == (2, 5)
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 16
    assert not c.use_qk_norm and not c.attn_temperature_tuning
    assert [c.layer_is_moe(i) for i in range(6)] == [False, True, False, True, False, True]


def test_no_rope_layers_both_forms():
    flags = dict(TINY_A, no_rope_layers=[1, 1, 1, 0])
    index = dict(TINY_A, no_rope_layers=[3])
    assert Llama4TextConfig.from_dict(flags).no_rope_layers == Llama4TextConfig.from_dict(index).no_rope_layers == (3,)
    absent = dict(TINY_A)
    absent.pop("no_rope_layers")
    assert Llama4TextConfig.from_dict(absent).no_rope_layers == (3,)          # every 4th layer
    c = Llama4TextConfig.from_dict(TINY_C)
    assert c.no_rope_layers == (1,) and c.moe_layers == (0, 2) and c.tie_word_embeddings


def test_qk_norm_eps_defaults_to_the_rms_eps_and_an_explicit_key_wins():
    base = dict(TINY_A, rms_norm_eps=3e-5)
    assert Llama4TextConfig.from_dict(base).qk_norm_eps == 1e-6               # Tiny A names its own
    base.pop("qk_norm_eps")
    assert Llama4TextConfig.from_dict(base).qk_norm_eps == 3e-5               # what a checkpoint's file gives
    from conftest import TINY_D
    d = Llama4TextConfig.from_dict(TINY_D)
    assert "qk_norm_eps" not in TINY_D and d.use_qk_norm and d.qk_norm_eps == d.rms_norm_eps == 1e-5


def test_interval_switch_and_whole_floor_scale():
    absent = dict(TINY_B, no_rope_layer_interval=3)
    absent.pop("no_rope_layers")
    assert Llama4TextConfig.from_dict(absent).no_rope_layers == (2, 5)
    # the temperature switch is written as a boolean or as a non-negative integer
    assert Llama4TextConfig.from_dict(dict(TINY_A, attn_temperature_tuning=4)).attn_temperature_tuning is True
    assert Llama4TextConfig.from_dict(dict(TINY_A, attn_temperature_tuning=0)).attn_temperature_tuning is False
    with pytest.raises(ConfigError):
        Llama4TextConfig.from_dict(dict(TINY_A, attn_temperature_tuning="yes"))
    with pytest.raises(ConfigError):
        Llama4TextConfig.from_dict(dict(TINY_A, no_rope_layer_interval=0, no_rope_layers=None))
    out = Llama4TextConfig.from_dict(TINY_A).to_dict()
    assert out["floor_scale"] == 8 and isinstance(out["floor_scale"], int)
    assert Llama4TextConfig.from_dict(dict(TINY_A, floor_scale=2.5)).to_dict()["floor_scale"] == 2.5


def test_explicit_moe_layers_wins():
    c = Llama4TextConfig.from_dict(dict(TINY_B, moe_layers=[0, 4]))
    assert c.moe_layers == (0, 4)


def test_text_config_member_and_round_trip():
    nested = {"architectures": ["Llama4ForConditionalGeneration"], "text_config": dict(TINY_B)}
    arch, c = resolve(nested)
    assert arch.name == "Llama4ForCausalLM"
    assert c == Llama4TextConfig.from_dict(TINY_B)
    assert Llama4TextConfig.from_dict(c.to_dict()) == c


def test_all_problems_in_one_error():
    bad = dict(TINY_A, num_attention_heads=5, num_experts_per_tok=2, head_dim=15)
    bad.pop("vocab_size")
    with pytest.raises(ConfigError) as exc:
        Llama4TextConfig.from_dict(bad)
    text = str(exc.value)
    assert "vocab_size" in text
    bad2 = dict(TINY_A, num_attention_heads=5, num_experts_per_tok=2, head_dim=15)
    with pytest.raises(ConfigError) as exc:
        Llama4TextConfig.from_dict(bad2)
    text = str(exc.value)
    assert "multiple of num_key_value_heads" in text and "num_experts_per_tok" in text and "head_dim" in text


@pytest.mark.parametrize("key,value", [("hidden_size", "64"), ("use_qk_norm", 1), ("rope_theta", "x"),
                                       ("no_rope_layers", [9]), ("moe_layers", [7]), ("attention_chunk_size", 0),
                                       ("hidden_act", "gelu"), ("attention_bias", "yes")])
def test_bad_values(key, value):
    with pytest.raises(ConfigError):
        Llama4TextConfig.from_dict(dict(TINY_A, **{key: value}))


def test_attention_bias_declares_the_bias_tensors():
    from sharpinference_b200.weights.loading import declared_tensors
    c = Llama4TextConfig.from_dict(dict(TINY_A, attention_bias=True))
    assert c.attention_bias and Llama4TextConfig.from_dict(c.to_dict()) == c
    names = {d.name: d.shape for d in declared_tensors(get_architecture("Llama4ForCausalLM"), c)}
    assert names["model.layers.0.self_attn.q_proj.bias"] == (64,) and names["model.layers.3.self_attn.k_proj.bias"] == (32,)
    assert names["model.layers.1.self_attn.o_proj.bias"] == (64,)
    plain = {d.name for d in declared_tensors(get_architecture("Llama4ForCausalLM"), Llama4TextConfig.from_dict(TINY_A))}
    assert not any(n.endswith(".bias") for n in plain)


def test_unsupported_rope_type():
    bad = copy.deepcopy(TINY_B)
    bad["rope_scaling"]["rope_type"] = "yarn"
    with pytest.raises(ConfigError, match="yarn"):
        Llama4TextConfig.from_dict(bad)


def test_registry_unknown_lists_known():
    assert "Llama4ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="Llama4ForCausalLM"):
        get_architecture("NoSuchModel")
    with pytest.raises(ConfigError, match="architectures"):
        resolve({"vocab_size": 3})


def test_registry_accepts_new_architecture():
    class Cfg:
        architecture = "ToyArch"

        @classmethod
        def from_dict(cls, obj, where="config.json"):
            return cls()

    register_architecture("ToyArch", Cfg, lambda config, weights: None)
    try:
        arch, cfg = resolve({"architectures": ["ToyArch"]})
        assert arch.name == "ToyArch" and isinstance(cfg, Cfg)
    finally:
        unregister_architecture("ToyArch")


def test_command_line_keeps_the_reference_option_names():
    from sharpinference_b200.cli import build_parser, parse_prompts
    ns = build_parser().parse_args(["-m", "dir", "-p", "5 17 3; 9,9", "-n", "8", "--temp", "0", "--top-k", "5",
                                    "--top-p", "0.5", "--min-p", "0.1", "-s", "7", "-c", "256", "--rep-penalty", "1.3",
                                    "--repeat-last-n", "32", "--verbose-prompt", "--no-display-prompt"])
    assert (ns.model, ns.n_predict, ns.temp, ns.top_k, ns.top_p, ns.min_p) == ("dir", 8, 0.0, 5, 0.5, 0.1)
    assert (ns.seed, ns.ctx_size, ns.repeat_penalty, ns.repeat_last_n) == (7, 256, 1.3, 32)
    assert ns.verbose_prompt and ns.no_display_prompt
    defaults = build_parser().parse_args([])
    assert (defaults.n_predict, defaults.temp, defaults.top_k, defaults.top_p, defaults.min_p, defaults.seed) == \
        (512, 0.7, 40, 0.95, 0.05, -1)
    assert parse_prompts("5 17 3; 9,9") == [[5, 17, 3], [9, 9]]
    # --device in the reference's spellings (an index, a name) and torch's; --min-batch-blas as there
    from sharpinference_b200.cli import parse_device
    assert [parse_device(t) for t in (None, "auto", "0", "1", "CUDA0", "cuda:2", "cuda3")] == \
        ["cuda:0", "cuda:0", "cuda:0", "cuda:1", "cuda:0", "cuda:2", "cuda:3"]
    assert parse_device("none") is None and parse_device("Vulkan1") is None and parse_device("gpu") is None
    assert defaults.min_batch_blas == 0 and defaults.device is None
    assert build_parser().parse_args(["--min-batch-blas", "9", "--device", "CUDA0"]).min_batch_blas == 9
