"""Configuration and registry (no device)."""
import pytest

import transformer_b200 as tb
from transformer_b200.config import ConfigError, LlamaMeta, architecture_for, registered_architectures
from tiny import TINY_A, TINY_B, TINY_DENSE


def test_reads_every_size_from_the_file():
    m = LlamaMeta.from_dict(TINY_B)
    assert (m.nblk, m.d, m.nh, m.nkvh, m.dh, m.di) == (3, 96, 3, 1, 32, 80)
    assert (m.nexp, m.nexp_use, m.nctx, m.nvoc) == (6, 3, 256, 384)
    assert m.epsilon == 1e-6 and m.theta == 500000.0 and m.tied and m.rope_pairing == "half"


def test_defaults_are_the_references():
    cfg = {"model_type": "llama", "num_hidden_layers": 1, "hidden_size": 64, "num_attention_heads": 4,
           "intermediate_size": 32, "max_position_embeddings": 16, "vocab_size": 10}
    m = LlamaMeta.from_dict(cfg)
    assert m.nkvh == 4 and m.dh == 16 and m.nexp == 0 and m.nexp_use == 0
    assert m.epsilon == 1e-5 and m.theta == 1e4 and not m.tied and not m.is_moe


def test_gguf_spelling_is_accepted():
    cfg = {"general.architecture": "llama", "llama.block_count": 2, "llama.embedding_length": 64,
           "llama.attention.head_count": 4, "llama.attention.head_count_kv": 2, "llama.feed_forward_length": 128,
           "llama.expert_count": 4, "llama.expert_used_count": 2, "llama.context_length": 128,
           "llama.vocab_size": 256, "llama.rope.freq_base": 10000.0}
    m = LlamaMeta.from_dict(cfg)
    assert m.is_moe and m.dh == 16 and architecture_for(cfg).name == "llama"


def test_round_trip():
    for cfg in (TINY_A, TINY_B, TINY_DENSE):
        m = LlamaMeta.from_dict(cfg)
        assert LlamaMeta.from_dict(m.to_dict()) == m


@pytest.mark.parametrize("change, word", [
    ({"num_hidden_layers": None}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "share"),
    ({"head_dim": 15}, "even"),
    ({"num_experts_per_tok": 9}, "experts per token"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"vocab_size": "many"}, "number"),
    ({"hidden_size": 64.5}, "integer"),
    ({"rope_pairing": "spiral"}, "rope_pairing"),
    ({"attention_bias": True}, "bias"),
    ({"sliding_window": 128}, "window"),
    ({"eos_token_id": 999}, "vocabulary"),
])
def test_bad_configs_are_refused(change, word):
    cfg = dict(TINY_A)
    cfg.update(change)
    with pytest.raises(ConfigError, match=word):
        LlamaMeta.from_dict(cfg)


def test_unknown_architecture_lists_the_known():
    with pytest.raises(ConfigError, match="llama"):
        architecture_for({"model_type": "gpt2"})
    with pytest.raises(ConfigError, match="names no architecture"):
        architecture_for({"hidden_size": 3})
    assert "llama" in registered_architectures()


def test_spec_is_data():
    from transformer_b200.architectures.llama import build_spec
    spec = build_spec(LlamaMeta.from_dict(TINY_A))
    spec.validate()
    assert len(spec.layers) == 2 and [e.layer for e in spec.order] == [0, 1]
    assert spec.layers[0].mixer.kind == "attention" and spec.layers[0].feed_forward.kind == "moe"
    assert spec.layers[0].feed_forward.get()["nexp"] == 4
    dense = build_spec(LlamaMeta.from_dict(TINY_DENSE))
    assert dense.layers[0].feed_forward.kind == "swiglu"


def test_sample_args_rules():
    tb.SampleArgs(0.0, 1.0, 0)
    tb.SampleArgs(0.8, 0.9, 40)
    for bad in ((-1.0, 1.0, 0), (1.0, 0.0, 0), (1.0, 1.5, 0), (1.0, 1.0, -2), (float("nan"), 1.0, 0)):
        with pytest.raises(tb.SampleArgsError):
            tb.SampleArgs(*bad)
