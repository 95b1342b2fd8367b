"""MAL parser, defaults, JSON form, presets, parameter estimator, validation."""
import json

import pytest

from summa_b200 import mal


def test_presets_parse_and_param_counts():
    names = mal.list_wellknown_models()
    for n in ["nano", "tiny", "llama_7b", "mistral_7b", "retriever_100m", "retriever_300m_moe_sleep"]:
        assert n in names
    assert abs(mal.get_builtin_model("retriever_100m").estimated_params() - 115.8e6) < 0.1e6
    assert abs(mal.get_builtin_model("llama_7b").estimated_params() - 6.738e9) < 5e6
    m = mal.get_builtin_model("retriever-100m")
    assert m.pattern and len(m.pattern) == 3 and m.pattern[0].is_ssm() and not m.pattern[2].is_ssm()
    assert m.padded_vocab_size() == 50304 and m.embeddings.tie_weights


def test_defaults_and_aliases():
    m = mal.parse_mal("""
        # comment
        model x-1 { d_model: 256 n_layers: 3 context_length: 99
          block: { attention: { n_heads: 4 kv_heads: 2 position_encoding: rope { base: 5e5 rope_scaling: 2.0 } }
                   ffn: { intermediate_size: 512 activation: gelu_tanh gate: false } norm: layernorm { norm_eps: 1e-6 }
                   norm_position: post } }
    """)
    assert (m.name, m.hidden_size, m.num_layers, m.max_seq_len, m.vocab_size) == ("x-1", 256, 3, 99, 32000)
    b = m.block
    assert b.num_heads() == 4 and b.num_kv_heads() == 2 and b.head_dim(256) == 64
    assert b.rope_theta() == 5e5 and b.rope_scaling() == 2.0
    assert b.ffn.activation == "gelu_tanh" and not b.ffn.gate and b.norm.norm_type == "layernorm"
    assert b.norm_eps() == 1e-6 and b.norm_position == "post"
    d = mal.ModelDef()
    assert d.block.num_heads() == 12 and d.block.intermediate_size(768) == 3072 and d.block.norm_eps() == 1e-5


def test_json_roundtrip_uses_serde_enum_encoding():
    m = mal.get_builtin_model("retriever_300m_moe_sleep")
    j = m.to_json()
    assert j["block"]["attention"]["position_encoding"] == {"Rope": {"theta": 100000.0, "scaling": None}}
    assert j["block"]["norm"]["norm_type"] == "RmsNorm" and j["block"]["ffn"]["activation"] == "SwiGLU"
    assert j["pattern"][1]["memory"]["tiers"][1]["residual_init"] == "ResidualZero"
    m2 = mal.ModelDef.from_json(json.dumps(j))
    assert m2.to_json() == j and m2.estimated_params() == m.estimated_params()


@pytest.mark.parametrize("src,msg", [
    ("attention a { } attention a { }", "duplicate attention"),
    ("block b { attention: nope }", "undefined attention"),
    ("model m { pattern: [x] }", "undefined block"),
    ("attention a { }", "no model"),
    ("model a { } model b { }", "multiple model"),
    ("model m { bogus: 1 }", "unknown property"),
    ("model m { vocab_size: 1.5 }", "expected integer"),
    ("memory mm { tier t { reserve_experts { capacity: 1 rank: 2 top_k: 1 } } }", "requires an ffn"),
])
def test_errors(src, msg):
    with pytest.raises(mal.MalError) as e:
        mal.parse_mal(src)
    assert msg in str(e.value)


def test_references_resolve_only_backwards():
    with pytest.raises(mal.MalError):
        mal.parse_mal("block b { ffn: f } ffn f { } model m { block: b }")


def test_model_time_validation():
    from summa_b200.models import validate_config
    bad = mal.parse_mal("model m { hidden_size: 100 block: { attention: { num_heads: 3 } } }")
    with pytest.raises(ValueError):
        validate_config(bad)
    alibi = mal.parse_mal("model m { hidden_size: 64 block: { attention: { num_heads: 2 position_encoding: alibi { slopes: fixed } } } }")
    with pytest.raises(ValueError):
        validate_config(alibi)
    moe = mal.parse_mal("model m { hidden_size: 64 block: { attention: { num_heads: 2 } ffn: { moe { experts: 4 top_k: 5 } } } }")
    with pytest.raises(ValueError):
        validate_config(moe)
