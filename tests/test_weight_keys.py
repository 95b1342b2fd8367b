"""`weights.safetensors` keys: this package's parameter names against the module paths the reference's store writes.

The reference saves through Burn's SafeTensors store with enum variants skipped (`summa-llm/src/model/weights.rs:41-46,
69-75`), so a key is the chain of struct FIELD names down to the parameter. The expected names below are spelled from
those struct definitions, not from this package: `transformer.rs:367-375` (embedding, layers, final_norm, lm_head,
tied_output_bias), `block.rs:25-31` (attention, ssm, feed_forward, memory, attn_norm, ffn_norm), `attention.rs:43-48`
(qkv_proj, o_proj, q_norm, k_norm), `mamba.rs:28-37` (in_proj, conv1d, x_proj, dt_proj, a_log, d, out_proj),
`ffn.rs:35-61,149-152,450-452` (in_proj, down_proj, moe.router, moe.experts.in_weight / down_weight [/ in_bias /
down_bias], moe.shared_experts.N), `memory.rs:155-161,297,657-658,700` (tiers.N.feed_forward, tiers.N.reserve.slots.K
with router, a, b, active, generation); leaf names are Burn's (`Linear`: weight `[in, out]`, bias; `RmsNorm`: gamma;
`LayerNorm`: gamma, beta; `Embedding`: weight; `Conv1d`: weight `[channels, 1, kernel]`, bias)."""
import torch

from summa_b200 import mal
from summa_b200.models import Transformer

MAL = """
  attention a { num_heads: 4 num_kv_heads: 2 qk_norm: true bias: true }
  ssm s { state_dim: 8 conv_kernel: 4 expand: 2 }
  ffn f { hidden_dim: 64 bias: true }
  ffn fm { hidden_dim: 64 moe { experts: 4 top_k: 2 shared_experts: 1 } }
  memory mm {
    tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
    tier slow { ffn: f residual_init: zero reserve_experts { capacity: 1 rank: 4 top_k: 1 } }
  }
  block b1 { attention: a ffn: fm norm: rmsnorm { eps: 1e-5 } }
  block b2 { ssm: s ffn: f norm: layernorm { eps: 1e-5 } }
  block b3 { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
  model t { vocab_size: 64 max_seq_len: 32 hidden_size: 32 num_layers: 3 pattern: [b1, b2, b3] }"""


def linear(prefix, d_in, d_out, bias):
    out = {f"{prefix}.weight": (d_in, d_out)}
    if bias:
        out[f"{prefix}.bias"] = (d_out,)
    return out


def attention(prefix):
    out = {}
    out.update(linear(f"{prefix}.qkv_proj", 32, 4 * 8 + 2 * 2 * 8, True))
    out.update(linear(f"{prefix}.o_proj", 32, 32, True))
    out.update({f"{prefix}.q_norm.gamma": (8,), f"{prefix}.k_norm.gamma": (8,)})
    return out


def dense_ffn(prefix, bias):
    out = linear(f"{prefix}.in_proj", 32, 128, bias)          # gate and up fused along the output dimension
    out.update(linear(f"{prefix}.down_proj", 64, 32, bias))
    return out


def expected():
    k = {"embedding.weight": (64, 32), "final_norm.gamma": (32,), "lm_head.weight": (32, 64)}
    # block 0: attention + MoE feed-forward, RMSNorm
    k.update({"layers.0.attn_norm.gamma": (32,), "layers.0.ffn_norm.gamma": (32,)})
    k.update(attention("layers.0.attention"))
    k.update(linear("layers.0.feed_forward.moe.router", 32, 4, False))
    k.update({"layers.0.feed_forward.moe.experts.in_weight": (4, 32, 128), "layers.0.feed_forward.moe.experts.down_weight": (4, 64, 32)})
    k.update(dense_ffn("layers.0.feed_forward.moe.shared_experts.0", False))
    # block 1: Mamba mixer + dense feed-forward, LayerNorm
    for n in ("attn_norm", "ffn_norm"):
        k.update({f"layers.1.{n}.gamma": (32,), f"layers.1.{n}.beta": (32,)})
    k.update({"layers.1.ssm.a_log": (64, 8), "layers.1.ssm.d": (64,), "layers.1.ssm.conv1d.weight": (64, 1, 4), "layers.1.ssm.conv1d.bias": (64,)})
    k.update(linear("layers.1.ssm.in_proj", 32, 128, False))
    k.update(linear("layers.1.ssm.x_proj", 64, 2 + 2 * 8, False))
    k.update(linear("layers.1.ssm.dt_proj", 2, 64, True))
    k.update(linear("layers.1.ssm.out_proj", 64, 32, False))
    k.update(dense_ffn("layers.1.feed_forward", True))
    # block 2: attention + memory chain
    k.update({"layers.2.attn_norm.gamma": (32,), "layers.2.ffn_norm.gamma": (32,)})
    k.update(attention("layers.2.attention"))
    for tier, slots in ((0, 2), (1, 1)):
        k.update(dense_ffn(f"layers.2.memory.tiers.{tier}.feed_forward", True))
        for s in range(slots):
            p = f"layers.2.memory.tiers.{tier}.reserve.slots.{s}"
            k.update({f"{p}.router.weight": (32, 1), f"{p}.a": (32, 4), f"{p}.b": (4, 32), f"{p}.active": (1,), f"{p}.generation": (1,)})
    return k


def test_parameter_names_and_shapes_are_the_reference_module_paths(tmp_path):
    model = Transformer(mal.parse_mal(MAL))
    got = {n: tuple(p.shape) for n, p in model.named_parameters()}
    want = expected()
    assert sorted(got) == sorted(want)
    assert got == want
    slot = model.layers[2].memory.tiers[0].reserve.slots[0]
    assert slot.active.dtype == torch.bool and slot.generation.dtype == torch.int64
    # the file this package writes carries exactly those keys, and its strict loader refuses anything else
    from summa_b200.models import weights as W
    path = str(tmp_path / "w.safetensors")
    W.save_safetensors(model, path)
    import json
    import struct
    raw = open(path, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    assert sorted(k for k in header if k != "__metadata__") == sorted(want)
    assert {k: tuple(v["shape"]) for k, v in header.items() if k != "__metadata__"} == want
    W.load_safetensors(Transformer(mal.parse_mal(MAL)), path)


def test_tied_embeddings_drop_the_head_and_keep_an_optional_bias_name():
    tied = Transformer(mal.parse_mal("""
      attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
      block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 64 max_seq_len: 32 hidden_size: 32 num_layers: 1 block: b embeddings { tie_weights: true } }"""))
    names = [n for n, _ in tied.named_parameters()]
    assert "lm_head.weight" not in names and "embedding.weight" in names
    assert all(n == "tied_output_bias" or not n.startswith("tied") for n in names)
