"""Model trace bundle (`summa_model_trace` version 1) for the visualisation lab, in the reference's shape.

A bounded diagnostic pass over at most `token_limit` tokens (the LAST ones of prompt + continuation)
records, per stage (`embedding`, one `block` per layer, `final_norm`): a row-binned activation heat-map
(`channel_limit` signed channel-bin means per token), tensor statistics, per-token RMS and the RMS of
the change against the previous stage; for attention layers the probability maps of the first
`attention_head_limit` heads; for Mamba layers the final recurrent state binned over channels. The
bundle also carries the architecture (`model.layers[]`), the decoded prompt / continuation with the
sampling settings, an evenly sub-sampled copy of a metrics journal (`training`) and what was cut
(`capture`). Field names, nesting and the binning / sub-sampling arithmetic follow
`summa-llm/src/trace.rs:61-268` (structures) and `:272-800` (capture), so the reference's Model Lab
reads these files and this package's lab reads the reference's.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

import torch

TRACE_KIND = "summa_model_trace"
TRACE_VERSION = 1
MAX_TOKENS = 128          # default token limit (kept as a module constant for the lab server)


@dataclass
class TraceOptions:
    token_limit: int = 128
    channel_limit: int = 64
    attention_head_limit: int = 4
    metrics_row_limit: int = 2000

    def validate(self) -> None:
        if self.token_limit <= 0:
            raise ValueError("trace token limit must be positive")
        if self.channel_limit <= 0:
            raise ValueError("trace channel limit must be positive")
        if self.attention_head_limit <= 0:
            raise ValueError("trace attention-head limit must be positive")
        if self.metrics_row_limit < 2:
            raise ValueError("trace metrics-row limit must be at least 2")


@dataclass
class TraceGeneration:
    max_new_tokens: int = 0
    temperature: float = 0.0
    top_k: Optional[int] = None
    repetition_penalty: float = 1.0
    seed: int = 0
    stop_at_eos: bool = True


# ---------------------------------------------------------------------------- helpers
def _bin_bounds(b: int, bins: int, columns: int):
    start = b * columns // bins
    end = max((b + 1) * columns // bins, start + 1)
    return start, end


def _channel_labels(columns: int, bins: int) -> List[str]:
    out = []
    for b in range(bins):
        s, e = _bin_bounds(b, bins, columns)
        out.append(str(s) if e == s + 1 else f"{s}..{e - 1}")
    return out


def _finite(values: torch.Tensor, name: str) -> torch.Tensor:
    v = values.detach().float().cpu()
    if not bool(torch.isfinite(v).all()):
        raise ValueError(f"{name} contains non-finite values")
    return v


def _heatmap(values: List[float], rows: int, cols: int, row_labels, col_labels, kind: str, orig_rows: int, orig_cols: int):
    return {"rows": rows, "cols": cols, "row_labels": list(row_labels), "col_labels": list(col_labels), "values": values,
            "min": min(values), "max": max(values), "value_kind": kind, "original_rows": orig_rows,
            "original_cols": orig_cols}


def _row_binned(x: torch.Tensor, channel_limit: int, row_labels: Sequence[str]):
    """`[rows, cols]` -> heat-map of `min(cols, channel_limit)` signed bin means per row."""
    rows, cols = x.shape
    bins = min(cols, channel_limit)
    cols_out = [x[:, s:e].mean(dim=1) for s, e in (_bin_bounds(b, bins, cols) for b in range(bins))]
    red = torch.stack(cols_out, dim=1)
    return _heatmap(red.reshape(-1).tolist(), rows, bins, row_labels, _channel_labels(cols, bins), "signed_mean", rows, cols)


def _stats(x: torch.Tensor) -> Dict[str, float]:
    lo, hi = float(x.min()), float(x.max())
    return {"mean": float(x.mean()), "rms": float(x.pow(2).mean().sqrt()), "min": lo, "max": hi,
            "abs_max": max(abs(lo), abs(hi))}


def visible_token(piece: str) -> str:
    v = piece.replace(" ", "·").replace("Ġ", "·").replace("▁", "·").replace("\n", "↵").replace("\r", "⏎").replace("\t", "⇥")
    if len(v) > 18:
        return v[:18] + "…"
    return v if v else "∅"


def _stage(stage: str, label: str, layer_index: Optional[int], mixer: Optional[str], x: torch.Tensor,
           previous: Optional[torch.Tensor], token_labels, channel_limit: int):
    v = _finite(x[0], label)
    out: Dict[str, Any] = {"stage": stage, "label": label}
    if layer_index is not None:
        out["layer_index"] = layer_index
    if mixer is not None:
        out["mixer"] = mixer
    out["activation"] = _row_binned(v, channel_limit, token_labels)
    out["stats"] = _stats(v)
    out["token_rms"] = v.pow(2).mean(dim=1).sqrt().tolist()
    if previous is not None:
        out["token_delta_rms"] = (v - previous).pow(2).mean(dim=1).sqrt().tolist()
    return out, v


def model_trace(cfg) -> Dict[str, Any]:
    """`model` member: the resolved architecture, one entry per layer (one-based `index`)."""
    pattern_len = len(cfg.pattern) if getattr(cfg, "pattern", None) else None
    layers = []
    for i in range(cfg.num_layers):
        b = cfg.block_for_layer(i)
        if b.ssm is not None:
            mixer = {"kind": "mamba", "state_dim": b.ssm.state_dim, "conv_kernel": b.ssm.conv_kernel,
                     "expand": b.ssm.expand, "dt_rank": cfg.dt_rank(b.ssm), "inner_size": b.ssm.expand * cfg.hidden_size}
        else:
            a = b.attention
            heads = a.num_heads
            mixer = {"kind": "attention", "num_heads": heads, "num_kv_heads": a.num_kv_heads or heads,
                     "head_dim": a.head_dim or cfg.hidden_size // heads, "causal": a.causal}
            if a.window_size is not None:
                mixer["window_size"] = a.window_size
            mixer["qk_norm"] = bool(a.qk_norm)
            mixer["position_encoding"] = a.position_encoding.kind
        ffn = b.ffn if b.ffn is not None else (b.memory.tiers[0].ffn if b.memory is not None else None)
        layer = {"index": i + 1, "name": b.name}
        if pattern_len:
            layer["pattern_index"] = i % pattern_len
        layer.update({"mixer": mixer,
                      "ffn_hidden_size": (ffn.hidden_dim or 4 * cfg.hidden_size) if ffn is not None else 0,
                      "ffn_activation": ffn.activation if ffn is not None else "none",
                      "ffn_gated": bool(ffn.gate) if ffn is not None else False,
                      "norm": b.norm.norm_type, "norm_position": b.norm_position, "residual": bool(b.residual),
                      "dropout": float(b.dropout)})
        layers.append(layer)
    out = {"name": cfg.name}
    if getattr(cfg, "description", None):
        out["description"] = cfg.description
    out.update({"vocab_size": cfg.vocab_size, "max_seq_len": cfg.max_seq_len, "hidden_size": cfg.hidden_size,
                "num_layers": cfg.num_layers, "estimated_parameters": cfg.estimated_params(),
                "tied_embeddings": bool(cfg.embeddings.tie_weights), "layers": layers})
    return out


def selected_rows(total: int, limit: int) -> List[int]:
    """Evenly spaced row indices that always keep the first and the last row."""
    if total <= limit:
        return list(range(total))
    return sorted({round(i * (total - 1) / (limit - 1)) for i in range(limit)})


def load_training_trace(path: str, row_limit: int) -> Dict[str, Any]:
    with open(path, "r", encoding="utf-8") as f:
        lines = [l for l in f if l.strip()]
    if not lines:
        raise ValueError(f"metrics file {path} is empty")
    rows_all = []
    for i, line in enumerate(lines):
        try:
            v = json.loads(line)
        except json.JSONDecodeError as e:
            raise ValueError(f"metrics line {i + 1} of {path} is not JSON: {e}")
        if not isinstance(v, dict):
            raise ValueError(f"metrics line {i + 1} of {path} is not an object")
        rows_all.append(v)
    keep = selected_rows(len(rows_all), row_limit)
    rows = [rows_all[i] for i in keep]
    return {"source": path, "total_rows": len(rows_all), "captured_rows": len(rows),
            "dropped_rows": len(rows_all) - len(rows),
            "sampling_stride": 0.0 if len(rows) <= 1 else (len(rows_all) - 1) / (len(rows) - 1), "rows": rows}


@torch.no_grad()
def forward_diagnostic(model, tokens: torch.Tensor, head_limit: int) -> Dict[str, Any]:
    """One forward pass that keeps what the lab draws: the embedding, every block's output, the attention
    probabilities of the first `head_limit` heads, every Mamba mixer's final state, and the final norm."""
    from ..ops import reference
    dev = tokens.device
    x = model.embed(tokens)
    rope = model.rope(dev)
    n_tok = tokens.shape[1]
    out: Dict[str, Any] = {"embedding": x, "layers": []}
    for blk in model.layers:
        entry: Dict[str, Any] = {}
        state = None
        if blk.attention is not None:
            a = blk.attention
            n = blk.attn_norm(x) if blk.pre_norm else x
            q, k, _ = a._split(a.qkv_proj(n).float())
            cos, sin = rope if (a.use_rope and rope is not None) else (None, None)
            qg = a.q_norm.gamma if a.q_norm is not None else None
            kg = a.k_norm.gamma if a.k_norm is not None else None
            q, k = reference.qk_norm_rope(q, k, qg, kg, a.eps, cos, sin, 0)
            g = a.num_heads // a.num_kv_heads
            mask = reference.attention_mask(n_tok, n_tok, a.causal, a.window, 0, dev)
            heads = []
            for h in range(min(head_limit, a.num_heads)):
                s = (q[0, :, h] @ k[0, :, h // g].t()) / math.sqrt(a.head_dim)
                if mask is not None:
                    s = s.masked_fill(mask, float("-inf"))
                heads.append(torch.softmax(s, dim=-1))
            entry["attention_weights"] = torch.stack(heads)
            entry["total_attention_heads"] = a.num_heads
        else:
            state = blk.ssm.make_state(1, dev, x.dtype)
        x, _ = blk(x, rope, state, None)
        if state is not None:
            entry["mamba_state"] = state.h           # [1, d_inner, N]
        entry["activation"] = x
        out["layers"].append(entry)
    out["final_norm"] = model.final_norm(x)
    return out


@torch.no_grad()
def capture_bundle(model, tokenizer, prompt: str, prompt_token_count: int, output_tokens: Sequence[int],
                   generation: Optional[TraceGeneration] = None, metrics_path: Optional[str] = None,
                   options: Optional[TraceOptions] = None) -> Dict[str, Any]:
    """`output_tokens` = prompt tokens followed by the generated continuation."""
    options = options or TraceOptions()
    options.validate()
    generation = generation or TraceGeneration()
    output_tokens = [int(t) for t in output_tokens]
    if not output_tokens:
        raise ValueError("cannot trace an empty token sequence")
    if prompt_token_count > len(output_tokens):
        raise ValueError(f"prompt token count {prompt_token_count} exceeds output token count {len(output_tokens)}")
    cfg = model.cfg
    limit = min(options.token_limit, cfg.max_seq_len)
    captured = min(len(output_tokens), limit)
    offset = len(output_tokens) - captured
    ids = output_tokens[offset:]
    tokens = []
    for j, t in enumerate(ids):
        piece = tokenizer.id_to_token(t) if tokenizer is not None else None
        piece = piece if piece is not None else str(t)
        shown = tokenizer.decode([t]) if tokenizer is not None else piece
        tokens.append({"original_index": offset + j, "id": t, "piece": piece, "display": visible_token(shown),
                       "source": "prompt" if offset + j < prompt_token_count else "generated"})
    labels = [f"{t['original_index']}:{t['display']}" for t in tokens]
    dev = model.embedding.weight.device
    raw = forward_diagnostic(model, torch.tensor([ids], device=dev), options.attention_head_limit)

    stages = []
    st, prev = _stage("embedding", "Token embedding", None, None, raw["embedding"], None, labels, options.channel_limit)
    stages.append(st)
    for i, layer in enumerate(raw["layers"]):
        mixer = "mamba" if cfg.block_for_layer(i).ssm is not None else "attention"
        st, prev = _stage("block", f"Layer {i + 1} · {mixer}", i + 1, mixer, layer["activation"], prev, labels,
                          options.channel_limit)
        if "attention_weights" in layer:
            w = _finite(layer["attention_weights"], "attention weights")
            st["attention"] = {"total_heads": layer["total_attention_heads"], "captured_heads": w.shape[0],
                               "heads": [_heatmap(w[h].reshape(-1).tolist(), captured, captured, labels, labels,
                                                  "probability", captured, captured) for h in range(w.shape[0])]}
        if "mamba_state" in layer:
            s = _finite(layer["mamba_state"][0], "Mamba recurrent state")        # [channels, N]
            channels, n_state = s.shape
            bins = min(channels, options.channel_limit)
            red = torch.stack([s[a:b].mean(dim=0) for a, b in (_bin_bounds(x, bins, channels) for x in range(bins))], dim=1)
            st["mamba_state"] = _heatmap(red.reshape(-1).tolist(), n_state, bins, [f"state {j}" for j in range(n_state)],
                                         _channel_labels(channels, bins), "signed_mean", n_state, channels)
        stages.append(st)
    st, _ = _stage("final_norm", "Final norm", None, None, raw["final_norm"], prev, labels, options.channel_limit)
    stages.append(st)

    training = load_training_trace(metrics_path, options.metrics_row_limit) if metrics_path else None
    gen_tokens = output_tokens[prompt_token_count:]
    sampling = {"max_new_tokens": generation.max_new_tokens, "temperature": float(generation.temperature)}
    if generation.top_k is not None:
        sampling["top_k"] = generation.top_k
    sampling.update({"repetition_penalty": float(generation.repetition_penalty), "seed": int(generation.seed),
                     "stop_at_eos": bool(generation.stop_at_eos)})
    dec = (lambda t: tokenizer.decode(t, True)) if tokenizer is not None else (lambda t: " ".join(map(str, t)))
    bundle: Dict[str, Any] = {
        "kind": TRACE_KIND, "version": TRACE_VERSION, "model": model_trace(cfg),
        "inference": {"prompt": prompt, "generated_text": dec(gen_tokens), "full_text": dec(output_tokens),
                      "original_token_count": len(output_tokens), "prompt_token_count": prompt_token_count,
                      "generated_token_count": len(gen_tokens), "token_offset": offset, "tokens": tokens,
                      "sampling": sampling, "stages": stages}}
    if training is not None:
        bundle["training"] = training
    capture = {"requested_token_limit": options.token_limit, "original_tokens": len(output_tokens),
               "captured_tokens": captured, "dropped_leading_tokens": offset, "tokens_truncated": offset > 0,
               "original_hidden_channels": cfg.hidden_size,
               "captured_hidden_channels": min(cfg.hidden_size, options.channel_limit),
               "channels_reduced": cfg.hidden_size > options.channel_limit,
               "requested_attention_head_limit": options.attention_head_limit}
    if training is not None:
        capture["metrics_total_rows"] = training["total_rows"]
        capture["metrics_captured_rows"] = training["captured_rows"]
    bundle["capture"] = capture
    return bundle


def validate_bundle(b: Dict[str, Any]) -> Dict[str, Any]:
    """The checks the lab's viewer applies before drawing (`summa-model-lab/src/trace-utils.js` `validateTrace`):
    kind / version, a model header whose layer list matches `num_layers`, token rows, and stages whose
    heat-maps are rectangular with one row per captured token."""
    if not isinstance(b, dict) or b.get("kind") != TRACE_KIND:
        raise ValueError(f"trace kind must be {TRACE_KIND}")
    if b.get("version") != TRACE_VERSION:
        raise ValueError(f"unsupported trace version {b.get('version')}")
    m = b.get("model") or {}
    if not isinstance(m.get("name"), str) or len(m.get("layers") or []) != m.get("num_layers"):
        raise ValueError("model header is inconsistent")
    inf = b.get("inference") or {}
    n = len(inf.get("tokens") or [])
    if n == 0 or n != (b.get("capture") or {}).get("captured_tokens"):
        raise ValueError("token rows do not match the capture record")
    stages = inf.get("stages") or []
    if len(stages) != m["num_layers"] + 2 or stages[0]["stage"] != "embedding" or stages[-1]["stage"] != "final_norm":
        raise ValueError("stage list must be embedding, one block per layer, final_norm")
    for s in stages:
        maps = [s["activation"]] + list((s.get("attention") or {}).get("heads", []))
        if s.get("mamba_state") is not None:
            maps.append(s["mamba_state"])
        for h in maps:
            if len(h["values"]) != h["rows"] * h["cols"] or len(h["row_labels"]) != h["rows"] or len(h["col_labels"]) != h["cols"]:
                raise ValueError(f"heat-map of stage `{s['label']}` is not rectangular")
        if s["activation"]["rows"] != n or len(s["token_rms"]) != n:
            raise ValueError(f"stage `{s['label']}` does not have one row per token")
    return b
