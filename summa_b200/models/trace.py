"""Model trace bundle (`summa_model_trace` v1) for the visualisation lab: a bounded
diagnostic pass (<= 128 tokens, <= 64 channel bins, <= 4 heads) that records per-layer
residual-stream statistics, attention maps and top next-token candidates
(`summa-llm/src/trace.rs:23-68,272-571`, `docs/llm-visualization-lab.md:41-60`)."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

MAX_TOKENS, MAX_BINS, MAX_HEADS, TOP_CANDIDATES = 128, 64, 4, 8


def _bins(x: torch.Tensor, bins: int) -> List[List[float]]:
    """[S, H] → [S, bins] mean absolute activation per channel bin."""
    S, H = x.shape
    b = min(bins, H)
    edges = [round(i * H / b) for i in range(b + 1)]
    cols = [x[:, edges[i]:edges[i + 1]].abs().mean(dim=1) for i in range(b)]
    return torch.stack(cols, dim=1).tolist()


@torch.no_grad()
def capture_bundle(model, tokens: List[int], tokenizer=None, metrics: Optional[List[Dict[str, Any]]] = None) -> Dict[str, Any]:
    from ..ops import reference
    cfg = model.cfg
    toks = tokens[:MAX_TOKENS]
    dev = model.embedding.weight.device
    x = model.embed(torch.tensor([toks], device=dev))
    rope = model.rope(dev)
    layers = []
    for i, blk in enumerate(model.layers):
        entry: Dict[str, Any] = {"index": i, "mixer": "ssm" if blk.ssm is not None else "attention"}
        if blk.attention is not None:
            a = blk.attention
            n = blk.attn_norm(x) if blk.pre_norm else x
            qkv = a.qkv_proj(n).float()
            q, k, _ = a._split(qkv)
            cos, sin = rope if (a.use_rope and rope is not None) else (None, None)
            qg = a.q_norm.gamma if a.q_norm is not None else None
            kg = a.k_norm.gamma if a.k_norm is not None else None
            q, k = reference.qk_norm_rope(q, k, qg, kg, a.eps, cos, sin, 0)
            g = a.num_heads // a.num_kv_heads
            heads = []
            for h in range(min(MAX_HEADS, a.num_heads)):
                s = (q[0, :, h] @ k[0, :, h // g].t()) / math.sqrt(a.head_dim)
                m = reference.attention_mask(len(toks), len(toks), a.causal, a.window, 0, dev)
                if m is not None:
                    s = s.masked_fill(m, float("-inf"))
                heads.append(torch.softmax(s, dim=-1).tolist())
            entry["attention"] = heads
        x, _ = blk(x, rope, None, None)
        xf = x[0].float()
        entry["residual_norm"] = xf.norm(dim=-1).tolist()
        entry["channels"] = _bins(xf, MAX_BINS)
        layers.append(entry)
    h = model.final_norm(x)
    logits = (h[0, -1].float() @ model.output_weight().float())[:cfg.vocab_size]
    probs = torch.softmax(logits, dim=-1)
    top = torch.topk(probs, min(TOP_CANDIDATES, cfg.vocab_size))
    cands = [{"id": int(i), "probability": float(p),
              "text": tokenizer.decode([int(i)]) if tokenizer is not None else None}
             for p, i in zip(top.values, top.indices)]
    return {"format": "summa_model_trace", "version": 1,
            "model": {"name": cfg.name, "hidden_size": cfg.hidden_size, "num_layers": cfg.num_layers,
                      "vocab_size": cfg.vocab_size, "parameters": cfg.estimated_params()},
            "tokens": [{"id": t, "text": tokenizer.decode([t]) if tokenizer is not None else None} for t in toks],
            "layers": layers, "next_token": cands, "metrics": (metrics or [])[-2048:]}
