"""Text generation: prefill once, then cached single-token steps.

Semantics follow `summa-llm/src/generate.rs:13-250`: the KV / recurrent state is sized
to `prompt + max_new - 1` (capped at `max_seq_len`); when the cache overflows the last
`max_seq_len / 2` tokens are re-prefilled; temperature <= 0 is greedy (argmax on the
device, one scalar crosses to the host per token); otherwise top-k sampling with a
sign-aware repetition penalty applied once per distinct seen token, driven by a seeded
generator; generation stops at EOS.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class SamplingConfig:
    max_new_tokens: int = 64
    temperature: float = 0.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    seed: int = 0
    stop_at_eos: bool = True


class TextGenerator:
    def __init__(self, model, tokenizer=None, eos_id: Optional[int] = None):
        self.model = model
        self.tokenizer = tokenizer
        self.eos_id = eos_id if eos_id is not None else (tokenizer.eos_id() if tokenizer is not None else None)

    @torch.no_grad()
    def generate_ids(self, prompt: List[int], cfg: SamplingConfig) -> List[int]:
        model = self.model
        dev = model.embedding.weight.device
        max_len = model.cfg.max_seq_len
        if not prompt:
            raise ValueError("prompt must contain at least one token")
        if len(prompt) > max_len:
            prompt = prompt[-max_len:]
        capacity = min(max_len, len(prompt) + max(cfg.max_new_tokens, 1) - 1)
        gen = torch.Generator(device="cpu").manual_seed(cfg.seed)
        tokens = list(prompt)
        out: List[int] = []
        state = model.make_state(1, capacity)
        logits = model.forward_next_logits_with_state(torch.tensor([tokens], device=dev), state)
        for _ in range(cfg.max_new_tokens):
            nxt = self._select(logits[0], tokens, cfg, gen)
            out.append(nxt)
            tokens.append(nxt)
            if cfg.stop_at_eos and self.eos_id is not None and nxt == self.eos_id:
                break
            if len(out) == cfg.max_new_tokens:
                break
            if state.pos + 1 > capacity:
                keep = tokens[-(max_len // 2):]
                capacity = min(max_len, len(keep) + cfg.max_new_tokens - len(out))
                state = model.make_state(1, capacity)
                logits = model.forward_next_logits_with_state(torch.tensor([keep], device=dev), state)
            else:
                logits = model.forward_next_logits_with_state(torch.tensor([[nxt]], device=dev), state)
        return out

    def _select(self, logits: torch.Tensor, seen: List[int], cfg: SamplingConfig, gen) -> int:
        if cfg.temperature <= 0.0 and cfg.repetition_penalty == 1.0:
            return int(torch.argmax(logits))
        if logits.is_cuda and 0 <= cfg.top_k <= 64:
            # device path: penalty, temperature and top-k in one kernel; the uniform draw comes from
            # the seeded host generator so a (seed, prompt) pair stays reproducible
            from .. import ops
            bm = ops.seen_bitmap([seen], logits.shape[-1], logits.device) if cfg.repetition_penalty != 1.0 else None
            u = torch.rand(1, generator=gen).to(logits.device) if cfg.temperature > 0.0 else None
            return int(ops.sample_rows(logits.reshape(1, -1), bm, u, cfg.repetition_penalty, cfg.temperature, cfg.top_k)[0])
        lf = logits.float().cpu().clone()
        if cfg.repetition_penalty != 1.0:
            ids = torch.tensor(sorted(set(seen)), dtype=torch.long)
            v = lf[ids]
            lf[ids] = torch.where(v > 0, v / cfg.repetition_penalty, v * cfg.repetition_penalty)
        if cfg.temperature <= 0.0:
            return int(torch.argmax(lf))
        lf = lf / cfg.temperature
        if cfg.top_k and cfg.top_k < lf.numel():
            vals, idx = torch.topk(lf, cfg.top_k)
            probs = torch.softmax(vals, dim=-1)
            return int(idx[torch.multinomial(probs, 1, generator=gen)])
        probs = torch.softmax(lf, dim=-1)
        return int(torch.multinomial(probs, 1, generator=gen))

    def generate(self, prompt: str, cfg: SamplingConfig) -> str:
        ids = self.tokenizer.encode(prompt, False)
        out = self.generate_ids(ids, cfg)
        if out and self.eos_id is not None and out[-1] == self.eos_id:
            out = out[:-1]
        return self.tokenizer.decode(out)
