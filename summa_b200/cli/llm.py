"""`python -m summa_b200.cli.llm <command>`: generate, trace, lab, info, export
(`summa-llm/src/main.rs:235-539`)."""
from __future__ import annotations

import argparse
import json
import os
import sys


def _load(args, need_weights=True):
    import torch
    from .. import mal
    from ..models import Transformer
    from ..models import weights as W
    from ..tokenizer import Tokenizer
    from ..utils.remote import resolve
    tok = Tokenizer.from_file(resolve(args.tokenizer)) if getattr(args, "tokenizer", None) else None
    cfg = mal.load_model_def(resolve(args.model))
    if tok is not None:
        if cfg.vocab_size != tok.vocab_size() and not getattr(args, "adopt_tokenizer_vocab", True):
            raise SystemExit(f"tokenizer vocabulary {tok.vocab_size()} != model vocabulary {cfg.vocab_size}")
        cfg.vocab_size = tok.vocab_size()
    model = Transformer(cfg)
    if need_weights and getattr(args, "weights", None):
        W.load_safetensors(model, resolve(args.weights))
    if need_weights and getattr(args, "archive", None):
        from ..models.quantized import load_archive
        load_archive(model, args.archive)
    dev = torch.device(getattr(args, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = model.to(dev).eval()
    if dev.type == "cuda":
        model.prepare_inference(torch.bfloat16)
    return model, tok, cfg


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="summa-llm")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("generate", "trace", "lab"):
        p = sub.add_parser(name)
        p.add_argument("--model", "--config", dest="model", required=True)
        p.add_argument("--tokenizer", "-t", required=True)
        p.add_argument("--weights", "--checkpoint", "-c", dest="weights")
        p.add_argument("--archive", help="directory written by `summa_b200.cli.train quantize`")
        p.add_argument("--device")
        if name != "lab":
            p.add_argument("--prompt", "-p", required=True)
        if name in ("generate", "trace"):
            p.add_argument("--max-new-tokens", "--max-tokens", "-m", dest="max_new_tokens", type=int, default=64 if name == "generate" else 16)
            p.add_argument("--no-eos", action="store_true", help="keep decoding past the end-of-sequence token")
            p.add_argument("--temperature", type=float, default=0.0)
            p.add_argument("--top-k", type=int, default=0)
            p.add_argument("--repetition-penalty", type=float, default=1.0)
            p.add_argument("--seed", type=int, default=0)
        if name == "trace":
            p.add_argument("--output", "-o", required=True)
            p.add_argument("--metrics")
            p.add_argument("--token-limit", "--trace-tokens", dest="token_limit", type=int, default=128)
            p.add_argument("--channel-limit", "--channel-bins", dest="channel_limit", type=int, default=64)
            p.add_argument("--attention-head-limit", "--attention-heads", dest="attention_head_limit", type=int, default=4)
            p.add_argument("--metrics-row-limit", "--metrics-points", dest="metrics_row_limit", type=int, default=2000)
        if name == "lab":
            p.add_argument("--port", type=int, default=8787)
            p.add_argument("--static")
            p.add_argument("--metrics")
    i = sub.add_parser("info")
    i.add_argument("--model", required=True)
    e = sub.add_parser("export")
    e.add_argument("--model", required=True)
    e.add_argument("--output", required=True)
    args = ap.parse_args(argv)

    if args.cmd == "info":
        from .. import mal
        cfg = mal.load_model_def(args.model)
        print(json.dumps({"name": cfg.name, "parameters": cfg.estimated_params(), "hidden_size": cfg.hidden_size,
                          "num_layers": cfg.num_layers, "vocab_size": cfg.vocab_size,
                          "padded_vocab_size": cfg.padded_vocab_size(), "max_seq_len": cfg.max_seq_len,
                          "presets": mal.list_wellknown_models()}))
        return 0
    if args.cmd == "export":
        from .. import mal
        mal.load_model_def(args.model).save_json(args.output)
        return 0
    model, tok, cfg = _load(args)
    if args.cmd == "generate":
        from ..models.generate import SamplingConfig, TextGenerator
        gen = TextGenerator(model, tok)
        text = gen.generate(args.prompt, SamplingConfig(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
                                                        repetition_penalty=args.repetition_penalty, seed=args.seed,
                                                        stop_at_eos=not args.no_eos))
        print(text)
        return 0
    if args.cmd == "trace":
        from ..models.generate import SamplingConfig, TextGenerator
        from ..models.trace import TraceGeneration, TraceOptions, capture_bundle
        prompt_ids = tok.encode(args.prompt, False)
        sc = SamplingConfig(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
                            repetition_penalty=args.repetition_penalty, seed=args.seed, stop_at_eos=not args.no_eos)
        new_ids = TextGenerator(model, tok).generate_ids(prompt_ids, sc) if args.max_new_tokens > 0 else []
        bundle = capture_bundle(model, tok, args.prompt, len(prompt_ids), prompt_ids + new_ids,
                                TraceGeneration(args.max_new_tokens, args.temperature, args.top_k or None,
                                                args.repetition_penalty, args.seed, not args.no_eos),
                                args.metrics, TraceOptions(args.token_limit, args.channel_limit,
                                                           args.attention_head_limit, args.metrics_row_limit))
        os.makedirs(os.path.dirname(os.path.abspath(args.output)), exist_ok=True)
        with open(args.output, "w") as f:
            json.dump(bundle, f, indent=2)
        return 0
    if args.cmd == "lab":
        from ..models.lab import make_server
        from ..models.lab import DEFAULT_UI
        srv = make_server(model, tok, port=args.port, static_dir=args.static or DEFAULT_UI, metrics_path=args.metrics)
        print(f"lab listening on http://127.0.0.1:{srv.server_address[1]}", flush=True)
        srv.serve_forever()
    return 0


if __name__ == "__main__":
    sys.exit(main())
