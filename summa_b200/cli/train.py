"""`python -m summa_b200.cli.train <command>`: the training-side command line.

Commands mirror the reference binary (`summa-train/src/main.rs:116-216`): train, eval,
generate-eval, validate-workflow, run-workflow, verify-checkpoint, quantize,
upgrade-memory-checkpoint.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="summa-train")
    sub = ap.add_subparsers(dest="cmd", required=True)

    t = sub.add_parser("train")
    t.add_argument("--model", "--config", dest="model", required=True, help=".mal / ModelDef .json / preset name")
    t.add_argument("--tokenizer", required=True)
    t.add_argument("--workflow", required=True)
    t.add_argument("--output", required=True)
    t.add_argument("--lr", type=float, default=3e-4)
    t.add_argument("--weight-decay", type=float, default=0.1)
    t.add_argument("--clip", "--grad-clip", dest="clip", type=float, default=1.0)
    t.add_argument("--warmup", "--warmup-steps", dest="warmup", type=int, default=1000)
    t.add_argument("--layer-metrics-every", type=int, default=0,
                   help="record the pre-clip gradient L2 norm of every layer every N optimizer steps; 0 disables")
    t.add_argument("--schedule", choices=["wsd", "cosine"], default="wsd")
    t.add_argument("--checkpoint-every", type=int, default=500)
    t.add_argument("--seed", type=int, default=42)
    t.add_argument("--checkpoint")
    t.add_argument("--resume", action="store_true")
    t.add_argument("--optimizer", choices=["adamw", "muon"], default="muon")
    t.add_argument("--device")
    t.add_argument("--max-steps", type=int)
    t.add_argument("--print-run-signature", action="store_true")
    t.add_argument("--gpu-metrics-interval-ms", type=int, default=None,
                   help="nvidia-smi sampling period; 0 disables (default: 1000 on CUDA, disabled elsewhere)")
    t.add_argument("--gpu-physical-device", default="0", help="physical index, GPU UUID or PCI bus id for nvidia-smi")
    t.add_argument("--sleep-runtime", help="sleep-runtime JSON (periodic shape) of a memory-enabled model; needs --sleep-runtime-sha256")
    t.add_argument("--sleep-runtime-sha256", help="`sha256:` identity of the --sleep-runtime file's bytes")
    t.add_argument("--no-token-cache", action="store_true", help="tokenise causal data on every epoch instead of replaying <output>/.token-cache/")

    v = sub.add_parser("validate-workflow")
    v.add_argument("workflow_path", nargs="?", metavar="workflow")
    v.add_argument("--workflow", help="same as the positional argument")
    v.add_argument("--config", "--model", dest="model", help="MAL model: also check the workflow against this exact topology")
    v.add_argument("--signature-only", action="store_true", help="print the workflow signature alone; nothing is written")

    c = sub.add_parser("verify-checkpoint", help="verify an exact-resume checkpoint with the trainer's strict schema")
    c.add_argument("output", nargs="?", help="same as --root")
    c.add_argument("--root", help="checkpoint output root containing current.json and generations/")
    c.add_argument("--generation", help="a materialised immutable generation directory")
    c.add_argument("--generation-name", help="content-addressed sha256-... name of --generation")
    c.add_argument("--manifest-sha256", help="lowercase SHA-256 of --generation's generation-manifest.json")
    c.add_argument("--metrics", help="metric journal whose committed checkpoint prefix must be valid")
    c.add_argument("--exact-metrics", action="store_true", help="the journal must end exactly at the committed prefix")
    c.add_argument("--format", choices=["json", "tsv"], default="json", help="tsv: step, generation, manifest digest, metric records")

    e = sub.add_parser("eval", help="held-out loss / perplexity / in-batch retrieval metrics as a deterministic JSON report")
    e.add_argument("--config", "--model", dest="model", required=True, help="MAL source or exported JSON model configuration")
    e.add_argument("--tokenizer", "-t", required=True)
    e.add_argument("--checkpoint", required=True, help="safetensors weights, loaded strictly against --config")
    e.add_argument("--data", required=True, action="append", help="held-out shard, repeatable")
    e.add_argument("--objective", choices=["causal_lm", "contrastive_retrieval", "summarization", "instruction_tuning",
                                           "qa_reasoning", "retrieval_planning"])
    e.add_argument("--task", help="a complete task JSON instead of --objective and its options")
    e.add_argument("--sequence-length", type=int, default=512)
    e.add_argument("--batch-size", type=int, default=8)
    e.add_argument("--max-batches", type=int)
    e.add_argument("--shuffle-buffer", type=int, default=0)
    e.add_argument("--seed", type=int, default=0)
    e.add_argument("--recall-k", type=int, default=10)
    e.add_argument("--retrieval-layer", type=int)
    e.add_argument("--temperature", type=float)
    e.add_argument("--instruction")
    e.add_argument("--require-reasoning", action="store_true")
    e.add_argument("--output", "-o", help="JSON report path; the report is also printed")
    e.add_argument("--device")

    rp = sub.add_parser("retrieval-pool-eval", help="rank every query against the global pool of distinct documents")
    rp.add_argument("--config", "--model", dest="model", required=True)
    rp.add_argument("--tokenizer", "-t", required=True)
    rp.add_argument("--checkpoint", required=True)
    rp.add_argument("--data", required=True, action="append", help="query shard (records with document_id), repeatable")
    rp.add_argument("--distractors", action="append", help="shard whose documents only enlarge the pool, repeatable")
    rp.add_argument("--task", help="a retrieval_representation task JSON (prefixes); default: the trainer's defaults")
    rp.add_argument("--sequence-length", type=int, default=512)
    rp.add_argument("--batch-size", type=int, default=32)
    rp.add_argument("--recall-k", type=int, default=10)
    rp.add_argument("--retrieval-layer", type=int)
    rp.add_argument("--output", "-o")
    rp.add_argument("--device")

    pc = sub.add_parser("prepare-corpus")
    pc.add_argument("--recipe", required=True, help="production recipe {corpus (version 2), search_api, postgres?}; or the offline form "
                                                     "{name, queries, page_size?, docs_per_shard?, records: path, search: path} with "
                                                     "records = JSONL {key, text} and search = JSON {query: [keys]}")
    pc.add_argument("--tokenizer", "-t", required=True)
    pc.add_argument("--output", "-o", required=True)
    pc.add_argument("--work-directory", help="restart state of a production build (defaults to a hidden folder beside the output)")
    pc.add_argument("--max-pages", type=int)

    cc = sub.add_parser("compose-curriculum")
    cc.add_argument("--config", help="versioned composition file with a content-pinned source manifest; writes one sealed stage "
                                     "directory per stage under --output")
    cc.add_argument("--work-directory", help="transient stratum spools of --config")
    cc.add_argument("--corpus", help="published corpus directory")
    cc.add_argument("--strata", help='JSON list: [{"name", "weight", "label": {"key": "value"}}]; '
                                                    "an empty label matches everything")
    cc.add_argument("--token-budget", type=int)
    cc.add_argument("--output", "-o", required=True, help="parent directory of the curriculum (--config) or the token-cache file of the "
                                                          "composed stage (--corpus/--strata)")

    g = sub.add_parser("generate-eval", help="decode held-out prompts of a supervised-generation objective and report text statistics")
    g.add_argument("--config", "--model", dest="model", required=True)
    g.add_argument("--tokenizer", "-t", required=True)
    g.add_argument("--checkpoint", required=True)
    g.add_argument("--data", required=True, action="append", help="held-out shard, repeatable")
    g.add_argument("--objective", choices=["summarization", "instruction_tuning", "qa_reasoning", "retrieval_planning"])
    g.add_argument("--task", help="a complete task JSON instead of --objective and its options")
    g.add_argument("--sequence-length", type=int, default=512)
    g.add_argument("--max-new-tokens", type=int, default=60)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--max-records", "--limit", dest="max_records", type=int)
    g.add_argument("--instruction")
    g.add_argument("--require-reasoning", action="store_true")
    g.add_argument("--samples", help="write the verbatim decodes to this file")
    g.add_argument("--output", "-o")
    g.add_argument("--device")

    q = sub.add_parser("quantize")
    q.add_argument("--model", required=True)
    q.add_argument("--checkpoint", required=True)
    q.add_argument("--tokenizer", help="tokenizer.json that defined the vocabulary (default: the model file's)")
    q.add_argument("--format", required=True, type=lambda v: v.replace("-", "_"),
                   choices=["binary_g128", "ternary_g128", "ternary_entropy_g128", "int4_g128"], help="also spelled with hyphens (binary-g128)")
    q.add_argument("--output", "-o", required=True)
    boolean = lambda v: {"true": True, "false": False}[v.lower()]
    q.add_argument("--quantize-embeddings", type=boolean, default=True, metavar="true|false")
    q.add_argument("--quantize-lm-head", type=boolean, default=True, metavar="true|false")
    q.add_argument("--ternary-warmup-steps", type=int, default=0, help="recorded in the archive: ternary steps that preceded a binary target")
    q.add_argument("--distillation-weight", type=float, default=0.0, help="recorded in the archive: weight of the teacher KL during training")

    u = sub.add_parser("upgrade-memory-checkpoint")
    u.add_argument("--model", "--target-config", dest="model", required=True, help="memory-chain model definition")
    u.add_argument("--source-config", help="the ordinary model the checkpoint was trained as; the checkpoint must fit it exactly")
    u.add_argument("--checkpoint", required=True)
    u.add_argument("--output", "-o", required=True)

    r = sub.add_parser("run-workflow")
    r.add_argument("--workflow", required=True)
    r.add_argument("--state", required=True)
    r.add_argument("--initial-checkpoint", "--initial-checkpoint-uri", dest="initial_checkpoint")
    r.add_argument("--initial-checkpoint-sha256", help="`sha256:` identity the initial checkpoint's bytes must have")
    r.add_argument("--worker", nargs="+", help="phase worker executable and arguments (the route of every phase "
                                               "without a native one; the only route without --native)")
    r.add_argument("--executor", help="phase worker executable (with --executor-arg, the same as --worker)")
    r.add_argument("--executor-arg", action="append", default=[], dest="executor_arguments", help="one worker argument, repeatable")
    r.add_argument("--timeout", "--executor-timeout-seconds", dest="timeout", type=float, default=3600.0)
    r.add_argument("--run-id", help="run id of the --metrics journal (default: derived from the workflow signature)")
    r.add_argument("--native", action="store_true",
                   help="embedded host: typed post_training, standalone sleep and periodic-wake phases run in this "
                        "process through the first-party adapters; routing is validated before any state is written")
    r.add_argument("--resume", action="store_true", help="--native: reopen an existing --state (journal cut back to "
                                                         "the committed prefix)")
    r.add_argument("--model", help="--native: model definition (.mal) of the phase checkpoints")
    r.add_argument("--tokenizer", help="--native: tokenizer.json (default: byte-level)")
    r.add_argument("--output", help="--native: directory for the candidates the in-process phases publish")
    r.add_argument("--replay", help="--native: JSONL of {\"tokens\": [...]} rows for standalone sleep phases")
    r.add_argument("--sleep-runtime", help="--native: sleep-runtime JSON (standalone shape) instead of --replay; needs --sleep-runtime-sha256")
    r.add_argument("--sleep-runtime-sha256", help="--native: `sha256:` identity of the --sleep-runtime file's bytes")
    r.add_argument("--metrics", help="--native: metrics.jsonl journal")
    r.add_argument("--update-budget", type=int, help="--native: yield after this many applied post-training updates")
    r.add_argument("--device", default="cpu")
    r.add_argument("--lr", type=float, default=1e-5, help="--native: post-training learning rate")

    args = ap.parse_args(argv)

    if args.cmd == "train":
        from ..train.trainer import TrainArgs, train
        res = train(TrainArgs(model=args.model, tokenizer=args.tokenizer, workflow=args.workflow, output=args.output,
                              lr=args.lr, weight_decay=args.weight_decay, max_grad_norm=args.clip,
                              warmup_steps=args.warmup, schedule=args.schedule, checkpoint_every=args.checkpoint_every,
                              seed=args.seed, checkpoint=args.checkpoint, resume=args.resume, optimizer=args.optimizer,
                              device=args.device, max_steps_override=args.max_steps,
                              print_run_signature=args.print_run_signature, layer_metrics_every=args.layer_metrics_every,
                              gpu_metrics_interval_ms=args.gpu_metrics_interval_ms,
                              gpu_physical_device=args.gpu_physical_device, token_cache=not args.no_token_cache,
                              sleep_runtime=args.sleep_runtime, sleep_runtime_sha256=args.sleep_runtime_sha256))
        if not args.print_run_signature and int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(res))
        return 0
    if args.cmd == "validate-workflow":
        from ..train.workflow import load_workflow, validate_against_model
        if (args.workflow is None) == (args.workflow_path is None):
            raise SystemExit("validate-workflow takes the workflow file once: positionally or as --workflow")
        wf = load_workflow(args.workflow or args.workflow_path)
        if args.model:
            from .. import mal
            from ..models import validate_config
            model_def = mal.load_model_def(args.model)
            validate_config(model_def)
            validate_against_model(wf, model_def)
        print("sha256:" + wf.signature() if args.signature_only else json.dumps({"phases": len(wf.phases), "signature": wf.signature()}))
        return 0
    if args.cmd == "verify-checkpoint":
        from ..train import checkpoint as C
        root = args.root or args.output
        try:
            if root and not args.generation:
                if args.root and args.output:
                    raise C.CheckpointError("name the checkpoint root once")
                verified = C.verify_checkpoint_root(root)
            elif args.generation and args.generation_name and args.manifest_sha256 and not root:
                verified = C.verify_checkpoint_generation(args.generation, args.generation_name, args.manifest_sha256)
            elif args.generation:
                raise C.CheckpointError("--generation requires both --generation-name and --manifest-sha256")
            else:
                raise C.CheckpointError("provide either --root, or --generation with --generation-name and --manifest-sha256")
            if args.exact_metrics and not args.metrics:
                raise C.CheckpointError("--exact-metrics requires --metrics")
            if args.metrics:
                C.validate_checkpoint_metrics(verified, args.metrics, args.exact_metrics)
        except C.CheckpointError as e:
            print(str(e), file=sys.stderr)
            return 1
        if args.format == "tsv":
            print("\t".join(str(verified[k]) for k in ("global_step", "generation", "manifest_sha256", "metric_records")))
        else:
            print(json.dumps(verified, sort_keys=True))
        return 0
    if args.cmd == "eval":
        from ..train.eval import eval_command
        print(json.dumps(eval_command(args), sort_keys=True))
        return 0
    if args.cmd == "retrieval-pool-eval":
        from ..train.eval import retrieval_pool_command
        print(json.dumps(retrieval_pool_command(args), sort_keys=True))
        return 0
    if args.cmd == "prepare-corpus":
        from ..tokenizer import Tokenizer
        from ..train import corpus as C
        with open(args.recipe) as f:
            rc = json.load(f)
        if "corpus" in rc:
            from ..train import corpus_backends as B
            from ..train import corpus_recipe as R
            from ..train.data import file_sha256 as D_file_sha256
            unknown = set(rc) - {"corpus", "search_api", "postgres"}
            if unknown or "search_api" not in rc:
                raise SystemExit(f"a production recipe holds `corpus`, `search_api` and optionally `postgres`; got {sorted(rc)}")
            recipe = R.CorpusRecipe.decode(rc["corpus"])
            search = B.SearchApiClient(rc["search_api"])
            materializer = (B.PostgresRecordMaterializer(rc["postgres"], B.connect_postgres(rc["postgres"])) if "postgres" in rc
                            else B.InlineRecordMaterializer())
            out = R.build_corpus(recipe, search, materializer, Tokenizer.from_file(args.tokenizer), args.output,
                                 work_directory=args.work_directory, max_batches=args.max_pages,
                                 tokenizer_identity="sha256:" + D_file_sha256(args.tokenizer))
            print(json.dumps({"published": out}))
            return 0
        base = os.path.dirname(os.path.abspath(args.recipe))
        with open(os.path.join(base, rc["search"])) as f:
            search = C.ListSearchBackend(json.load(f))
        records = {}
        with open(os.path.join(base, rc["records"])) as f:
            for line in f:
                if line.strip():
                    row = json.loads(line)
                    records[row["key"]] = row["text"]
        cfg = C.CorpusConfig(rc["name"], rc["queries"], rc.get("page_size", 64), rc.get("docs_per_shard", 256),
                             rc.get("min_chars", 1), rc.get("metadata", {}))
        tok = Tokenizer.from_file(args.tokenizer)
        out = C.CorpusPipeline(cfg, search, C.DictMaterializer(records), tok, C.SqliteDeduplicator).run(
            args.output, max_pages=args.max_pages)
        print(json.dumps({"published": out}))
        return 0
    if args.cmd == "compose-curriculum" and args.config:
        from ..train import corpus_recipe as R
        with open(args.config) as f:
            cfg = R.CompositionConfig.decode(json.load(f), os.path.dirname(os.path.abspath(args.config)))
        print(json.dumps({"published": R.compose_curriculum(cfg, args.output, args.work_directory)}))
        return 0
    if args.cmd == "compose-curriculum":
        if not (args.corpus and args.strata and args.token_budget):
            raise SystemExit("compose-curriculum needs --config, or --corpus with --strata and --token-budget")
        from ..train import corpus as C
        from ..train.data import write_token_cache
        manifest, docs = C.open_corpus(args.corpus)
        labels = [r["labels"] for sh in manifest["shards"] for r in sh["records"]]
        with open(args.strata) as f:
            spec = json.load(f)
        strata = [C.Stratum(x["name"], float(x["weight"]),
                            (lambda want: (lambda l: all(l.get(k) == v for k, v in want.items())))(x.get("label", {})))
                  for x in spec]
        stage = C.compose_stage(zip(labels, docs()), strata, args.token_budget)
        write_token_cache(args.output, [ids for _, ids in stage])
        counts = {}
        for name, ids in stage:
            counts[name] = counts.get(name, 0) + len(ids)
        print(json.dumps({"documents": len(stage), "tokens_by_stratum": counts}, sort_keys=True))
        return 0
    if args.cmd == "generate-eval":
        from ..train.eval import generate_eval_command
        print(json.dumps(generate_eval_command(args), sort_keys=True))
        return 0
    if args.cmd == "quantize":
        from ..train.quantization import quantize_command
        print(json.dumps(quantize_command(args), sort_keys=True))
        return 0
    if args.cmd == "upgrade-memory-checkpoint":
        from .. import mal
        from ..models import Transformer
        from ..models import weights as W
        cfg = mal.load_model_def(args.model)
        mm = Transformer(cfg)
        data = open(args.checkpoint, "rb").read()
        if args.source_config:
            src_cfg = mal.load_model_def(args.source_config)
            src_cfg.vocab_size = cfg.vocab_size
            W.load_safetensors_bytes(Transformer(src_cfg), data)       # strict: missing, extra or mis-shaped tensors are refused
        with open(args.output, "wb") as f:
            f.write(W.upgrade_safetensors_to_memory(data, mm))
        return 0
    if args.cmd == "run-workflow":
        from ..train.runtime import run_workflow_command
        if args.executor:
            if args.worker:
                raise SystemExit("give the phase worker once: --worker, or --executor with --executor-arg")
            args.worker = [args.executor, *args.executor_arguments]
        elif args.executor_arguments:
            raise SystemExit("--executor-arg needs --executor")
        if args.initial_checkpoint_sha256:
            import hashlib
            if not args.initial_checkpoint:
                raise SystemExit("--initial-checkpoint-sha256 needs --initial-checkpoint-uri")
            from ..utils.remote import resolve
            args.initial_checkpoint = resolve(args.initial_checkpoint)
            with open(args.initial_checkpoint, "rb") as f:
                digest = hashlib.sha256(f.read()).hexdigest()
            if digest != args.initial_checkpoint_sha256.removeprefix("sha256:"):
                raise SystemExit(f"the initial checkpoint hashes to sha256:{digest}, expected {args.initial_checkpoint_sha256}")
        print(json.dumps(run_workflow_command(args), sort_keys=True))
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
