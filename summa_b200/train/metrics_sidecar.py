"""Metrics sidecar: follows a run's append-only `metrics.jsonl` and forwards every event to
Weights & Biases when the `wandb` package and credentials are available, otherwise to a flat
`metrics.sidecar.tsv` next to the journal. It never writes to the journal and a failure here
never touches the trainer (`summa-train/scripts/relaunch.sh:2469-3343`, sidecar section).

    python -m summa_b200.train.metrics_sidecar --metrics RUN/metrics.jsonl [--project NAME] [--once]
"""
from __future__ import annotations

import argparse
import json
import os
import time


def flatten(event: dict, prefix: str = "") -> dict:
    out = {}
    for k, v in event.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(flatten(v, key + "."))
        elif isinstance(v, (int, float)) and not isinstance(v, bool):
            out[key] = v
    return out


def follow(path: str, once: bool, sink) -> int:
    pos, n = 0, 0
    while True:
        if os.path.exists(path):
            with open(path) as f:
                f.seek(pos)
                while True:
                    line = f.readline()
                    if not line or not line.endswith("\n"):
                        break                      # a partial last line is picked up on the next pass
                    pos = f.tell()
                    try:
                        ev = json.loads(line)
                    except json.JSONDecodeError:
                        continue
                    sink(ev)
                    n += 1
        if once:
            return n
        time.sleep(2.0)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--metrics", required=True)
    ap.add_argument("--project", default="summa_b200")
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args(argv)
    run = None
    try:
        import wandb                                  # optional
        if os.environ.get("WANDB_API_KEY"):
            run = wandb.init(project=a.project, resume="allow")
    except Exception:
        run = None
    tsv = open(os.path.join(os.path.dirname(os.path.abspath(a.metrics)), "metrics.sidecar.tsv"), "a") if run is None else None

    def sink(ev):
        flat = flatten(ev)
        step = ev.get("global_step", ev.get("step"))
        if run is not None:
            run.log(flat, step=step)
        else:
            tsv.write(f"{ev.get('event', ev.get('type', ''))}\t{step}\t{json.dumps(flat, sort_keys=True)}\n")
            tsv.flush()

    n = follow(a.metrics, a.once, sink)
    if tsv is not None:
        tsv.close()
    print(json.dumps({"forwarded": n}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
