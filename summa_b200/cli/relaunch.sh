#!/usr/bin/env bash
# Relaunch supervisor for long training runs: one lock per output directory, verify the
# sealed checkpoint, resume from it, restart on failure with back-off, mirror sealed
# generations to a second location with a compare-and-swap pointer, and run the metrics
# sidecar beside the trainer. Behaviour follows `summa-train/scripts/relaunch.sh:1-140`.
#
#   relaunch.sh --output RUN_DIR [--mirror DIR] [--max-restarts N] [--sidecar] -- <summa-train train args>
#
# Everything after `--` is passed to `python -m summa_b200.cli.train train`; `--output RUN_DIR`
# and, once a checkpoint exists, `--resume` are added here.
set -euo pipefail

OUTPUT=""; MIRROR=""; MAX_RESTARTS=20; SIDECAR=0
while [[ $# -gt 0 ]]; do
  case "$1" in
    --output) OUTPUT="$2"; shift 2 ;;
    --mirror) MIRROR="$2"; shift 2 ;;
    --max-restarts) MAX_RESTARTS="$2"; shift 2 ;;
    --sidecar) SIDECAR=1; shift ;;
    --) shift; break ;;
    *) echo "relaunch.sh: unknown option $1" >&2; exit 2 ;;
  esac
done
[[ -n "$OUTPUT" ]] || { echo "relaunch.sh: --output is required" >&2; exit 2; }
mkdir -p "$OUTPUT"
PY="${PYTHON:-python}"

# one supervisor per run directory
exec 9>"$OUTPUT/.relaunch.lock"
flock -n 9 || { echo "relaunch.sh: another supervisor holds $OUTPUT/.relaunch.lock" >&2; exit 3; }

mirror_sync() {
  [[ -n "$MIRROR" && -f "$OUTPUT/current.json" ]] || return 0
  mkdir -p "$MIRROR/generations"
  local gen
  gen="$("$PY" -c 'import json,sys; print(json.load(open(sys.argv[1]))["generation"])' "$OUTPUT/current.json")"
  if [[ ! -d "$MIRROR/generations/$gen" ]]; then
    # generations are immutable: copy to a temporary name, then publish with one rename
    cp -r "$OUTPUT/generations/$gen" "$MIRROR/generations/.$gen.partial"
    mv "$MIRROR/generations/.$gen.partial" "$MIRROR/generations/$gen"
  fi
  # compare-and-swap of the pointer: only replace it if it still names what we last saw
  local seen="$MIRROR/.last_seen_pointer"
  if [[ -f "$MIRROR/current.json" && -f "$seen" ]] && ! cmp -s "$MIRROR/current.json" "$seen"; then
    echo "relaunch.sh: mirror pointer changed under us; not overwriting" >&2
    return 0
  fi
  cp "$OUTPUT/current.json" "$MIRROR/.current.json.tmp"
  mv "$MIRROR/.current.json.tmp" "$MIRROR/current.json"
  cp "$MIRROR/current.json" "$seen"
}

SIDECAR_PID=""
start_sidecar() {
  [[ "$SIDECAR" -eq 1 ]] || return 0
  "$PY" -m summa_b200.train.metrics_sidecar --metrics "$OUTPUT/metrics.jsonl" &
  SIDECAR_PID=$!
}
stop_sidecar() { [[ -z "$SIDECAR_PID" ]] || kill "$SIDECAR_PID" 2>/dev/null || true; }
trap stop_sidecar EXIT

restarts=0
start_sidecar
while :; do
  resume=()
  if [[ -f "$OUTPUT/current.json" ]]; then
    if "$PY" -m summa_b200.cli.train verify-checkpoint "$OUTPUT" >/dev/null; then
      resume=(--resume)
    else
      echo "relaunch.sh: sealed checkpoint in $OUTPUT failed verification; refusing to continue" >&2
      exit 4
    fi
  fi
  set +e
  "$PY" -m summa_b200.cli.train train --output "$OUTPUT" "${resume[@]}" "$@"
  rc=$?
  set -e
  mirror_sync
  if [[ $rc -eq 0 ]]; then
    echo "relaunch.sh: training finished"; exit 0
  fi
  restarts=$((restarts + 1))
  if [[ $restarts -gt $MAX_RESTARTS ]]; then
    echo "relaunch.sh: giving up after $MAX_RESTARTS restarts (last exit $rc)" >&2; exit "$rc"
  fi
  delay=$(( restarts < 6 ? 5 * restarts : 30 ))
  echo "relaunch.sh: trainer exited with $rc; restart $restarts/$MAX_RESTARTS in ${delay}s" >&2
  sleep "$delay"
done
