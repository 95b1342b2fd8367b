#!/usr/bin/env bash
# Relaunch supervisor for long training runs (shell entry point). The supervisor itself is
# `summa_b200/cli/relaunch.py`: single-owner lock, verify -> resume, restart with a delay, remote
# synchronisation of sealed generations (immutable objects, read back and verified) with a
# compare-and-swap pointer that never moves backwards, restore on a fresh machine, metrics sidecar.
#
#   relaunch.sh --output RUN_DIR [--remote file:///mirror | gs://bucket/prefix] [--max-restarts N]
#               [--restart-delay S] [--sync-interval S] [--sidecar] -- <trainer command ...>
#
# Everything after `--` is the trainer command (default: `python -m summa_b200.cli.train train`);
# `--output RUN_DIR` and, once a sealed checkpoint verifies, `--resume` are added by the supervisor.
set -euo pipefail
has_output=0
for a in "$@"; do
  [[ "$a" == "--" ]] && break
  [[ "$a" == "--output" ]] && has_output=1
done
[[ $has_output -eq 1 ]] || { echo "relaunch.sh: --output is required" >&2; exit 2; }
exec "${PYTHON:-python}" -m summa_b200.cli.relaunch "$@"
