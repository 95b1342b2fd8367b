"""Relaunch supervisor: keeps one training run alive across process failures and machine changes.

    python -m summa_b200.cli.relaunch --output RUN_DIR [--remote file:///mirror | gs://bucket/prefix]
        [--sync-interval 900] [--restart-delay 30] [--max-restarts 0] [--verifier CMD ...] [--sidecar]
        -- <trainer command ...>

Behaviour follows the reference's supervisor (`summa-train/scripts/relaunch.sh:1-140` for the
configuration rules and the lock, `:2469-3343` for verification, remote synchronisation and the loops):

  * one supervisor per run (an exclusive `flock`; a second one exits 0 with "nothing to do");
  * the supervisor owns `--output` and `--resume`: they are refused inside the trainer command and added
    here, `--resume` only when a sealed checkpoint exists AND verifies;
  * before the first launch the newest of {local checkpoint, remote checkpoint} is chosen; a fresh machine
    restores the remote generation into a staging directory, verifies it and renames it into place;
  * a synchronisation loop uploads every newly sealed generation as IMMUTABLE objects (an existing object
    with the same bytes is reused, one with different bytes is an error, creation is create-only), verifies
    the remote copy by reading it back, and only then advances the remote pointer with a compare-and-swap
    that never moves it backwards (`same` / `advance` / `newer` / conflict);
  * the trainer is restarted after a failure with a delay, up to `--max-restarts` (0 = no limit); a sealed
    checkpoint that fails verification stops the supervisor instead of training on top of it;
  * the metrics sidecar runs beside the trainer and is restarted when it exits;
  * SIGTERM / SIGINT stop the children's process groups, run one last synchronisation and exit.

The trainer, the verifier and `gcloud` are plain executables, so tests substitute fakes for all three
(the reference's `relaunch_test.sh:16-60` method)."""
from __future__ import annotations

import argparse
import fcntl
import hashlib
import json
import os
import shutil
import signal
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional, Tuple

POINTER = "current.json"
GENERATIONS = "generations"
MANIFEST = "generation-manifest.json"


class SupervisorError(RuntimeError):
    pass


def log(msg: str) -> None:
    sys.stderr.write(time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()) + " summa-relaunch: " + msg + "\n")
    sys.stderr.flush()


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def verify_file(path: str, nbytes: int, sha: str) -> bool:
    return (os.path.isfile(path) and not os.path.islink(path) and os.path.getsize(path) == nbytes
            and sha256_file(path) == sha)


# ---------------------------------------------------------------------------------------------- pointers
def read_pointer(path: str) -> Optional[Dict]:
    if not os.path.exists(path):
        return None
    ptr = json.load(open(path))
    if ptr.get("version") != 1 or not str(ptr.get("generation", "")).startswith("sha256-"):
        raise SupervisorError(f"{path} is not a version-1 checkpoint pointer")
    return ptr


def compare_pointers(candidate: Dict, cand_step: int, existing: Optional[Dict], exist_step: Optional[int]) -> str:
    """`same`: both name the same generation; `advance`: the candidate is strictly later; `newer`: the existing
    pointer is strictly later (it must stay); `conflict`: two different generations of the same step."""
    if existing is None:
        return "advance"
    if (existing["generation"], existing.get("manifest_sha256")) == (candidate["generation"], candidate.get("manifest_sha256")):
        return "same"
    if exist_step is None:
        return "conflict"
    if cand_step > exist_step:
        return "advance"
    if cand_step < exist_step:
        return "newer"
    return "conflict"


# ---------------------------------------------------------------------------------------------- remotes
class FileRemote:
    """`file://` remote: a directory tree (another disk, an NFS mount). Create-only installs use `os.link`,
    which fails when the name exists; the pointer is replaced under an exclusive lock on the remote root."""

    def __init__(self, url: str):
        self.root = url[len("file://"):]
        os.makedirs(self.root, exist_ok=True)

    def _p(self, rel: str) -> str:
        p = os.path.normpath(os.path.join(self.root, rel))
        if not p.startswith(os.path.normpath(self.root) + os.sep):
            raise SupervisorError(f"remote path escapes the remote root: {rel}")
        return p

    def download(self, rel: str, dst: str) -> bool:
        src = self._p(rel)
        if not os.path.isfile(src) or os.path.islink(src):
            return False
        shutil.copyfile(src, dst)
        return True

    def upload_immutable(self, src: str, rel: str, nbytes: int, sha: str) -> None:
        if not verify_file(src, nbytes, sha):
            raise SupervisorError(f"{src} does not match its manifest entry")
        dst = self._p(rel)
        if os.path.lexists(dst):
            if verify_file(dst, nbytes, sha):
                return
            raise SupervisorError(f"immutable remote object already exists with different bytes: {rel}")
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        fd, tmp = tempfile.mkstemp(prefix=".upload-", dir=os.path.dirname(dst))
        try:
            with os.fdopen(fd, "wb") as out, open(src, "rb") as inp:
                shutil.copyfileobj(inp, out)
                out.flush()
                os.fsync(out.fileno())
            try:
                os.link(tmp, dst)                     # create-only: loses to a concurrent writer
            except FileExistsError:
                if not verify_file(dst, nbytes, sha):
                    raise SupervisorError(f"immutable remote object already exists with different bytes: {rel}")
        finally:
            os.unlink(tmp)
        if not verify_file(dst, nbytes, sha):
            raise SupervisorError(f"remote copy of {rel} failed verification")

    def publish_pointer(self, candidate_path: str, step_of) -> str:
        cand = read_pointer(candidate_path)
        with open(os.path.join(self.root, ".pointer.lock"), "a+") as lk:
            fcntl.flock(lk, fcntl.LOCK_EX)
            existing = read_pointer(self._p(POINTER))
            state = compare_pointers(cand, step_of(cand), existing, step_of(existing) if existing else None)
            if state != "advance":
                return state
            fd, tmp = tempfile.mkstemp(prefix=".current-", dir=self.root)
            with os.fdopen(fd, "wb") as out, open(candidate_path, "rb") as inp:
                shutil.copyfileobj(inp, out)
                out.flush()
                os.fsync(out.fileno())
            os.replace(tmp, self._p(POINTER))
            return "published"


class GcsRemote:
    """`gs://` remote through the `gcloud storage` command line: create-only uploads with
    `--if-generation-match=0`, pointer replacement with `--if-generation-match=<generation read before>`."""

    def __init__(self, url: str, gcloud: str, scratch: str):
        self.url, self.gcloud, self.scratch = url.rstrip("/"), gcloud, scratch

    def _u(self, rel: str) -> str:
        return self.url + "/" + rel.lstrip("/")

    def _run(self, *args) -> subprocess.CompletedProcess:
        return subprocess.run([self.gcloud, "storage", *args], capture_output=True, text=True)

    def download(self, rel: str, dst: str) -> bool:
        return self._run("cp", self._u(rel), dst).returncode == 0 and os.path.isfile(dst)

    def _object_generation(self, rel: str) -> Optional[int]:
        r = self._run("objects", "describe", self._u(rel), "--format=value(generation)")
        if r.returncode != 0:
            return None
        v = r.stdout.strip()
        if not v.isdigit() or int(v) <= 0:
            raise SupervisorError(f"unexpected object generation {v!r} for {rel}")
        return int(v)

    def upload_immutable(self, src: str, rel: str, nbytes: int, sha: str) -> None:
        if not verify_file(src, nbytes, sha):
            raise SupervisorError(f"{src} does not match its manifest entry")
        probe = os.path.join(self.scratch, "remote-object.probe")
        if self.download(rel, probe):
            ok = verify_file(probe, nbytes, sha)
            os.unlink(probe)
            if ok:
                return
            raise SupervisorError(f"immutable remote object already exists with different bytes: {rel}")
        # never replace an object written by another supervisor: if a concurrent writer wins the
        # precondition, the read-back below accepts its bytes only when they are the same bytes
        self._run("cp", "--if-generation-match=0", src, self._u(rel))
        ok = self.download(rel, probe) and verify_file(probe, nbytes, sha)
        if os.path.exists(probe):
            os.unlink(probe)
        if not ok:
            raise SupervisorError(f"remote copy of {rel} failed verification")

    def publish_pointer(self, candidate_path: str, step_of) -> str:
        cand = read_pointer(candidate_path)
        existing_path = os.path.join(self.scratch, "existing-current.json")
        for _ in range(12):
            before = self._object_generation(POINTER)
            if before is not None:
                if not self.download(POINTER, existing_path) or self._object_generation(POINTER) != before:
                    continue                          # replaced while we were reading it
                existing = read_pointer(existing_path)
                state = compare_pointers(cand, step_of(cand), existing, step_of(existing))
                if state != "advance":
                    return state
            else:
                before = 0
                if self.download(POINTER, existing_path):
                    continue                          # appeared between the two reads
            if self._run("cp", f"--if-generation-match={before}", candidate_path, self._u(POINTER)).returncode == 0:
                if self.download(POINTER, existing_path) and read_pointer(existing_path) == cand:
                    return "published"
                raise SupervisorError("the remote pointer does not hold what was just published")
        raise SupervisorError("could not publish the remote pointer in 12 attempts")


def open_remote(url: str, gcloud: str, scratch: str):
    if url.startswith("file://"):
        return FileRemote(url)
    if url.startswith("gs://"):
        if shutil.which(gcloud) is None:
            raise SupervisorError(f"gcloud is required for {url}: {gcloud}")
        return GcsRemote(url, gcloud, scratch)
    raise SupervisorError("remote URL must use gs:// or file://")


# ---------------------------------------------------------------------------------------------- supervisor
class Supervisor:
    def __init__(self, output: str, command: List[str], remote: str = "", state_dir: str = "", sync_interval: float = 900,
                 restart_delay: float = 30, max_restarts: int = 0, verifier: Optional[List[str]] = None,
                 gcloud: str = "gcloud", sidecar: Optional[List[str]] = None, sidecar_restart_delay: float = 15):
        for a in command:
            if a in ("--resume", "--output", "-o") or a.startswith("--output="):
                raise SupervisorError(f"leave {a} out of the trainer command; the supervisor owns resume and output")
        if not command:
            raise SupervisorError("the trainer command is empty")
        if shutil.which(command[0]) is None:
            raise SupervisorError(f"trainer is unavailable: {command[0]}")
        if verifier and shutil.which(verifier[0]) is None:
            raise SupervisorError(f"checkpoint verifier is unavailable: {verifier[0]}")
        self.output = output.rstrip("/")
        self.command, self.verifier = list(command), verifier
        self.state_dir = state_dir or os.path.join(self.output, ".relaunch")
        os.makedirs(self.output, exist_ok=True)
        os.makedirs(self.state_dir, exist_ok=True)
        self.sync_interval, self.restart_delay, self.max_restarts = sync_interval, restart_delay, max_restarts
        self.remote = open_remote(remote, gcloud, self.state_dir) if remote else None
        self.sidecar, self.sidecar_restart_delay = sidecar, sidecar_restart_delay
        self.train_log = os.path.join(self.state_dir, "train.log")
        self._lock_file = None
        self._stop = threading.Event()
        self._children: List[subprocess.Popen] = []
        self._sync_lock = threading.Lock()
        self._synced: Optional[str] = None
        self.launches: List[List[str]] = []            # the command lines that were started (for tests and the log)

    # ---- single owner
    def acquire_lock(self) -> bool:
        self._lock_file = open(os.path.join(self.state_dir, "lock"), "a+")
        try:
            fcntl.flock(self._lock_file, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except OSError:
            self._lock_file.close()
            self._lock_file = None
            return False
        return True

    # ---- local checkpoint
    def _gen_dir(self, name: str) -> str:
        return os.path.join(self.output, GENERATIONS, name)

    def local_pointer(self) -> Optional[Dict]:
        return read_pointer(os.path.join(self.output, POINTER))

    def _manifest_of(self, name: str, root: Optional[str] = None) -> Dict:
        return json.load(open(os.path.join(root or self._gen_dir(name), MANIFEST)))

    def verify_local(self) -> Optional[str]:
        """Name of the sealed local generation after verification, None without a checkpoint."""
        ptr = self.local_pointer()
        if ptr is None:
            return None
        if self.verifier:
            r = subprocess.run(self.verifier + [self.output], capture_output=True, text=True)
            if r.returncode != 0:
                raise SupervisorError(f"sealed checkpoint in {self.output} failed verification: {r.stderr.strip()[-400:]}")
        else:
            verify_generation_dir(self._gen_dir(ptr["generation"]), ptr["generation"])
        return ptr["generation"]

    # ---- artifact closure
    def closure_of(self, name: str) -> Dict:
        """Everything outside the generation directory that the sealed training state refers to and a replacement host
        needs to resume: the tier optimizer bundles its optimizer scopes name, the files of every published candidate it
        lists, and the committed prefix of the metric journal. Objects are named by content (`objects/sha256-<hash>`);
        paths are kept relative to the output root, artifacts outside it are deployment-owned inputs and stay out."""
        try:
            with open(os.path.join(self._gen_dir(name), "training-state.json"), "r", encoding="utf-8") as f:
                state = json.load(f)
        except (OSError, ValueError):
            state = None
        if not isinstance(state, dict):                     # a generation of another writer: nothing is known to refer outside it
            return {"version": 1, "generation": name, "objects": [], "metrics": None}
        wanted: List[str] = []
        scopes = (state.get("memory_update") or {}).get("optimizer_scopes") or {}
        for tier in scopes.get("tiers", []):
            if tier.get("artifact"):
                wanted.append(os.path.join(self.output, "tier-optimizers", tier["artifact"]["path"]))
        for art in state.get("artifacts") or []:
            root = os.path.dirname(art.get("manifest", ""))
            if root and os.path.isdir(root):
                for base, _dirs, files in os.walk(root):
                    wanted += [os.path.join(base, n) for n in files]
        objects = []
        out_root = os.path.realpath(self.output)
        for path in sorted(set(wanted)):
            real = os.path.realpath(path)
            if not real.startswith(out_root + os.sep) or os.path.islink(path) or not os.path.isfile(path):
                continue
            objects.append({"path": os.path.relpath(real, out_root), "bytes": os.path.getsize(real), "sha256": sha256_file(real)})
        closure = {"version": 1, "generation": name, "objects": objects, "metrics": None}
        journal, records = os.path.join(self.output, "metrics.jsonl"), int(state.get("metric_records") or 0)
        if records and os.path.isfile(journal):
            prefix = os.path.join(self.state_dir, f"metrics-prefix-{name}.jsonl")
            with open(journal, "rb") as src, open(prefix, "wb") as dst:
                for _ in range(records):
                    line = src.readline()
                    if not line.endswith(b"\n"):
                        raise SupervisorError("the metric journal is shorter than the prefix the checkpoint committed")
                    dst.write(line)
            closure["metrics"] = {"records": records, "bytes": os.path.getsize(prefix), "sha256": sha256_file(prefix), "staged": prefix}
        return closure

    def _upload_closure(self, name: str) -> None:
        closure = self.closure_of(name)
        for obj in closure["objects"]:
            self.remote.upload_immutable(os.path.join(self.output, obj["path"]), f"objects/sha256-{obj['sha256']}", obj["bytes"], obj["sha256"])
        metrics = closure["metrics"]
        if metrics:
            staged = metrics.pop("staged")
            self.remote.upload_immutable(staged, f"checkpoint-metrics/{name}/metrics.jsonl", metrics["bytes"], metrics["sha256"])
            os.unlink(staged)
        path = os.path.join(self.state_dir, f"closure-{name}.json")
        with open(path, "w") as f:
            json.dump(closure, f, indent=1, sort_keys=True)
        self.remote.upload_immutable(path, f"closures/{name}.json", os.path.getsize(path), sha256_file(path))

    def _restore_closure(self, name: str) -> None:
        """Installs the closure of a restored generation; a local file that differs from the recorded object is never
        overwritten."""
        path = os.path.join(self.state_dir, f"remote-closure-{name}.json")
        if not self.remote.download(f"closures/{name}.json", path):
            return                                          # a generation published without generated artifacts
        closure = json.load(open(path))
        if closure.get("version") != 1 or closure.get("generation") != name:
            raise SupervisorError(f"remote closure of {name} names another generation")

        def install(remote_rel: str, rel: str, nbytes: int, sha: str) -> None:
            if os.path.isabs(rel) or ".." in rel.split("/") or rel.split("/")[0] in (GENERATIONS, POINTER):
                raise SupervisorError(f"remote closure names an unsafe path: {rel}")
            dst = os.path.join(self.output, rel)
            if os.path.lexists(dst):
                if os.path.islink(dst) or not verify_file(dst, nbytes, sha):
                    raise SupervisorError(f"{rel} exists locally and differs from the checkpoint's artifact: not overwritten")
                return
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            tmp = dst + ".restoring"
            if not self.remote.download(remote_rel, tmp) or not verify_file(tmp, nbytes, sha):
                if os.path.exists(tmp):
                    os.unlink(tmp)
                raise SupervisorError(f"remote artifact {rel} is missing or differs from its recorded identity")
            os.replace(tmp, dst)
        for obj in closure["objects"]:
            install(f"objects/sha256-{obj['sha256']}", obj["path"], obj["bytes"], obj["sha256"])
        metrics = closure.get("metrics")
        journal = os.path.join(self.output, "metrics.jsonl")
        if metrics and not os.path.exists(journal):         # an existing journal is the trainer's to cut back on resume
            install(f"checkpoint-metrics/{name}/metrics.jsonl", "metrics.jsonl", metrics["bytes"], metrics["sha256"])

    # ---- remote
    def _step_of_remote(self, ptr: Dict) -> int:
        """global_step of a pointer's generation: from the local copy when present, else from the remote manifest."""
        name = ptr["generation"]
        local = os.path.join(self._gen_dir(name), MANIFEST)
        if os.path.isfile(local):
            return int(json.load(open(local))["global_step"])
        tmp = os.path.join(self.state_dir, "remote-manifest.json")
        if not self.remote.download(f"{GENERATIONS}/{name}/{MANIFEST}", tmp):
            raise SupervisorError(f"remote generation {name} has no manifest")
        data = open(tmp, "rb").read()
        os.unlink(tmp)
        if "sha256-" + hashlib.sha256(data).hexdigest() != name:
            raise SupervisorError(f"remote manifest of {name} does not hash to its name")
        return int(json.loads(data)["global_step"])

    def sync_once(self) -> str:
        """Uploads the sealed generation (immutable objects, read back and verified) and then advances the remote
        pointer. Returns `none` / `same` / `published` / `newer`; raises on corruption or conflict."""
        if self.remote is None:
            return "none"
        with self._sync_lock:
            name = self.verify_local()
            if name is None:
                return "none"
            if self._synced == name:
                return "same"
            manifest = self._manifest_of(name)
            mpath = os.path.join(self._gen_dir(name), MANIFEST)
            for f in manifest["files"]:
                self.remote.upload_immutable(os.path.join(self._gen_dir(name), f["path"]),
                                             f"{GENERATIONS}/{name}/{f['path']}", f["bytes"], f["sha256"])
            self.remote.upload_immutable(mpath, f"{GENERATIONS}/{name}/{MANIFEST}", os.path.getsize(mpath),
                                         sha256_file(mpath))
            self._upload_closure(name)                      # every referenced artifact is up before the pointer moves
            state = self.remote.publish_pointer(os.path.join(self.output, POINTER), self._step_of_remote)
            if state == "conflict":
                raise SupervisorError("the remote pointer names a different generation of the same step")
            if state in ("published", "same"):
                self._synced = name
            log(f"remote synchronisation: {state} ({name})")
            return state

    def restore_from_remote(self) -> Optional[str]:
        """Installs the remote generation when there is no local checkpoint or the remote one is later.
        Returns the installed generation name, or None when the local state stays."""
        if self.remote is None:
            return None
        rp = os.path.join(self.state_dir, "remote-current.json")
        if not self.remote.download(POINTER, rp):
            return None
        remote_ptr = read_pointer(rp)
        local_ptr = self.local_pointer()
        if local_ptr is not None:
            state = compare_pointers(local_ptr, self._step_of_remote(local_ptr), remote_ptr, self._step_of_remote(remote_ptr))
            if state != "newer":
                return None
        name = remote_ptr["generation"]
        gens = os.path.join(self.output, GENERATIONS)
        os.makedirs(gens, exist_ok=True)
        if not os.path.isdir(self._gen_dir(name)):
            staging = tempfile.mkdtemp(prefix=".restore-", dir=gens)
            try:
                if not self.remote.download(f"{GENERATIONS}/{name}/{MANIFEST}", os.path.join(staging, MANIFEST)):
                    raise SupervisorError(f"remote generation {name} has no manifest")
                for f in self._manifest_of(name, staging)["files"]:
                    if "/" in f["path"] or f["path"].startswith("."):
                        raise SupervisorError(f"remote manifest names an unsafe member: {f['path']}")
                    if not self.remote.download(f"{GENERATIONS}/{name}/{f['path']}", os.path.join(staging, f["path"])):
                        raise SupervisorError(f"remote generation {name} lacks {f['path']}")
                verify_generation_dir(staging, name)
                os.rename(staging, self._gen_dir(name))
            except BaseException:
                shutil.rmtree(staging, ignore_errors=True)
                raise
        verify_generation_dir(self._gen_dir(name), name)
        self._restore_closure(name)
        fd, tmp = tempfile.mkstemp(prefix=".current-", dir=self.output)
        with os.fdopen(fd, "w") as out:
            json.dump(remote_ptr, out, indent=2, sort_keys=True)
            out.flush()
            os.fsync(out.fileno())
        os.replace(tmp, os.path.join(self.output, POINTER))
        self._synced = name
        log(f"restored generation {name} from the remote")
        return name

    # ---- children
    def _spawn(self, argv: List[str], logfile: str) -> subprocess.Popen:
        out = open(logfile, "ab")
        p = subprocess.Popen(argv, stdout=out, stderr=subprocess.STDOUT, start_new_session=True)
        out.close()
        self._children.append(p)
        return p

    def _kill_children(self) -> None:
        for p in self._children:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)      # the exact process group this supervisor started
                except ProcessLookupError:
                    pass
        for p in self._children:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass

    def _sync_loop(self) -> None:
        while not self._stop.wait(self.sync_interval):
            try:
                self.sync_once()
            except Exception as e:                       # the loop survives a bad pass; the next one retries
                log(f"remote synchronisation failed: {e}")

    def _sidecar_loop(self) -> None:
        while not self._stop.is_set():
            p = self._spawn(self.sidecar, os.path.join(self.state_dir, "sidecar.log"))
            while p.poll() is None and not self._stop.wait(0.2):
                pass
            if self._stop.wait(self.sidecar_restart_delay):
                return

    # ---- main loop
    def run(self) -> int:
        if not self.acquire_lock():
            log(f"another supervisor already owns {self.state_dir}/lock; nothing to do")
            return 0
        threads = []
        try:
            self.restore_from_remote()
            if self.remote is not None:
                threads.append(threading.Thread(target=self._sync_loop, daemon=True))
            if self.sidecar:
                threads.append(threading.Thread(target=self._sidecar_loop, daemon=True))
            for t in threads:
                t.start()
            restarts = 0
            while not self._stop.is_set():
                resume = ["--resume"] if self.verify_local() is not None else []
                argv = self.command + ["--output", self.output] + resume
                self.launches.append(argv)
                log("starting trainer: " + " ".join(argv))
                p = self._spawn(argv, self.train_log)
                while p.poll() is None and not self._stop.wait(0.1):
                    pass
                if self._stop.is_set():
                    break
                rc = p.returncode
                if rc == 0:
                    log("training finished")
                    self._final_sync()
                    return 0
                restarts += 1
                if self.max_restarts and restarts > self.max_restarts:
                    log(f"giving up after {self.max_restarts} restarts (last exit {rc})")
                    self._final_sync()
                    return rc if rc > 0 else 1
                log(f"trainer exited with {rc}; restart {restarts} in {self.restart_delay}s")
                try:
                    self.sync_once()
                except Exception as e:
                    log(f"remote synchronisation failed: {e}")
                if self._stop.wait(self.restart_delay):
                    break
            self._final_sync()
            return 130
        except SupervisorError as e:
            log(f"error: {e}")
            return 4
        finally:
            self._stop.set()
            self._kill_children()
            for t in threads:
                t.join(timeout=5)

    def _final_sync(self) -> None:
        try:
            self.sync_once()
        except Exception as e:
            log(f"final remote synchronisation failed: {e}")

    def stop(self, *_a) -> None:
        self._stop.set()


def verify_generation_dir(d: str, name: str) -> Dict:
    """The checks of `train/checkpoint.py::verify_generation` on an arbitrary directory (a restore staging
    directory has no `generations/` parent yet): manifest hash = name, member set = manifest, sizes, sha256."""
    mp = os.path.join(d, MANIFEST)
    if not os.path.isfile(mp):
        raise SupervisorError(f"generation {name} has no manifest")
    data = open(mp, "rb").read()
    if "sha256-" + hashlib.sha256(data).hexdigest() != name:
        raise SupervisorError(f"generation {name}: manifest hash does not match its name")
    manifest = json.loads(data)
    listed = {f["path"] for f in manifest["files"]}
    present = {n for n in os.listdir(d) if n != MANIFEST}
    if listed != present:
        raise SupervisorError(f"generation {name}: members {sorted(present)} differ from manifest {sorted(listed)}")
    for f in manifest["files"]:
        if not verify_file(os.path.join(d, f["path"]), f["bytes"], f["sha256"]):
            raise SupervisorError(f"generation {name}: {f['path']} failed verification")
    return manifest


def parse_relaunch_conf(text: str) -> dict:
    """The supervisor's configuration file (`summa-train/scripts/relaunch.conf.example`) read as DATA, never executed:
    `SUMMA_TRAIN_<NAME>=value` lines (optionally quoted) and one `SUMMA_TRAIN_COMMAND=( ... )` array whose words may
    span lines; `#` starts a comment. Anything else (substitutions, other statements) is refused."""
    import shlex
    out, lines, i = {}, text.splitlines(), 0
    while i < len(lines):
        line = lines[i].strip()
        i += 1
        if not line or line.startswith("#"):
            continue
        key, eq, rest = line.partition("=")
        if not eq or not key.startswith("SUMMA_TRAIN_") or not key.replace("_", "").isalnum():
            raise SupervisorError(f"configuration line {i} is not a SUMMA_TRAIN_<NAME>=value assignment")
        if rest.startswith("("):
            body = rest[1:]
            while ")" not in shlex.split(body, comments=True) and not body.rstrip().endswith(")"):
                if i >= len(lines):
                    raise SupervisorError(f"configuration array {key} is not closed")
                body += "\n" + lines[i]
                i += 1
            words = shlex.split(body.rstrip().removesuffix(")"), comments=True)
            value = words
        else:
            words = shlex.split(rest, comments=True)
            if len(words) > 1:
                raise SupervisorError(f"configuration value of {key} must be one word (quote it)")
            value = words[0] if words else ""
        for w in (value if isinstance(value, list) else [value]):
            if "$" in w or "`" in w:
                raise SupervisorError(f"configuration value of {key} uses a shell substitution; write the value out")
        out[key] = value
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="summa-relaunch")
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and not argv[0].startswith("-"):
        # `relaunch <file>`: the reference supervisor's calling convention
        try:
            with open(argv[0], "r", encoding="utf-8") as f:
                conf = parse_relaunch_conf(f.read())
            if not conf.get("SUMMA_TRAIN_OUTPUT") or not conf.get("SUMMA_TRAIN_COMMAND"):
                raise SupervisorError("the configuration needs SUMMA_TRAIN_OUTPUT and SUMMA_TRAIN_COMMAND")
        except (OSError, SupervisorError) as e:
            log(f"error: configuration {argv[0]}: {e}")
            return 2
        translated = ["--output", conf["SUMMA_TRAIN_OUTPUT"]]
        for key, flag in (("SUMMA_TRAIN_REMOTE_URL", "--remote"), ("SUMMA_TRAIN_STATE_DIR", "--state-dir"), ("SUMMA_TRAIN_SYNC_INTERVAL", "--sync-interval"),
                          ("SUMMA_TRAIN_RESTART_DELAY", "--restart-delay"), ("SUMMA_TRAIN_MAX_RESTARTS", "--max-restarts"), ("SUMMA_TRAIN_GCLOUD", "--gcloud")):
            if conf.get(key):
                translated += [flag, conf[key]]
        if conf.get("SUMMA_TRAIN_WANDB_ENV"):
            translated.append("--sidecar")
        argv = translated + argv[1:] + ["--", *conf["SUMMA_TRAIN_COMMAND"]]
    ap.add_argument("--output", required=True)
    ap.add_argument("--remote", default=os.environ.get("SUMMA_TRAIN_REMOTE_URL", ""))
    ap.add_argument("--state-dir", default="")
    ap.add_argument("--sync-interval", type=float, default=900)
    ap.add_argument("--restart-delay", type=float, default=30)
    ap.add_argument("--max-restarts", type=int, default=0)
    ap.add_argument("--verifier", nargs="+", help="checkpoint verifier command (the run directory is appended); "
                                                  "default: verify in this process")
    ap.add_argument("--gcloud", default=os.environ.get("SUMMA_TRAIN_GCLOUD", "gcloud"))
    ap.add_argument("--sidecar", action="store_true", help="run the metrics sidecar beside the trainer")
    ap.add_argument("command", nargs=argparse.REMAINDER, help="-- trainer command (default: this package's `train`)")
    a = ap.parse_args(argv)
    cmd = [c for c in a.command if c != "--"] or [sys.executable, "-m", "summa_b200.cli.train", "train"]
    if a.sync_interval <= 0 or a.restart_delay < 0 or a.max_restarts < 0:
        ap.error("--sync-interval must be positive, --restart-delay and --max-restarts non-negative")
    sidecar = ([sys.executable, "-m", "summa_b200.train.metrics_sidecar", "--metrics",
                os.path.join(a.output, "metrics.jsonl")] if a.sidecar else None)
    try:
        sup = Supervisor(a.output, cmd, a.remote, a.state_dir, a.sync_interval, a.restart_delay, a.max_restarts,
                         a.verifier, a.gcloud, sidecar)
    except SupervisorError as e:
        log(f"error: {e}")
        return 2
    signal.signal(signal.SIGTERM, sup.stop)
    signal.signal(signal.SIGINT, sup.stop)
    return sup.run()


if __name__ == "__main__":
    sys.exit(main())
