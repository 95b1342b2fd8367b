"""The relaunch supervisor against fake executables (trainer, verifier, gcloud), the way the reference tests its
shell supervisor (`summa-train/scripts/relaunch_test.sh:16-60`): restart with `--resume`, remote restore on a
fresh machine, pointer races, corruption, immutable-object conflicts, the single-owner lock."""
import hashlib
import json
import os
import stat
import sys
import textwrap

import pytest

from summa_b200.cli import relaunch as R

FILES = ("weights.safetensors", "adamw-state.bpk", "muon-state.bpk", "training-state.json", "training-accounting.json")

SEAL = textwrap.dedent("""
    import hashlib, json, os
    FILES = %r
    def seal(out, step, tag=""):
        gens = os.path.join(out, "generations"); os.makedirs(gens, exist_ok=True)
        tmp = os.path.join(gens, ".staging-%%d" %% os.getpid()); os.makedirs(tmp, exist_ok=True)
        files = []
        for n in FILES:
            data = ("%%s step %%d %%s" %% (n, step, tag)).encode()
            open(os.path.join(tmp, n), "wb").write(data)
            files.append({"path": n, "bytes": len(data), "sha256": hashlib.sha256(data).hexdigest()})
        m = json.dumps({"version": 1, "training_state_version": 2, "global_step": step, "phase": 0, "phase_id": "p",
                        "files": files}, indent=2, sort_keys=True).encode()
        open(os.path.join(tmp, "generation-manifest.json"), "wb").write(m)
        name = "sha256-" + hashlib.sha256(m).hexdigest()
        final = os.path.join(gens, name)
        if not os.path.exists(final):
            os.rename(tmp, final)
        ptr = {"version": 1, "generation": name, "manifest_sha256": hashlib.sha256(m).hexdigest()}
        open(os.path.join(out, ".current.tmp"), "w").write(json.dumps(ptr, indent=2, sort_keys=True))
        os.replace(os.path.join(out, ".current.tmp"), os.path.join(out, "current.json"))
        return name
""") % (FILES,)
exec(SEAL)          # `seal` for the test process too

TRAINER = "#!" + sys.executable + "\n" + SEAL + textwrap.dedent("""
    import sys
    args = sys.argv[1:]
    out = args[args.index("--output") + 1]
    plan_path = args[args.index("--plan") + 1]
    plan = json.load(open(plan_path))
    calls = plan_path + ".calls"
    n = len(open(calls).read().splitlines()) if os.path.exists(calls) else 0
    open(calls, "a").write(json.dumps(args) + "\\n")
    act = plan[min(n, len(plan) - 1)]
    if "seal" in act:
        seal(out, act["seal"])
    sys.exit(act.get("exit", 0))
""")

GCLOUD = "#!" + sys.executable + "\n" + textwrap.dedent("""
    import json, os, shutil, sys
    root = os.environ["FAKE_GCS_ROOT"]
    def local(url):
        assert url.startswith("gs://bucket/"), url
        return os.path.join(root, url[len("gs://bucket/"):])
    def gen_path(p):
        g = os.path.join(root, ".gens", os.path.relpath(p, root))
        os.makedirs(os.path.dirname(g), exist_ok=True)
        return g
    def gen_of(p):
        return int(open(gen_path(p)).read()) if os.path.exists(gen_path(p)) else 0
    a = sys.argv[1:]
    assert a[0] == "storage"
    open(os.path.join(root, "calls.log"), "a").write(" ".join(a) + "\\n")
    if a[1] == "objects" and a[2] == "describe":
        p = local(a[3])
        if not os.path.exists(p): sys.exit(1)
        print(gen_of(p)); sys.exit(0)
    if a[1] == "cp":
        rest = a[2:]; match = None
        if rest[0].startswith("--if-generation-match="):
            match = int(rest[0].split("=")[1]); rest = rest[1:]
        src, dst = rest
        if dst.startswith("gs://"):
            p = local(dst)
            race = os.path.join(root, "race-once")              # another writer replaces the object first
            if os.path.exists(race) and dst.endswith("current.json"):
                os.unlink(race)
                bumped = gen_of(p) + 1
                open(gen_path(p), "w").write(str(bumped))
            cur = gen_of(p) if os.path.exists(p) else 0
            if match is not None and match != cur: sys.exit(1)
            os.makedirs(os.path.dirname(p), exist_ok=True)
            shutil.copyfile(src, p); open(gen_path(p), "w").write(str(cur + 1)); sys.exit(0)
        p = local(src)
        if not os.path.exists(p): sys.exit(1)
        shutil.copyfile(p, dst); sys.exit(0)
    sys.exit(2)
""")


def _exe(path, text):
    path.write_text(text)
    path.chmod(path.stat().st_mode | stat.S_IXUSR)
    return str(path)


def _sup(tmp_path, out, plan, remote="", **kw):
    trainer = _exe(tmp_path / f"trainer-{len(list(tmp_path.iterdir()))}.py", TRAINER)
    plan_path = tmp_path / f"plan-{os.path.basename(out)}.json"
    plan_path.write_text(json.dumps(plan))
    kw.setdefault("restart_delay", 0.01)
    kw.setdefault("sync_interval", 0.05)
    return R.Supervisor(out, [trainer, "--plan", str(plan_path)], remote, **kw), str(plan_path)


def _calls(plan_path):
    return [json.loads(l) for l in open(plan_path + ".calls").read().splitlines()]


def test_restart_passes_resume_and_mirrors_sealed_generations(tmp_path):
    out, remote = str(tmp_path / "run"), "file://" + str(tmp_path / "mirror")
    sup, plan = _sup(tmp_path, out, [{"seal": 1, "exit": 3}, {"seal": 2, "exit": 0}], remote)
    assert sup.run() == 0
    calls = _calls(plan)
    assert len(calls) == 2 and "--resume" not in calls[0] and calls[1][-1] == "--resume"
    assert calls[0][calls[0].index("--output") + 1] == out
    ptr = json.load(open(tmp_path / "mirror" / "current.json"))
    assert ptr == json.load(open(os.path.join(out, "current.json")))
    R.verify_generation_dir(str(tmp_path / "mirror" / "generations" / ptr["generation"]), ptr["generation"])
    # a fresh machine: empty run directory, same remote -> restored, verified, resumed
    out2 = str(tmp_path / "run2")
    sup2, plan2 = _sup(tmp_path, out2, [{"exit": 0}], remote)
    assert sup2.run() == 0
    assert _calls(plan2)[0][-1] == "--resume"
    assert json.load(open(os.path.join(out2, "current.json"))) == ptr
    R.verify_generation_dir(os.path.join(out2, "generations", ptr["generation"]), ptr["generation"])


def test_pointer_never_moves_backwards_and_conflicts_are_errors(tmp_path):
    remote = "file://" + str(tmp_path / "mirror")
    ahead, _ = _sup(tmp_path, str(tmp_path / "ahead"), [{"exit": 0}], remote)
    seal(ahead.output, 5)
    assert ahead.sync_once() == "published" and ahead.sync_once() == "same"
    behind, _ = _sup(tmp_path, str(tmp_path / "behind"), [{"exit": 0}], remote)
    seal(behind.output, 2)
    before = open(tmp_path / "mirror" / "current.json").read()
    assert behind.sync_once() == "newer"                       # its objects are uploaded, the pointer stays
    assert open(tmp_path / "mirror" / "current.json").read() == before
    fork, _ = _sup(tmp_path, str(tmp_path / "fork"), [{"exit": 0}], remote)
    seal(fork.output, 5, tag="other run")
    with pytest.raises(R.SupervisorError, match="different generation of the same step"):
        fork.sync_once()
    assert open(tmp_path / "mirror" / "current.json").read() == before
    # a supervisor whose local checkpoint is older than the remote adopts the remote one before launching
    assert behind.restore_from_remote() == json.loads(before)["generation"]
    assert json.load(open(os.path.join(behind.output, "current.json"))) == json.loads(before)


def test_immutable_objects_and_corruption(tmp_path):
    remote = "file://" + str(tmp_path / "mirror")
    sup, plan = _sup(tmp_path, str(tmp_path / "run"), [{"exit": 0}], remote)
    name = seal(sup.output, 1)
    # a remote object of that name with other bytes: refuse, and do not publish a pointer
    bad = tmp_path / "mirror" / "generations" / name
    bad.mkdir(parents=True)
    (bad / "weights.safetensors").write_text("someone else's bytes")
    with pytest.raises(R.SupervisorError, match="already exists with different bytes"):
        sup.sync_once()
    assert not (tmp_path / "mirror" / "current.json").exists()
    # a corrupted local generation stops the supervisor before the trainer is started
    with open(os.path.join(sup.output, "generations", name, "adamw-state.bpk"), "ab") as f:
        f.write(b"x")
    assert sup.run() == 4 and not os.path.exists(plan + ".calls")
    # a remote generation that fails verification is not installed
    out2 = str(tmp_path / "run2")
    good, _ = _sup(tmp_path, str(tmp_path / "good"), [{"exit": 0}], "file://" + str(tmp_path / "mirror2"))
    gname = seal(good.output, 3)
    assert good.sync_once() == "published"
    with open(tmp_path / "mirror2" / "generations" / gname / "muon-state.bpk", "ab") as f:
        f.write(b"tampered")
    fresh, plan3 = _sup(tmp_path, out2, [{"exit": 0}], "file://" + str(tmp_path / "mirror2"))
    assert fresh.run() == 4 and not os.path.exists(plan3 + ".calls")
    assert not os.path.exists(os.path.join(out2, "current.json"))
    assert [n for n in os.listdir(os.path.join(out2, "generations")) if not n.startswith("sha256-")] == []


def test_lock_limits_and_refused_arguments(tmp_path):
    out = str(tmp_path / "run")
    first, _ = _sup(tmp_path, out, [{"exit": 0}])
    assert first.acquire_lock()
    second, plan2 = _sup(tmp_path, out, [{"exit": 0}])
    assert second.run() == 0 and second.launches == []          # "nothing to do"
    first._lock_file.close()
    failing, plan = _sup(tmp_path, str(tmp_path / "failing"), [{"exit": 7}], max_restarts=2)
    assert failing.run() == 7 and len(_calls(plan)) == 3         # the first launch and two restarts
    for bad in (["--resume"], ["--output", "x"], ["--output=x"], ["-o"]):
        with pytest.raises(R.SupervisorError, match="owns resume and output"):
            R.Supervisor(out, [sys.executable] + bad)
    with pytest.raises(R.SupervisorError, match="trainer is unavailable"):
        R.Supervisor(out, ["/nonexistent/trainer"])
    with pytest.raises(R.SupervisorError, match="gs:// or file://"):
        R.Supervisor(out, [sys.executable], remote="s3://bucket")
    # a verifier executable that rejects the checkpoint: refuse to resume on top of it
    verifier = _exe(tmp_path / "verifier.py", "#!" + sys.executable + "\nimport sys\nsys.stderr.write('bad seal')\nsys.exit(1)\n")
    guarded, plan4 = _sup(tmp_path, str(tmp_path / "guarded"), [{"exit": 0}], verifier=[verifier])
    seal(guarded.output, 1)
    assert guarded.run() == 4 and not os.path.exists(plan4 + ".calls")


def test_gcs_backend_uses_create_only_uploads_and_pointer_compare_and_swap(tmp_path, monkeypatch):
    gcs = tmp_path / "gcs"
    gcs.mkdir()
    monkeypatch.setenv("FAKE_GCS_ROOT", str(gcs))
    gcloud = _exe(tmp_path / "gcloud", GCLOUD)
    sup, _ = _sup(tmp_path, str(tmp_path / "run"), [{"exit": 0}], "gs://bucket/runs/a", gcloud=gcloud)
    name = seal(sup.output, 1)
    assert sup.sync_once() == "published"
    log = open(gcs / "calls.log").read()
    assert log.count("--if-generation-match=0") == len(FILES) + 3          # every member, the manifest, the closure, the first pointer
    R.verify_generation_dir(str(gcs / "runs" / "a" / "generations" / name), name)
    # the next generation: the pointer is replaced only if it still has the generation that was read
    name2 = seal(sup.output, 2)
    (gcs / "race-once").write_text("")          # somebody bumps the pointer object between our read and our write
    assert sup.sync_once() == "published"       # the first compare-and-swap fails, the loop re-reads and wins
    assert json.load(open(gcs / "runs" / "a" / "current.json"))["generation"] == name2
    assert "--if-generation-match=1" in open(gcs / "calls.log").read()
    # a fresh machine restores through the same command line tool
    fresh, plan = _sup(tmp_path, str(tmp_path / "fresh"), [{"exit": 0}], "gs://bucket/runs/a", gcloud=gcloud)
    assert fresh.run() == 0 and _calls(plan)[0][-1] == "--resume"
    assert json.load(open(os.path.join(fresh.output, "current.json")))["generation"] == name2


def test_command_line_entry(tmp_path, capsys):
    trainer = _exe(tmp_path / "trainer.py", TRAINER)
    plan = tmp_path / "plan.json"
    plan.write_text(json.dumps([{"seal": 1, "exit": 0}]))
    rc = R.main(["--output", str(tmp_path / "run"), "--remote", "file://" + str(tmp_path / "m"), "--restart-delay", "0",
                 "--", trainer, "--plan", str(plan)])
    assert rc == 0 and (tmp_path / "m" / "current.json").exists()
    assert R.main(["--output", str(tmp_path / "run"), "--", trainer, "--resume"]) == 2


def test_configuration_file_is_read_as_data():
    """The reference's `relaunch.conf` shape: assignments and one command array over several lines with comments."""
    from summa_b200.cli import relaunch as R
    conf = R.parse_relaunch_conf("""
# supervisor settings
SUMMA_TRAIN_OUTPUT=/opt/run/checkpoint
SUMMA_TRAIN_REMOTE_URL="gs://bucket/run name"
SUMMA_TRAIN_COMMAND=(
  /opt/run/bin/summa-train
  train
  --config /opt/run/model.mal
  --checkpoint-every 500
  # --sleep-runtime /opt/run/sleep-runtime.json
)
SUMMA_TRAIN_MAX_RESTARTS=0   # forever
""")
    assert conf["SUMMA_TRAIN_OUTPUT"] == "/opt/run/checkpoint" and conf["SUMMA_TRAIN_REMOTE_URL"] == "gs://bucket/run name" and conf["SUMMA_TRAIN_MAX_RESTARTS"] == "0"
    assert conf["SUMMA_TRAIN_COMMAND"] == ["/opt/run/bin/summa-train", "train", "--config", "/opt/run/model.mal", "--checkpoint-every", "500"]
    assert R.parse_relaunch_conf("SUMMA_TRAIN_COMMAND=(a b)")["SUMMA_TRAIN_COMMAND"] == ["a", "b"]
    import pytest
    for bad in ("rm -rf /", "SUMMA_TRAIN_OUTPUT=$(hostname)", "SUMMA_TRAIN_OUTPUT=a b", "SUMMA_TRAIN_COMMAND=(a", "PATH=/x"):
        with pytest.raises(R.SupervisorError):
            R.parse_relaunch_conf(bad)
    ref = os.path.join(os.environ.get("SUMMA_REFERENCE_TREE", os.path.join(os.sep, "root", "reference", "summa-train")), "scripts", "relaunch.conf.example")
    if os.path.exists(ref):
        parsed = R.parse_relaunch_conf(open(ref).read())
        assert parsed["SUMMA_TRAIN_COMMAND"][1] == "train" and "--resume" not in parsed["SUMMA_TRAIN_COMMAND"] and parsed["SUMMA_TRAIN_SYNC_INTERVAL"] == "900"


def test_supervisor_runs_from_a_configuration_file(tmp_path):
    import subprocess
    import sys
    conf = tmp_path / "relaunch.conf"
    conf.write_text(f"""SUMMA_TRAIN_OUTPUT={tmp_path}/out
SUMMA_TRAIN_STATE_DIR={tmp_path}/state
SUMMA_TRAIN_COMMAND=(
  {sys.executable} -c "import sys; open(sys.argv[sys.argv.index('--output') + 1] + '.seen', 'w').write('x')"
)
SUMMA_TRAIN_RESTART_DELAY=0
SUMMA_TRAIN_MAX_RESTARTS=1
""")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "summa_b200.cli.relaunch", str(conf)], cwd=root, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and os.path.exists(f"{tmp_path}/out.seen"), r.stderr[-2000:]
    conf.write_text("SUMMA_TRAIN_OUTPUT=$(pwd)\\nSUMMA_TRAIN_COMMAND=(x)\\n")
    r = subprocess.run([sys.executable, "-m", "summa_b200.cli.relaunch", str(conf)], cwd=root, capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "shell substitution" in (r.stderr + r.stdout)


def test_artifact_closure_travels_with_the_generation(tmp_path):
    """What the sealed training state refers to outside its generation (tier optimizer bundles, a published candidate's
    files, the committed metric prefix) is uploaded before the pointer moves and installed on a replacement host; a
    local file that differs is never overwritten."""
    import hashlib
    from summa_b200.cli import relaunch as R
    out = str(tmp_path / "a" / "run")
    os.makedirs(os.path.join(out, "tier-optimizers", "generations"))
    os.makedirs(os.path.join(out, "quantized-candidates", "q.step-4", "archive"))
    bundle = b"tier bundle bytes"
    bname = "sha256-" + hashlib.sha256(bundle).hexdigest() + ".bpk"
    open(os.path.join(out, "tier-optimizers", "generations", bname), "wb").write(bundle)
    cand = os.path.join(out, "quantized-candidates", "q.step-4")
    for rel, body in (("candidate.json", b"{}"), ("weights.safetensors", b"w" * 10), ("archive/archive-manifest.json", b"[]")):
        open(os.path.join(cand, rel), "wb").write(body)
    open(os.path.join(out, "metrics.jsonl"), "w").write("".join(json.dumps({"sequence": i}) + "\n" for i in range(5)))
    state = {"global_step": 4, "metric_records": 3, "artifacts": [{"kind": "hquant_candidate", "manifest": os.path.join(cand, "candidate.json"), "hash": "sha256:" + "0" * 64}],
             "memory_update": {"type": "wake_only", "config": {}, "optimizer_scopes": {"wake_parameter_ids": [], "tiers": [
                 {"tier": 0, "artifact": {"path": "generations/" + bname, "sha256": "sha256:" + hashlib.sha256(bundle).hexdigest(), "bytes": len(bundle)}},
                 {"tier": 1, "artifact": None}]}}}
    # seal a generation by hand around that state
    gens = os.path.join(out, "generations")
    stage = os.path.join(gens, ".stage")
    os.makedirs(stage)
    files = []
    for n in FILES:
        data = json.dumps(state).encode() if n == "training-state.json" else n.encode()
        open(os.path.join(stage, n), "wb").write(data)
        files.append({"path": n, "bytes": len(data), "sha256": hashlib.sha256(data).hexdigest()})
    m = json.dumps({"version": 1, "training_state_version": 2, "global_step": 4, "phase": 0, "phase_id": "p", "files": files}, indent=2, sort_keys=True).encode()
    open(os.path.join(stage, "generation-manifest.json"), "wb").write(m)
    name = "sha256-" + hashlib.sha256(m).hexdigest()
    os.rename(stage, os.path.join(gens, name))
    json.dump({"version": 1, "generation": name, "manifest_sha256": hashlib.sha256(m).hexdigest()}, open(os.path.join(out, "current.json"), "w"))
    remote = "file://" + str(tmp_path / "mirror")
    sup = R.Supervisor(out, [sys.executable], remote)
    assert sup.sync_once() == "published"
    mirror = str(tmp_path / "mirror")
    closure = json.load(open(os.path.join(mirror, "closures", name + ".json")))
    assert sorted(o["path"] for o in closure["objects"]) == sorted([
        "tier-optimizers/generations/" + bname, "quantized-candidates/q.step-4/candidate.json", "quantized-candidates/q.step-4/weights.safetensors",
        "quantized-candidates/q.step-4/archive/archive-manifest.json"]) and closure["metrics"]["records"] == 3
    assert open(os.path.join(mirror, "checkpoint-metrics", name, "metrics.jsonl")).read().count("\n") == 3
    # a replacement host gets the generation AND its closure
    out2 = str(tmp_path / "b" / "run")
    sup2 = R.Supervisor(out2, [sys.executable], remote)
    assert sup2.restore_from_remote() == name
    assert open(os.path.join(out2, "tier-optimizers", "generations", bname), "rb").read() == bundle
    assert open(os.path.join(out2, "quantized-candidates", "q.step-4", "archive", "archive-manifest.json"), "rb").read() == b"[]"
    assert open(os.path.join(out2, "metrics.jsonl")).read().count("\n") == 3
    # a host whose local artifact differs refuses the restore instead of overwriting it
    out3 = str(tmp_path / "c" / "run")
    os.makedirs(os.path.join(out3, "tier-optimizers", "generations"))
    open(os.path.join(out3, "tier-optimizers", "generations", bname), "wb").write(b"something else")
    with pytest.raises(R.SupervisorError, match="not overwritten"):
        R.Supervisor(out3, [sys.executable], remote).restore_from_remote()
    assert not os.path.exists(os.path.join(out3, "current.json"))
