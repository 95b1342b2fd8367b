"""Failure detection on CPU ranks (gloo): a rank that leaves between steps is seen through its
heartbeat before the next launch; a collective whose peer never joins ends with an error instead
of hanging; no GPU is involved."""
import os
import subprocess
import sys
import textwrap
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_heartbeat_detects_silent_and_departed_ranks(tmp_path):
    sys.path.insert(0, ROOT)
    from summa_b200.parallel.health import Heartbeat, RankFailure
    d = str(tmp_path / "hb")
    a = Heartbeat(0, 3, directory=d, interval=0.05, timeout=0.6).start()
    b = Heartbeat(1, 3, directory=d, interval=0.05, timeout=0.6).start()
    c = Heartbeat(2, 3, directory=d, interval=0.05, timeout=0.6).start()
    time.sleep(0.2)
    a.guard(0)                                        # everyone alive
    b.leave()                                         # orderly departure: seen at once
    with pytest.raises(RankFailure) as e:
        a.guard(1)
    assert e.value.ranks == [1]
    c.stop()                                          # silent death: seen after the timeout
    assert a.dead_ranks() == [1]
    time.sleep(0.9)
    assert a.dead_ranks() == [1, 2]
    a.stop()


def test_watched_collective_times_out_and_passes_results():
    sys.path.insert(0, ROOT)
    from summa_b200.parallel.health import RankFailure, watched_collective
    assert watched_collective(lambda: 7, 1.0) == 7
    with pytest.raises(RankFailure, match="did not finish"):
        watched_collective(lambda: time.sleep(5), 0.2)
    with pytest.raises(RankFailure, match="failed"):
        watched_collective(lambda: (_ for _ in ()).throw(RuntimeError("peer reset")), 1.0)


WORKER = textwrap.dedent("""
    import datetime, os, sys, time, torch, torch.distributed as dist
    sys.path.insert(0, %r)
    from summa_b200.parallel.health import Heartbeat, RankFailure, watched_collective
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
    rank, world = dist.get_rank(), dist.get_world_size()
    hb = Heartbeat(rank, world, directory=sys.argv[1], interval=0.05, timeout=1.0).start()
    t = torch.ones(4)
    done = 0
    try:
        for step in range(6):
            hb.guard(step)                             # before any launch of this step
            if rank == 1 and step == 3:
                hb.leave()                             # rank 1 goes away BETWEEN steps, nothing in flight
                os._exit(0)
            watched_collective(lambda: dist.all_reduce(t), 5.0, "all_reduce")
            done += 1
            time.sleep(0.15)
    except RankFailure as e:
        print("RANK", rank, "STOPPED_AFTER", done, "CAUSE", str(e).split(":")[0], flush=True)
        os._exit(0)                                    # the supervisor restarts from the last sealed generation
    print("RANK", rank, "FINISHED", done, flush=True)
""") % ROOT


def test_survivor_stops_before_the_next_launch(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29551", str(script), str(tmp_path / "hb")],
                       capture_output=True, text=True, env=env, timeout=120)
    lines = [l for l in r.stdout.splitlines() if l.startswith("RANK 0")]
    assert lines, (r.stdout[-2000:], r.stderr[-3000:])
    # rank 0 completed the three joint steps and then stopped on the host: either its guard saw the
    # departure, or (if it was already inside the collective) the short process-group timeout ended it
    assert "STOPPED_AFTER 3" in lines[0], lines
    assert "peer heartbeat lost" in lines[0] or "all_reduce" in lines[0]
