"""Failure detection on the host: heartbeats and failure notes in a key-value store.  The
failures are made on the host (a rank raises, leaves, or never joins); no GPU is involved."""

import multiprocessing as mp
import os
import time

import pytest
import torch.distributed as dist

from lorafusion_b200.parallel.health import HealthMonitor, PeerFailure


class _Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_silent_and_missing_peers_are_detected_with_a_fake_clock():
    store, clock = dist.HashStore(), _Clock()
    mons = [HealthMonitor(store, r, 3, timeout=5.0, clock=clock) for r in range(3)]
    mons[0].beat(), mons[1].beat()            # rank 2 never joins
    assert mons[0].failed_peers() == {}       # still within the grace period
    clock.t = 3.0
    mons[1].beat()
    assert mons[0].failed_peers() == {}
    clock.t = 6.0                             # rank 2 missing for > timeout; rank 1 beat 3 s ago
    assert mons[0].failed_peers() == {2: "never joined"}
    clock.t = 9.5                             # rank 1 silent for 6.5 s
    bad = mons[0].failed_peers()
    assert set(bad) == {1, 2} and bad[1].startswith("no heartbeat")
    with pytest.raises(PeerFailure) as e:
        mons[0].check()
    assert e.value.ranks == [1, 2]


def test_failure_note_is_seen_before_the_next_step():
    store = dist.HashStore()
    a, b = HealthMonitor(store, 0, 2), HealthMonitor(store, 1, 2)
    a.beat(), b.beat()

    def boom():
        raise ValueError("loss is nan")

    with pytest.raises(ValueError):
        b.guarded(boom)
    with pytest.raises(PeerFailure, match="rank 1: ValueError: loss is nan"):
        a.guarded(lambda: 1)                  # the step is not even started
    # an orderly leave looks the same to the peers
    store2 = dist.HashStore()
    c, d = HealthMonitor(store2, 0, 2), HealthMonitor(store2, 1, 2)
    c.beat(), d.beat()
    d.leave()
    with pytest.raises(PeerFailure, match="left the job"):
        c.check()


def _rank_main(rank, world, path, q):
    store = dist.FileStore(path, world)
    mon = HealthMonitor(store, rank, world, interval=0.1, timeout=1.0).start()
    try:
        for step in range(200):
            mon.check()
            if rank == 1 and step == 3:
                os._exit(0)                   # dies between steps without a word
            time.sleep(0.05)
        q.put((rank, "finished"))
    except PeerFailure as e:
        q.put((rank, f"detected {e.ranks} at step {step}"))
    finally:
        mon.stop()


def test_rank_that_dies_between_steps_is_noticed_by_heartbeat_timeout(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    path = str(tmp_path / "store")
    procs = [ctx.Process(target=_rank_main, args=(r, 2, path, q)) for r in range(2)]
    for p in procs:
        p.start()
    rank, msg = q.get(timeout=60)
    for p in procs:
        p.join(timeout=30)
    assert rank == 0 and msg.startswith("detected [1]"), msg


_STORE_CHILD = r"""
import time, torch.distributed as dist
from lorafusion_b200.parallel.health import HealthMonitor, PeerFailure
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
h = HealthMonitor(dist.distributed_c10d._get_default_store(), rank, world, interval=0.1, timeout=2.0).start()
time.sleep(0.4)
h.check()
dist.barrier()
if rank == 1:
    h.report_failure("boom")
dist.barrier()
if rank == 0:
    try:
        h.check()
        raise SystemExit("rank 0 did not see the failure note")
    except PeerFailure as e:
        assert e.ranks == [1] and "boom" in str(e)
dist.barrier()
h.stop()
dist.destroy_process_group()
print("ok", rank)
"""


def test_health_monitor_on_the_rendezvous_store_of_a_process_group(tmp_path):
    """Same checks through the store ``init_process_group`` creates (what ``cli.train`` uses)."""
    import socket
    import subprocess
    import sys

    script = tmp_path / "child.py"
    script.write_text(_STORE_CHILD)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   PYTHONPATH=os.pathsep.join([os.getcwd(), os.environ.get("PYTHONPATH", "")]))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o[-2000:]}"
