"""Failure detection on the host: heartbeat records, watchdog decisions (fake clock), the store after a killed writer,
and ranks that learn of a lost peer (gloo child processes). No test faults, traps or hangs a GPU."""
import os
import signal
import subprocess
import sys
import time

import numpy as np
import pytest

from llm_distillery_b200.obs.watchdog import Heartbeat, RankFailure

HERE = os.path.dirname(os.path.abspath(__file__))


class Clock:
    def __init__(self):
        self.t = 1000.0

    def __call__(self):
        return self.t


def _trio(tmp_path, **kw):
    clk = Clock()
    hbs = [Heartbeat(str(tmp_path), r, 3, timeout=10.0, clock=clk, start_threads=False, **kw) for r in range(3)]
    return clk, hbs


def test_silent_rank_is_reported_after_the_timeout_and_only_then(tmp_path):
    clk, hbs = _trio(tmp_path)
    for step in range(3):
        clk.t += 4.0
        for hb in hbs[:2]:
            hb.beat(step, "train")
        if step == 0:
            hbs[2].beat(step, "train")       # rank 2 beats once, then goes silent
        if step < 2:
            hbs[0].check()                   # 4 s and 8 s of silence: inside the limit
    clk.t += 4.0                             # 12 s of silence
    with pytest.raises(RankFailure) as e:
        hbs[0].check()
    assert e.value.ranks == [2] and "stopped beating" in str(e.value)
    assert hbs[1].scan().keys() == {2}


def test_done_ranks_are_never_reported_and_failed_ranks_at_once(tmp_path):
    clk, hbs = _trio(tmp_path)
    hbs[1].close("done")
    hbs[2].close("failed")
    clk.t += 1.0
    assert hbs[0].scan() == {2: "reported a failure"}
    clk.t += 100.0
    hbs[0].failed.clear()
    assert set(hbs[0].scan()) == {2}         # rank 1 finished: silence is fine


def test_rank_that_never_starts_and_stale_records_of_an_older_run(tmp_path):
    clk = Clock()
    old = Heartbeat(str(tmp_path), 1, 2, timeout=10.0, clock=clk, start_threads=False)
    old.close("failed")                      # record of an earlier run under the same id
    clk.t += 500.0
    hb = Heartbeat(str(tmp_path), 0, 2, timeout=10.0, clock=clk, start_threads=False)
    assert hb.scan() == {}                   # stale record ignored, rank 1 may still be starting
    clk.t += 11.0
    assert "never wrote" in hb.scan()[1]


def test_alive_but_stalled_rank_and_escalation_callback(tmp_path):
    clk = Clock()
    seen = []
    a = Heartbeat(str(tmp_path), 0, 2, timeout=10.0, stall_timeout=20.0, clock=clk, start_threads=False,
                  on_failure=seen.append, grace=5.0)
    b = Heartbeat(str(tmp_path), 1, 2, timeout=10.0, clock=clk, start_threads=False)
    b.beat(7, "train")
    for _ in range(5):                       # b's process stays alive (record refreshed) but its step never moves
        clk.t += 5.0
        b._write()
    assert "made no progress" in a.scan()[1]
    # the watchdog thread's rule: escalate once, after the grace period, if check() was never reached
    clk.t += 6.0
    failed = a.scan()
    if failed and not a._handled and clk() - a._first_failure_at > a.grace:
        a._handled = True
        a.on_failure(failed)
    assert len(seen) == 1 and 1 in seen[0]


def test_threads_detect_a_dead_process_in_real_time(tmp_path):
    a = Heartbeat(str(tmp_path), 0, 2, interval=0.05, timeout=0.5)
    b = Heartbeat(str(tmp_path), 1, 2, interval=0.05, timeout=0.5)
    time.sleep(0.3)
    a.check()
    b._stop.set()                            # b's process "dies": no more records, no goodbye
    deadline = time.time() + 5.0
    while time.time() < deadline and not a.failed:
        time.sleep(0.05)
    with pytest.raises(RankFailure):
        a.check()
    a.close()


def test_store_survives_a_killed_writer(tmp_path):
    """SIGKILL a process that is writing conversations: the file reopens with every flushed conversation readable."""
    code = f"""
import sys, numpy as np
sys.path.insert(0, {os.path.dirname(HERE)!r})
from llm_distillery_b200.data.h5store import H5Store
from llm_distillery_b200.data.convo import TeacherRows
st = H5Store({str(tmp_path)!r})
rng = np.random.default_rng(0)
i = 0
while True:
    st.write_batch([TeacherRows(i, rng.standard_normal((64, 32)).astype(np.float16),
                                rng.integers(0, 32000, (64, 32)).astype(np.int64), 'sha%d' % i, 's')])
    i += 1
    if i % 10 == 0:
        st.wait(); st.flush(); print(i, flush=True)
"""
    p = subprocess.Popen([sys.executable, "-c", code], stdout=subprocess.PIPE, text=True)
    flushed = 0
    while flushed < 50:
        line = p.stdout.readline()
        assert line, "writer ended early"
        flushed = int(line)
    time.sleep(0.05)
    os.kill(p.pid, signal.SIGKILL)           # the exact process started above
    p.wait()
    from llm_distillery_b200.data.h5store import H5Store
    st = H5Store(str(tmp_path))
    ids = st.get_dataset_ids()
    assert len(ids) >= flushed
    for cid in ids:
        v, ix = st.load_id(cid)
        assert v.shape == (64, 32) and ix.shape == (64, 32) and np.isfinite(v.astype(np.float32)).all()
    st.close()


def test_truncated_store_is_refused_cleanly(tmp_path):
    from llm_distillery_b200.data.convo import TeacherRows
    from llm_distillery_b200.data.h5store import H5Store
    st = H5Store(str(tmp_path))
    st.write_batch([TeacherRows(1, np.zeros((8, 4), np.float16), np.zeros((8, 4), np.int64), "x", "s")])
    st.close()
    p = os.path.join(str(tmp_path), "distributions.hdf5")
    data = open(p, "rb").read()
    q = os.path.join(str(tmp_path), "cut.hdf5")
    open(q, "wb").write(data[: len(data) // 2])
    with pytest.raises(IOError):
        H5Store(q)


def test_ranks_learn_of_a_lost_peer_and_leave(tmp_path):
    """Three gloo ranks; rank 2 leaves between steps without a goodbye. The others either see its heartbeat stop
    before their next collective or get an error out of that collective, attribute it through the heartbeat, and
    leave in order."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_worker.py"), "cpu_rank_loss", str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, OMP_NUM_THREADS="1", B200_NO_PROGRESS="1"))
    assert r.stdout.count("SURVIVOR_OK") == 2, (r.stdout[-2000:], r.stderr[-3000:])
