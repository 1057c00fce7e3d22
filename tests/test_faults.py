"""Failure detection, all on the host (no GPU is made to fault, trap or hang).

A rank that dies, never joins, stalls or aborts must turn into an error code on the other ranks within
a bounded time: ncclRemoteError (6) when the watchdog saw the peer go, ncclInternalError (3) when a
transfer made no progress for the configured timeout, ncclSystemError (2) for a failed join. The
device-side counterpart (a kernel wait that runs out and reports through the status block) is in
tests/test_gpu_emu.py::test_bounded_wait_returns_a_status.
"""
import os
import time

from dccl_b200.utils.launch import python_ranks

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "workers", "fault_worker.py")


def results(res):
    out = []
    for p in res:
        lines = [ln for ln in p.stdout.splitlines() if ln.startswith("RESULT")]
        out.append(lines[-1] if lines else "")
    return out


def test_rank_that_exits_is_detected_by_the_watchdog():
    t0 = time.time()
    res = python_ranks(WORKER, ["--mode", "exit_mid_run", "--victim", "2"], 4, timeout=60, env_extra={"DCCL_TIMEOUT_MS": "20000"})
    took = time.time() - t0
    r = results(res)
    assert res[2].returncode == 9
    for i in (0, 1, 3):
        assert r[i].startswith("RESULT error"), (i, r[i], res[i].stderr[-500:])
        assert "code=6" in r[i], r[i]                     # ncclRemoteError: the heartbeat watchdog flagged the dead rank
        assert "rank 2" in r[i]
    assert took < 30, "survivors must not wait for the 20 s transfer timeout"


def test_stalled_rank_runs_into_the_transfer_timeout():
    res = python_ranks(WORKER, ["--mode", "stall", "--victim", "1"], 3, timeout=60, env_extra={"DCCL_TIMEOUT_MS": "500"})
    r = results(res)
    assert any("code=3" in x for x in (r[0], r[2])), r      # ncclInternalError: no progress for 500 ms


def test_rank_that_never_joins_fails_the_join():
    t0 = time.time()
    res = python_ranks(WORKER, ["--mode", "none"], 3, timeout=60,
                       env_extra={"DCCL_FAULT": "drop_hello@1", "DCCL_INIT_TIMEOUT_MS": "2000"})
    r = results(res)
    assert all("init_failed code=2" in x for x in r), r
    assert time.time() - t0 < 30


def test_rank_that_exits_during_a_control_operation():
    # rank 1 leaves the process at its second control operation (the join barrier is the first)
    res = python_ranks(WORKER, ["--mode", "none"], 3, timeout=60,
                       env_extra={"DCCL_FAULT": "exit_at_barrier=1@1", "DCCL_INIT_TIMEOUT_MS": "5000", "DCCL_BOOTSTRAP_TIMEOUT_MS": "5000"})
    r = results(res)
    assert res[1].returncode == 17
    assert all(("init_failed" in r[i]) or ("error" in r[i]) for i in (0, 2)), r


def test_slow_rank_only_delays():
    res = python_ranks(WORKER, ["--mode", "none"], 3, timeout=120, env_extra={"DCCL_FAULT": "delay_ms=30@2"})
    r = results(res)
    assert all(x == "RESULT completed code=0" for x in r), r


def test_local_abort_unblocks_everybody():
    res = python_ranks(WORKER, ["--mode", "abort_local", "--victim", "0"], 3, timeout=60, env_extra={"DCCL_TIMEOUT_MS": "20000"})
    r = results(res)
    assert all(x.startswith("RESULT error") for x in r), r


def test_survivors_shrink_the_group_and_carry_on():
    """Rank 1 of 4 dies; ranks 0, 2, 3 become ranks 0, 1, 2 of a new group and reduce again. With rank 0 as the
    victim the lowest survivor leads the new rendezvous instead."""
    for victim in (1, 0):
        res = python_ranks(WORKER, ["--mode", "exit_then_shrink", "--victim", str(victim)], 4, timeout=90, env_extra={"DCCL_TIMEOUT_MS": "20000"})
        r = results(res)
        assert res[victim].returncode == 9
        for i in range(4):
            if i != victim:
                assert r[i].startswith("RESULT shrunk ok=1 world=3"), (victim, i, r[i], res[i].stderr[-800:])
