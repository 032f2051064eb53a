"""Failure detection and recovery on the host (no GPU involved): heartbeat logic against a fake
store and clock, a Gloo job in which one rank dies between steps, and an elastic restart that resumes
from the last complete checkpoint."""
import os
import subprocess
import sys
import tempfile

import pytest

from dist_utils import ROOT, TINY, free_port, run_trainer


class _FakeStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_heartbeat_detects_silent_and_failed_peers():
    from train_large_model_from_scratch_b200.utils.health import Heartbeat, PeerFailure
    store, now = _FakeStore(), [100.0]
    clock = lambda: now[0]
    a = Heartbeat(0, 2, timeout_s=5.0, store=store, clock=clock)
    b = Heartbeat(1, 2, timeout_s=5.0, store=store, clock=clock)
    a.check(); b.check()
    a.beat(0); b.beat(0)
    now[0] += 4.0
    a.check()                                            # within the limit
    a.beat(1)
    now[0] += 6.0                                        # rank 1's heartbeat has not changed for 6 s on rank 0's clock
    with pytest.raises(PeerFailure) as e:
        a.check()
    assert e.value.rank == 1 and "no heartbeat" in str(e.value)
    b.check()                                            # rank 0 is fresh from rank 1's point of view
    b.beat(1)
    a.check()
    b.announce_failure("ValueError: boom")
    with pytest.raises(PeerFailure) as e:
        a.check()
    assert e.value.rank == 1 and "boom" in str(e.value)


def test_long_pause_between_steps_is_not_a_failure_but_a_missing_peer_is():
    """Evaluation, a checkpoint or set-up between two steps may outlast the heartbeat limit on every rank:
    `enter_step` judges liveness by the rendezvous itself (the peer arrives within the limit counted from
    now), not by the age of the last heartbeat."""
    from train_large_model_from_scratch_b200.utils.health import Heartbeat, PeerFailure
    store, now = _FakeStore(), [0.0]

    def clock():
        now[0] += 0.05
        return now[0]
    a = Heartbeat(0, 2, timeout_s=3.0, store=store, clock=clock)
    b = Heartbeat(1, 2, timeout_s=3.0, store=store, clock=clock)
    a.beat(0); b.beat(0)
    a.check(); b.check()
    now[0] += 500.0                                      # both ranks spend 500 s in evaluation + save
    store.set("tlm/enter/0", "1")                        # rank 0 arrives at step 1 ...
    b.enter_step(1, poll_s=0.0)                          # ... and rank 1 joins without complaint
    a.enter_step(1, poll_s=0.0)
    a.beat(1)
    with pytest.raises(PeerFailure) as e:                # rank 1 never arrives at step 2
        a.enter_step(2, poll_s=0.0)
    assert e.value.rank == 1 and "did not arrive" in str(e.value)


def test_device_timeout_aborts_the_step_before_it_is_logged_or_saved(tmp_path, monkeypatch):
    """A nonzero device status word after a step (a kernel gave up on a flag wait, so its exchange did not
    happen) must end the run before the step is committed: no log line, no checkpoint."""
    import torch
    from train_large_model_from_scratch_b200.training import Trainer, build_config, parse_args
    from train_large_model_from_scratch_b200.utils.health import DeviceTimeout
    flags = TINY + ["--log_dir", str(tmp_path), "--total_batch_size", "512", "--batch_size", "2",
                    "--do_save", "--save_every_steps", "1", "--sep_size", "1"]
    trainer = Trainer(build_config(parse_args(flags)))
    calls = {"n": 0}

    def fake_status():
        calls["n"] += 1
        return (41 << 8) | 1 if calls["n"] == 2 else 0       # the second step's reduce-scatter timed out

    monkeypatch.setattr(trainer, "_read_device_status", fake_status)
    with pytest.raises(DeviceTimeout) as e:
        trainer.train()
    assert e.value.status == (41 << 8) | 1 and "site 41" in str(e.value)
    log = open(trainer.log_file).read().splitlines()
    assert len(log) == 1 and log[0].startswith("0 train")      # step 1 was never logged
    import glob
    assert not glob.glob(str(tmp_path / "*" / "00001_meta.pt"))
    trainer.close()


def test_wait_for_step_times_out_on_a_lagging_peer():
    from train_large_model_from_scratch_b200.utils.health import Heartbeat, PeerFailure
    store, now = _FakeStore(), [0.0]

    def clock():
        now[0] += 0.3                                    # every look at the clock advances time
        return now[0]
    a = Heartbeat(0, 2, timeout_s=3.0, store=store, clock=clock)
    Heartbeat(1, 2, timeout_s=3.0, store=store, clock=clock)
    a.beat(0)
    with pytest.raises(PeerFailure) as e:
        a.wait_for_step(0, poll_s=0.0)
    assert e.value.rank == 1


def test_rank_death_between_steps_is_reported_by_the_survivor():
    tmp = tempfile.mkdtemp(prefix="tlm_fault_")
    flags = TINY + ["--log_dir", tmp, "--total_batch_size", "512", "--batch_size", "2", "--sep_size", "1",
                    "--use_distributed_optimizer", "--heartbeat_timeout_s", "4", "--dist_timeout_s", "30"]
    codes, logs = run_trainer(2, flags, {"TLM_EXIT_RANK": "1", "TLM_EXIT_BEFORE_STEP": "2"}, timeout=240,
                              expect_fail=True)
    assert codes[1] == 17                                 # the rank that left
    assert codes[0] not in (0, None), logs[0][-2000:]     # the survivor ends with an error, it does not hang
    assert "PeerFailure" in logs[0] and "rank 1" in logs[0], logs[0][-2000:]


def test_restart_after_rank_death_resumes_from_last_complete_checkpoint():
    """What an elastic launcher does after a failure: start every rank again with the same command.
    The second attempt must pick up after the last complete checkpoint and finish."""
    tmp = tempfile.mkdtemp(prefix="tlm_elastic_")
    flags = TINY + ["--log_dir", tmp, "--total_batch_size", "512", "--batch_size", "2", "--sep_size", "1",
                    "--use_distributed_optimizer", "--do_save", "--save_every_steps", "2",
                    "--heartbeat_timeout_s", "4", "--dist_timeout_s", "30"]
    codes, logs = run_trainer(2, flags, {"TLM_EXIT_RANK": "1", "TLM_EXIT_BEFORE_STEP": "5"}, timeout=240,
                              expect_fail=True)
    assert codes[1] == 17 and codes[0] not in (0, None)
    assert "PeerFailure" in logs[0]
    second = run_trainer(2, flags, timeout=240)
    assert second["start_step"] == 5                      # steps 0..4 were done; the step-4 checkpoint is complete
    assert max(int(k) for k in second["losses"]) == 7     # ran to the end (8 steps)
