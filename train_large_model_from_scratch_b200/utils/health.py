"""Host-side failure detection for multi-rank jobs.

The reference has none (a dead rank leaves the others blocked in their next
collective until the process-group timeout, `training/trainer.py:63`; recovery
is "run the same command again", `training/trainer.py:266-306`). Here every
rank publishes a heartbeat (its step counter and a wall-clock stamp) in the
job's key-value store between steps, and checks its peers' heartbeats BEFORE
it launches the next step, i.e. with none of its kernels or collectives in
flight. A rank whose heartbeat is older than the limit, or that announced a
failure, makes `check()` raise `PeerFailure` naming that rank, so the job ends
with a clear error (and a non-zero exit code, which an elastic launcher such as
`torchrun --max-restarts` turns into a restart from the last complete
checkpoint) instead of hanging in a collective.

Nothing here touches a GPU: a failure is always learned on the host.
"""
from __future__ import annotations

import time

import torch.distributed as dist


class PeerFailure(RuntimeError):
    """Another rank failed or stopped answering."""

    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} {reason}")
        self.rank, self.reason = rank, reason


class DeviceTimeout(RuntimeError):
    """A kernel of this rank gave up on a bounded wait (flag, barrier or mbarrier): `status` is the device
    status word, `site << 8 | detail`. The exchange the kernel was waiting for did not happen, so the data it
    would have produced (a gradient shard, a received tile) is stale and the step must not be kept."""

    def __init__(self, status: int):
        super().__init__(f"a kernel timed out waiting at site {status >> 8} (detail {status & 0xff}); "
                         f"the step's result is not valid")
        self.status = int(status)


class Heartbeat:
    """`enter_step(step)` before each step, `beat(step)` after it (and after anything long that runs between
    steps: evaluation, a checkpoint); `check()` at any time.

    Ages are measured on the READER's clock: a peer's heartbeat is as old as the time since this rank first
    saw its current value, so clocks of different hosts are never compared.

    `store` is any c10d store shared by the job (default: the store of the
    default process group). Keys: `tlm/hb/<rank>` = "<step>:<unix time>",
    `tlm/enter/<rank>` = "<step>", `tlm/failed/<rank>` = reason."""

    def __init__(self, rank: int, world_size: int, timeout_s: float, store=None, clock=time.time, prefix: str = "tlm"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store, self.rank, self.world, self.timeout, self.clock = store, rank, world_size, float(timeout_s), clock
        self.prefix = prefix
        self._seen: dict = {}               # peer rank -> (raw heartbeat value, local time it was first seen)
        self.beat(-1)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self, step: int) -> None:
        self.last_step = step
        self.store.set(self._key("hb", self.rank), f"{step}:{self.clock():.3f}")

    def announce_failure(self, reason: str) -> None:
        """Called by a rank that is about to leave (e.g. from an exception handler)."""
        try:
            self.store.set(self._key("failed", self.rank), reason[:200] or "failed")
        except Exception:                                    # the store may already be gone
            pass

    def peer_state(self, rank: int):
        """(step, age in seconds) of `rank`'s last heartbeat, or None before its first one. The age counts from
        the moment THIS rank first read the current value (its own clock), not from the writer's time stamp."""
        key = self._key("hb", rank)
        if not self.store.check([key]):
            return None
        raw = self.store.get(key).decode()
        now = self.clock()
        seen = self._seen.get(rank)
        if seen is None or seen[0] != raw:
            seen = self._seen[rank] = (raw, now)
        return int(raw.split(":")[0]), now - seen[1]

    def check(self, ages: bool = True) -> None:
        """Raise `PeerFailure` if a peer announced a failure or (`ages`) has been silent for longer than the
        limit."""
        for r in range(self.world):
            if r == self.rank:
                continue
            fkey = self._key("failed", r)
            if self.store.check([fkey]):
                raise PeerFailure(r, f"reported a failure: {self.store.get(fkey).decode()}")
            if not ages:
                continue
            st = self.peer_state(r)
            if st is not None and self.timeout > 0 and st[1] > self.timeout:
                raise PeerFailure(r, f"sent no heartbeat for {st[1]:.1f} s (limit {self.timeout:.1f} s, last step {st[0]})")

    def enter_step(self, step: int, poll_s: float = 0.02) -> None:
        """Rendezvous on the host before a step: publish "I am about to run `step`" and wait until every
        peer has published the same (or a later) step. A peer that died or stalled after its last heartbeat
        never does, so this raises `PeerFailure` after the limit, before anything is launched.
        Liveness is judged by this rendezvous alone (and by announced failures), not by heartbeat ages: set-up,
        evaluation or a checkpoint between two steps may take longer than the limit on every rank, and a
        healthy peer that is still busy with them simply arrives late, within the limit counted from now."""
        self.beat(self.last_step)
        self.store.set(self._key("enter", self.rank), str(step))
        t0 = self.clock()
        while True:
            self.check(ages=False)
            late = []
            for r in range(self.world):
                if r == self.rank:
                    continue
                key = self._key("enter", r)
                if not self.store.check([key]) or int(self.store.get(key).decode()) < step:
                    late.append(r)
            if not late:
                return
            if self.timeout > 0 and self.clock() - t0 > self.timeout:
                raise PeerFailure(late[0], f"did not arrive at step {step} within {self.timeout:.1f} s")
            time.sleep(poll_s)

    def wait_for_step(self, step: int | None = None, poll_s: float = 0.05) -> None:
        """Block (on the host) until every peer has finished `step` (default: the last step this rank
        finished itself), checking health while waiting. Used before a step whose collectives would
        otherwise be the first to notice a dead peer."""
        if step is None:
            step = self.last_step
        t0 = self.clock()
        while True:
            self.check()
            states = [self.peer_state(r) for r in range(self.world) if r != self.rank]
            if all(s is not None and s[0] >= step for s in states):
                return
            if self.timeout > 0 and self.clock() - t0 > self.timeout:
                lag = [r for r in range(self.world) if r != self.rank
                       and (self.peer_state(r) is None or self.peer_state(r)[0] < step)]
                raise PeerFailure(lag[0], f"did not reach step {step} within {self.timeout:.1f} s")
            time.sleep(poll_s)
