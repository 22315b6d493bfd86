"""Rank health: heartbeats through the rendezvous store, failure detection between steps, and host-side fault injection.

The reference is single-process and has none of this (its failure handling is OaStatus propagation and the device
admission canary).  A multi-GPU job needs one more thing: when a rank dies, the others must learn of it on the HOST,
between steps, before they launch a kernel that would wait on the dead rank's memory.  Every rank therefore publishes a
heartbeat (its step counter and a wall-clock stamp) under its own key of the process group's store, and checks its
peers' stamps before each step:

    monitor = OaRankMonitor(store, rank, world, timeout_s=5.0)
    for step in range(n):
        monitor.Beat(step)
        st = monitor.Check()             # OaStatus: Unavailable names the silent ranks
        if not st.IsOk(): break          # leave between steps: nothing of ours is in flight
        train_step()

A rank that finishes on purpose calls `Leave()` so that its silence is not taken for a failure.  `OaFaultInjector` makes
failures on the host only (a rank that raises, exits, stops beating or delays a beat at a chosen step); nothing here
touches a device, so the tests run as CPU processes.
"""
from __future__ import annotations

import os
import struct
import sys
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from ..core.types import OaStatus, OaStatusCode

_BEAT = struct.Struct("<qdB")            # step, wall-clock seconds, state (0 alive, 1 left on purpose, 2 reported failure)
ALIVE, LEFT, FAILED = 0, 1, 2


class OaRankFailure(RuntimeError):
    def __init__(self, ranks: List[int], message: str):
        super().__init__(message)
        self.Ranks = ranks


@dataclass
class OaRankState:
    Rank: int
    Step: int = -1
    Stamp: float = 0.0
    State: int = ALIVE
    Seen: bool = False

    def Age(self, now: Optional[float] = None) -> float:
        return (now if now is not None else time.time()) - self.Stamp if self.Seen else float("inf")


class OaRankMonitor:
    """`store` is any object with set(key, bytes) / get(key) -> bytes that raises (or blocks at most its own timeout) on
    a missing key: the TCPStore / FileStore behind a process group, or a dict-backed stand-in in tests."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 10.0, prefix: str = "oa/health", clock: Callable[[], float] = time.time):
        self._store, self.Rank, self.World, self.TimeoutS, self._prefix, self._clock = store, rank, world, float(timeout_s), prefix, clock
        self._start = clock()
        self._last: Dict[int, OaRankState] = {r: OaRankState(r) for r in range(world)}

    def _key(self, rank: int) -> str: return f"{self._prefix}/{rank}"

    def _publish(self, step: int, state: int) -> None:
        self._store.set(self._key(self.Rank), _BEAT.pack(int(step), self._clock(), state))

    def Beat(self, step: int) -> None: self._publish(step, ALIVE)
    def Leave(self, step: int = -1) -> None: self._publish(step, LEFT)
    def ReportFailure(self, step: int = -1) -> None: self._publish(step, FAILED)

    def _read(self, rank: int) -> OaRankState:
        st = self._last[rank]
        try:
            check = getattr(self._store, "check", None)
            if check is not None and not check([self._key(rank)]):
                return st                                     # never published: do not block on the key
            blob = bytes(self._store.get(self._key(rank)))
            step, stamp, state = _BEAT.unpack(blob[:_BEAT.size])
            st.Step, st.Stamp, st.State, st.Seen = step, stamp, state, True
        except Exception:                                     # missing key or a store that went away with its host rank
            pass
        return st

    def Peers(self) -> List[OaRankState]:
        return [self._read(r) for r in range(self.World)]

    def WaitForPeers(self, timeout_s: float = 60.0, poll_s: float = 0.05) -> OaStatus:
        """Start-up rendezvous: publish a first beat and wait until every peer has published one, so that process start-up
        skew is not mistaken for a failure.  The silence clock of every peer starts when this returns."""
        self.Beat(-1)
        deadline = self._clock() + timeout_s
        while True:
            missing = [s.Rank for s in self.Peers() if not s.Seen]
            if not missing:
                break
            if self._clock() > deadline:
                return OaStatus(OaStatusCode.DeadlineExceeded, f"rank(s) {missing} never published a heartbeat")
            time.sleep(poll_s)
        self._start = self._clock()
        self.Beat(-1)
        return OaStatus.Ok()

    def Check(self) -> OaStatus:
        """Ok while every peer is alive (or left on purpose); Unavailable naming the ranks that reported a failure or have
        been silent for longer than the timeout (a rank that never published counts from this monitor's creation)."""
        now = self._clock()
        bad = []
        for s in self.Peers():
            if s.Rank == self.Rank or s.State == LEFT:
                continue
            # silence counts from the later of the peer's last beat and the end of this rank's own rendezvous: a beat that
            # aged while this rank was still waiting for a slower third rank is start-up skew, not a failure
            silent = (now - max(s.Stamp, self._start)) if s.Seen else (now - self._start)
            if s.State == FAILED or silent > self.TimeoutS:
                bad.append(s.Rank)
        self.LastBad = bad                       # the ranks this pass found gone (Guard reports exactly these)
        if bad:
            return OaStatus(OaStatusCode.Unavailable, f"rank(s) {bad} failed or stopped responding (timeout {self.TimeoutS:.1f} s)")
        return OaStatus.Ok()

    def Guard(self, step: int) -> None:
        """Beat, then raise OaRankFailure if a peer is gone: call it first thing in every step."""
        self.Beat(step)
        st = self.Check()
        if not st.IsOk():
            raise OaRankFailure(list(self.LastBad), st.message)     # one pass over the store: list and message agree

    def SlowestPeer(self) -> Optional[OaRankState]:
        alive = [s for s in self.Peers() if s.Seen and s.State == ALIVE]
        return min(alive, key=lambda s: s.Step) if alive else None


class OaFaultKind:
    Raise = "raise"            # the rank raises an exception at the step
    Exit = "exit"              # the rank's process exits without a word
    Silence = "silence"        # the rank keeps running but stops publishing heartbeats
    Delay = "delay"            # the rank's next heartbeat is late by `Seconds`


@dataclass
class OaFault:
    Rank: int
    Step: int
    Kind: str = OaFaultKind.Raise
    Seconds: float = 0.0


class OaFaultInjector:
    """Host-side faults by schedule.  `OA_FAULT="rank:step:kind[:seconds],..."` configures it from the environment."""

    def __init__(self, faults: Optional[List[OaFault]] = None):
        self.Faults = list(faults or [])
        self.Silenced = False

    @staticmethod
    def FromEnv(name: str = "OA_FAULT") -> "OaFaultInjector":
        out = []
        kinds = (OaFaultKind.Raise, OaFaultKind.Exit, OaFaultKind.Silence, OaFaultKind.Delay)
        for item in filter(None, (x.strip() for x in os.environ.get(name, "").split(","))):
            p = item.split(":")
            try:
                if not 2 <= len(p) <= 4:
                    raise ValueError("expected rank:step[:kind[:seconds]]")
                fault = OaFault(int(p[0]), int(p[1]), p[2] if len(p) > 2 else OaFaultKind.Raise, float(p[3]) if len(p) > 3 else 0.0)
                if fault.Kind not in kinds:
                    raise ValueError(f"unknown kind {fault.Kind!r} (one of {', '.join(kinds)})")
                if fault.Rank < 0 or fault.Seconds < 0:
                    raise ValueError("rank and seconds must not be negative")
            except ValueError as e:
                raise ValueError(f"{name}: bad item {item!r}: {e}") from None
            out.append(fault)
        return OaFaultInjector(out)

    def AtStep(self, rank: int, step: int, monitor: Optional[OaRankMonitor] = None) -> None:
        """Call between steps (nothing in flight).  Applies the faults scheduled for (rank, step)."""
        for f in self.Faults:
            if f.Rank != rank or f.Step != step:
                continue
            if f.Kind == OaFaultKind.Raise:
                if monitor is not None:
                    monitor.ReportFailure(step)
                raise RuntimeError(f"injected failure on rank {rank} at step {step}")
            if f.Kind == OaFaultKind.Exit:
                sys.stdout.flush()
                os._exit(17)
            if f.Kind == OaFaultKind.Silence:
                self.Silenced = True
            if f.Kind == OaFaultKind.Delay:
                time.sleep(f.Seconds)

    def Beat(self, monitor: OaRankMonitor, step: int) -> None:
        """The heartbeat a faulty rank would (not) send."""
        if not self.Silenced:
            monitor.Beat(step)
