"""Weight-sync rounds as a state machine (tunix/experimental/weight_sync/weight_sync_coordinator.py:500-600).

A round moves trainer weights of one policy version to a set of rollout workers:

    PREPARING -> TRANSFERRING -> COMMITTING -> COMMITTED
         \\            \\             \\
          +-> ABORTED  +-> ABORTED   +-> UNKNOWN_TRANSFER_STATE

Every phase has a timeout. A failure before any worker was told to commit aborts the round and every prepared
worker rolls back to the version it had; a failure while commits are in flight leaves the set of workers in an
unknown mix of versions, which poisons the round: the coordinator refuses further rounds until the caller has
re-established a known state (`reset_after_unknown`). The transport is whatever `WeightSyncParticipant`
implements: in this framework `rl.reshard.WeightReshard.run` for the transfer itself."""
from __future__ import annotations

import enum
import time
from typing import Callable, Optional, Protocol, Sequence


class RoundState(str, enum.Enum):
    IDLE = "idle"
    PREPARING = "preparing"
    TRANSFERRING = "transferring"
    COMMITTING = "committing"
    COMMITTED = "committed"
    ABORTED = "aborted"
    UNKNOWN_TRANSFER_STATE = "unknown_transfer_state"


PHASE_TIMEOUTS_S = {RoundState.PREPARING: 120.0, RoundState.TRANSFERRING: 600.0, RoundState.COMMITTING: 120.0}


class WeightSyncParticipant(Protocol):
    worker_id: str

    def prepare(self, version: int) -> None: ...       # pause admission, allocate staging
    def transfer(self, version: int) -> None: ...      # receive the weights into staging
    def commit(self, version: int) -> None: ...        # swap staging in, resume
    def rollback(self) -> None: ...                    # drop staging, resume on the old version


class WeightSyncError(RuntimeError):
    pass


class WeightSyncCoordinator:
    def __init__(self, participants: Sequence[WeightSyncParticipant], timeouts: Optional[dict] = None,
                 clock: Callable[[], float] = time.monotonic):
        self.participants = list(participants)
        self.timeouts = dict(PHASE_TIMEOUTS_S, **(timeouts or {}))
        self.clock = clock
        self.state = RoundState.IDLE
        self.version = 0
        self.history: list = []

    def _phase(self, state: RoundState, fn: Callable, done: list) -> None:
        self.state = state
        t0 = self.clock()
        for p in self.participants:
            fn(p)
            done.append(p)
            if self.clock() - t0 > self.timeouts[state]:
                raise TimeoutError(f"{state.value} exceeded {self.timeouts[state]} s")

    def run_round(self, version: int) -> RoundState:
        if self.state == RoundState.UNKNOWN_TRANSFER_STATE:
            raise WeightSyncError("a previous round ended in an unknown transfer state; call reset_after_unknown() first")
        prepared, transferred, committed = [], [], []
        try:
            self._phase(RoundState.PREPARING, lambda p: p.prepare(version), prepared)
            self._phase(RoundState.TRANSFERRING, lambda p: p.transfer(version), transferred)
        except BaseException as e:
            for p in prepared:
                try:
                    p.rollback()
                except BaseException:
                    pass
            self.state = RoundState.ABORTED
            self.history.append((version, self.state, repr(e)))
            return self.state
        try:
            self._phase(RoundState.COMMITTING, lambda p: p.commit(version), committed)
        except BaseException as e:
            # some workers run the new version, some the old one, one of them possibly half-way
            self.state = RoundState.UNKNOWN_TRANSFER_STATE
            self.history.append((version, self.state, repr(e)))
            return self.state
        self.state, self.version = RoundState.COMMITTED, version
        self.history.append((version, self.state, ""))
        return self.state

    def reset_after_unknown(self, known_version: int) -> None:
        """The caller has restarted or re-synchronised every worker to `known_version`."""
        if self.state != RoundState.UNKNOWN_TRANSFER_STATE:
            raise WeightSyncError("nothing to reset")
        self.state, self.version = RoundState.IDLE, known_version
