"""Concrete participants of a weight-sync round (the work-unit side of
tunix/experimental/weight_sync/weight_sync.py:401-523: stage, commit, roll back).

`EngineParticipant` updates the model behind a continuous-batching engine server without ever letting a request
see half-updated weights:

    prepare   pause the server (admission stops, running requests finish and are delivered)
    transfer  pull the new tensors from `source()` into STAGING buffers on the rollout device, checking names,
              shapes and dtypes; the live parameters are untouched, so a failure here costs nothing
    commit    copy staging -> parameters (device-to-device, in place, so fused views and captured graphs keep
              their addresses), drop staging, resume the server (it re-reads fused / packed copies)
    rollback  drop staging and resume on the old weights

Staging doubles the rollout model's footprint for the length of the round; with `stage=False` the transfer phase
only validates and `commit` copies straight from the source (no extra memory, but a failure inside commit leaves
mixed weights, which the coordinator reports as UNKNOWN_TRANSFER_STATE)."""
from __future__ import annotations

from typing import Callable, Iterable, Optional

import torch


class EngineParticipant:
    def __init__(self, worker_id: str, model: torch.nn.Module, source: Callable[[], Iterable], server=None, *,
                 stage: bool = True, pause_timeout: Optional[float] = 120.0, strict: bool = True,
                 key_map: Optional[Callable[[str], Optional[str]]] = None):
        """`source()` yields `(name, tensor)` of the new weights (a trainer's `named_parameters()`, a LoRA-merged
        export, a resharding plan's output). `key_map` renames source names to this model's (None drops one)."""
        self.worker_id, self.model, self.source, self.server = worker_id, model, source, server
        self.stage, self.pause_timeout, self.strict, self.key_map = stage, pause_timeout, strict, key_map
        self.version = 0
        self._staged: Optional[dict] = None
        self._paused = False
        self.bytes_last_round = 0

    def _targets(self) -> dict:
        return dict(self.model.named_parameters())

    def _pairs(self):
        for name, t in self.source():
            if self.key_map is not None:
                name = self.key_map(name)
                if name is None:
                    continue
            yield name, t

    def prepare(self, version: int) -> None:
        if self._staged is not None or self._paused:
            raise RuntimeError(f"{self.worker_id}: a round is already open")
        if self.server is not None:
            if not self.server.pause(self.pause_timeout):
                self.server.resume()
                raise TimeoutError(f"{self.worker_id}: running requests did not drain in {self.pause_timeout} s")
            self._paused = True
        self._staged = {}

    def transfer(self, version: int) -> None:
        if self._staged is None:
            raise RuntimeError(f"{self.worker_id}: transfer before prepare")
        targets, seen, nbytes = self._targets(), set(), 0
        for name, t in self._pairs():
            dst = targets.get(name)
            if dst is None:
                if self.strict:
                    raise KeyError(f"{self.worker_id}: the source has {name!r}, the model does not")
                continue
            if tuple(t.shape) != tuple(dst.shape):
                raise ValueError(f"{self.worker_id}: {name}: shape {tuple(t.shape)} does not fit {tuple(dst.shape)}")
            seen.add(name)
            nbytes += dst.numel() * dst.element_size()
            if self.stage:
                self._staged[name] = t.detach().to(device=dst.device, dtype=dst.dtype, copy=True)
        missing = set(targets) - seen
        if self.strict and missing:
            raise KeyError(f"{self.worker_id}: the source lacks {sorted(missing)[:4]}{' ...' if len(missing) > 4 else ''}")
        self.bytes_last_round = nbytes

    @torch.no_grad()
    def commit(self, version: int) -> None:
        if self._staged is None:
            raise RuntimeError(f"{self.worker_id}: commit before prepare")
        targets = self._targets()
        pairs = self._staged.items() if self.stage else ((n, t) for n, t in self._pairs() if n in targets)
        for name, t in pairs:
            targets[name].copy_(t)
        self.version = version
        self._finish()

    def rollback(self) -> None:
        self._finish()

    def _finish(self) -> None:
        self._staged = None
        if self._paused and self.server is not None:
            self.server.resume()
        self._paused = False
