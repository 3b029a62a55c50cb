"""`rl.Trainer`: PeftTrainer + RL aux-metric plumbing + `{global_step, role}` checkpoint metadata
(tunix/rl/trainer.py:29-125)."""
from __future__ import annotations

from typing import Any, Optional

from ..sft.peft_trainer import PeftTrainer


class Trainer(PeftTrainer):
    def __init__(self, model, optimizer, training_config, metrics_logger=None, perf_tracer=None, role: str = "actor"):
        super().__init__(model, optimizer, training_config, metrics_logger, perf_tracer)
        self.role = role
        self.rl_metrics_to_log: dict = {}
        self.restored_global_step = int((self._restored_custom_metadata or {}).get("global_step", 0))
        self.global_step = self.restored_global_step
        self.is_managed_externally = True
        self._last_aux: Optional[dict] = None

    def with_rl_metrics_to_log(self, rl_metrics_to_log: dict) -> "Trainer":
        """{aux key: reducer} of loss-aux entries to forward to the metrics logger."""
        self.rl_metrics_to_log = rl_metrics_to_log
        return self

    def _shard_and_move(self, batch):
        """RL examples are produced on this rank from this rank's own rollouts: they are moved to the device but
        never sliced by rank (the SFT trainer slices a global batch that every rank received in full)."""
        import dataclasses

        from ..sft.peft_trainer import _to_device
        if dataclasses.is_dataclass(batch) and not isinstance(batch, type):
            return dataclasses.replace(batch, **{f.name: _to_device(getattr(batch, f.name), self.device)
                                                 for f in dataclasses.fields(batch)})
        if isinstance(batch, dict):
            return {k: _to_device(v, self.device) for k, v in batch.items()}
        return batch

    def set_global_step(self, step: int) -> None:
        self.global_step = step

    def _checkpoint_metadata(self) -> dict:
        return {"global_step": self.global_step, "role": self.role}

    def _post_process_train_step(self, aux: Any) -> None:
        self._last_aux = aux if isinstance(aux, dict) else None

    def _aux_metrics(self, aux):
        out = super()._aux_metrics(aux) or {}
        if self.rl_metrics_to_log and isinstance(aux, dict):
            for k, op in self.rl_metrics_to_log.items():
                if k in aux:
                    v = aux[k]
                    out[k] = (v[0], v[1]) if isinstance(v, tuple) else (v, op)
        return out or None
