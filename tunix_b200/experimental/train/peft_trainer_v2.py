"""`TrainerV2`: the split-step protocol on top of `PeftTrainer` (tunix/experimental/train/peft_trainer_v2.py).

`PeftTrainer.train` owns its loop (data iterator, accumulation count, checkpoint cadence). The distributed engine
instead calls `fwd_bwd` per micro-batch, as they arrive from the batch assembler, and `update` when a mini-batch
is complete, so the number of micro-batches per step may vary (filtered groups, ragged tails). Loss function, input
preparation, optimizer (sharded or not), metrics logger and checkpoint manager are the wrapped trainer's."""
from __future__ import annotations

from typing import Any, Optional

import torch

from ...sft.peft_trainer import PeftTrainer
from ...sft.utils import WeightedMetric
from .abstract_trainer import AbstractTrainer


def _scalar(metric) -> float:
    if isinstance(metric, WeightedMetric):
        return float(metric.value().item())
    return float(metric.item()) if hasattr(metric, "item") else float(metric)


class TrainerV2(AbstractTrainer):
    def __init__(self, trainer: PeftTrainer):
        self.trainer = trainer
        self._pending = 0
        self._closed_last = False

    @property
    def train_steps(self) -> int:
        return self.trainer.train_steps

    def fwd_bwd(self, batch: Any, is_last_microbatch: bool = False) -> dict:
        """`is_last_microbatch` lets a sharded optimizer overlap its gradient reduction with this backward pass;
        it must be set on the last micro-batch before `update` when the optimizer is sharded."""
        tr = self.trainer
        batch = tr._prepare_inputs(batch)
        inputs = tr.gen_model_input_fn(batch)
        out = tr.loss_fn(tr.model, **inputs)
        to_diff, metric, denom, aux = tr._unpack_loss(out)
        prepare = getattr(tr.optimizer, "prepare_backward", None)
        if prepare is not None:
            prepare(is_last_microbatch)
        to_diff.backward()
        tr.optimizer.buffers.collect_autograd_grads()
        tr._denoms.append(denom.detach() if denom is not None else None)
        self._pending += 1
        self._closed_last = is_last_microbatch
        return {"loss": _scalar(metric), "aux": aux, "pending_microbatches": self._pending}

    def update(self) -> dict:
        tr = self.trainer
        if self._pending == 0:
            raise RuntimeError("update() without a preceding fwd_bwd()")
        if getattr(tr.optimizer, "is_sharded", False) and not self._closed_last:
            raise RuntimeError("a sharded optimizer reduces gradients during the last backward pass: "
                               "call fwd_bwd(..., is_last_microbatch=True) before update()")
        local = False
        if tr._denoms and tr._denoms[0] is not None:
            denominator, local = tr._reduce_denominator(torch.stack([d.float() for d in tr._denoms]).sum())
        else:
            denominator = float(len(tr._denoms))
        grad_norm = tr._optimizer_step(denominator, local)
        tr.optimizer.zero_grad()
        tr._denoms = []
        n, self._pending = self._pending, 0
        tr._train_steps += 1
        gn = float(grad_norm.item()) if hasattr(grad_norm, "item") else grad_norm
        return {"step": tr._train_steps, "grad_norm": gn, "microbatches": n}

    def eval_step(self, batch: Any) -> dict:
        tr = self.trainer
        was = tr.model.training
        tr.model.eval()
        try:
            metric, aux = tr._eval_step(tr._prepare_inputs(batch))
        finally:
            tr.model.train(was)
        return {"loss": _scalar(metric), "aux": aux}

    @torch.no_grad()
    def fwd_only(self, batch: Any, fn=None) -> Any:
        """`fn(model, **inputs)` under no_grad; by default the model's forward on the prepared inputs."""
        tr = self.trainer
        inputs = tr.gen_model_input_fn(tr._prepare_inputs(batch))
        if fn is not None:
            return fn(tr.model, **inputs)
        return tr.model(inputs["input_tokens"], positions=inputs.get("positions"), segment_ids=inputs.get("segment_ids"))[0]

    def save_checkpoint(self, step: Optional[int] = None, force: bool = False, custom_metadata: Optional[dict] = None) -> bool:
        tr = self.trainer
        meta = dict(tr._checkpoint_metadata())
        meta.update(custom_metadata or {})
        return bool(tr.checkpoint_manager.save(tr._train_steps if step is None else step, tr.model, tr.optimizer,
                                               save_only_lora_params=tr._lora, force=force, custom_metadata=meta))

    def restore_checkpoint(self, step: Optional[int] = None) -> int:
        tr = self.trainer
        got, meta = tr.checkpoint_manager.maybe_restore(tr.model, tr.optimizer, step=step, restore_only_lora_params=tr._lora)
        if got:
            tr._train_steps = got
            tr._restored_custom_metadata = meta
        self._restored_step = int(got or 0)
        return got

    def wait_for_checkpoints(self) -> None:
        """Block until background checkpoint writes have finished."""
        self.trainer.checkpoint_manager.wait_until_finished()

    def restored_metadata(self) -> Optional[dict]:
        """The custom metadata of the checkpoint that the last `restore_checkpoint` read (None if there was none),
        with the restored optimizer step under `step` when the writer did not record one."""
        if not getattr(self, "_restored_step", 0):
            return None
        out = dict(getattr(self.trainer, "_restored_custom_metadata", None) or {})
        out.setdefault("step", self._restored_step)
        return out

    def get_metrics(self) -> dict:
        """Optimizer steps taken and micro-batches waiting for `update`."""
        return {"train_steps": self.trainer._train_steps, "pending_microbatches": self._pending}
