"""PeftTrainer: the training loop behind SFT, DPO, distillation and every RL actor / critic.

Behaviour follows tunix/sft/peft_trainer.py:284-1194:
  * trainable set = LoRA parameters when the model has adapters, else all parameters (:340-342);
  * a loss function returns a scalar, `(loss, aux)` or a `LossOutput` whose `WeightedMetric` carries the
    unreduced sum and the denominator; the sum is differentiated and gradients are divided by the summed
    denominator of all micro-batches of the update, which gives the exact token-weighted mean (:489-575);
  * an update happens every `gradient_accumulation_steps` micro-batches, or when a batch carries
    `is_update_step=True`;
  * metrics of step k are written while step k+1 runs (one-step delay, :784-801): the loss stays on the
    device until then, so logging never stalls the stream;
  * checkpoints: restore in the constructor, skip already-consumed batches on resume (:921-924), save on
    update steps, forced save in `close()`;
  * hooks, progress bar, profiler window, in-flight throttling, periodic eval.

One process per GPU: with `torch.distributed` initialised each rank consumes its slice of the global
batch (`sharding_utils.shard_input`) and the optimizer comes from `parallel.fsdp` (sharded states,
fused reduce-scatter + AdamW); single-process runs use `optim.py` directly.
"""
from __future__ import annotations

import dataclasses
import math
import time
from typing import Any, Callable, Iterable, Optional

import numpy as np
import torch

from .. import optim as optim_lib
from ..common.configs import TrainingConfig
from ..common.datatypes import Mode
from ..lora import is_lora_enabled, is_lora_param_name
from . import checkpoint_manager as ckpt_lib
from . import hooks as hooks_lib
from . import inflight_throttler, metrics_logger as ml, profiler as profiler_lib, progress_bar, sharding_utils
from .utils import LossOutput, WeightedMetric, weighted_metric_mean


@dataclasses.dataclass
class TrainingInput:
    """input_tokens [B,T] int, input_mask [B,T] (1 = contributes to the loss / is a real token)."""
    input_tokens: Any
    input_mask: Any
    images: Any = None


@dataclasses.dataclass
class MetricsBuffer:
    step: int
    losses: list = dataclasses.field(default_factory=list)
    additional_metrics: dict = dataclasses.field(default_factory=dict)
    grad_norm: Any = None
    step_time: Optional[float] = None        # host seconds since the previous optimizer step was issued
    tokens: int = 0                          # tokens of the step's micro-batches on this rank

    @property
    def loss(self) -> float:
        if self.losses and isinstance(self.losses[0], WeightedMetric):
            return weighted_metric_mean(self.losses)
        return float(np.mean([float(l) for l in self.losses])) if self.losses else 0.0


_MULTIMODAL_KEYS = ("images", "pixel_values", "pixel_position_ids", "input_features", "input_features_mask")


def _default_loss_fn(model, input_tokens, input_mask, positions=None, attention_mask=None, segment_ids=None,
                     **extra) -> LossOutput:
    """Next-token NLL: sum_t -log p(x_{t+1}) * mask_{t+1} over sum_t mask_{t+1} (:1197-1230).

    Uses the fused lm_head log-prob path, so [B,T,V] logits are never materialised. Image / audio inputs of a
    batch (`images` of `TrainingInput`, or the Gemma-4 patch and feature arrays) go to a multimodal model's
    forward; other extra fields are ignored."""
    mm = {k: v for k, v in extra.items() if k in _MULTIMODAL_KEYS and v is not None}
    if mm:
        hidden, _ = model(input_tokens, positions=positions, segment_ids=segment_ids, skip_lm_head=True, **mm)
    else:
        hidden, _ = model(input_tokens, positions=positions, attention_mask=attention_mask, segment_ids=segment_ids,
                          skip_lm_head=True)
    from ..parallel.tp import local_batch   # under tensor parallelism `hidden` covers this rank's sequences only
    cp = getattr(model, "cp", None)
    if cp is not None and cp.world > 1:
        # context parallel: `hidden` covers this rank's tokens; targets are shifted over the full sequence first
        targets, mask = cp.shift_and_slice(input_tokens, input_mask)
        mask = mask.to(torch.float32)
        logp, _ = model.token_logprobs(hidden, targets)
    else:
        targets = local_batch(model, input_tokens)[:, 1:]
        mask = local_batch(model, input_mask)[:, 1:].to(torch.float32)
        logp, _ = model.token_logprobs(hidden[:, :-1], targets)
    nll_sum = -(logp * mask).sum()
    aux = model.aux_loss() if hasattr(model, "aux_loss") else None
    if aux is not None:
        nll_sum = nll_sum + aux * mask.sum()
    return LossOutput(WeightedMetric(nll_sum, mask.sum(), eps=1e-8))


def _to_device(x, device, non_blocking=True):
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    if isinstance(x, torch.Tensor):
        return x.to(device, non_blocking=non_blocking)
    return x


class PeftTrainer:
    def __init__(self, model, optimizer: optim_lib.Optimizer, training_config: TrainingConfig,
                 metrics_logger: Optional[ml.MetricsLogger] = None, perf_tracer=None):
        self.model = model
        self.config = training_config
        self._lora = is_lora_enabled(model)
        self.device = next(model.parameters()).device
        named = [(n, p) for n, p in model.named_parameters()
                 if p.requires_grad and (not self._lora or is_lora_param_name(n))]
        if self._lora:
            for n, p in model.named_parameters():
                p.requires_grad_(is_lora_param_name(n))
        self.grad_accum_steps = training_config.get_with_default("gradient_accumulation_steps", 1)
        self.optimizer = optimizer
        if optimizer.buffers is None:
            grad_dtype = torch.float32 if (self.grad_accum_steps > 1 or self.device.type != "cuda") else None
            optimizer.bind(named, grad_dtype=grad_dtype)
        if hasattr(optimizer, "install_hooks"):
            optimizer.install_hooks(model)
        self.loss_fn: Callable = _default_loss_fn
        self.eval_loss_fn: Callable = _default_loss_fn
        self.gen_model_input_fn: Callable = lambda x: x if isinstance(x, dict) else {
            "input_tokens": x.input_tokens, "input_mask": x.input_mask,
            **({"images": x.images} if getattr(x, "images", None) is not None else {})}
        self._has_aux = False
        # the ranks that train this model: a sharded optimizer knows its group (a disaggregated RL job trains on a
        # subset of the job's ranks); otherwise every rank of the job
        self.checkpoint_manager = ckpt_lib.CheckpointManager(training_config.checkpoint_root_directory,
                                                             training_config.checkpointing_options,
                                                             group=getattr(optimizer, "group", None))
        self.metrics_logger = metrics_logger or ml.MetricsLogger(training_config.metrics_logging_options)
        self.metrics_prefix = training_config.metrics_prefix
        self.perf_tracer = perf_tracer
        self.training_hooks: Optional[hooks_lib.TrainingHooks] = None
        self.data_hooks: Optional[hooks_lib.DataHooks] = None
        self._mode = Mode.TRAIN
        self._train_steps = 0       # optimizer updates done
        self._iter_steps = 0        # micro-batches consumed
        self._restored_custom_metadata: dict = {}
        self._buffered_train_metrics: Optional[MetricsBuffer] = None
        self._prev_buffered_train_metrics: Optional[MetricsBuffer] = None
        self._denoms: list = []
        self._throttler = inflight_throttler.InflightThrottler(training_config.max_inflight_computations)
        self._pbar = None
        self._last_step_time = None
        self._num_params: Optional[int] = None
        self._step_tokens = 0
        self.is_managed_externally = False
        if training_config.resume_from_checkpoint_on_init:
            self._train_steps, self._restored_custom_metadata = self.checkpoint_manager.maybe_restore(
                self.model, self.optimizer, restore_only_lora_params=self._lora)
            if self._train_steps:
                self.optimizer.sync_master_from_params() if "master" not in self.optimizer._state_tensors() else None
            self._iter_steps = self._train_steps * self.grad_accum_steps

    # ------------------------------------------------------------ configuration
    def with_loss_fn(self, loss_fn: Callable, has_aux: bool = False) -> "PeftTrainer":
        self.loss_fn = loss_fn
        self.eval_loss_fn = loss_fn
        self._has_aux = has_aux
        return self

    def with_gen_model_input_fn(self, fn: Callable) -> "PeftTrainer":
        self.gen_model_input_fn = fn
        return self

    def with_training_hooks(self, hooks: hooks_lib.TrainingHooks) -> "PeftTrainer":
        self.training_hooks = hooks
        return self

    def with_data_hooks(self, hooks: hooks_lib.DataHooks) -> "PeftTrainer":
        self.data_hooks = hooks
        return self

    @property
    def train_steps(self) -> int:
        return self._train_steps

    @property
    def iter_steps(self) -> int:
        return self._iter_steps

    # --------------------------------------------------------------- one step
    def _prepare_inputs(self, batch: Any) -> Any:
        return batch

    def _post_process_train_step(self, aux: Any) -> None:
        pass

    def _post_process_eval_step(self, aux: Any) -> None:
        pass

    def _unpack_loss(self, out):
        """-> (tensor to differentiate, metric value for logging, denominator or None, aux)."""
        aux = None
        if isinstance(out, LossOutput):
            aux = out.aux
            out = out.loss
        elif isinstance(out, tuple):
            out, aux = out
            if isinstance(out, LossOutput):
                aux = out.aux if aux is None else aux
                out = out.loss
        if isinstance(out, WeightedMetric):
            return out.sum, out, out.denominator, aux
        return out, out, None, aux

    def _train_step(self, batch: Any, is_update_step: bool):
        """Forward + backward of one micro-batch; optimizer update when `is_update_step`."""
        inputs = self.gen_model_input_fn(batch)
        out = self.loss_fn(self.model, **inputs)
        to_diff, metric, denom, aux = self._unpack_loss(out)
        prepare = getattr(self.optimizer, "prepare_backward", None)
        if prepare is not None:
            prepare(is_update_step)   # sharded optimizers overlap the gradient reduction with this backward
        to_diff.backward()
        self.optimizer.buffers.collect_autograd_grads()
        self._denoms.append(denom.detach() if denom is not None else None)
        grad_norm = None
        if is_update_step:
            local = False
            if self._denoms and self._denoms[0] is not None:
                total = torch.stack([d.float() for d in self._denoms]).sum()
                denominator, local = self._reduce_denominator(total)
            else:
                denominator = float(len(self._denoms))
            grad_norm = self._optimizer_step(denominator, local)
            self.optimizer.zero_grad()
            self._denoms = []
        if isinstance(metric, WeightedMetric):
            metric = WeightedMetric(metric.sum.detach(), metric.denominator.detach(), metric.eps,
                                    metric.min_denominator)
        else:
            metric = metric.detach()
        return metric, aux, grad_norm

    def _reduce_denominator(self, total: torch.Tensor):
        """Denominator of the update -> (value, is_local). On a CUDA device the value stays a device tensor that
        the update kernel divides by, so no step waits for the host to read it (the reference's jitted step keeps
        it on the device as well, tunix/sft/peft_trainer.py:517-548). A sharded optimizer that sums denominators
        together with its gradient norm gets this rank's part (`is_local`); otherwise the sum over the
        data-parallel ranks is taken here."""
        import torch.distributed as dist
        multi = dist.is_initialized() and dist.get_world_size() > 1
        sharded = getattr(self.optimizer, "is_sharded", False)
        tp = getattr(self.model, "tp", None)
        dps = getattr(self.model, "dp_shard", None)
        local = False
        if multi and sharded:
            if getattr(self.optimizer, "reduces_denominator", False) and not (tp is not None and tp.world > 1):
                local = True
            else:
                dist.all_reduce(total, group=getattr(self.optimizer, "group", None))
        if tp is not None and tp.world > 1:
            dist.all_reduce(total, group=tp.group)      # every tp rank scored its own sequences
            rep = getattr(self.model, "dp_replica_group", None)
            if rep is not None:
                dist.all_reduce(total, group=rep)
        if dps is not None and dps.world > 1 and not sharded:
            dist.all_reduce(total, group=dps.group)
        if total.is_cuda:
            return total.reshape(1), local
        return float(max(total.item(), 1e-8)), local

    def _optimizer_step(self, denominator, denominator_is_local: bool = False):
        if denominator_is_local:
            return self.optimizer.step(denominator, denominator_is_local=True)
        tp = getattr(self.model, "tp", None)
        if tp is not None and tp.world > 1:
            from ..parallel import strategy, tp as tp_lib
            self.optimizer.buffers.collect_autograd_grads()
            strategy.sum_replica_grads(self.model, self.optimizer)      # data-parallel replicas of the tp group
            tp_lib.allreduce_replicated_grads(self.model, tp)
            return self.optimizer.step(denominator, sumsq=tp_lib.grad_sumsq(self.model, tp))
        dps = getattr(self.model, "dp_shard", None)
        if dps is not None and dps.world > 1:
            from ..parallel import fsdp3
            self.optimizer.buffers.collect_autograd_grads()
            fsdp3.sync_replicated_grads(self.model, dps)
            return self.optimizer.step(denominator, sumsq=fsdp3.grad_sumsq(self.model, dps))
        return self.optimizer.step(denominator)

    @torch.no_grad()
    def _eval_step(self, batch: Any):
        inputs = self.gen_model_input_fn(batch)
        out = self.eval_loss_fn(self.model, **inputs)
        _, metric, _, aux = self._unpack_loss(out)
        return metric, aux

    # ------------------------------------------------------------------ metrics
    def _log_metrics(self, loss: float, step: Optional[int], additional: Optional[dict] = None, grad_norm=None):
        lg, pf = self.metrics_logger, self.metrics_prefix
        lg.log(pf, "loss", loss, self._mode, step)
        lg.log(pf, "perplexity", math.exp(min(loss, 80.0)), self._mode, step)
        if self._mode == Mode.TRAIN:
            lg.log(pf, "learning_rate", self.optimizer.learning_rate_at(max((step or 1) - 1, 0)), self._mode, step)
            if grad_norm is not None:
                lg.log(pf, "grad_norm", float(grad_norm), self._mode, step)
        for k, v in (additional or {}).items():
            if k.startswith(("sampler_trainer/", "sampler_is/", "sampler_rs/")):
                prefix, name = k.split("/", 1)
                lg.log(prefix, name, v, self._mode, step)
            else:
                lg.log(pf, k, v, self._mode, step)

    def _buffer_metrics(self, buf: Optional[MetricsBuffer], loss, step: int, additional: Optional[dict] = None):
        if buf is None:
            buf = MetricsBuffer(step=step)
        buf.losses.append(loss)
        for k, (v, op) in (additional or {}).items():
            buf.additional_metrics.setdefault(k, ([], op))[0].append(v)
        return buf

    def _write_metrics(self, buf: MetricsBuffer):
        def to_host(v):
            if isinstance(v, WeightedMetric):
                return v
            if isinstance(v, torch.Tensor):
                return v.detach().float().cpu().numpy()
            return v

        additional = {}
        for k, (vals, op) in buf.additional_metrics.items():
            if vals and isinstance(vals[0], WeightedMetric):
                additional[k] = weighted_metric_mean(vals)
            else:
                additional[k] = op([to_host(v) for v in vals])
        self._log_metrics(buf.loss, buf.step, additional, buf.grad_norm)
        if buf.step_time and buf.step_time > 0 and self._mode == Mode.TRAIN:
            # host time between the issue of consecutive optimizer steps: with asynchronous launches this is the
            # steady-state time per step (the in-flight throttle keeps the host at most a few steps ahead)
            lg, pf = self.metrics_logger, self.metrics_prefix
            lg.log(pf, "step_time_sec", buf.step_time, self._mode, buf.step)
            lg.log(pf, "steps_per_sec", 1.0 / buf.step_time, self._mode, buf.step)
            if buf.tokens:
                if self._num_params is None:
                    self._num_params = sum(p.numel() for p in self.model.parameters())
                from .system_metrics_calculator import approximate_tflops_per_step
                lg.log(pf, "tflops_per_step", approximate_tflops_per_step(self._num_params, buf.tokens, buf.step_time),
                       self._mode, buf.step)

    def _write_train_metrics(self):
        """Write the metrics of the previous update (one-step delay so host IO overlaps device work)."""
        if self._prev_buffered_train_metrics is not None:
            prev = self._prev_buffered_train_metrics
            prev.step += 1
            self._write_metrics(prev)
            self._may_update_pbar(step=prev.step, loss=prev.loss)
        self._prev_buffered_train_metrics = self._buffered_train_metrics
        self._buffered_train_metrics = None

    def _may_update_pbar(self, step=None, loss=None):
        if self._pbar is not None:
            self._pbar.update_metrics(["loss", "perplexity", "learning_rate"], self._mode)
            self._pbar.update()
        if self.training_hooks and self._mode == Mode.TRAIN:
            self.training_hooks.on_train_step_end(self, step, loss)

    # --------------------------------------------------------------------- eval
    def _run_eval(self, eval_ds: Iterable[Any]):
        prev_mode, self._mode = self._mode, Mode.EVAL
        was_training = self.model.training
        self.model.eval()
        buf = None
        try:
            it = iter(eval_ds) if eval_ds is not None else None
            while True:
                if self.training_hooks:
                    self.training_hooks.on_eval_step_start(self)
                if self.data_hooks:
                    batch = self.data_hooks.load_next_eval_batch(self)
                    if batch is None:
                        break
                else:
                    try:
                        batch = next(it)
                    except StopIteration:
                        break
                batch = self._shard_and_move(self._prepare_inputs(batch))
                metric, aux = self._eval_step(batch)
                self._post_process_eval_step(aux)
                buf = self._buffer_metrics(buf, metric, self._train_steps)
            if buf is not None:
                self._write_metrics(buf)
                if self.training_hooks:
                    self.training_hooks.on_eval_step_end(self, buf.loss)
        finally:
            self._mode = prev_mode
            self.model.train(was_training)
        return None if buf is None else buf.loss

    def _shard_and_move(self, batch):
        tp, cp = getattr(self.model, "tp", None), getattr(self.model, "cp", None)
        # ranks of one tensor- or context-parallel group work on the same sequences
        batch = sharding_utils.shard_input(batch, self.config.data_sharding_axis,
                                           model_parallel=(tp.world if tp else 1) * (cp.world if cp else 1))
        if dataclasses.is_dataclass(batch) and not isinstance(batch, type):
            return dataclasses.replace(batch, **{f.name: _to_device(getattr(batch, f.name), self.device)
                                                 for f in dataclasses.fields(batch)})
        if isinstance(batch, dict):
            return {k: _to_device(v, self.device) for k, v in batch.items()}
        return batch

    # -------------------------------------------------------------------- train
    def train(self, train_ds: Iterable[Any], eval_ds: Optional[Iterable[Any]] = None, skip_jit: bool = False):
        cfg = self.config
        self.model.train()
        self._last_step_time, self._step_tokens = None, 0     # step times are measured inside one call, not across calls
        watchdog = self._start_watchdog()
        prof = profiler_lib.Profiler(self._train_steps, cfg.max_steps, cfg.profiler_options)
        if cfg.pbar_description and self._pbar is None and not self.is_managed_externally:
            self._pbar = progress_bar.ProgressBar(self.metrics_logger, self._train_steps, cfg.max_steps,
                                                  cfg.pbar_description, self.metrics_prefix,
                                                  disable=not ml._is_main_process())
        if self.training_hooks:
            self.training_hooks.on_train_start(self)
        it = iter(train_ds) if train_ds is not None else None
        index = 0
        if eval_ds is not None and self._train_steps == 0 and not self.is_managed_externally:
            self._run_eval(eval_ds)
        while True:
            if cfg.max_steps is not None and self._train_steps >= cfg.max_steps and not self.is_managed_externally:
                break
            prof.maybe_activate(self._train_steps)
            if self.data_hooks:
                batch = self.data_hooks.load_next_train_batch(self)
                if batch is None:
                    break
            else:
                try:
                    batch = next(it)
                except StopIteration:
                    break
            # resume: skip batches that were consumed before the restored checkpoint
            if not self.is_managed_externally and index < self._iter_steps and self._restored_custom_metadata is not None \
                    and self._resume_skip:
                index += 1
                continue
            index += 1
            if watchdog is not None:
                try:
                    watchdog.check()        # between steps, nothing of this rank in flight that waits for a peer
                except BaseException:
                    watchdog.stop()
                    raise
            batch = self._prepare_inputs(batch)
            batch = self._shard_and_move(batch)
            self._throttler.wait_for_next()
            if self.training_hooks:
                self.training_hooks.on_train_step_start(self)
            explicit = getattr(batch, "is_update_step", None)
            if isinstance(batch, dict):
                explicit = batch.get("is_update_step", explicit)
            if explicit is not None:
                is_update = bool(explicit)
            else:
                is_update = (self._iter_steps + 1) % self.grad_accum_steps == 0
            span = self.perf_tracer.span("peft_train_step", device=True) if self.perf_tracer else None
            if span:
                span.__enter__()
            metric, aux, grad_norm = self._train_step(batch, is_update)
            if span:
                span.__exit__(None, None, None)
            if self.device.type == "cuda":
                ev = torch.cuda.Event()
                ev.record()
                self._throttler.add_computation(ev)
            self._iter_steps += 1
            self._post_process_train_step(aux)
            self._buffered_train_metrics = self._buffer_metrics(self._buffered_train_metrics, metric,
                                                                self._train_steps, self._aux_metrics(aux))
            self._step_tokens += _count_tokens(batch)
            if is_update:
                self._buffered_train_metrics.grad_norm = grad_norm
                now = time.perf_counter()
                if self._last_step_time is not None:
                    self._buffered_train_metrics.step_time = now - self._last_step_time
                self._last_step_time = now
                self._buffered_train_metrics.tokens, self._step_tokens = self._step_tokens, 0
                self._train_steps += 1
                self._write_train_metrics()
                if self.checkpoint_manager.should_save(self._train_steps):
                    self._params_ready()
                self.checkpoint_manager.save(self._train_steps, self.model, self.optimizer,
                                             save_only_lora_params=self._lora,
                                             custom_metadata=self._checkpoint_metadata())
                if eval_ds is not None and cfg.eval_every_n_steps and self._train_steps % cfg.eval_every_n_steps == 0:
                    self._run_eval(eval_ds)
            prof.maybe_deactivate(self._train_steps)
        self._throttler.wait_for_all()
        self._params_ready()
        if watchdog is not None:
            watchdog.stop()
        if self.training_hooks:
            self.training_hooks.on_train_end(self)
        if not self.is_managed_externally:
            self.close()

    _resume_skip = True

    def _start_watchdog(self):
        """Heartbeats through the job's store when `rank_failure_timeout_s` is set and there is more than one rank."""
        timeout = getattr(self.config, "rank_failure_timeout_s", None)
        if not timeout:
            return None
        import torch.distributed as dist
        if not dist.is_initialized() or dist.get_world_size() < 2:
            return None
        from ..parallel.watchdog import Watchdog
        return Watchdog(interval_s=min(1.0, timeout / 4), timeout_s=timeout).start()

    def _params_ready(self) -> None:
        """Order the current stream after any parameter transfer that the optimizer left running on a side stream
        (a sharded optimizer pulls the updated shards while the next forward pass already runs)."""
        wait = getattr(self.optimizer, "wait_params", None)
        if wait is not None:
            wait()

    def _aux_metrics(self, aux) -> Optional[dict]:
        """aux dict of scalars -> {name: (value, reducer)} for the metrics buffer."""
        if not isinstance(aux, dict):
            return None
        out = {}
        for k, v in aux.items():
            if isinstance(v, tuple) and len(v) == 2 and callable(v[1]):
                out[k] = v
            elif isinstance(v, (WeightedMetric, float, int)) or (isinstance(v, torch.Tensor) and v.numel() == 1):
                out[k] = (v, lambda xs: float(np.mean([float(np.asarray(x)) for x in xs])))
        return out

    def _checkpoint_metadata(self) -> dict:
        return {}

    def close(self):
        """Flush the delayed metrics, force a last checkpoint, close loggers."""
        if self._buffered_train_metrics is not None or self._prev_buffered_train_metrics is not None:
            self._write_train_metrics()
            if self._prev_buffered_train_metrics is not None:
                self._write_train_metrics()
        self.checkpoint_manager.save(self._train_steps, self.model, self.optimizer, save_only_lora_params=self._lora,
                                     force=True, custom_metadata=self._checkpoint_metadata())
        self.checkpoint_manager.close()
        if self._pbar is not None:
            self._pbar.close()
            self._pbar = None
        self.metrics_logger.close()


def _count_tokens(batch) -> int:
    """Tokens in a prepared batch (`input_tokens` of a `TrainingInput` or dict; 0 when the batch has another shape)."""
    toks = batch.get("input_tokens") if isinstance(batch, dict) else getattr(batch, "input_tokens", None)
    if toks is None:
        ex = batch.get("train_example") if isinstance(batch, dict) else getattr(batch, "train_example", None)
        ex = ex if ex is not None else batch
        p, c = getattr(ex, "prompt_ids", None), getattr(ex, "completion_ids", None)
        return int(p.numel() + c.numel()) if p is not None and c is not None and hasattr(p, "numel") else 0
    return int(toks.numel()) if hasattr(toks, "numel") else int(np.size(toks))


class GradientAccumulator:
    """fp32 accumulation of gradients with a loss denominator (tunix/sft/peft_trainer.py:164-281).

    The flat `main_grad` buffer of the optimizer plays this role inside `PeftTrainer`; this class offers the
    same arithmetic for code that manages gradients itself: `add(grads, denom)`, `get()` = sum(grad)/sum(denom)
    cast back to the parameter dtype, `reset()`.
    """

    def __init__(self, params: list[torch.Tensor]):
        self._params = params
        self._acc = [torch.zeros_like(p, dtype=torch.float32) for p in params]
        self._denom = 0.0

    def add(self, grads: list[torch.Tensor], denom: float = 1.0) -> None:
        for a, g in zip(self._acc, grads):
            if g is not None:
                a.add_(g.float())
        self._denom += float(denom)

    def get(self) -> list[torch.Tensor]:
        d = max(self._denom, 1e-8)
        return [(a / d).to(p.dtype) for a, p in zip(self._acc, self._params)]

    def reset(self) -> None:
        for a in self._acc:
            a.zero_()
        self._denom = 0.0
