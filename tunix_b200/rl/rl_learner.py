"""RLLearner: the outer RL loop shared by GRPO / PPO learners (tunix/rl/rl_learner.py:54-850).

    global step -> (rollout + scoring on the producer thread) -> mini-batch steps -> micro-batch steps

* `_prepare_data` (producer, :278-503): merges prompt micro-batches up to lcm(rollout_mb, logps_mb), repeats
  every prompt G times, calls the algorithm's `_generate_and_compute_advantage`, splits the result into
  train micro-batches and enqueues them; repeats the same data `num_iterations` times (mu) with an optional
  seeded shuffle; a `None` sentinel ends the step. It runs on a thread so that, when rollout and actor live
  on different ranks, generation of the next batch overlaps training of the current one; in the colocated
  layout the queue degenerates to a synchronous hand-off (:151-156).
* the consumer (main thread, :722-841) pulls micro-batches, optionally packs them, and calls
  `rl_cluster.update_actor` (and `update_critic`);
* after every global step: weight sync, metric flush, perf export (:627-658);
* resume: the first `restored_global_step` batches of the dataset are skipped (:404-411).
"""
from __future__ import annotations

import abc
import math
import threading
from concurrent import futures
from typing import Any, Callable, Iterable, Iterator, Optional, Sequence

import numpy as np
import torch

from ..common.datatypes import Mode
from . import algo_core, common, function_registry, reward_manager as _reward_manager, utils as rl_utils  # noqa: F401 (registrations)
from .queue.data_queue import SimpleDataQueue
from .rl_cluster import RLCluster


class RLLearner(abc.ABC):
    def __init__(self, rl_cluster: RLCluster, algo_config, reward_fns=None, metric_fns: Optional[Sequence[Callable]] = None,
                 data_shuffle_seed: Optional[int] = None):
        self.rl_cluster = rl_cluster
        self.algo_config = algo_config
        self.metric_fns = list(metric_fns or [])
        self.tcfg = rl_cluster.cluster_config.training_config
        rc = rl_cluster._rollout_config(Mode.TRAIN)
        self.algo_config.temperature = rc.temperature if rc.temperature and rc.temperature > 0 else None
        self.reward_manager = None
        if reward_fns is not None:
            cls = function_registry.get_reward_manager(algo_config.reward_manager)
            self.reward_manager = cls(reward_fns, algo_config)
        self.grad_acc_steps = self.tcfg.get_with_default("gradient_accumulation_steps", 1)
        self._data_shuffle_seed = data_shuffle_seed
        self._iter_steps = 0
        self._eval_iter_steps = 0
        if not rl_cluster.is_controller:
            raise RuntimeError("this rank hosts no part of the training loop: call rl_cluster.serve() on it instead of "
                               "building a learner")
        self.should_sync_weights = not rl_cluster._rollout_shares_weights
        self._producer_error: Optional[BaseException] = None
        self.pad_id = rl_cluster.tokenizer.pad_id()
        self.eos_id = rl_cluster.tokenizer.eos_id()
        self.device = next(rl_cluster.train_actor.parameters()).device
        # generation on other ranks: open the next batch's round before training on the current one
        self.rollout_is_remote = not rl_cluster.exchange.is_local("rollout")
        self.off_policy_steps = int(getattr(algo_config, "off_policy_steps", 1 if self.rollout_is_remote else 0))

    # ---------------------------------------------------------- to implement
    @abc.abstractmethod
    def _generate_and_compute_advantage(self, training_input: dict, mode: Mode = Mode.TRAIN) -> common.TrainExample: ...

    @abc.abstractmethod
    def _num_generations(self) -> int: ...

    @abc.abstractmethod
    def _num_iterations(self) -> int: ...

    def _compute_trajectory_ids(self, batch: dict, step: int) -> list[str]:
        n = len(batch["prompts"])
        G = self._num_generations()
        return [f"{step}_{i // G}_{i % G}" for i in range(n)]

    # ------------------------------------------------------------- rewards
    def _compute_rewards(self, prompts: list, completions: list, mode: Mode, **kwargs) -> np.ndarray:
        if self.reward_manager is None:
            raise ValueError("no reward functions configured")
        out = self.reward_manager(prompts, completions, **kwargs)
        r = out["rewards"]
        m = {"rewards/score/mean": (float(r.mean()), np.mean), "rewards/score/max": (float(r.max()), np.max),
             "rewards/score/min": (float(r.min()), np.min)}
        for name, col in out["per_fn"].items():
            m[f"rewards/{name}"] = (float(np.mean(col)), np.mean)
        self.rl_cluster.buffer_metrics(m, mode)
        return r

    # ------------------------------------------------------------- producer
    def _repeat(self, batch: dict, G: int) -> dict:
        out = {}
        for k, v in batch.items():
            if isinstance(v, (list, tuple)):
                out[k] = [x for x in v for _ in range(G)]
            elif isinstance(v, np.ndarray):
                out[k] = np.repeat(v, G, axis=0)
            elif isinstance(v, torch.Tensor):
                out[k] = v.repeat_interleave(G, dim=0)
            else:
                out[k] = v
        return out

    @staticmethod
    def _item_size(batch: dict) -> int:
        for key in ("prompts", "prompt_token_ids"):
            if batch.get(key) is not None:
                return len(batch[key])
        return len(next(iter(batch.values())))

    @staticmethod
    def _merge_items(items: list) -> dict:
        """Several prompt batches as one: lists are concatenated, arrays / tensors stacked along dim 0."""
        if len(items) == 1:
            return items[0]
        out = {}
        for k in items[0]:
            vals = [it[k] for it in items]
            v0 = vals[0]
            if isinstance(v0, (list, tuple)):
                out[k] = [x for v in vals for x in v]
            elif isinstance(v0, np.ndarray):
                out[k] = np.concatenate(vals, 0)
            elif isinstance(v0, torch.Tensor):
                out[k] = torch.cat(vals, 0)
            else:
                out[k] = v0
        return out

    def _service_target(self) -> int:
        """Prompts to collect before one generate-and-score pass: the least common multiple of the rollout and the
        log-prob micro-batch sizes, so that neither service runs a ragged last micro-batch
        (tunix/rl/rl_learner.py:278-330)."""
        a, b = self.tcfg.rollout_micro_batch_size or 1, self.tcfg.compute_logps_micro_batch_size or 1
        return math.lcm(int(a), int(b))

    def _prepare_data(self, iterator: Iterator, data_queue: SimpleDataQueue, mode: Mode, num_batches: int) -> None:
        """Producer: consume `num_batches` prompt batches, enqueue train micro-batches, then a None sentinel.

        Batches smaller than the service target (a dataset that yields micro-batches) are merged until they reach
        it, generated and scored in one pass, and split again into train micro-batches; a remainder at the end of
        the step is processed as it is."""
        try:
            G, mu = self._num_generations(), self._num_iterations()
            mb = self.tcfg.train_micro_batch_size
            target = self._service_target()
            produced: list[common.TrainExample] = []
            held: list = []
            held_n = 0

            def flush():
                nonlocal held, held_n
                if not held:
                    return
                batch = self._repeat(self._merge_items(held), G)
                held, held_n = [], 0
                with torch.no_grad():
                    ex = self._generate_and_compute_advantage(batch, mode)
                n = ex.completion_ids.shape[0]
                step_mb = (mb * G) if mb else n
                for sl in rl_utils.chunk_slices(n, step_mb):
                    produced.append(rl_utils.slice_example(ex, sl))

            for _ in range(num_batches):
                try:
                    batch = next(iterator)
                except StopIteration:
                    break
                held.append(batch)
                held_n += self._item_size(batch)
                if held_n >= target:
                    flush()
            flush()
            # one pass over the step's micro-batches updates every `gradient_accumulation_steps` of them and, whatever
            # that count is, at its last one: a global step never ends with gradients left unapplied
            acc = max(int(self.grad_acc_steps or 1), 1)
            for k, piece in enumerate(produced):
                if piece.is_update_step is None:
                    piece.is_update_step = ((k + 1) % acc == 0) or k == len(produced) - 1
                data_queue.put(piece)
            if mode == Mode.TRAIN:
                for it in range(1, mu):
                    order = list(range(len(produced)))
                    if self._data_shuffle_seed is not None:
                        np.random.default_rng(self._data_shuffle_seed + it).shuffle(order)
                    for i in order:
                        data_queue.put(produced[i])
        except BaseException as e:  # forwarded to the consumer
            self._producer_error = e
        finally:
            data_queue.put(None)

    # ------------------------------------------------------------- consumer
    def _batches_from_queue(self, q: SimpleDataQueue) -> Iterator[common.TrainExample]:
        while True:
            item = q.get()
            if item is None:
                if self._producer_error is not None:
                    e, self._producer_error = self._producer_error, None
                    raise RuntimeError("rollout producer failed") from e
                return
            yield item

    def _maybe_pack(self, examples: Iterable[common.TrainExample]) -> Iterable[common.TrainExample]:
        if not self.tcfg.sequence_packing_enabled:
            return examples
        budget = self.tcfg.max_seq_token_per_tpu
        return rl_utils.pack_sequences(examples, budget, pack_size=max(self.tcfg.train_micro_batch_size or 1, 1),
                                       pad_id=self.pad_id, device=self.device,
                                       max_segments=self.tcfg.max_segments_per_packed_row)

    def _train_on(self, examples: Iterable[common.TrainExample]) -> None:
        self.rl_cluster.update_actor(self._maybe_pack(examples), None)

    def train(self, train_ds: Iterable[dict], eval_ds: Optional[Iterable[dict]] = None, skip_jit: bool = False) -> None:
        """`train_ds` yields dicts with at least `prompts` (list[str]) or `prompt_token_ids`; one item = one
        global batch of prompts (mini_batch_size prompts)."""
        it = iter(train_ds)
        max_steps = self.tcfg.max_steps
        # a dataset may yield whole global batches or micro-batches of them: a global step takes as many items as
        # make up `mini_batch_size` prompts
        first = next(it, None)
        if first is None:
            return
        import itertools
        it = itertools.chain([first], it)
        mini = self.tcfg.mini_batch_size
        self._items_per_step = max(1, int(mini) // max(self._item_size(first), 1)) if mini else 1
        # resume: skip consumed prompt batches
        for _ in range(self.rl_cluster.global_steps * self._items_per_step):
            try:
                next(it)
            except StopIteration:
                return
        if self.rollout_is_remote:
            try:
                self._train_remote_rollout(it, eval_ds)
            finally:
                self.rl_cluster.close()
                if self.reward_manager is not None and hasattr(self.reward_manager, "close"):
                    self.reward_manager.close()
            return
        executor = futures.ThreadPoolExecutor(max_workers=1, thread_name_prefix="rl-producer")
        try:
            while True:
                if max_steps is not None and self.rl_cluster.global_steps >= max_steps:
                    break
                q: SimpleDataQueue = SimpleDataQueue()
                got_any = False

                def counted():
                    nonlocal got_any
                    for ex in self._batches_from_queue(q):
                        got_any = True
                        self._iter_steps += 1
                        yield ex
                with self._step_group() as step_span:
                    fut = executor.submit(self._prepare_data, it, q, Mode.TRAIN, self._items_per_step)
                    self._train_on(counted())
                    fut.result()
                    if not got_any:
                        break
                    self.rl_cluster.sync_weights()
                self._export_perf(step_span)
                self.rl_cluster.flush_metrics()
                if eval_ds is not None and self.tcfg.eval_every_n_steps and \
                        self.rl_cluster.global_steps % self.tcfg.eval_every_n_steps == 0:
                    self._run_eval(eval_ds)
        finally:
            executor.shutdown(wait=True)
            self.rl_cluster.close()
            if self.reward_manager is not None and hasattr(self.reward_manager, "close"):
                self.reward_manager.close()

    def _step_group(self):
        """Span group around one global step (a no-op context without a tracer)."""
        import contextlib
        perf = self.rl_cluster.perf
        return perf.span_group("global_step", step=self.rl_cluster.global_steps) if perf is not None \
            else contextlib.nullcontext()

    def _export_perf(self, step_span) -> None:
        """Reduce the step's spans to the layout's perf metrics and hand them to the metrics buffer (:627-658)."""
        perf = self.rl_cluster.perf
        if perf is None or step_span is None:
            return
        fn = getattr(self, "_perf_export_fn", None)
        if fn is None:
            from ..perf.export import PerfMetricsExport
            opts = self.tcfg.perf_metrics_options
            custom = getattr(opts, "custom_export_fn", None) if opts is not None else None
            fn = custom or PerfMetricsExport.from_cluster_config(self.rl_cluster.cluster_config, self.rl_cluster.placement)
            self._perf_export_fn = fn
        opts = self.tcfg.perf_metrics_options
        if opts is None or getattr(opts, "enable_perf_v1", True):        # the per-step `perf/...` scalars
            metrics = fn(perf, step_span)
            self.rl_cluster.buffer_metrics({k: (v, np.mean) for k, v in metrics.items()}, Mode.TRAIN,
                                           step=self.rl_cluster.global_steps - 1)
        if opts is not None and getattr(opts, "enable_perf_v2", False) and getattr(opts, "enable_trace_writer", False) \
                and getattr(opts, "log_dir", None):
            exp = getattr(self, "_trace_exporter", None)
            if exp is None:
                from ..perf.experimental.bridge import StepTraceExporter
                pl = self.rl_cluster.placement
                from .placement import Role
                roles = {r.value: list(pl.ranks(r)) for r in (Role.ACTOR, Role.ROLLOUT, Role.REFERENCE)}
                exp = self._trace_exporter = StepTraceExporter(opts.log_dir, roles, device_id=getattr(pl, "rank", 0))
            exp.step(perf, step_span, self.rl_cluster.global_steps - 1)

    def _open_round(self, batch: dict) -> None:
        """Send the prompts of `batch` to the rollout ranks now; `_generate_and_compute_advantage` picks the result up."""
        rep = self._repeat(batch, self._num_generations())
        mb = self.tcfg.rollout_micro_batch_size and self.tcfg.rollout_micro_batch_size * self._num_generations()
        self.rl_cluster.generate_begin(rep.get("prompts"), mode=Mode.TRAIN, micro_batch_size=mb,
                                       prompt_token_ids=rep.get("prompt_token_ids"))

    def _train_remote_rollout(self, it: Iterator, eval_ds) -> None:
        """The loop when the sampler lives on other ranks (tunix/rl/rl_learner.py:151-156: rollout and training
        overlap when their meshes differ). With `off_policy_steps` >= 1 the round for batch k+1 is opened before
        the update on batch k, so the rollout ranks generate while this rank trains; the weights they use are then
        one update old. With 0 every batch is generated from the latest weights and nothing overlaps."""
        max_steps = self.tcfg.max_steps
        ahead = self.off_policy_steps >= 1
        nxt = next(it, None)
        if nxt is not None and ahead:
            self._open_round(nxt)
        while nxt is not None:
            if max_steps is not None and self.rl_cluster.global_steps >= max_steps:
                break
            cur = nxt
            q: SimpleDataQueue = SimpleDataQueue()
            got_any = False

            def counted():
                nonlocal got_any
                for ex in self._batches_from_queue(q):
                    got_any = True
                    self._iter_steps += 1
                    yield ex
            with self._step_group() as step_span:
                self._prepare_data(iter([cur]), q, Mode.TRAIN, 1)          # closes the round of `cur`, scores it
                nxt = next(it, None)
                last = max_steps is not None and self.rl_cluster.global_steps + 1 >= max_steps
                if nxt is not None and ahead and not last:
                    self._open_round(nxt)
                self._train_on(counted())
                if not got_any:
                    break
                self.rl_cluster.sync_weights()       # closes an open round first: rounds do not nest
            self._export_perf(step_span)
            self.rl_cluster.flush_metrics()
            if eval_ds is not None and self.tcfg.eval_every_n_steps and \
                    self.rl_cluster.global_steps % self.tcfg.eval_every_n_steps == 0:
                self._run_eval(eval_ds)

    def _run_eval(self, eval_ds: Iterable[dict]) -> None:
        rewards = []
        for batch in eval_ds:
            with torch.no_grad():
                ex = self._generate_and_compute_advantage(dict(batch), Mode.EVAL)
            rewards.append(float(ex.advantages.float().mean()))
            self._eval_iter_steps += 1
        self.rl_cluster.flush_metrics()
