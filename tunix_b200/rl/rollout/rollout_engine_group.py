"""Several rollout engines behind one `BaseRollout` (tunix/rl/rollout/rollout_engine_group.py).

Prompts of a `generate` call are split over the engines in contiguous slices, the engines run on their own
threads (each engine is bound to its own device or stream), and the outputs are stitched back in prompt order.
Weight updates go to every engine."""
from __future__ import annotations

import concurrent.futures as cf
from typing import Sequence

import numpy as np

from .base_rollout import BaseRollout, RolloutOutput


class RolloutEngineGroup(BaseRollout):
    def __init__(self, engines: Sequence[BaseRollout]):
        if not engines:
            raise ValueError("a rollout group needs at least one engine")
        self.engines = list(engines)
        self._pool = cf.ThreadPoolExecutor(max_workers=len(self.engines), thread_name_prefix="rollout-engine")

    def generate(self, prompts, rollout_config, **kwargs) -> RolloutOutput:
        ids = kwargs.pop("prompt_token_ids", None)
        n = len(ids) if ids is not None else len(prompts)
        bounds = np.linspace(0, n, len(self.engines) + 1).astype(int)
        futs = []
        for e, (a, b) in zip(self.engines, zip(bounds[:-1], bounds[1:])):
            if a == b:
                continue
            kw = dict(kwargs)
            if ids is not None:
                kw["prompt_token_ids"] = ids[a:b]
            futs.append(self._pool.submit(e.generate, None if prompts is None else prompts[a:b], rollout_config, **kw))
        outs = [f.result() for f in futs]
        if len(outs) == 1:
            return outs[0]

        def cat(name):
            vals = [getattr(o, name) for o in outs]
            if any(v is None for v in vals):
                return None
            if isinstance(vals[0], np.ndarray) and all(v.shape[1:] == vals[0].shape[1:] for v in vals):
                return np.concatenate(vals)
            return [x for v in vals for x in v]
        import dataclasses
        return RolloutOutput(**{f.name: cat(f.name) for f in dataclasses.fields(RolloutOutput)})

    def update_params(self, params, filter_types=None) -> None:
        for e in self.engines:
            e.update_params(params, filter_types)

    def get_per_token_logps(self, *a, **kw):
        return self.engines[0].get_per_token_logps(*a, **kw)

    def pad_id(self) -> int:
        return self.engines[0].pad_id()

    def eos_id(self) -> int:
        return self.engines[0].eos_id()

    def model(self):
        return self.engines[0].model()
