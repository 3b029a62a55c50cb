"""The asynchronous sampler protocol of the distributed rollout path and its adapter over this framework's engines
(tunix/experimental/rollout/sampler.py:28-238, vanilla_sampler_adapter.py:35-360).

A rollout worker talks to its generation engine only through `AsyncSampler`: `sample` a list of requests,
`pause` / `resume` admission, the four weight-sync hooks, and `get_load_info` for routing. `EngineSamplerAdapter`
implements it over an `EngineServer` (every request joins the running batch on its own) or, without one, over a
batch callable with the `Sampler` / `PagedEngine` signature (requests of one call with equal sampling parameters are
generated as one batch). A request that fails is answered with `error` set; the others of the call are not
affected."""
from __future__ import annotations

import asyncio
import dataclasses
import time
from typing import Optional, Protocol, Sequence

import numpy as np


@dataclasses.dataclass
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 1.0
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    seed: Optional[int] = None
    return_logprobs: bool = True


@dataclasses.dataclass
class SamplingRequest:
    request_id: str
    prompt_token_ids: Sequence[int]
    sampling_params: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    route_key: Optional[str] = None
    metadata: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class SamplingResponse:
    request_id: str
    token_ids: list = dataclasses.field(default_factory=list)
    logprobs: Optional[list] = None
    text: Optional[str] = None
    finish_reason: str = "stop"
    policy_version: int = 0
    latency_s: float = 0.0
    error: Optional[BaseException] = None

    def __post_init__(self):
        if self.logprobs is not None and len(self.logprobs) != len(self.token_ids):
            raise ValueError(f"{self.request_id}: {len(self.logprobs)} logprobs for {len(self.token_ids)} tokens")


@dataclasses.dataclass
class LoadInfo:
    inflight: int = 0
    served: int = 0
    paused: bool = False
    policy_version: int = 0


class AsyncSampler(Protocol):
    def initialize(self) -> None: ...
    async def start(self) -> None: ...
    async def stop(self) -> None: ...
    async def pause(self) -> bool: ...
    async def resume(self) -> None: ...
    async def sample(self, requests: Sequence[SamplingRequest]) -> list: ...
    async def pre_weight_sync(self, version: int) -> None: ...
    async def weight_sync(self, version: int) -> None: ...
    async def post_weight_sync(self, version: int) -> None: ...
    async def abort_weight_sync(self) -> None: ...
    async def get_load_info(self) -> LoadInfo: ...


class EngineSamplerAdapter:
    def __init__(self, engine, *, tokenizer=None, participant=None, eos_tokens: Optional[Sequence[int]] = None,
                 max_threads: int = 64, batch_window_s: float = 0.0, max_batch: int = 64):
        """`engine`: an `EngineServer` (has `submit`) or a batch callable. `participant`: an
        `experimental.weight_sync.participants.EngineParticipant` that knows where new weights come from.
        `batch_window_s` > 0 (batch callables only): requests that arrive within the window and share their sampling
        settings are served by ONE engine call of up to `max_batch` prompts, with the shortest token limit among them
        and the first request's seed; episodes that run concurrently then decode together instead of one after the
        other. 0 keeps one engine call, and the request's own seed, per request."""
        from concurrent.futures import ThreadPoolExecutor
        self.engine, self.tokenizer, self.participant = engine, tokenizer, participant
        self.eos_tokens = list(eos_tokens or [])
        self._server = hasattr(engine, "submit")
        self._pool = ThreadPoolExecutor(max_threads, thread_name_prefix="sampler-adapter")
        self._inflight = self._served = 0
        self._paused = False
        self._gate: Optional[asyncio.Event] = None
        self.policy_version = 0
        self._window, self._max_batch = float(batch_window_s), max(int(max_batch), 1)
        self._pending: list = []
        self._flusher: Optional[asyncio.Task] = None
        self.engine_calls = 0

    # ------------------------------------------------------------------ lifecycle
    def initialize(self) -> None:
        pass

    async def start(self) -> None:
        self._gate = asyncio.Event()
        self._gate.set()

    async def stop(self) -> None:
        if hasattr(self.engine, "close"):
            await asyncio.get_running_loop().run_in_executor(self._pool, self.engine.close)
        self._pool.shutdown(wait=False)

    async def pause(self) -> bool:
        self._paused = True
        if self._gate is not None:
            self._gate.clear()
        if hasattr(self.engine, "pause"):
            return bool(await asyncio.get_running_loop().run_in_executor(self._pool, self.engine.pause, 600.0))
        while self._inflight:                               # a batch callable: wait for the calls in flight
            await asyncio.sleep(0.005)
        return True

    async def resume(self) -> None:
        if hasattr(self.engine, "resume"):
            self.engine.resume()
        self._paused = False
        if self._gate is not None:
            self._gate.set()

    # ------------------------------------------------------------------ sampling
    def _finish(self, toks) -> str:
        return "stop" if len(toks) and int(toks[-1]) in self.eos_tokens else "length"

    def _one(self, req: SamplingRequest) -> SamplingResponse:
        t0 = time.perf_counter()
        try:
            sp = req.sampling_params
            if self._server:
                toks, lps = self.engine.generate(list(req.prompt_token_ids), sp.max_tokens)
            else:
                out = self.engine(prompt_token_ids=[list(req.prompt_token_ids)], max_generation_steps=sp.max_tokens,
                                  temperature=sp.temperature, top_p=sp.top_p, top_k=sp.top_k, seed=sp.seed,
                                  return_logprobs=sp.return_logprobs, **({"eos_tokens": self.eos_tokens} if self.eos_tokens else {}))
                toks, lps = np.asarray(out.tokens[0]), (None if out.logprobs is None else out.logprobs[0])
            toks = [int(t) for t in toks]
            return SamplingResponse(req.request_id, toks, None if lps is None or not sp.return_logprobs else [float(x) for x in lps],
                                    self.tokenizer.decode(toks) if self.tokenizer is not None else None, self._finish(toks),
                                    self.policy_version, time.perf_counter() - t0)
        except BaseException as e:
            return SamplingResponse(req.request_id, error=e, finish_reason="error", policy_version=self.policy_version,
                                    latency_s=time.perf_counter() - t0)

    def _many(self, reqs: Sequence[SamplingRequest]) -> list:
        """One engine call for requests that share their sampling settings."""
        t0 = time.perf_counter()
        try:
            sp = reqs[0].sampling_params
            limit = min(r.sampling_params.max_tokens for r in reqs)
            out = self.engine(prompt_token_ids=[list(r.prompt_token_ids) for r in reqs], max_generation_steps=limit,
                              temperature=sp.temperature, top_p=sp.top_p, top_k=sp.top_k, seed=sp.seed, return_logprobs=sp.return_logprobs,
                              **({"eos_tokens": self.eos_tokens} if self.eos_tokens else {}))
            res = []
            for i, r in enumerate(reqs):
                toks = [int(t) for t in np.asarray(out.tokens[i])]
                lps = None if out.logprobs is None or not sp.return_logprobs else [float(x) for x in np.asarray(out.logprobs[i])[:len(toks)]]
                res.append(SamplingResponse(r.request_id, toks, lps, self.tokenizer.decode(toks) if self.tokenizer is not None else None,
                                            self._finish(toks), self.policy_version, time.perf_counter() - t0))
            return res
        except BaseException as e:
            return [SamplingResponse(r.request_id, error=e, finish_reason="error", policy_version=self.policy_version,
                                     latency_s=time.perf_counter() - t0) for r in reqs]

    async def _flush_later(self) -> None:
        await asyncio.sleep(self._window)
        loop = asyncio.get_running_loop()
        while self._pending:
            first = self._pending[0][0].sampling_params
            key = (first.temperature, first.top_p, first.top_k, first.return_logprobs)
            take = [p for p in self._pending if (p[0].sampling_params.temperature, p[0].sampling_params.top_p, p[0].sampling_params.top_k,
                                                 p[0].sampling_params.return_logprobs) == key][: self._max_batch]
            ids = {id(p) for p in take}
            self._pending = [p for p in self._pending if id(p) not in ids]
            self.engine_calls += 1
            outs = await loop.run_in_executor(self._pool, self._many, [p[0] for p in take])
            for (_, fut), o in zip(take, outs):
                if not fut.done():
                    fut.set_result(o)

    async def _batched(self, req: SamplingRequest) -> SamplingResponse:
        fut = asyncio.get_running_loop().create_future()
        self._pending.append((req, fut))
        if self._flusher is None or self._flusher.done():
            self._flusher = asyncio.create_task(self._flush_later())
        return await fut

    async def sample(self, requests: Sequence[SamplingRequest]) -> list:
        if self._gate is None:
            await self.start()
        await self._gate.wait()                             # no admission during a weight sync
        loop = asyncio.get_running_loop()
        self._inflight += len(requests)
        try:
            if self._window > 0 and not self._server:
                out = await asyncio.gather(*(self._batched(r) for r in requests))
            else:
                self.engine_calls += len(requests)
                out = await asyncio.gather(*(loop.run_in_executor(self._pool, self._one, r) for r in requests))
        finally:
            self._inflight -= len(requests)
        self._served += len(requests)
        return list(out)

    # ------------------------------------------------------------------ weight sync
    async def pre_weight_sync(self, version: int) -> None:
        self._paused = True
        if self._gate is not None:
            self._gate.clear()
        if self.participant is not None:
            await asyncio.get_running_loop().run_in_executor(self._pool, self.participant.prepare, version)
        else:
            await self.pause()

    async def weight_sync(self, version: int) -> None:
        if self.participant is not None:
            await asyncio.get_running_loop().run_in_executor(self._pool, self.participant.transfer, version)

    async def post_weight_sync(self, version: int) -> None:
        if self.participant is not None:
            await asyncio.get_running_loop().run_in_executor(self._pool, self.participant.commit, version)
        self.policy_version = version
        self._open()

    async def abort_weight_sync(self) -> None:
        if self.participant is not None:
            await asyncio.get_running_loop().run_in_executor(self._pool, self.participant.rollback)
        self._open()

    def _open(self) -> None:
        if self.participant is None and hasattr(self.engine, "resume"):
            self.engine.resume()
        self._paused = False
        if self._gate is not None:
            self._gate.set()

    async def get_load_info(self) -> LoadInfo:
        return LoadInfo(self._inflight, self._served, self._paused, self.policy_version)
