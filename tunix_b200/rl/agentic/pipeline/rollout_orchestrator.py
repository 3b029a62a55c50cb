"""Bounded-concurrency pool of per-episode runners (tunix/rl/agentic/pipeline/rollout_orchestrator.py:47-393).

`run_producers_from_stream(pairs)` starts at most `max_concurrency` episodes at a time; finished
`TrajectoryItem`s go to a `GroupQueueManager`; `yield_batches` hands complete groups to the consumer.
Exceptions inside an episode mark that trajectory FAILED; exceptions of the pipeline itself are forwarded to
the consumer through the queue (:176-192, :336-340); cancellation is graceful."""
from __future__ import annotations

import asyncio
from typing import Any, AsyncIterator, Callable, Iterable, Optional

from ..agents.agent_types import TrajectoryItem
from ..queue_manager.group_queue_manager import GroupQueueManager


class RolloutOrchestrator:
    def __init__(self, *, engine_factory: Callable[[Any, Any], Any], group_size: int, max_concurrency: int = 8,
                 max_open_buckets: Optional[int] = None, collect_mode: str = "Token"):
        self.engine_factory = engine_factory
        self.max_concurrency = max_concurrency
        self.collect_mode = collect_mode
        self.queue = GroupQueueManager(group_size=group_size, max_open_buckets=max_open_buckets)
        self._tasks: set = set()
        self._stop = False

    async def _run_one(self, idx: int, agent, env, group_id, episode_id: int, sem: asyncio.Semaphore, start_step: int):
        try:
            engine = self.engine_factory(agent, env)
            traj = await engine.collect(self.collect_mode)
            await self.queue.put(TrajectoryItem(pair_index=idx, group_id=group_id, episode_id=episode_id,
                                                start_step=start_step, traj=traj), group_key=group_id)
        except asyncio.CancelledError:
            raise
        except Exception as e:
            await self.queue.put_exception(e)
        finally:
            sem.release()

    async def run_producers_from_stream(self, pairs: Iterable, start_step: int = 0) -> None:
        """pairs yields (agent, env, group_id); episodes of one group share `group_id`."""
        sem = asyncio.Semaphore(self.max_concurrency)
        counts: dict = {}
        try:
            for idx, (agent, env, gid) in enumerate(pairs):
                if self._stop:
                    break
                await sem.acquire()
                ep = counts.get(gid, 0)
                counts[gid] = ep + 1
                t = asyncio.create_task(self._run_one(idx, agent, env, gid, ep, sem, start_step))
                self._tasks.add(t)
                t.add_done_callback(self._tasks.discard)
            if self._tasks:
                await asyncio.gather(*list(self._tasks), return_exceptions=True)
        except Exception as e:
            await self.queue.put_exception(e)
        finally:
            await self.queue.close()

    async def yield_batches(self, n_groups: int = 1) -> AsyncIterator[list]:
        while True:
            groups = await self.queue.get_batch(n_groups)
            if not groups:
                return
            yield groups

    async def cancel(self) -> None:
        self._stop = True
        for t in list(self._tasks):
            t.cancel()
        await asyncio.gather(*list(self._tasks), return_exceptions=True)
        await self.queue.close()
