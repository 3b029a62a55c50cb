"""The compute primitives an RL program is written against (tunix/experimental/orchestrator/rl_engine_interface.py:29-206).

An engine hides WHERE the models run (in-process workers, workers behind gRPC, one GPU or many): a program only
dispatches rollouts, polls finished ones, scores, asks for log-probs, feeds micro-batches to a trainer role, syncs
weights and saves / restores checkpoints. Everything is a coroutine so that the stages of a program overlap on one
event loop. `DistributedRLEngine` (`distributed_rl_engine.py`) is the implementation over this package's workers; a
test double only needs these methods."""
from __future__ import annotations

from typing import Any, Mapping, Optional, Protocol, Sequence, runtime_checkable

from ..common.datatypes import GenerationArgs, Role


@runtime_checkable
class AbstractRLEngine(Protocol):
    @property
    def restored_checkpoint_metadata(self) -> Optional[dict]:
        """Metadata of the checkpoint that the last `resume_from_checkpoint` restored, if any."""
        ...

    async def dispatch_rollout_requests(self, requests: Sequence[Any]) -> list:
        """Send pre-formed `RolloutRequest`s (unique `request_id`, non-empty `group_id`); returns their ids at once."""
        ...

    async def dispatch_rollouts(self, prompts: Sequence[Any], *, num_generations: int = 1, policy_version: int = 0,
                                generation_args: Optional[GenerationArgs] = None,
                                route_metadata: Optional[Mapping[str, Any]] = None, **kwargs: Any) -> list:
        """Expand every prompt (which MUST carry a unique `prompt_id`) into `num_generations` requests with ids
        `req_<prompt_id>_g<index>_v<version>` and dispatch them."""
        ...

    async def poll_rollouts(self, timeout_s: float = 1.0) -> list:
        """Rollouts that have finished since the last poll (waits up to `timeout_s` for the first)."""
        ...

    async def generate(self, prompts: Sequence[Any], generation_args: Optional[GenerationArgs] = None,
                       route_metadata: Optional[Mapping[str, Any]] = None) -> list:
        """Blocking generation: one response per prompt, in order."""
        ...

    async def score(self, role: Role, items: Sequence[Any], **kwargs: Any) -> list:
        ...

    async def per_token_logps(self, role: Role, items: Any, **kwargs: Any) -> Any:
        ...

    async def train_step(self, batch: Any, role: Role = Role.ACTOR, accumulate_gradients: bool = False,
                         apply_optimizer: bool = True, **kwargs: Any) -> Any:
        """Forward + backward on one micro-batch; with `apply_optimizer` the optimizer step follows."""
        ...

    async def get_metrics(self, role: Role = Role.ACTOR, **kwargs: Any) -> Any:
        ...

    def configure_worker(self, role: Role = Role.ACTOR, *, algo: Any, assembler: Any, **kwargs: Any) -> None:
        ...

    async def prepare_rollout_policy(self, role: Role = Role.ACTOR, sync_weights: bool = True,
                                     policy_version: Optional[int] = None, **kwargs: Any) -> Optional[int]:
        """Make the rollout workers hold the trainer's weights before the first dispatch."""
        ...

    async def sync_weights(self, role: Role = Role.ACTOR, target_roles: Optional[Sequence[Role]] = None,
                           policy_version: Optional[int] = None, **kwargs: Any) -> int:
        ...

    async def save_checkpoint(self, role: Role = Role.ACTOR, metadata: Any = None, **kwargs: Any) -> Any:
        ...

    async def resume_from_checkpoint(self, role: Role = Role.ACTOR, resync_rollout_weights: bool = True) -> int:
        """Restore the trainer's latest checkpoint, set the policy version to the restored step boundary and
        (optionally) push the restored weights to the rollout workers. Returns the restored step (0 = fresh run)."""
        ...

    async def close(self) -> None:
        ...
