"""The layered distributed RL run: engine primitives over workers, the four-stage program on top
(test model: tunix/experimental/orchestrator/{distributed_rl_engine,rl_program}_test.py). CPU, tiny model; worker
failures are scripted on the host."""
import asyncio
import os
import time

import numpy as np
import pytest
import torch

from tunix_b200.experimental.common.datatypes import GenerationArgs, Role, RolloutRequest, RolloutResponse
from tunix_b200.experimental.orchestrator.algorithm_adapter import GRPOAdapter
from tunix_b200.experimental.orchestrator.batch_assembly import BatchConfig
from tunix_b200.experimental.orchestrator.distributed_rl_engine import DistributedRLEngine
from tunix_b200.experimental.orchestrator.rl_engine_interface import AbstractRLEngine
from tunix_b200.experimental.orchestrator.rl_program import StandardRLProgram, _generation_metrics, prompt_coordinates, tag_prompt


from tunix_b200.experimental.common import test_utils as doubles


class _EchoRollout(doubles.EchoRolloutWorker):
    def __init__(self, worker_id, fail=False, n=4):
        super().__init__(worker_id, n=n, fail=fail)


class _Trainer(doubles.RecordingTrainerWorker):
    pass


def _prompts(n):
    return doubles.make_prompts(n)


def test_engine_builds_requests_routes_by_prompt_and_reports_failures():
    a, b = _EchoRollout("r0"), _EchoRollout("r1")
    eng = DistributedRLEngine([a, b], {Role.ACTOR: _Trainer({})}, export_weights=lambda: "W")
    assert isinstance(eng, AbstractRLEngine)

    async def go():
        with pytest.raises(ValueError, match="lacks 'prompt_id'"):
            await eng.dispatch_rollouts([{"prompt_ids": [1, 2]}])
        ids = await eng.dispatch_rollouts(_prompts(3), num_generations=4, policy_version=2,
                                          generation_args=GenerationArgs(max_tokens=3, temperature=0.7))
        assert ids[:2] == ["req_p0_g0_v2", "req_p0_g1_v2"] and len(ids) == 12
        got = []
        while len(got) < 12:
            got += await eng.poll_rollouts(timeout_s=1.0)
        assert await eng.poll_rollouts(timeout_s=0.01) == []
        # the generations of one prompt share a worker; seeds differ inside a group and repeat across runs
        owner = {}
        for w in (a, b):
            for r in w.seen:
                owner.setdefault(r.group_id, set()).add(w.worker_id)
                assert r.max_tokens == 3 and r.temperature == 0.7 and r.metadata["lineage"].events[0].operation == "rollout"
        assert all(len(v) == 1 for v in owner.values())
        seeds = sorted(r.seed for w in (a, b) for r in w.seen if r.group_id == "p0")
        assert len(set(seeds)) == 4 and seeds == list(range(seeds[0], seeds[0] + 4))
        assert all(r.metadata["is_valid"] and r.metadata["num_generations"] == 4 for r in got)
        # both workers down: the request comes back as an invalid response instead of disappearing
        a.fail = b.fail = True
        await eng.dispatch_rollouts(_prompts(1), num_generations=2)
        bad = []
        while len(bad) < 2:
            bad += await eng.poll_rollouts(timeout_s=1.0)
        assert all(r.finish_reason == "error" and r.metadata["is_valid"] is False for r in bad)
        with pytest.raises(TypeError, match="Unexpected generate kwargs"):
            await eng.generate(_prompts(1), temperature=1.0)
        eng.rollout_pool.mark_up("r0"); eng.rollout_pool.mark_up("r1")
        a.fail = b.fail = False
        out = await eng.generate(_prompts(2), GenerationArgs(max_tokens=2))
        assert [r.group_id for r in out] == ["p0", "p1"] and all(len(r.tokens) == 2 for r in out)
        assert await eng.sync_weights() == 1 and a.synced == [(1, "W")] and eng.policy_version == 1
        with pytest.raises(ValueError, match="No inference worker"):
            await eng.score(Role.REWARD, [])
        assert (await eng.get_metrics(Role.ROLLOUT))["policy_version"] == 1
        assert (await eng.get_metrics(Role.ACTOR))["train_steps"] == 0
        await eng.close()
    asyncio.run(go())


def test_engine_resume_policy_version_rules():
    async def resume(meta, **kw):
        disk = {"latest": meta} if meta is not None else {}
        r = _EchoRollout("r0")
        eng = DistributedRLEngine([r], {"actor": _Trainer(disk)})
        step = await eng.resume_from_checkpoint(**kw)
        await eng.close()
        return step, eng.policy_version, r.synced, eng.restored_checkpoint_metadata
    assert asyncio.run(resume(None)) == (0, 0, [], None)
    step, version, synced, meta = asyncio.run(resume({"step": 3, "global_step": 3, "policy_version": 3}))
    assert (step, version, synced) == (3, 3, [(3, None)]) and meta["global_step"] == 3
    # a version recorded inside a step is ignored unless the checkpoint carries off-policy state
    assert asyncio.run(resume({"step": 6, "global_step": 3, "policy_version": 5}))[:2] == (3, 3)
    assert asyncio.run(resume({"step": 6, "global_step": 3, "policy_version": 5, "committed_prompt_ids": ["p0"]}))[:2] == (3, 5)
    assert asyncio.run(resume({"step": 2}, resync_rollout_weights=False))[:3] == (2, 2, [])
    assert asyncio.run(resume({"step": "x"}))[0] == 0


def test_coordinates_and_generation_metrics():
    assert prompt_coordinates(7, 4) == {"prompt_idx": 7, "batch_idx": 1, "intra_batch_idx": 3}
    item = {"prompt_id": "a", "metadata": {"k": 1}}
    assert tag_prompt(item, prompt_coordinates(0, 2))["metadata"] == {"k": 1, "prompt_idx": 0, "batch_idx": 0, "intra_batch_idx": 0}
    assert item["metadata"] == {"k": 1}
    mk = lambda n, c: RolloutResponse("r", [], metadata={"raw_length": n, "clipped": c})
    m = _generation_metrics([[mk(10, True), mk(20, False)], [mk(4, False)], [RolloutResponse("r", [])]])
    assert m == {"rollout/completions/clip_ratio": 0.25, "rollout/completions/mean_raw_length": 9.5,
                 "rollout/completions/max_raw_length": 20.0, "rollout/completions/min_raw_length": 4.0}
    assert _generation_metrics([[RolloutResponse("r", [])]]) == {}


def _program(dataset, max_steps, **kw):
    algo = GRPOAdapter(reward_fn=lambda item, r: float(sum(t % 5 for t in r.tokens)), drop_uniform_groups=True)
    return StandardRLProgram(algo, dataset, max_steps, num_generations=4, batch_size=2,
                             batch_config=BatchConfig(rows_per_microbatch=2, max_packed_len=48), generation_args=GenerationArgs(max_tokens=4),
                             poll_timeout_s=0.05, **kw)


def test_program_runs_steps_checkpoints_and_resumes():
    disk = {}
    a, b, tr = _EchoRollout("r0"), _EchoRollout("r1", fail=True), _Trainer(disk)
    eng = DistributedRLEngine([a, b], {Role.ACTOR: tr}, export_weights=lambda: "W")
    begun, ended = [], []
    prog = _program(_prompts(10), 3, on_step_begin=begun.append, on_step_end=lambda s, r: ended.append((s, r["train_step"])))
    hist = prog.run(eng)
    assert [h["step"] for h in hist] == [0, 1, 2] and begun == [0, 1, 2] and ended == [(0, 1), (1, 2), (2, 3)]
    assert [h["policy_version"] for h in hist] == [1, 2, 3] and prog.step == 3 and prog.last_step_result.step == 2
    assert all(h["num_rollouts"] == 8 and h["num_microbatches"] >= 1 and 0 <= h["padding_ratio"] < 1 for h in hist)
    assert all(h["staleness_max"] == 0 for h in hist)                                 # max_staleness = 0: strictly on-policy
    # every optimizer step: the micro-batches before the last accumulate, the last one closes the step
    fb = [last for op, last in tr.ops if op == "fwd_bwd"]
    assert fb.count(True) == 3 and [op for op, _ in tr.ops].count("update") == 3
    for i, (op, last) in enumerate(tr.ops):
        if op == "update":
            assert tr.ops[i - 1] == ("fwd_bwd", True)
    assert a.synced[0] == (0, "W") and [v for v, _ in a.synced][-3:] == [1, 2, 3]      # bootstrap sync, then one per step
    assert b.seen == [] and eng.rollout_pool.stats()["r1"]["down"]                    # the dead worker was routed around
    assert disk["latest"]["global_step"] == 3 and disk["latest"]["policy_version"] == 3
    asyncio.run(eng.close())
    # a new process: fresh engine and program over the same checkpoint continue with step 3 and the unseen prompts
    a2, tr2 = _EchoRollout("r0"), _Trainer(disk)
    eng2 = DistributedRLEngine([a2], {Role.ACTOR: tr2})
    prog2 = _program(_prompts(10), 5)
    hist2 = prog2.run(eng2)
    assert [h["step"] for h in hist2] == [3, 4] and tr2.steps == 5 and [v for v, _ in a2.synced] == [3, 4, 5]
    seen = {r.group_id for r in a2.seen}
    trained = {r.group_id for r in a.seen}
    assert seen.isdisjoint({f"p{i}" for i in range(6)}) and seen <= {f"p{i}" for i in range(6, 10)}
    assert trained >= {f"p{i}" for i in range(6)}
    asyncio.run(eng2.close())


def test_program_replaces_filtered_groups_and_stops_at_dataset_end():
    class Uniform(_EchoRollout):
        def submit(self, req):
            out = super().submit(req)
            if req.group_id in ("p1", "p2"):            # identical responses: no learning signal
                out.tokens = [7, 7]
            return out
    r, tr = Uniform("r0"), _Trainer({})
    eng = DistributedRLEngine([r], {Role.ACTOR: tr})
    prog = _program(_prompts(7), None, checkpoint_every=0, sync_weights=False)
    hist = prog.run(eng)
    consumed = sum(h["num_rollouts"] for h in hist) // 4
    assert consumed == 5 and sum(h["filtered_groups"] for h in hist) == 2
    assert prog.dispatch_window.skipped_prompt_ids == {"p1", "p2"}
    assert prog.dispatch_window.committed_prompt_ids == {"p0", "p3", "p4", "p5", "p6"}
    assert hist[-1]["num_rollouts"] == 4                                             # the dataset ran out inside the last step
    assert all(v == 0 for v, _ in r.synced) and tr.steps == len(hist) == 3
    asyncio.run(eng.close())


def test_program_surfaces_stage_errors():
    class BadTrainer(_Trainer):
        def submit(self, req):
            if req["op"] == "update":
                raise RuntimeError("optimizer exploded")
            return super().submit(req)
    eng = DistributedRLEngine([_EchoRollout("r0")], {Role.ACTOR: BadTrainer({})})
    with pytest.raises(RuntimeError, match="optimizer exploded"):
        _program(_prompts(4), 2, sync_weights=False).run(eng)
    asyncio.run(eng.close())


def test_program_on_real_workers_with_checkpoint_resume(tmp_path):
    """Sampler-backed rollout workers, a split-step trainer worker over a tiny model and its checkpoint manager: two
    steps, then a second process-worth of objects resumes from the checkpoint directory."""
    from tests.test_sampler_cpu import CharTok
    from tunix_b200 import optim
    from tunix_b200.common.configs import CacheConfig, TrainingConfig
    from tunix_b200.experimental.train.peft_trainer_v2 import TrainerV2
    from tunix_b200.experimental.worker.rollout_worker import RolloutWorker, TrainerWorker
    from tunix_b200.generate.sampler import Sampler
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.sft.peft_trainer import PeftTrainer
    from tunix_b200.sft.utils import LossOutput, WeightedMetric
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16,
                                           num_kv_heads=1)

    def pg_loss(model, input_tokens, completion_mask, advantages, segment_ids=None, positions=None, **_):
        hidden, _ = model(input_tokens[:, :-1], positions=None if positions is None else positions[:, :-1],
                          segment_ids=None if segment_ids is None else segment_ids[:, :-1], skip_lm_head=True)
        lp = model.token_logprobs(hidden.reshape(-1, hidden.shape[-1]), input_tokens[:, 1:].reshape(-1).long())[0]
        m = completion_mask[:, 1:]
        return LossOutput(loss=WeightedMetric(-(lp.view(input_tokens.shape[0], -1) * advantages[:, 1:] * m).sum(), m.sum()))

    def to_inputs(batch):
        out = {k: torch.as_tensor(v) for k, v in batch.items()}
        out["input_tokens"] = out["input_tokens"].long()
        return out

    def build():
        model = create_model(cfg, seed=0)
        trainer = PeftTrainer(model, optim.AdamW(5e-3), TrainingConfig(
            eval_every_n_steps=10 ** 9, pbar_description=None, resume_from_checkpoint_on_init=False,
            checkpoint_root_directory=str(tmp_path / "ckpt")))
        trainer.with_loss_fn(pg_loss).with_gen_model_input_fn(to_inputs)
        synced = []
        workers = [RolloutWorker("rollout-0", Sampler(model, CharTok(), CacheConfig(64, 1, 1, 16)), eos_tokens=[2],
                                 apply_weights=lambda v, p: synced.append(v)), TrainerWorker("trainer-0", TrainerV2(trainer))]
        for w in workers:
            w.start()
        return model, workers, synced, DistributedRLEngine([workers[0]], {Role.ACTOR: workers[1]})
    model, workers, synced, eng = build()
    before = torch.cat([p.detach().reshape(-1).clone() for p in model.parameters()])
    prog = StandardRLProgram(GRPOAdapter(reward_fn=lambda item, r: float(sum(t % 5 for t in r.tokens))), _prompts(8), 2,
                             num_generations=4, batch_size=2, batch_config=BatchConfig(rows_per_microbatch=2, max_packed_len=48),
                             generation_args=GenerationArgs(max_tokens=6, temperature=1.0), poll_timeout_s=0.05)
    hist = prog.run(eng)
    assert [h["step"] for h in hist] == [0, 1] and all(np.isfinite(h["loss"]) for h in hist)
    after = torch.cat([p.detach().reshape(-1).clone() for p in model.parameters()])
    assert not torch.equal(before, after) and synced == [0, 1, 2]
    assert (asyncio.run(eng.get_metrics(Role.ACTOR)))["train_steps"] == 2
    asyncio.run(eng.close())
    for w in workers:
        w.stop()
    model2, workers2, synced2, eng2 = build()
    prog2 = StandardRLProgram(GRPOAdapter(reward_fn=lambda item, r: float(sum(t % 5 for t in r.tokens))), _prompts(8), 3,
                              num_generations=4, batch_size=2, batch_config=BatchConfig(rows_per_microbatch=2, max_packed_len=48),
                              generation_args=GenerationArgs(max_tokens=6, temperature=1.0), poll_timeout_s=0.05)
    hist2 = prog2.run(eng2)
    assert [h["step"] for h in hist2] == [2] and synced2 == [2, 3]
    meta = eng2.restored_checkpoint_metadata
    assert meta["global_step"] == 2 and meta["policy_version"] == 2 and meta["num_rollouts"] == 8
    restored = torch.cat([p.detach().reshape(-1) for p in model2.parameters()])
    assert not torch.equal(restored, before)                      # weights came from the checkpoint, then one more step
    asyncio.run(eng2.close())
    for w in workers2:
        w.stop()


def test_program_logs_consumed_rollouts_to_a_step_level_store():
    from tunix_b200.experimental.trajectory.in_memory_store import InMemoryTrajectoryStore
    store = InMemoryTrajectoryStore()
    eng = DistributedRLEngine([_EchoRollout("r0")], {Role.ACTOR: _Trainer({})})
    hist = _program(_prompts(2), 1, trajectory_store=store, sync_weights=False, checkpoint_every=0).run(eng)
    metas = store.get_trajectories_metadata()
    assert len(metas) == hist[0]["num_rollouts"] == 8 and {m.prompt_id for m in metas} == {"p0", "p1"}
    full = store.get_trajectories([metas[0].trajectory_id])[0]
    assert len(full.steps) == 2 and len(full.steps[1].assistant_tokens) == 4 and full.extra["consumed_at_step"] == 0
    assert metas[0].trajectory_id.startswith("req_p") and sorted(m.group_index for m in metas if m.prompt_id == "p0") == [0, 1, 2, 3]
    asyncio.run(eng.close())


def test_multi_turn_episodes_through_the_distributed_stack():
    """FrozenLake episodes run on episode workers (agent + environment + sampler); the program trains on the model's
    tokens only, with the environment's reward; weights are swapped while episodes are in flight."""
    import threading
    from tests.test_sampler_cpu import CharTok
    from tunix_b200.experimental.common.datatypes import WorkerState
    from tunix_b200.experimental.orchestrator.algorithm_adapter import env_reward
    from tunix_b200.experimental.rl.agentic import registry as registries
    from tunix_b200.experimental.rollout import sampler as sampler_lib
    from tunix_b200.experimental.worker.agentic_rollout_worker import AgenticRolloutWorker
    from tunix_b200.rl.agentic.environments.frozenlake_environment import FrozenLakeAgent, FrozenLakeEnv, shortest_path
    from tunix_b200.rl.agentic.parser.chat_template_parser import get_parser
    for reg, name, cls in ((registries.AGENT_REGISTRY, "frozenlake", FrozenLakeAgent), (registries.ENV_REGISTRY, "frozenlake", FrozenLakeEnv)):
        if name not in reg:
            reg.register(name)(cls)
    tok = CharTok()

    class Scripted:
        """Walks the shortest path for even seeds, wanders for odd ones; counts calls per policy version."""
        def __init__(self):
            self.policy_version, self.calls, self.lock, self.hold, self.turns = 0, [], threading.Lock(), None, {}

        async def sample(self, requests):
            out = []
            for r in requests:
                if self.hold is not None:
                    await self.hold.wait()
                with self.lock:
                    self.calls.append((r.request_id, self.policy_version, r.sampling_params.seed))
                good = r.sampling_params.seed % 2 == 0
                turn = self.turns[r.request_id] = self.turns.get(r.request_id, -1) + 1
                seed = int(str(r.route_key).replace("lake", "").replace("held", "0"))
                path = shortest_path(FrozenLakeEnv({"seed": seed, "size": 4, "p": 0.8, "max_steps": 8}).grid)
                reply = f"```{path[min(turn, len(path) - 1)].capitalize() if good else 'Up'}```"
                ids = tok.encode(reply)
                out.append(sampler_lib.SamplingResponse(r.request_id, ids, [-0.3] * len(ids), reply, "stop", self.policy_version))
            return out

        async def pre_weight_sync(self, version): ...
        async def weight_sync(self, version): ...

        async def post_weight_sync(self, version):
            self.policy_version = version
    samplers = [Scripted(), Scripted()]
    workers = [AgenticRolloutWorker(f"ep-{i}", s, tok, chat_parser=get_parser("qwen"), eos_ids=[2], default_agent="frozenlake",
                                    default_env="frozenlake") for i, s in enumerate(samplers)]
    for w in workers:
        w.start()
    tr = _Trainer({})
    eng = DistributedRLEngine(workers, {Role.ACTOR: tr})
    data = [{"prompt_id": f"lake{i}", "task": {"seed": i, "size": 4, "p": 0.8, "max_steps": 8}, "max_turns": 8} for i in range(4)]
    prog = StandardRLProgram(GRPOAdapter(reward_fn=env_reward), data, 2, num_generations=4, batch_size=2,
                             batch_config=BatchConfig(rows_per_microbatch=2, max_packed_len=4096, max_prompt_length=1024,
                                                      max_response_length=2048),
                             generation_args=GenerationArgs(max_tokens=16, temperature=1.0), poll_timeout_s=0.05, checkpoint_every=0)
    seen_batches = []
    real = tr.submit

    def spy(req):
        if req.get("op") == "fwd_bwd":
            seen_batches.append(req["batch"])
        return real(req)
    tr.submit = spy
    hist = prog.run(eng)
    assert [h["step"] for h in hist] == [0, 1] and all(h["num_rollouts"] == 8 for h in hist)
    assert all(0.0 < h["reward_mean"] < 1.0 and h["reward_std"] > 0 for h in hist)          # half of each group reaches the goal
    b = seen_batches[0]
    m = np.asarray(b["completion_mask"])
    assert 0 < m.sum() < (np.asarray(b["input_tokens"]) != 0).sum()                         # environment and prompt tokens carry no loss
    assert all(w.state == WorkerState.READY and w.policy_version == 2 for w in workers) and sum(w.served for w in workers) == 16
    assert {v for s in samplers for _, v, _ in s.calls} == {0, 1}                            # step 1 was generated with version 1
    # a sync arriving while an episode waits for its model: the episode is held, then goes on under the new version
    hold = samplers[0].hold = asyncio.Event()
    req = eng._build_rollout_requests([dict(data[0], prompt_id="held")], num_generations=1, policy_version=2)[0]
    res = {}
    t = threading.Thread(target=lambda: res.setdefault("r", workers[0].submit(req)))
    t.start()
    deadline = time.monotonic() + 5
    while workers[0].state != WorkerState.BUSY and time.monotonic() < deadline:
        time.sleep(0.01)
    workers[0].sync_weights(3)
    assert workers[0].state == WorkerState.BUSY and workers[0].policy_version == 3
    workers[0]._loop.call_soon_threadsafe(hold.set)
    t.join(10)
    assert res["r"].metadata["is_valid"] and max(res["r"].metadata["policy_versions"]) == 3
    asyncio.run(eng.close())
    for w in workers:
        w.stop()
        assert w.state == WorkerState.STOPPED


def test_sampler_adapter_batches_concurrent_requests_within_its_window():
    from tunix_b200.experimental.rollout import sampler as sampler_lib
    calls = []

    class Engine:
        def __call__(self, prompt_token_ids, max_generation_steps, temperature, top_p, top_k, seed, return_logprobs, **kw):
            calls.append((len(prompt_token_ids), max_generation_steps, temperature, seed))
            import types
            return types.SimpleNamespace(tokens=[[p[0] + 1] * max_generation_steps for p in prompt_token_ids],
                                         logprobs=[[-1.0] * max_generation_steps for _ in prompt_token_ids], text=None)
    ad = sampler_lib.EngineSamplerAdapter(Engine(), batch_window_s=0.01, max_batch=3)
    mk = lambda i, t=1.0, n=4: sampler_lib.SamplingRequest(f"r{i}", [10 * i], sampler_lib.SamplingParams(max_tokens=n, temperature=t, seed=i))

    async def go():
        return await asyncio.gather(*(ad.sample([mk(i, n=4 + i)]) for i in range(4)), ad.sample([mk(9, t=0.5)]))
    out = asyncio.run(go())
    sizes = sorted(c[0] for c in calls)
    assert sizes == [1, 1, 3] and ad.engine_calls == 3                 # 3 + 1 of one setting (batch limit 3), 1 of another
    assert (3, 4, 1.0, 0) in calls                                     # shortest limit and the first request's seed
    assert [o[0].request_id for o in out] == ["r0", "r1", "r2", "r3", "r9"] and out[1][0].token_ids[0] == 11
    solo = sampler_lib.EngineSamplerAdapter(Engine())
    calls.clear()
    asyncio.run(solo.sample([mk(1), mk(2)]))
    assert sorted(c[3] for c in calls) == [1, 2] and all(c[0] == 1 for c in calls)      # without a window: own call, own seed


def test_polling_does_not_spin_while_nothing_is_in_flight():
    """A dispatcher parked at the window leaves nothing in flight; the polling stage must wait, not burn the loop."""
    class CountingEngine(DistributedRLEngine):
        polls = 0

        async def poll_rollouts(self, timeout_s=1.0):
            type(self).polls += 1
            return await super().poll_rollouts(timeout_s)

    class SlowTrainer(_Trainer):
        def submit(self, req):
            if req["op"] == "fwd_bwd":
                time.sleep(0.3)
            return super().submit(req)
    eng = CountingEngine([_EchoRollout("r0")], {Role.ACTOR: SlowTrainer({})})
    _program(_prompts(4), 2, sync_weights=False, checkpoint_every=0).run(eng)
    assert CountingEngine.polls < 200
    asyncio.run(eng.close())


def test_program_over_workers_behind_grpc():
    """The same engine and program with every worker in its own server on the loopback interface: requests, responses
    and weights cross the wire (`RemoteWorker`), one rollout server goes away mid-run."""
    pytest.importorskip("grpc")
    from tunix_b200.experimental.worker.remote_execution import RemoteWorker, serve_worker
    from tunix_b200.experimental.worker.rollout_worker import RolloutWorker

    class Out:
        def __init__(self, toks):
            self.tokens, self.logprobs, self.text = [toks], [[-0.5] * len(toks)], None

    def engine(prompt_token_ids, max_generation_steps, seed=None, **kw):
        rng = np.random.default_rng(seed)
        return Out(rng.integers(3, 60, max_generation_steps).tolist())
    synced = {"a": [], "b": []}
    locals_ = [RolloutWorker(f"rollout-{k}", engine, apply_weights=lambda v, p, k=k: synced[k].append((v, float(p["w"].sum()))), eos_tokens=[2])
               for k in "ab"]
    tr = _Trainer({})

    class TrainerFacade:
        """`_Trainer` behind the worker protocol (start / state / submit)."""
        worker_id, policy_version = "trainer-0", 0

        def start(self): ...
        def stop(self): ...

        def info(self):
            from tunix_b200.experimental.orchestrator.worker_registry import WorkerInfo
            return WorkerInfo(self.worker_id, ("trainer",))

        @property
        def state(self):
            from tunix_b200.experimental.common.datatypes import WorkerState
            return WorkerState.READY

        def submit(self, req):
            return tr.submit(req)

        def sync_weights(self, version, payload=None): ...
    servers = [serve_worker(w, "127.0.0.1:0", token="t") for w in locals_] + [serve_worker(TrainerFacade(), "127.0.0.1:0", token="t")]
    try:
        remotes = [RemoteWorker(s.address, token="t") for s in servers]
        for r in remotes[:2]:
            r.start()
        eng = DistributedRLEngine({"a": remotes[0], "b": remotes[1]}, {Role.ACTOR: remotes[2]},
                                  export_weights=lambda: {"w": np.full(1000, float(tr.steps), np.float32)})
        stopped = []

        def on_end(step, result):
            if step == 0:                                   # one rollout server disappears between steps
                servers[1].stop(grace=0)
                stopped.append(True)
        hist = _program(_prompts(6), 3, on_step_end=on_end).run(eng)
        assert [h["step"] for h in hist] == [0, 1, 2] and all(h["num_rollouts"] == 8 for h in hist) and stopped == [True]
        assert tr.steps == 3 and [v for v, _ in synced["a"]] == [0, 1, 2, 3]
        assert synced["a"][-1] == (3, 3000.0)               # the payload crossed the wire
        assert eng.rollout_pool.stats()["b"]["down"] and locals_[0].served > locals_[1].served
        asyncio.run(eng.close())
    finally:
        for s in servers:
            s.stop(grace=0)


def test_worker_that_cannot_take_weights_leaves_the_rotation():
    good, bad = _EchoRollout("good"), _EchoRollout("bad")
    bad.sync_weights = lambda v, p=None: (_ for _ in ()).throw(ConnectionError("gone"))
    eng = DistributedRLEngine([good, bad], {Role.ACTOR: _Trainer({})})
    assert asyncio.run(eng.sync_weights()) == 1 and good.synced == [(1, None)]
    assert eng.rollout_pool.live() == ["good"]
    good.sync_weights = bad.sync_weights
    with pytest.raises(RuntimeError, match="no rollout worker took policy version 2"):
        asyncio.run(eng.sync_weights())
    assert eng.policy_version == 1
    asyncio.run(eng.close())


def test_reference_logprobs_are_attached_to_every_micro_batch():
    class Ref:
        calls = 0

        def submit(self, req):
            assert req["op"] == "per_token_logps" and {"input_tokens", "completion_mask", "segment_ids", "positions"} <= set(req)
            Ref.calls += 1
            return np.full(np.asarray(req["input_tokens"]).shape, -2.0, np.float32).tolist()
    tr = _Trainer({})
    seen = []
    real = tr.submit
    tr.submit = lambda req: (seen.append(req["batch"]) if req.get("op") == "fwd_bwd" else None, real(req))[1]
    eng = DistributedRLEngine([_EchoRollout("r0")], {Role.ACTOR: tr}, inference_workers={Role.REFERENCE: Ref()})
    hist = _program(_prompts(2), 1, reference_kl=True, sync_weights=False, checkpoint_every=0).run(eng)
    assert Ref.calls == hist[0]["num_microbatches"] == len(seen)
    assert all(b["ref_per_token_logps"].shape == np.asarray(b["input_tokens"]).shape and (b["ref_per_token_logps"] == -2).all() for b in seen)
    asyncio.run(eng.close())
    with pytest.raises(ValueError, match="No worker registered for per_token_logps"):
        e2 = DistributedRLEngine([_EchoRollout("r0")], {Role.CRITIC: _Trainer({})})
        asyncio.run(e2.per_token_logps(Role.REFERENCE, {"input_tokens": [[1]]}))


@pytest.mark.parametrize("order", ["completion", "prompt_arrival"])
def test_group_order_decouples_training_order_from_rollout_timing(order):
    class Uneven(_EchoRollout):
        """Earlier prompts of a batch take longer, so groups finish in reverse."""
        def submit(self, req):
            i = int(req.group_id[1:])
            time.sleep(0.12 if i % 4 == 0 else 0.0)
            out = super().submit(req)
            if req.group_id == "p5":
                out.tokens = [9, 9]                      # a group without signal in the middle gives up its place
            return out
    w = Uneven("r0")
    w.max = 64
    eng = DistributedRLEngine([w], {Role.ACTOR: _Trainer({})}, max_threads=32)
    consumed = []
    prog = StandardRLProgram(GRPOAdapter(reward_fn=lambda item, r: float(sum(t % 5 for t in r.tokens))), _prompts(8), None,
                             num_generations=4, batch_size=4, batch_config=BatchConfig(rows_per_microbatch=2, max_packed_len=48),
                             generation_args=GenerationArgs(max_tokens=4), poll_timeout_s=0.02, checkpoint_every=0, sync_weights=False,
                             group_order=order)
    real = prog.dispatch_window.record_committed_groups
    prog.dispatch_window.record_committed_groups = lambda groups: (consumed.extend(g.prompt_id for g in groups), real(groups))[1]
    prog.run(eng)
    assert sorted(consumed) == sorted(f"p{i}" for i in range(8) if i != 5)
    if order == "prompt_arrival":
        assert consumed == [f"p{i}" for i in range(8) if i != 5]
    else:
        assert consumed[:4] != ["p0", "p1", "p2", "p3"]                     # the slow first prompt is not waited for
    asyncio.run(eng.close())
    with pytest.raises(ValueError, match="group_order"):
        _program(_prompts(1), 1, group_order="random")


def test_episode_worker_behind_grpc_serves_frozenlake_episodes():
    """An episode worker in a server on the loopback interface: the request (task, agent / environment names, lineage)
    and the response (conversation tokens, masks, environment reward, budget facts) cross the wire."""
    pytest.importorskip("grpc")
    from tests.test_sampler_cpu import CharTok
    from tunix_b200.experimental.rl.agentic import registry as registries
    from tunix_b200.experimental.rollout import sampler as sampler_lib
    from tunix_b200.experimental.worker.agentic_rollout_worker import AgenticRolloutWorker
    from tunix_b200.experimental.worker.remote_execution import RemoteWorker, serve_worker
    from tunix_b200.rl.agentic.environments.frozenlake_environment import FrozenLakeAgent, FrozenLakeEnv, shortest_path
    from tunix_b200.rl.agentic.parser.chat_template_parser import get_parser
    for reg, cls in ((registries.AGENT_REGISTRY, FrozenLakeAgent), (registries.ENV_REGISTRY, FrozenLakeEnv)):
        if "frozenlake" not in reg:
            reg.register("frozenlake")(cls)
    tok = CharTok()
    task = {"seed": 3, "size": 4, "p": 0.8, "max_steps": 8}
    path = shortest_path(FrozenLakeEnv(task).grid)

    class Walker:
        def __init__(self):
            self.turn = 0

        async def sample(self, requests):
            out = []
            for r in requests:
                reply = f"```{path[min(self.turn, len(path) - 1)].capitalize()}```"
                self.turn += 1
                ids = tok.encode(reply)
                out.append(sampler_lib.SamplingResponse(r.request_id, ids, [-0.2] * len(ids), reply, "stop", 0))
            return out
    local = AgenticRolloutWorker("episodes-0", Walker(), tok, chat_parser=get_parser("qwen"), eos_ids=[2])
    with serve_worker(local, "127.0.0.1:0", token="t") as srv:
        remote = RemoteWorker(srv.address, token="t")
        remote.start()
        eng = DistributedRLEngine([remote], {Role.ACTOR: _Trainer({})})
        item = {"prompt_id": "lake", "task": task, "agent": "frozenlake", "env": "frozenlake", "max_turns": 8, "max_response_length": 4096}
        (resp,) = asyncio.run(eng.generate([item], GenerationArgs(max_tokens=32, temperature=1.0)))
        md = resp.metadata
        assert md["is_valid"] and md["status"] == "SUCCEEDED" and md["trajectory_reward"] == 1.0 and md["num_turns"] == len(path)
        masks = np.asarray(md["conversation_masks"])
        assert len(masks) == len(resp.tokens) == len(resp.logprobs) and 0 < masks.sum() < len(masks)
        assert md["raw_length"] == len(resp.tokens) and md["clipped"] is False and len(md["prompt_token_ids"]) > 0
        assert md["lineage"].events[0].component == "engine.dispatch"
        asyncio.run(eng.close())
        remote.stop()


def test_factory_built_episode_worker_plays_and_takes_weights():
    from tunix_b200.experimental.worker.factories import export_state, make_agentic_rollout_worker
    w = make_agentic_rollout_worker("episodes-f", device="cpu", cache_size=1024, max_new_tokens=8)
    w.start()
    try:
        eng = DistributedRLEngine([w], {Role.ACTOR: _Trainer({})})
        item = {"prompt_id": "lake", "task": {"seed": 1, "size": 4, "p": 0.8, "max_steps": 2}, "max_turns": 2, "max_response_length": 24}
        out = asyncio.run(eng.generate([item, dict(item, prompt_id="lake2")], GenerationArgs(max_tokens=8, temperature=1.0)))
        assert len(out) == 2 and all(r.metadata["status"] in ("SUCCEEDED", "MAX_STEPS_REACHED", "MAX_CONTEXT_LIMIT_REACHED") for r in out)
        assert all(0 < sum(r.metadata["conversation_masks"]) <= 24 + 8 for r in out)
        before = torch.cat([p.detach().reshape(-1).clone() for p in w.model.parameters()])
        state = export_state(w.model)
        name = next(iter(state))
        kind, arr = state[name]
        state[name] = (kind, arr * 0)
        w.sync_weights(5, state)
        after = torch.cat([p.detach().reshape(-1) for p in w.model.parameters()])
        assert w.policy_version == 5 and not torch.equal(before, after)
        asyncio.run(eng.close())
    finally:
        w.stop()


def test_program_validation_reports_everything_at_once():
    from tunix_b200.experimental.orchestrator.startup_validation import StartupValidationError, validate_program
    eng = DistributedRLEngine([], {Role.CRITIC: _Trainer({})})
    prog = StandardRLProgram(GRPOAdapter(reward_fn=doubles.token_sum_reward), None, 1, num_generations=4, batch_size=2,
                             batch_config=BatchConfig(rows_per_microbatch=2, max_packed_len=16), generation_args=GenerationArgs(max_tokens=64),
                             max_staleness=1, sync_weights=False, reference_kl=True)
    with pytest.raises(StartupValidationError) as ei:
        validate_program(prog, eng)
    text = str(ei.value)
    for part in ("no rollout worker", "no trainer worker for the actor", "no worker serves the reference role", "cannot fit a packed row",
                 "sync_weights is off", "no dataset"):
        assert part in text, part
    assert len(ei.value.errors) == 6
    good = DistributedRLEngine([_EchoRollout("r0")], {Role.ACTOR: _Trainer({})})
    hist = _program(_prompts(2), 1, sync_weights=False, checkpoint_every=0).run(good, validate=True)
    assert len(hist) == 1
    with pytest.raises(StartupValidationError):
        _program(None, 1).run(good, validate=True)
    asyncio.run(good.close()); asyncio.run(eng.close())


def test_engine_rotation_follows_the_health_monitor():
    from tunix_b200.experimental.common.datatypes import HealthReport, WorkerState
    from tunix_b200.experimental.orchestrator.health_monitor import HealthMonitor
    now = [100.0]
    mon = HealthMonitor(heartbeat_timeout_s=5.0, clock=lambda: now[0])
    a, b = _EchoRollout("a"), _EchoRollout("b")
    eng = DistributedRLEngine([a, b], {Role.ACTOR: _Trainer({})})
    for w in ("a", "b"):
        mon.observe(HealthReport(w, WorkerState.READY, timestamp=now[0]))
    stop = eng.follow_health(mon, period_s=0.02)
    try:
        now[0] += 10.0                                         # both silent ...
        mon.observe(HealthReport("a", WorkerState.READY, timestamp=now[0]))        # ... then only "a" reports again
        deadline = time.monotonic() + 3
        while eng.rollout_pool.live() != ["a"] and time.monotonic() < deadline:
            time.sleep(0.02)
        assert eng.rollout_pool.live() == ["a"]
        out = asyncio.run(eng.generate(_prompts(4), GenerationArgs(max_tokens=2)))
        assert len(out) == 4 and b.seen == []                  # nothing was sent to the silent worker
        mon.observe(HealthReport("b", WorkerState.READY, timestamp=now[0]))
        deadline = time.monotonic() + 3
        while eng.rollout_pool.live() != ["a", "b"] and time.monotonic() < deadline:
            time.sleep(0.02)
        assert eng.rollout_pool.live() == ["a", "b"]
    finally:
        stop.set()
        asyncio.run(eng.close())


def test_program_writes_a_json_line_per_consumed_rollout(tmp_path):
    import json
    eng = DistributedRLEngine([_EchoRollout("r0")], {Role.ACTOR: _Trainer({})})
    prog = _program(_prompts(2), 1, trajectory_log_dir=str(tmp_path / "traj"), sync_weights=False, checkpoint_every=0)
    hist = prog.run(eng)
    prog.close()
    files = [f for f in os.listdir(tmp_path / "traj") if f.endswith(".jsonl")]
    rows = [json.loads(line) for f in files for line in open(tmp_path / "traj" / f)]
    assert len(rows) == hist[0]["num_rollouts"] == 8 and {r["prompt_id"] for r in rows} == {"p0", "p1"}
    assert all(len(r["tokens"]) == 4 and r["step"] == 0 and r["request_id"].startswith("req_p") for r in rows)
    asyncio.run(eng.close())


def test_eval_mode_scores_without_training():
    class Logger:
        def __init__(self):
            self.rows = []

        def log(self, prefix, name, value, mode, step):
            self.rows.append((prefix, name, str(mode), step))
    tr, r = _Trainer({"latest": {"step": 3, "global_step": 3}}), _EchoRollout("r0")
    eng = DistributedRLEngine([r], {Role.ACTOR: tr})
    lg = Logger()
    hist = _program(_prompts(4), None, mode="eval", metrics_logger=lg).run(eng)
    assert [h["step"] for h in hist] == [0, 1] and all(h["num_rollouts"] == 8 and h["num_microbatches"] == 0 and h["loss"] is None for h in hist)
    assert tr.ops == [] and r.synced == [] and "global_step" in tr.disk["latest"]          # no restore, no training, no sync, no save
    assert {m for _, _, m, _ in lg.rows} == {"eval"} and ("rewards", "mean", "eval", 1) in lg.rows
    asyncio.run(eng.close())
    with pytest.raises(ValueError, match="mode must be"):
        _program(_prompts(1), 1, mode="test")
