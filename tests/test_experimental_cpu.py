"""Control-plane pieces: worker lifecycle, health monitor, weight-sync rounds, KV page manager, trajectory store,
grouped queue, rank watchdog. All host-side; failures are scripted."""
import os
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_worker_lifecycle_and_health_monitor():
    from tunix_b200.experimental.common.datatypes import IllegalTransition, WorkerState, check_transition
    from tunix_b200.experimental.orchestrator.health_monitor import HealthMonitor
    from tunix_b200.experimental.worker.mock_worker import MockWorker
    now = [0.0]
    mon = HealthMonitor(heartbeat_timeout_s=5, state_deadlines={WorkerState.SYNCING: 10}, clock=lambda: now[0])
    w = MockWorker("w0", handler=lambda r: r * 2, needs_compile=True, on_report=mon.observe)
    w.start()
    assert w.state == WorkerState.READY and w.submit(21) == 42 and w.state == WorkerState.READY
    w.sync_weights(3)
    assert w.policy_version == 3 and mon.healthy_workers() == ["w0"]
    now[0] = 6.0
    assert [u.reason for u in mon.check()] == ["heartbeat"]
    bad = MockWorker("w1", fail_on_sync=True, on_report=mon.observe)
    bad.start()
    with pytest.raises(RuntimeError):
        bad.sync_weights(1)
    assert bad.state == WorkerState.FAILED and any(u.worker_id == "w1" and u.reason == "failed" for u in mon.check())
    with pytest.raises(RuntimeError):
        bad.submit(1)
    with pytest.raises(IllegalTransition):
        check_transition(WorkerState.STOPPED, WorkerState.READY)
    w.stop()
    assert w.state == WorkerState.STOPPED


def test_weight_sync_rounds_abort_and_poison():
    from tunix_b200.experimental.weight_sync.weight_sync_coordinator import RoundState, WeightSyncCoordinator, WeightSyncError

    class P:
        def __init__(self, wid, fail=None):
            self.worker_id, self.fail, self.version, self.staged, self.log = wid, fail, 0, None, []

        def _do(self, phase):
            self.log.append(phase)
            if self.fail == phase:
                raise RuntimeError(f"{self.worker_id} fails in {phase}")

        def prepare(self, v):
            self._do("prepare")
            self.staged = v

        def transfer(self, v):
            self._do("transfer")

        def commit(self, v):
            self._do("commit")
            self.version, self.staged = v, None

        def rollback(self):
            self.log.append("rollback")
            self.staged = None
    a, b = P("a"), P("b")
    c = WeightSyncCoordinator([a, b])
    assert c.run_round(1) == RoundState.COMMITTED and (a.version, b.version) == (1, 1)
    b.fail = "transfer"
    assert c.run_round(2) == RoundState.ABORTED and a.version == 1 and "rollback" in a.log and a.staged is None
    b.fail = "commit"
    assert c.run_round(3) == RoundState.UNKNOWN_TRANSFER_STATE and a.version == 3 and b.version == 1
    with pytest.raises(WeightSyncError):
        c.run_round(4)
    b.fail = None
    c.reset_after_unknown(1)
    assert c.run_round(4) == RoundState.COMMITTED


def test_kv_cache_manager_prefix_hits_lru_and_window():
    from tunix_b200.experimental.generate.kv_cache_manager import KVCacheManager, PagePool, PagePoolError
    pool = PagePool(6)
    m = KVCacheManager(pool, page_size=4)
    toks = list(range(10))
    pages, cached = m.allocate_for_request("r1", toks)
    assert cached == 0 and len(pages) == 3 and pool.num_free == 3
    m.cache_full_pages("r1", toks, 10)                              # two full pages get hashed
    pages2, cached2 = m.allocate_for_request("r2", toks + [99, 98])
    assert cached2 == 8 and pages2[0] is pages[0] and pages2[1] is pages[1] and pool.num_free == 2
    m.free_request("r1")
    assert pool.num_free == 3                                       # r1's unhashed tail page is freed, shared ones stay
    m.free_request("r2")
    assert pool.num_free == 4 and len(m._lru) == 2                  # hashed pages stay cached, unreferenced
    hit = m.find_longest_cache_hit(toks)
    assert len(hit) == 2
    m.allocate_for_request("r3", list(range(100, 124)))             # needs all 6 pages: evicts the cached ones
    assert pool.num_free == 0 and m.find_longest_cache_hit(toks) == []
    with pytest.raises(PagePoolError):
        m.allocate_for_request("r4", [1] * 4)
    with pytest.raises(PagePoolError):
        pool.free([0, 0][0:1] * 2 if False else [17])
    m.free_request("r3")
    sw = KVCacheManager(PagePool(8), page_size=4, window_size=6)
    assert sw.pages_in_window == 3
    sw.allocate_for_request("s", list(range(20)))
    assert sw.release_out_of_window("s", 20) == 3 and sw.page_table("s", 6)[:3] == [-1, -1, -1]


def test_trajectory_store_and_queue(tmp_path):
    from tunix_b200.experimental.queue_manager.trajectory_queue_manager import TrajectoryQueueManager
    from tunix_b200.experimental.trajectory.store import FileTrajectoryStore, InMemoryTrajectoryStore, new_record
    mem = InMemoryTrajectoryStore(capacity=2)
    ids = [mem.put(new_record([{"a": i}], reward=i, group_id="g", policy_version=i)) for i in range(3)]
    assert len(mem) == 2 and [r["reward"] for r in mem.query(min_policy_version=2)] == [2.0]
    with pytest.raises(KeyError):
        mem.get(ids[0])
    fs = FileTrajectoryStore(str(tmp_path / "t" / "traj.jsonl"))
    fs.put(new_record([{"tokens": torch.arange(3)}], reward=1.5))
    fs.close()
    assert [r["steps"][0]["tokens"] for r in fs.read()] == [[0, 1, 2]]
    q = TrajectoryQueueManager(group_size=2, max_staleness=1)
    q.put("a", 1, 0)
    q.put("b", 10, 5)
    q.put("a", 2, 0)
    q.put("b", 11, 5)
    q.set_policy_version(5)
    gid, items = q.get(timeout=1)
    assert gid == "b" and items == [10, 11] and q.dropped_stale == 1 and q.num_inflight == 1
    q.nack("b")
    assert q.get(timeout=1)[0] == "b"
    q.ack("b")
    assert q.get(timeout=0.05) is None
    oq = TrajectoryQueueManager(group_size=1, ordered=True)
    oq.put("x", 1)
    assert oq.get(timeout=1) == ("x", [1])


def _wd_rank(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200.parallel.watchdog import RankFailure, Watchdog
    wd = Watchdog(interval_s=0.1, timeout_s=0.6).start()
    dist.barrier()
    time.sleep(0.3)
    wd.check()                                   # everyone alive
    if rank == 1:
        wd.pause()                               # plays a rank that hung between steps
        time.sleep(2.5)
    else:
        seen = None
        t0 = time.time()
        while time.time() - t0 < 2.0 and seen is None:
            try:
                wd.check()
            except RankFailure as e:
                seen = e.ranks
            time.sleep(0.1)
        torch.save(seen, out)
        time.sleep(0.6)
    wd.stop()
    dist.destroy_process_group()


def test_watchdog_names_the_silent_rank(tmp_path):
    out = str(tmp_path / "seen.pt")
    mp.spawn(_wd_rank, args=(2, 29749, out), nprocs=2, join=True)
    assert torch.load(out) == [1]


def test_traffic_controller_gates_tasks_around_weight_sync():
    import asyncio
    from tunix_b200.experimental.common.datatypes import WorkerState
    from tunix_b200.experimental.worker.traffic_controller import TrafficController

    async def run():
        tc = TrafficController()
        gate = asyncio.Event()

        async def work():
            await gate.wait()
            return 1
        t1 = asyncio.ensure_future(work())
        assert tc.try_admit(t1) and tc.active_tasks() == [t1]
        tc.close_for_sync()
        assert tc.state == WorkerState.SYNCING and not tc.is_admission_open()
        t2 = asyncio.ensure_future(work())
        assert not tc.try_admit(t2)                  # rejected and cancelled
        waiter = asyncio.ensure_future(tc.wait_for_admission())
        await asyncio.sleep(0)
        assert t2.cancelled() or t2.cancelling() and not waiter.done()
        assert not await tc.drain(timeout_s=0.01)    # t1 still runs
        gate.set()
        assert await tc.drain(timeout_s=1.0) and t1.result() == 1
        assert tc.reopen()
        await asyncio.wait_for(waiter, 1.0)
        t3 = asyncio.ensure_future(asyncio.sleep(10))
        assert tc.try_admit(t3)
        assert tc.stop() == [t3]
        await asyncio.sleep(0)
        assert t3.cancelled() and tc.state == WorkerState.STOPPED and not tc.reopen()
        import pytest
        with pytest.raises(RuntimeError):
            tc.close_for_sync()
    asyncio.run(run())


def test_worker_registry_lineage_and_dispatch_window():
    import asyncio
    import numpy as np
    import pytest
    from tunix_b200.experimental.common.dispatch_window import DispatchWindow
    from tunix_b200.experimental.common.lineage import LineageContext, map_in_chunks
    from tunix_b200.experimental.orchestrator.worker_registry import WorkerInfo, WorkerRegistry

    class W:
        def __init__(self, wid, roles):
            self._i = WorkerInfo(wid, tuple(roles))

        def info(self):
            return self._i
    reg = WorkerRegistry()
    a, b, c = W("r1", ["rollout"]), W("r0", ["rollout", "inference"]), W("t0", ["trainer"])
    for w in (a, b, c):
        reg.register(w)
    assert [w.info().worker_id for w in reg.group("rollout")] == ["r0", "r1"] and len(reg.group("critic")) == 0
    assert reg.roles() == {"rollout", "inference", "trainer"} and "t0" in reg and len(reg) == 3
    with pytest.raises(ValueError):
        reg.register(W("r1", ["rollout"]))
    with pytest.raises(ValueError):
        reg.register(W("x", []))
    reg.register(W("r1", ["inference"]), override=True)
    assert [w.info().worker_id for w in reg.group("rollout")] == ["r0"]
    reg.unregister("t0")
    assert reg.worker_ids() == ["r0", "r1"]

    t0, t1 = LineageContext(tracking_id="traj_0"), LineageContext(tracking_id="traj_1")
    t0.add_event("worker.rollout", "generate", {"tokens": 5})
    batch = LineageContext.merge("batch_0", [t0, None, t1, t0], "orchestrator.assembler", "pack", {"rows": 2})
    assert batch.parent_tracking_ids == ["traj_0", "traj_1"] and batch.events[0].operation == "pack"
    out = map_in_chunks(lambda x, y: x.sum(-1) + y, 2, np.arange(10).reshape(5, 2), np.ones(5))
    assert out.tolist() == [2, 6, 10, 14, 18]

    async def run():
        consumed = [0]
        win = DispatchWindow(1, lambda: consumed[0], full_batch_size=2, out_of_order_resume=True)
        await asyncio.wait_for(win.wait_for(1), 0.1)             # within next_batch + staleness
        parked = asyncio.ensure_future(win.wait_for(2))
        await asyncio.sleep(0.01)
        assert not parked.done()
        consumed[0] = 1
        win.release()
        await asyncio.wait_for(parked, 0.5)
        # two filtered groups (= one full batch) move the window by one
        win.on_group_filtered([{"prompt_id": "p7"}])
        assert win.next_batch == 2
        win.on_group_filtered([{"prompt_id": "p9"}])
        assert win.next_batch == 2 and win.skipped_prompt_ids == {"p7", "p9"}
        win.record_committed_groups([[{"prompt_id": "p1"}], [{"prompt_id": "p2"}]])
        meta = win.checkpoint_metadata(pending_groups=[[{"prompt_id": "p3"}]])
        assert meta == {"committed_prompt_ids": ["p1", "p2", "p3"], "skipped_prompt_ids": ["p7", "p9"]}
        fresh = DispatchWindow(1, lambda: 0, full_batch_size=2, out_of_order_resume=True)
        assert fresh.dataset_skip_count == 0 and fresh.admit({"prompt_id": "p1"})
        assert fresh.restore_checkpoint_metadata(meta) and fresh.uses_prompt_id_resume
        assert not fresh.admit({"prompt_id": "p1"}) and not fresh.admit({"prompt_id": "p9"}) and fresh.admit({"prompt_id": "p4"})
    asyncio.run(run())


def test_workers_and_split_step_trainer():
    import numpy as np
    import torch
    from tests.test_sampler_cpu import CharTok
    from tunix_b200 import optim
    from tunix_b200.common.configs import CacheConfig, TrainingConfig
    from tunix_b200.experimental.common.datatypes import RolloutRequest, WorkerState
    from tunix_b200.experimental.common.lineage import LineageContext
    from tunix_b200.experimental.orchestrator.worker_registry import WorkerRegistry
    from tunix_b200.experimental.train.peft_trainer_v2 import TrainerV2
    from tunix_b200.experimental.worker.rollout_worker import InferenceWorker, RolloutWorker, TrainerWorker
    from tunix_b200.generate.sampler import Sampler
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.sft.peft_trainer import PeftTrainer
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16,
                                           num_kv_heads=1)
    model = create_model(cfg, seed=0)
    sampler = Sampler(model, CharTok(), CacheConfig(64, 1, 1, 16))
    synced = []
    rw = RolloutWorker("rollout-0", sampler, apply_weights=lambda v, p: synced.append((v, p)), eos_tokens=[2])
    trainer = PeftTrainer(model, optim.AdamW(1e-2), TrainingConfig(eval_every_n_steps=10 ** 9, pbar_description=None,
                                                                   resume_from_checkpoint_on_init=False))
    tw = TrainerWorker("trainer-0", TrainerV2(trainer))
    iw = InferenceWorker("ref-0", {"sum": lambda x: np.asarray(x).sum(-1)})
    reg = WorkerRegistry()
    for w in (rw, tw, iw):
        w.start()
        reg.register(w)
    assert [w.worker_id for w in reg.group("rollout")] == ["rollout-0"] and rw.state == WorkerState.READY
    lin = LineageContext(tracking_id="traj_0")
    resp = rw.submit(RolloutRequest("q0", [1, 5, 6, 7], group_id="g", max_tokens=6, temperature=0.0, metadata={"lineage": lin}))
    assert resp.request_id == "q0" and 1 <= len(resp.tokens) <= 6 and len(resp.logprobs) == len(resp.tokens)
    assert resp.finish_reason in ("stop", "length") and lin.events[0].component == "worker.rollout"
    rw.sync_weights(3, {"w": 1})
    assert synced == [(3, {"w": 1})] and rw.policy_version == 3 and rw.state == WorkerState.READY
    assert iw.submit({"op": "sum", "x": [[1, 2], [3, 4]]}).tolist() == [3, 7]
    # split-step training: three micro-batches of different sizes, one optimizer step
    before = torch.cat([p.detach().reshape(-1).clone() for p in model.parameters()])
    losses = []
    for n in (2, 1, 3):
        toks = torch.randint(3, 60, (n, 12))
        r = tw.submit({"op": "fwd_bwd", "batch": {"input_tokens": toks, "input_mask": torch.ones(n, 12)}})
        losses.append(r["loss"])
    assert r["pending_microbatches"] == 3 and all(np.isfinite(losses))
    up = tw.submit({"op": "update"})
    assert up["step"] == 1 and up["microbatches"] == 3 and tw.policy_version == 1
    after = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    assert not torch.equal(before, after)
    ev = tw.submit({"op": "eval_step", "batch": {"input_tokens": toks, "input_mask": torch.ones(3, 12)}})
    assert np.isfinite(ev["loss"])
    logits = tw.submit({"op": "fwd_only", "batch": {"input_tokens": toks, "input_mask": torch.ones(3, 12)}})
    assert logits.shape == (3, 12, 64)
    import pytest
    with pytest.raises(RuntimeError):
        tw.trainer.update()
    for w in (rw, tw, iw):
        w.stop()
        assert w.state == WorkerState.STOPPED


def test_rollout_manager_streams_episodes_and_syncs_between_them():
    import asyncio
    import time
    from tunix_b200.experimental.rollout.manager import RolloutManager
    from tunix_b200.experimental.worker.traffic_controller import AdmissionClosedError
    weights = {"v": 0}

    def generate(prompt, max_tokens):              # a blocking engine: echoes the weight version it ran with
        time.sleep(0.01 * len(prompt))
        return [weights["v"]] * (max_tokens or 1), [0.0] * (max_tokens or 1)

    async def episode(model_call, item):
        turns = []
        for _ in range(item["turns"]):
            out = await model_call(item["prompt"], 2)
            turns.append((out["tokens"][0], out["policy_version"]))
        if item.get("boom"):
            raise ValueError("environment failed")
        return turns

    async def run():
        mgr = RolloutManager(generate, episode, max_concurrency=2,
                             apply_weights=lambda v, p: weights.__setitem__("v", v), partial_rollout=False)
        items = [{"prompt": [1] * n, "turns": 1} for n in (5, 1, 3)] + [{"prompt": [1], "turns": 1, "boom": True}]
        got = [o async for o in mgr.as_completed(items)]
        assert len(got) == 4 and sum(o["error"] is not None for o in got) == 1
        assert [len(o["item"]["prompt"]) for o in got if o["error"] is None][0] == 1        # shortest finishes first
        # a sync round with an episode in flight: it drains first, new episodes are refused meanwhile
        mgr.start_episode({"prompt": [1] * 4, "turns": 2})
        await asyncio.sleep(0.005)
        pre = asyncio.ensure_future(mgr.pre_weight_sync())
        await asyncio.sleep(0.005)
        import pytest
        with pytest.raises(AdmissionClosedError):
            mgr.start_episode({"prompt": [1], "turns": 1})
        info = await pre
        assert info["in_flight_before"] == 1 and info["in_flight_after"] == 0 and info["drained"]
        assert (await mgr.pop_next_completed())["result"] == [(0, 0), (0, 0)]
        await mgr.weight_sync(7, None)
        assert await mgr.post_weight_sync() and mgr.policy_version == 7
        out = [o async for o in mgr.as_completed([{"prompt": [1], "turns": 1}])]
        assert out[0]["result"] == [(7, 7)]
        assert mgr.stats["episodes"] == 5 and mgr.stats["failed"] == 1
        # partial rollouts: the episode in flight is not drained; its next request waits for the new weights
        part = RolloutManager(generate, episode, max_concurrency=2,
                              apply_weights=lambda v, p: weights.__setitem__("v", v), partial_rollout=True)
        part.policy_version = 7
        part.start_episode({"prompt": [1] * 3, "turns": 2})
        await asyncio.sleep(0.005)
        info = await part.pre_weight_sync()
        assert info["in_flight_after"] == 1
        await asyncio.sleep(0.06)                    # first turn done, second one parked at the gate
        await part.weight_sync(8, None)
        await part.post_weight_sync()
        assert (await part.pop_next_completed())["result"] == [(7, 7), (8, 8)]
    asyncio.run(run())


def test_batch_assemblers_pad_and_pack():
    import numpy as np
    from tunix_b200.experimental.common.datatypes import RLTrainerPayload
    from tunix_b200.experimental.common.lineage import LineageContext
    from tunix_b200.experimental.orchestrator.batch_assembly import (BatchConfig, PaddingStats, create_batch_assembler,
                                                                    summarize_padding_stats)
    rng = np.random.default_rng(0)

    def traj(i, p, c):
        return RLTrainerPayload({"prompt_ids": rng.integers(3, 50, p), "completion_ids": rng.integers(3, 50, c),
                                 "old_per_token_logps": -np.ones(c, np.float32), "lineage": LineageContext(tracking_id=f"traj_{i}")},
                                policy_version=2, group_id=f"g{i // 2}", reward=float(i))
    items = [traj(i, p, c) for i, (p, c) in enumerate([(4, 6), (8, 3), (2, 9), (5, 5), (3, 2)])]
    pad = create_batch_assembler(BatchConfig(rows_per_microbatch=2, max_prompt_length=8, max_response_length=8), packed=False)
    out = list(pad.feed(items))
    assert [b.batch_id for b in out] == ["batch_0", "batch_1"] and out[0].arrays["input_tokens"].shape == (2, 16)
    b0 = out[0]
    assert b0.arrays["prompt_mask"][0].tolist() == [0] * 4 + [1] * 4 + [0] * 8          # left-padded prompt
    assert b0.arrays["completion_mask"][0].tolist() == [0] * 8 + [1] * 6 + [0] * 2      # right-padded completion
    assert b0.arrays["advantages"][1, 8:11].tolist() == [1.0] * 3 and b0.arrays["old_per_token_logps"][0, 8] == -1
    assert b0.stats.row_valid_tokens.tolist() == [10, 11] and b0.lineage.parent_tracking_ids == ["traj_0", "traj_1"]
    tail = list(pad.flush())
    assert len(tail) == 1 and tail[0].num_trajectories == 1 and tail[0].stats.row_num_sequences.tolist() == [1, 0]
    # packing: all five fit two rows of 24 tokens
    pk = create_batch_assembler(BatchConfig(rows_per_microbatch=2, max_packed_len=24), packed=True)
    assert list(pk.feed(items[:2])) == []                       # 21 tokens: below a full micro-batch, keeps buffering
    got = list(pk.feed(items[2:])) + list(pk.flush())
    assert sum(b.num_trajectories for b in got) == 5
    b = got[0]
    seg = b.arrays["segment_ids"]
    assert seg.shape == (2, 24) and b.stats.valid_tokens == int((seg > 0).sum()) and b.stats.row_capacity == 24
    row0 = b.arrays["positions"][0][seg[0] == 1]
    assert row0.tolist() == list(range(len(row0)))              # positions restart per segment
    assert set(b.lineage.parent_tracking_ids) <= {f"traj_{i}" for i in range(5)}
    summary = summarize_padding_stats([x.stats for x in got])
    assert summary["valid_tokens"] == 47 and summary["sequences"] == 5 and 0 <= summary["padding_ratio"] < 1
    import pytest
    with pytest.raises(ValueError):
        PaddingStats(row_valid_tokens=np.asarray([30]), row_num_sequences=np.asarray([1]), row_capacity=24)


def test_orchestrator_end_to_end_with_worker_failover():
    """Prompts -> rollout workers -> group advantages -> packed micro-batches -> split-step trainer -> weight sync, on
    a tiny CPU model; one of two rollout workers dies mid-run and the other takes over."""
    import numpy as np
    import torch
    from tests.test_sampler_cpu import CharTok
    from tunix_b200 import optim
    from tunix_b200.common.configs import CacheConfig, TrainingConfig
    from tunix_b200.experimental.common.datatypes import WorkerState
    from tunix_b200.experimental.common.dispatch_window import DispatchWindow
    from tunix_b200.experimental.orchestrator.batch_assembly import BatchConfig, create_batch_assembler
    from tunix_b200.experimental.orchestrator.orchestrator import AlgorithmAdapter, Orchestrator
    from tunix_b200.experimental.orchestrator.worker_registry import WorkerRegistry
    from tunix_b200.experimental.train.peft_trainer_v2 import TrainerV2
    from tunix_b200.experimental.worker.rollout_worker import RolloutWorker, TrainerWorker
    from tunix_b200.generate.sampler import Sampler
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.sft.peft_trainer import PeftTrainer
    from tunix_b200.sft.utils import LossOutput, WeightedMetric
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16,
                                           num_kv_heads=1)
    model = create_model(cfg, seed=0)
    cc = CacheConfig(64, 1, 1, 16)

    def pg_loss(model, input_tokens, completion_mask, advantages, segment_ids=None, positions=None, **_):
        hidden, _ = model(input_tokens[:, :-1], positions=None if positions is None else positions[:, :-1],
                          segment_ids=None if segment_ids is None else segment_ids[:, :-1], skip_lm_head=True)
        lp = model.token_logprobs(hidden.reshape(-1, hidden.shape[-1]), input_tokens[:, 1:].reshape(-1).long())[0]
        lp = lp.view(input_tokens.shape[0], -1)
        m = completion_mask[:, 1:]
        loss_sum = -(lp * advantages[:, 1:] * m).sum()
        return LossOutput(loss=WeightedMetric(loss_sum, m.sum()))

    def to_inputs(batch):
        out = {k: torch.as_tensor(v) for k, v in batch.items()}
        out["input_tokens"] = out["input_tokens"].long()
        return out
    trainer = PeftTrainer(model, optim.AdamW(5e-3), TrainingConfig(eval_every_n_steps=10 ** 9, pbar_description=None,
                                                                   resume_from_checkpoint_on_init=False))
    trainer.with_loss_fn(pg_loss).with_gen_model_input_fn(to_inputs)

    class Flaky:
        """A sampler that breaks after a number of calls (a host-side stand-in for a lost rollout worker)."""
        def __init__(self, inner, die_after):
            self.inner, self.left = inner, die_after

        def __call__(self, **kw):
            self.left -= 1
            if self.left < 0:
                raise ConnectionError("rollout worker lost")
            return self.inner(**kw)
    synced = []
    reg = WorkerRegistry()
    workers = [RolloutWorker("rollout-0", Flaky(Sampler(model, CharTok(), cc), die_after=5), eos_tokens=[2],
                             apply_weights=lambda v, p: synced.append(("rollout-0", v))),
               RolloutWorker("rollout-1", Sampler(model, CharTok(), cc), eos_tokens=[2],
                             apply_weights=lambda v, p: synced.append(("rollout-1", v))),
               TrainerWorker("trainer-0", TrainerV2(trainer))]
    for w in workers:
        w.start()
        reg.register(w)
    consumed = [0]
    window = DispatchWindow(0, lambda: consumed[0], full_batch_size=2, out_of_order_resume=True)
    orch = Orchestrator(reg, create_batch_assembler(BatchConfig(rows_per_microbatch=2, max_packed_len=48), packed=True),
                        AlgorithmAdapter(reward_fn=lambda item, r: float(sum(t % 5 for t in r.tokens)), drop_uniform_groups=True),
                        group_size=4, window=window, rollout_params={"max_tokens": 6, "temperature": 1.0, "seed": None},
                        export_weights=lambda: {"version_of": "actor"})
    before = torch.cat([p.detach().reshape(-1).clone() for p in model.parameters()])
    rng = np.random.default_rng(0)
    batches = [[{"prompt_id": f"p{s}_{i}", "prompt_ids": [1] + rng.integers(3, 60, 4).tolist()} for i in range(2)] for s in range(3)]
    for s, b in enumerate(batches):
        rec = orch.step(s, b)
        consumed[0] += 1
        assert rec["trajectories"] + 4 * rec["filtered_groups"] == 8
    hist = orch.history
    assert [h["policy_version"] for h in hist] == [1, 2, 3] and hist[-1]["train_step"] == 3
    assert all(np.isfinite(h["loss"]) and 0 <= h["padding_ratio"] < 1 for h in hist)
    after = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    assert not torch.equal(before, after)
    # rollout-0 died during the first step: marked FAILED, excluded, and only rollout-1 keeps receiving weights
    assert workers[0].state == WorkerState.FAILED and orch.excluded == {"rollout-0"}
    assert [s for s in synced if s[0] == "rollout-1"] == [("rollout-1", 1), ("rollout-1", 2), ("rollout-1", 3)]
    assert window.committed_prompt_ids | window.skipped_prompt_ids == {f"p{s}_{i}" for s in range(3) for i in range(2)}
    assert workers[1].served >= 19
    orch.close()


def test_remote_worker_over_grpc_loopback():
    """A worker served on 127.0.0.1 behaves like the local object: requests, weight sync with a payload larger
    than one chunk, remote exceptions, the token check, and registration in the worker registry."""
    import numpy as np
    import pytest
    pytest.importorskip("grpc")
    from tunix_b200.experimental.common.datatypes import RolloutRequest, WorkerState
    from tunix_b200.experimental.orchestrator.worker_registry import WorkerRegistry
    from tunix_b200.experimental.worker.remote_execution import RemoteError, RemoteWorker, serve_worker
    from tunix_b200.experimental.worker.rollout_worker import RolloutWorker

    class Out:
        def __init__(self, toks):
            self.tokens, self.logprobs, self.text = [toks], [[-0.5] * len(toks)], ["x"]
    seen = {}

    def engine(prompt_token_ids, max_generation_steps, **kw):
        if prompt_token_ids[0][0] == 99:
            raise ValueError("bad prompt")
        return Out([t + 1 for t in prompt_token_ids[0]][:max_generation_steps])
    local = RolloutWorker("rollout-7", engine, apply_weights=lambda v, p: seen.update(version=v, nbytes=p["w"].nbytes), eos_tokens=[2])
    with serve_worker(local, "127.0.0.1:0", token="s3cret") as srv:
        remote = RemoteWorker(srv.address, token="s3cret")
        remote.start()
        assert remote.state == WorkerState.READY and remote.worker_id == "rollout-7" and remote.info().roles == ("rollout",)
        resp = remote.submit(RolloutRequest("q", [5, 6, 7], max_tokens=2))
        assert resp.tokens == [6, 7] and resp.request_id == "q" and local.served == 1
        big = {"w": np.zeros(3 << 20, np.float32)}                    # 12 MB: goes over the chunked call
        remote.sync_weights(4, big)
        assert seen == {"version": 4, "nbytes": 12 << 20} and remote.policy_version == 4
        reg = WorkerRegistry()
        reg.register(remote)
        assert [w.worker_id for w in reg.group("rollout")] == ["rollout-7"]
        with pytest.raises(RemoteError) as ei:
            remote.submit(RolloutRequest("bad", [99], max_tokens=1))
        assert isinstance(ei.value.__cause__, ValueError) and remote.state == WorkerState.FAILED
        with pytest.raises(RemoteError):
            remote._invoke("_fail", None)                                 # private names are not callable remotely
        intruder = RemoteWorker(srv.address, token="guess")
        with pytest.raises(RemoteError, match="token"):
            intruder.info()
        # a frame without a valid tag is refused before any of it is unpickled: this payload would set the flag
        import cloudpickle, grpc
        from tunix_b200.experimental.worker import remote_execution as rex

        class Boom:
            def __reduce__(self):
                return (seen.update, ({"pwned": True},))
        for frame in (cloudpickle.dumps(("guess", "info", (Boom(),), {})),            # an untagged pickle
                      rex._seal(cloudpickle.dumps(("info", (Boom(),), {})), "guess")):   # tagged under the wrong token
            with pytest.raises(grpc.RpcError) as rpc:
                intruder._call(frame, timeout=10)
            assert rpc.value.code() == grpc.StatusCode.UNAUTHENTICATED
        assert "pwned" not in seen
        remote.close()
        intruder.close()


def test_orchestrator_with_a_remote_rollout_worker():
    """The orchestrator drives a rollout worker through its gRPC endpoint exactly as it drives a local one."""
    import numpy as np
    import pytest
    pytest.importorskip("grpc")
    import torch
    from tests.test_sampler_cpu import CharTok
    from tunix_b200 import optim
    from tunix_b200.common.configs import CacheConfig, TrainingConfig
    from tunix_b200.experimental.orchestrator.batch_assembly import BatchConfig, create_batch_assembler
    from tunix_b200.experimental.orchestrator.orchestrator import AlgorithmAdapter, Orchestrator
    from tunix_b200.experimental.orchestrator.worker_registry import WorkerRegistry
    from tunix_b200.experimental.train.peft_trainer_v2 import TrainerV2
    from tunix_b200.experimental.worker.remote_execution import RemoteWorker, serve_worker
    from tunix_b200.experimental.worker.rollout_worker import RolloutWorker, TrainerWorker
    from tunix_b200.generate.sampler import Sampler
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.sft.peft_trainer import PeftTrainer
    from tunix_b200.sft.utils import LossOutput, WeightedMetric
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16,
                                           num_kv_heads=1)
    model = create_model(cfg, seed=0)

    def loss(model, input_tokens, completion_mask, advantages, **_):
        hidden, _ = model(input_tokens[:, :-1], skip_lm_head=True)
        lp = model.token_logprobs(hidden.reshape(-1, hidden.shape[-1]), input_tokens[:, 1:].reshape(-1).long())[0]
        m = completion_mask[:, 1:]
        return LossOutput(loss=WeightedMetric(-(lp.view(m.shape) * advantages[:, 1:] * m).sum(), m.sum()))
    trainer = PeftTrainer(model, optim.AdamW(5e-3), TrainingConfig(eval_every_n_steps=10 ** 9, pbar_description=None,
                                                                   resume_from_checkpoint_on_init=False))
    trainer.with_loss_fn(loss).with_gen_model_input_fn(
        lambda b: {k: (torch.as_tensor(v).long() if k == "input_tokens" else torch.as_tensor(v)) for k, v in b.items()})
    versions = []
    served = RolloutWorker("rollout-r", Sampler(model, CharTok(), CacheConfig(64, 1, 1, 16)), eos_tokens=[2],
                           apply_weights=lambda v, p: versions.append(v))
    with serve_worker(served) as srv:
        remote = RemoteWorker(srv.address)
        tw = TrainerWorker("trainer-0", TrainerV2(trainer))
        remote.start()
        tw.start()
        reg = WorkerRegistry()
        reg.register(remote)
        reg.register(tw)
        orch = Orchestrator(reg, create_batch_assembler(BatchConfig(rows_per_microbatch=2, max_prompt_length=8,
                                                                    max_response_length=8), packed=False),
                            AlgorithmAdapter(reward_fn=lambda item, r: float(sum(t % 5 for t in r.tokens))), group_size=4,
                            rollout_params={"max_tokens": 6, "temperature": 1.0})
        rng = np.random.default_rng(1)
        rec = orch.step(0, [{"prompt_id": f"p{i}", "prompt_ids": [1] + rng.integers(3, 60, 4).tolist()} for i in range(2)])
        assert rec["trajectories"] + 4 * rec["filtered_groups"] == 8 and rec["policy_version"] == (1 if rec["microbatches"] else 0)
        assert served.served == 8 and versions == ([1] if rec["microbatches"] else [])
        orch.close()
        remote.close()


def test_launcher_starts_worker_processes_and_discovers_them():
    """Two worker processes come up, announce themselves to the controller's directory, serve requests through
    their own gRPC endpoints and leave when the controller shuts down."""
    import pytest
    pytest.importorskip("grpc")
    from tunix_b200.experimental.common.datatypes import WorkerState
    from tunix_b200.experimental.orchestrator.worker_registry import WorkerRegistry
    from tunix_b200.experimental.runtime.launcher import Launcher
    lau = Launcher(token="t0k")
    try:
        factory = "tunix_b200.experimental.worker.mock_worker:make_echo_worker"
        procs = [lau.launch(factory, "rollout-0", scale=2), lau.launch(factory, "trainer-0", role="trainer", scale=3)]
        entries = lau.wait_for(["rollout-0", "trainer-0"], timeout=120)
        assert entries["trainer-0"]["roles"] == ("trainer",) and entries["rollout-0"]["address"].startswith("127.0.0.1:")
        workers = lau.workers()
        reg = WorkerRegistry()
        for w in workers.values():
            reg.register(w)
        assert [w.worker_id for w in reg.group("rollout")] == ["rollout-0"]
        assert workers["rollout-0"].submit(21) == 42 and workers["trainer-0"].submit(5) == 15
        assert workers["rollout-0"].state == WorkerState.READY
        workers["rollout-0"].sync_weights(3, None)
        assert workers["rollout-0"].policy_version == 3
    finally:
        lau.shutdown()
    assert all(p.poll() is not None for p in procs)


def test_sql_trajectory_store_converter_and_explorer(tmp_path):
    import io
    import numpy as np
    from tunix_b200.experimental.trajectory import explorer
    from tunix_b200.experimental.trajectory.store import (FileTrajectoryStore, SqliteTrajectoryStore, new_record,
                                                          record_from_trajectory)
    from tunix_b200.rl.agentic.agents.agent_types import Action, Step, Trajectory, TrajectoryStatus
    db = str(tmp_path / "runs" / "traj.db")
    st = SqliteTrajectoryStore(db)
    ids = st.put_many([new_record([{"model_response": f"answer {i}", "reward": i / 4}], reward=i / 4, group_id=f"g{i % 2}",
                                  policy_version=i // 2) for i in range(6)])
    assert len(st) == 6 and st.get(ids[3])["steps"][0]["model_response"] == "answer 3"
    assert [r["reward"] for r in st.query(group_id="g1")] == [0.25, 0.75, 1.25]
    assert [r["reward"] for r in st.query(min_policy_version=1, min_reward=0.6, max_reward=1.1)] == [0.75, 1.0]
    assert len(list(st.query(limit=2))) == 2 and next(st.query(newest_first=True, limit=1))["reward"] in (1.25,)
    assert [r["reward"] for r in st.query(predicate=lambda r: r["reward"] > 1.0)] == [1.25]
    stats = st.stats()
    assert stats[0]["count"] == 2 and abs(stats[2]["reward_mean"] - 1.125) < 1e-9 and stats[1]["steps_mean"] == 1.0
    with pytest.raises(KeyError):
        st.get("nope")
    # an agent trajectory with token arrays converts to a record that survives the JSON round trip
    traj = Trajectory(task={"question": "2+2"}, reward=1.0, status=TrajectoryStatus.SUCCEEDED, steps=[
        Step(model_response="<think>easy</think> 4", thought="easy", action=Action(action="4"), observation="2+2", reward=1.0,
             done=True, assistant_tokens=np.array([5, 6, 7]), assistant_masks=np.array([1, 1, 1]), logprobs=np.array([-0.1, -0.2, -0.3]))])
    traj.steps[0].chat_completions = [{"role": "user", "content": "2+2?"}]
    rec = record_from_trajectory(traj, group_id="g9", policy_version=3, env="math")
    worse = record_from_trajectory(traj, group_id="g9", policy_version=3)
    worse["reward"] = 0.25
    st.put(worse)
    tid = st.put(rec)
    back = st.get(tid)
    assert back["steps"][0]["assistant_tokens"] == [5, 6, 7] and back["steps"][0]["action"] == "4"
    assert back["metadata"]["status"] == "SUCCEEDED" and back["metadata"]["env"] == "math" and back["policy_version"] == 3
    st.close()
    # the explorer on the SQL store, then exported to JSON lines and explored again
    out = io.StringIO()
    assert explorer.main([db, "stats"], out) == 0 and out.getvalue().count("\n") == 5           # header + versions 0, 1, 2, 3
    sft = str(tmp_path / "sft.jsonl")                       # good conversations as chat rows for SFT (rejection sampling)
    assert explorer.main([db, "export-sft", sft, "--best-of-group"], io.StringIO()) == 0
    rows = [__import__("json").loads(l) for l in open(sft)]
    assert len(rows) == 1 and rows[0]["reward"] == 1.0 and rows[0]["trajectory_id"] == tid
    assert rows[0]["messages"] == [{"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "<think>easy</think> 4"}]
    assert explorer.main([db, "export-sft", sft, "--min-reward", "0.2"], io.StringIO()) == 0 and len(open(sft).readlines()) == 2
    out = io.StringIO()
    assert explorer.main([db, "list", "--min-reward", "1.0"], out) == 0
    assert out.getvalue().count("\n") == 3 and "answer 5" in out.getvalue()
    out = io.StringIO()
    assert explorer.main([db, "show", tid], out) == 0 and "model_response: <think>easy</think> 4" in out.getvalue()
    assert explorer.main([db, "show", "missing"], io.StringIO()) == 1
    jl = str(tmp_path / "copy.jsonl")
    assert explorer.main([db, "export", jl], io.StringIO()) == 0
    fs = FileTrajectoryStore(jl)
    assert len(list(fs.read())) == 8
    fs.close()
    out = io.StringIO()
    assert explorer.main([jl, "list", "--group", "g9"], out) == 0 and out.getvalue().count("\n") == 2
    out1, out2 = io.StringIO(), io.StringIO()
    explorer.main([jl, "stats"], out1), explorer.main([db, "stats"], out2)
    assert out1.getvalue() == out2.getvalue()


def test_routing_pool_sticky_keys_failover_and_round_robin():
    import subprocess
    import sys
    from concurrent.futures import ThreadPoolExecutor
    from tunix_b200.experimental.worker.routing import NoWorkerAvailable, RoutingPool, stable_route_hash

    class W:
        def __init__(self, name):
            self.name, self.fail, self.seen = name, False, []

        def submit(self, req):
            if self.fail:
                raise ConnectionError(self.name)
            self.seen.append(req.get("route_key"))
            return self.name

    ws = {f"w{i}": W(f"w{i}") for i in range(4)}
    pool = RoutingPool(ws)
    keys = [f"conv-{i}" for i in range(200)]
    first = {k: pool.submit({"route_key": k}) for k in keys}
    assert all(pool.submit({"route_key": k}) == first[k] for k in keys)                    # sticky
    assert min(sum(v == n for v in first.values()) for n in ws) >= 25                      # and spread (50 each expected)
    # the digest does not depend on the process (Python's hash() does)
    other = subprocess.run([sys.executable, "-c", "from tunix_b200.experimental.worker.routing import stable_route_hash as h;"
                            "print(h('conv-7', 'w1'))"], capture_output=True, text=True, check=True).stdout.strip()
    assert int(other) == stable_route_hash("conv-7", "w1")
    # a worker fails: its keys move, nobody else's do
    ws["w2"].fail = True
    second = {k: pool.submit({"route_key": k}) for k in keys}
    assert all(second[k] == first[k] for k in keys if first[k] != "w2") and "w2" not in second.values()
    assert pool.stats()["w2"]["down"] and pool.live() == ["w0", "w1", "w3"]
    ws["w2"].fail = False
    pool.mark_up("w2")
    assert all(pool.submit({"route_key": k}) == first[k] for k in keys)                    # and come back
    # no key: round robin over the live workers
    before = {n: s["served"] for n, s in pool.stats().items()}
    with ThreadPoolExecutor(4) as ex:
        list(ex.map(lambda i: pool.submit({"i": i}), range(40)))
    gained = {n: pool.stats()[n]["served"] - before[n] for n in ws}
    assert sum(gained.values()) == 40 and min(gained.values()) >= 5
    # the pool follows a health monitor: a silent worker leaves the rotation before a request fails on it
    from tunix_b200.experimental.common.datatypes import HealthReport, WorkerState
    from tunix_b200.experimental.orchestrator.health_monitor import HealthMonitor
    now = [0.0]
    mon = HealthMonitor(heartbeat_timeout_s=10.0, clock=lambda: now[0])
    for n in ws:
        mon.observe(HealthReport(n, WorkerState.READY))
    assert pool.apply_health(mon) == ([], [])
    now[0] = 8.0
    for n in ("w0", "w1", "w3"):
        mon.observe(HealthReport(n, WorkerState.READY))
    now[0] = 12.0                                           # w2 has been silent for 12 s
    assert pool.apply_health(mon) == (["w2"], []) and pool.live() == ["w0", "w1", "w3"]
    assert all(pool.submit({"route_key": k}) != "w2" for k in keys[:50]) and not ws["w2"].seen[-1:] == ["never"]
    mon.observe(HealthReport("w2", WorkerState.READY))
    assert pool.apply_health(mon) == ([], ["w2"]) and pool.live() == ["w0", "w1", "w2", "w3"]
    # a custom router wins over the key; everything down is an error, not a hang
    routed = RoutingPool(ws, router=lambda req, names: "w3" if req.get("big") else None)
    assert routed.submit({"big": True, "route_key": "conv-1"}) == "w3"
    for w in ws.values():
        w.fail = True
    with pytest.raises(NoWorkerAvailable):
        pool.submit({"route_key": "x"})
    with pytest.raises(NoWorkerAvailable):
        pool.submit({"route_key": "x"})                                                    # now nobody is live


def test_tiered_page_pool_moves_pages_between_device_and_host():
    import torch
    from tunix_b200.experimental.generate.tiered_page_pool import PageLocation, TieredPagePool, TieredPoolError
    pool = TieredPagePool(["k", "v"], page_shape=(4, 2, 8), dtype=torch.float32, num_device_pages=4, num_host_pages=3)
    ids = pool.allocate_device_pages(4)
    assert pool.num_free_device_pages == 0 and sorted(pool.device_indices(ids)) == [0, 1, 2, 3]
    for p in ids:                                           # a recognisable pattern per logical page and partition
        pool.dev["k"][pool.page_idx(p)] = float(p + 1)
        pool.dev["v"][pool.page_idx(p)] = -float(p + 1)
    with pytest.raises(TieredPoolError):
        pool.allocate_device_pages(1)
    pool.offload([ids[1], ids[3]])
    assert pool.page_location(ids[1]) is PageLocation.HOST and pool.num_free_device_pages == 2 and pool.num_free_host_pages == 1
    assert float(pool.host["k"][pool.page_idx(ids[3])].mean()) == ids[3] + 1
    with pytest.raises(TieredPoolError, match="load it first"):
        pool.device_indices(ids)
    more = pool.allocate_device_pages(2)                    # the freed device slots are reused...
    for p in more:
        pool.dev["k"][pool.page_idx(p)] = 100.0 + p
        pool.dev["v"][pool.page_idx(p)] = -100.0 - p
    with pytest.raises(TieredPoolError):                    # ...so nothing fits until something else leaves
        pool.load([ids[1]])
    assert pool.page_location(ids[1]) is PageLocation.HOST  # a refused move changes nothing
    pool.offload([more[0]])
    with pytest.raises(TieredPoolError):                    # the host tier is full now: 3 pages
        pool.offload([more[1]])
    pool.free([more[1]])
    pool.load([ids[1]])
    assert pool.page_location(ids[1]) is PageLocation.DEVICE
    assert float(pool.dev["k"][pool.page_idx(ids[1])].mean()) == ids[1] + 1 and float(pool.dev["v"][pool.page_idx(ids[1])].mean()) == -(ids[1] + 1)
    assert float(pool.dev["k"][pool.page_idx(ids[0])].mean()) == ids[0] + 1                 # untouched neighbours
    page_bytes = 4 * 2 * 8 * 4 * 2
    assert pool.bytes_offloaded == 3 * page_bytes and pool.bytes_loaded == page_bytes
    with pytest.raises(TieredPoolError):
        pool.offload([ids[3]])                              # already on the host
    with pytest.raises(TieredPoolError):
        pool.free([ids[0], ids[0]])
    with pytest.raises(TieredPoolError):
        pool.free([12345])
    pool.free([ids[0], ids[1], ids[2], ids[3], more[0]])
    assert pool.num_free_device_pages == 4 and pool.num_free_host_pages == 3
    # adopting existing pools checks their geometry
    with pytest.raises(ValueError):
        TieredPagePool(["k"], (4, 2, 8), torch.float32, 4, 2, device_pages={"k": torch.zeros(3, 4, 2, 8)})


def test_lifecycle_driver_and_startup_validation():
    import types
    from tunix_b200.experimental.common.datatypes import WorkerState
    from tunix_b200.experimental.orchestrator.lifecycle import LifecycleDriver, LifecycleError
    from tunix_b200.experimental.orchestrator.startup_validation import (RegistryValidator, StartupValidationError,
                                                                         validate_startup)
    from tunix_b200.experimental.orchestrator.worker_registry import WorkerRegistry
    from tunix_b200.experimental.worker.mock_worker import MockWorker, make_echo_worker

    def registry(*workers):
        reg = WorkerRegistry()
        for w in workers:
            reg.register(w)
        return reg

    good = [make_echo_worker("r0"), make_echo_worker("r1"), make_echo_worker("t0", role="trainer")]
    reg = registry(*good)
    drv = LifecycleDriver(reg)
    drv.bring_up()
    assert all(w.state == WorkerState.READY for w in good)
    drv.shutdown()
    assert all(w.state == WorkerState.STOPPED for w in good)
    # one worker fails to initialise: the others are stopped again and the error names the failure
    ok1, ok2 = make_echo_worker("a"), make_echo_worker("c")
    bad = MockWorker("b", fail_on_init=True)
    bad.role = "rollout"
    with pytest.raises(LifecycleError, match="b: RuntimeError") as ei:
        LifecycleDriver(registry(ok1, bad, ok2)).bring_up()
    assert [wid for wid, _ in ei.value.failures] == ["b"] and ei.value.phase == "bring_up"
    assert ok1.state == WorkerState.STOPPED and ok2.state == WorkerState.STOPPED and bad.state == WorkerState.FAILED
    # shutdown is best effort and reports every worker that could not be stopped
    s1, s2 = make_echo_worker("s1"), make_echo_worker("s2")
    reg2 = registry(s1, s2)
    LifecycleDriver(reg2).bring_up()
    s1._drain = lambda: (_ for _ in ()).throw(OSError("stuck"))
    with pytest.raises(LifecycleError, match="shutdown failed on 1 worker") as ei:
        LifecycleDriver(reg2).shutdown()
    assert ei.value.failures[0][0] == "s1" and s2.state == WorkerState.STOPPED
    # startup validation gathers every problem in one error
    alg = types.SimpleNamespace(num_generations=4, algo_variant="grpo", max_response_length=256)
    tc = types.SimpleNamespace(mini_batch_size=16, train_micro_batch_size=4, rollout_micro_batch_size=8, compute_logps_micro_batch_size=None)
    validate_startup(reg, alg, tc)
    alg_bad = types.SimpleNamespace(num_generations=1, algo_variant="grpo", max_response_length=0)
    tc_bad = types.SimpleNamespace(mini_batch_size=10, train_micro_batch_size=4, rollout_micro_batch_size=True, compute_logps_micro_batch_size=5)
    with pytest.raises(StartupValidationError) as ei:
        validate_startup(registry(make_echo_worker("only")), alg_bad, tc_bad)
    msgs = "\n".join(ei.value.errors)
    for part in ("max_response_length must be a positive integer", "not divisible by train_micro_batch_size 4",
                 "rollout_micro_batch_size must be a positive integer", "num_generations must be > 1 for 'grpo'",
                 "role 'trainer': 0 worker(s) registered, 1 needed"):
        assert part in msgs, part
    assert "compute_logps_micro_batch_size 5" not in msgs                    # 10 % 5 == 0
    tc_pack = types.SimpleNamespace(mini_batch_size=16, train_micro_batch_size=3, sequence_packing=True)
    validate_startup(reg, alg, tc_pack)                                       # token-sized micro-batches need not divide
    with pytest.raises(StartupValidationError, match="2 needed"):
        validate_startup(reg, alg, tc, validators=[RegistryValidator(min_counts={"trainer": 2})])


def test_algorithm_adapters_grpo_variants_and_ppo_gae():
    import numpy as np
    import torch
    from tunix_b200.experimental.common.datatypes import RolloutResponse
    from tunix_b200.experimental.orchestrator.algorithm_adapter import GRPOAdapter, PPOAdapter
    from tunix_b200.experimental.orchestrator.batch_assembly import BatchConfig, create_batch_assembler
    item = {"prompt_ids": [1, 5, 6], "prompt_id": "p0"}
    resp = [RolloutResponse(f"p0/{i}", tokens=list(range(10, 10 + n)), logprobs=[-0.5] * n, group_id="p0", policy_version=2)
            for i, n in enumerate((2, 4, 3, 1))]
    reward = lambda it, r: float(len(r.tokens))
    r = np.array([2, 4, 3, 1], np.float32)
    g = GRPOAdapter(reward).create_payloads(item, resp)
    np.testing.assert_allclose([p.example["advantages"][0] for p in g], (r - r.mean()) / (r.std() + 1e-6), rtol=1e-5)
    assert all(len(p.example["advantages"]) == len(p.example["completion_ids"]) for p in g) and g[1].policy_version == 2
    d = GRPOAdapter(reward, estimator="drgrpo").create_payloads(item, resp)
    np.testing.assert_allclose([p.example["advantages"][0] for p in d], r - r.mean(), rtol=1e-6)
    l = GRPOAdapter(reward, estimator="rloo").create_payloads(item, resp)
    np.testing.assert_allclose([p.example["advantages"][0] for p in l], r - (r.sum() - r) / 3, rtol=1e-6)
    assert GRPOAdapter(lambda it, rr: 1.0).create_payloads(item, resp) == []            # uniform group: nothing to learn
    # PPO: reward on the last token, KL charged per token, GAE over the response; compare with the recurrence
    values = lambda p, c: [0.1 * (k + 1) for k in range(len(c))]
    ref = lambda p, c: [-0.7] * len(c)
    ppo = PPOAdapter(reward, values, ref_logps_fn=ref, gamma=0.9, gae_lambda=0.8, kl_coef=0.5, whiten=False)
    out = ppo.create_payloads(item, resp)
    for p, rr in zip(out, resp):
        n = len(rr.tokens)
        rew = np.full(n, -0.5 * (-0.5 + 0.7), np.float32)
        rew[-1] += n
        v = np.array(values(None, rr.tokens), np.float32)
        adv, last = np.zeros(n, np.float32), 0.0
        for t in range(n - 1, -1, -1):
            nv = v[t + 1] if t + 1 < n else 0.0
            last = rew[t] + 0.9 * nv - v[t] + 0.9 * 0.8 * last
            adv[t] = last
        np.testing.assert_allclose(p.example["advantages"], adv, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(p.example["returns"], adv + v, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(p.example["values"], v)
    # the assembler carries the per-token PPO fields into the micro-batch
    asm = create_batch_assembler(BatchConfig(rows_per_microbatch=4, max_prompt_length=4, max_response_length=4), packed=False)
    batches = list(asm.feed(out)) + list(asm.flush())
    assert len(batches) == 1 and {"returns", "values", "old_per_token_logps"} <= set(batches[0].arrays)
    assert batches[0].arrays["returns"].shape == batches[0].arrays["advantages"].shape


def test_deployments_local_processes_and_jobset_manifest():
    """The same role specs start local worker processes or render a Kubernetes JobSet; a pod-style worker (own
    bind / advertised address, no parent pipe) runs until it is terminated and withdraws from the directory."""
    import signal
    import subprocess
    import sys
    import time
    import yaml
    pytest.importorskip("grpc")
    from tunix_b200.experimental.runtime.deployment import LocalDeployment, RoleSpec, jobset_manifest, to_yaml
    from tunix_b200.experimental.runtime.launcher import Launcher
    factory = "tunix_b200.experimental.worker.mock_worker:make_echo_worker"
    roles = [RoleSpec("rollout", factory, replicas=2, gpus_per_worker=1, args={"scale": 2}),
             RoleSpec("trainer", factory, replicas=1, gpus_per_worker=8, args={"scale": 5}, env={"NCCL_NVLS_ENABLE": 0})]
    dep = LocalDeployment(roles, token="s3")
    try:
        workers = dep.start(timeout=120)
        assert sorted(workers) == ["rollout-0", "rollout-1", "trainer-0"]
        assert workers["rollout-1"].submit(4) == 8 and workers["trainer-0"].submit(4) == 20
        assert workers["trainer-0"].info().roles == ("trainer",)
    finally:
        dep.shutdown()
    man = yaml.safe_load(to_yaml(jobset_manifest("grpo-run", "registry.local/tunix-b200:1", roles,
                                                 directory_address="controller.default.svc:4000", token_secret="run-token",
                                                 node_selector={"gpu": "b200"})))
    assert man["kind"] == "JobSet" and [j["name"] for j in man["spec"]["replicatedJobs"]] == ["rollout", "trainer"]
    rj, tj = (j["template"]["spec"] for j in man["spec"]["replicatedJobs"])
    assert rj["parallelism"] == rj["completions"] == 2 and rj["completionMode"] == "Indexed"
    tc = tj["template"]["spec"]["containers"][0]
    assert tc["resources"]["limits"]["nvidia.com/gpu"] == 8 and tj["template"]["spec"]["nodeSelector"] == {"gpu": "b200"}
    cmd = tc["command"]
    assert cmd[cmd.index("--worker-id") + 1] == "trainer-$(JOB_COMPLETION_INDEX)" and "--stay" in cmd
    assert cmd[cmd.index("--advertise") + 1] == "$(POD_IP):50051" and cmd[cmd.index("--token") + 1] == "$(TUNIX_B200_TOKEN)"
    assert {"name": "NCCL_NVLS_ENABLE", "value": "0"} in tc["env"] and "scale=5" in cmd
    assert any(e.get("valueFrom", {}).get("secretKeyRef", {}).get("name") == "run-token" for e in tc["env"])
    with pytest.raises(ValueError, match="DNS label"):
        jobset_manifest("Bad_Name", "img", roles, directory_address="x:1")
    # a pod-style worker: explicit bind and advertised addresses, leaves on SIGTERM
    lau = Launcher(token="s3")
    proc = None
    try:
        proc = subprocess.Popen([sys.executable, "-m", "tunix_b200.experimental.runtime.launcher", "--factory", factory,
                                 "--worker-id", "rollout-7", "--directory", lau.address, "--token", "s3", "--bind", "127.0.0.1:0",
                                 "--stay", "--arg", "scale=3"], stdin=subprocess.DEVNULL)
        lau._procs["rollout-7"] = proc
        lau.wait_for(["rollout-7"], timeout=120)
        assert lau.workers()["rollout-7"].submit(5) == 15               # stdin at end of file did not end it
        proc.send_signal(signal.SIGTERM)
        assert proc.wait(30) == 0
        deadline = time.time() + 5
        while "rollout-7" in lau.directory.entries() and time.time() < deadline:
            time.sleep(0.05)
        assert "rollout-7" not in lau.directory.entries()
    finally:
        if proc is not None and proc.poll() is None:
            proc.kill()
        lau._procs.clear()
        lau.shutdown()


def test_engine_participants_stage_commit_and_roll_back_weight_rounds():
    """Two rollout engines behind a coordinator: a good round swaps both models while their servers are paused; a
    round whose second transfer fails leaves BOTH on the old weights and serving again."""
    import threading
    import torch
    from tunix_b200.experimental.weight_sync.participants import EngineParticipant
    from tunix_b200.experimental.weight_sync.weight_sync_coordinator import RoundState, WeightSyncCoordinator

    class Server:                                           # the pause / resume face of generate.engine.EngineServer
        def __init__(self, drains=True):
            self.paused, self.drains, self.log = False, drains, []

        def pause(self, timeout=None):
            self.paused = True
            self.log.append("pause")
            return self.drains

        def resume(self):
            self.paused = False
            self.log.append("resume")

    torch.manual_seed(0)
    trainer = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))
    rollouts = [torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4)).to(torch.bfloat16) for _ in range(2)]
    servers = [Server(), Server()]
    seen_paused = []

    def source():
        seen_paused.append([s.paused for s in servers])
        return trainer.named_parameters()

    parts = [EngineParticipant(f"r{i}", m, source, s) for i, (m, s) in enumerate(zip(rollouts, servers))]
    coord = WeightSyncCoordinator(parts)
    addr = [p.data_ptr() for p in rollouts[0].parameters()]
    assert coord.run_round(1) is RoundState.COMMITTED
    for m in rollouts:
        for (n, p), (_, q) in zip(m.named_parameters(), trainer.named_parameters()):
            assert torch.equal(p, q.to(torch.bfloat16)), n                        # cast into the rollout dtype
    assert [p.data_ptr() for p in rollouts[0].parameters()] == addr                # in place: captured graphs stay valid
    assert all(all(row) for row in seen_paused) and [s.log for s in servers] == [["pause", "resume"]] * 2
    assert parts[0].version == 1 and parts[0].bytes_last_round == sum(p.numel() * 2 for p in rollouts[0].parameters())
    # second round: the trainer moved on, but the second engine's transfer fails on a shape -> nobody changes
    before = [[p.clone() for p in m.parameters()] for m in rollouts]
    with torch.no_grad():
        for p in trainer.parameters():
            p.add_(1.0)
    parts[1].source = lambda: [("0.weight", torch.zeros(3, 3))]
    assert coord.run_round(2) is RoundState.ABORTED and "shape" in coord.history[-1][2]
    for m, old in zip(rollouts, before):
        assert all(torch.equal(p, o) for p, o in zip(m.parameters(), old))
    assert not any(s.paused for s in servers) and parts[0].version == 1 and parts[0]._staged is None
    # a missing tensor is an error under strict, fine otherwise; a key map renames
    parts[1].source = lambda: [(n, p) for n, p in trainer.named_parameters() if n != "1.bias"]
    assert coord.run_round(3) is RoundState.ABORTED and "lacks" in coord.history[-1][2]
    parts[1].strict = False
    parts[1].source = lambda: [("model." + n, p) for n, p in trainer.named_parameters() if n != "1.bias"]
    parts[1].key_map = lambda n: n[len("model."):]
    assert coord.run_round(4) is RoundState.COMMITTED
    assert torch.equal(rollouts[1][0].weight, trainer[0].weight.to(torch.bfloat16)) and torch.equal(rollouts[1][1].bias, before[1][3])
    # requests that do not drain in time abort the round and the server is admitted again
    stuck = EngineParticipant("r9", rollouts[0], trainer.named_parameters, Server(drains=False), pause_timeout=0.01)
    c2 = WeightSyncCoordinator([stuck])
    assert c2.run_round(1) is RoundState.ABORTED and stuck.server.log == ["pause", "resume"]
    # without staging nothing is held between transfer and commit
    direct = EngineParticipant("r8", rollouts[0], trainer.named_parameters, None, stage=False)
    assert WeightSyncCoordinator([direct]).run_round(7) is RoundState.COMMITTED and direct.version == 7
    assert torch.equal(rollouts[0][1].bias, trainer[1].bias.to(torch.bfloat16))


def test_distributed_grpo_example_runs_across_processes(capsys):
    """Rollout workers in their own processes (launched, discovered, driven over gRPC, weights pushed as a payload),
    trainer in this one: the example's loop runs and the weight payload round-trips bit-exactly, bf16 included."""
    import importlib.util
    import os
    import torch
    import yaml
    pytest.importorskip("grpc")
    from tunix_b200.experimental.worker.factories import ByteTokenizer, export_state, install_state, toy_config
    from tunix_b200.models.transformer import create_model
    tok = ByteTokenizer()
    assert tok.decode(tok.encode("héllo")) == "héllo"
    for dtype in (torch.float32, torch.bfloat16):
        a, b = create_model(toy_config(dtype=dtype), seed=0), create_model(toy_config(dtype=dtype), seed=1)
        assert install_state(b, export_state(a)) == len(list(a.parameters()))
        assert all(torch.equal(p, q) for p, q in zip(a.parameters(), b.parameters()))
    with pytest.raises(KeyError):
        install_state(b, {})
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "experimental", "distributed_grpo.py")
    spec = importlib.util.spec_from_file_location("distributed_grpo_example", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    hist = mod.main(["--steps", "2", "--rollout-workers", "2", "--prompts-per-step", "2"])
    assert [h["policy_version"] for h in hist] == [2, 3] and all(h["trajectories"] + 4 * h["filtered_groups"] == 8 for h in hist)
    capsys.readouterr()
    assert mod.main(["--print-jobset"]) is None
    man = yaml.safe_load(capsys.readouterr().out)
    assert man["kind"] == "JobSet" and man["spec"]["replicatedJobs"][0]["template"]["spec"]["parallelism"] == 2


def test_bulk_plane_striped_transfers_and_remote_weight_sync():
    import os
    import threading
    import numpy as np
    pytest.importorskip("grpc")
    from tunix_b200.experimental.worker.network import (ArrayBundle, BulkReceiver, join_arrays, send_bulk, split_arrays)
    from tunix_b200.experimental.worker.mock_worker import MockWorker
    from tunix_b200.experimental.worker.remote_execution import RemoteWorker, serve_worker
    rng = np.random.default_rng(0)
    payload = {"layers": [{"w": rng.standard_normal((601, 301)).astype(np.float32), "b": rng.integers(-9, 9, 77).astype(np.int16)}],
               "head": ("bf16", rng.integers(0, 2 ** 15, (1000, 33)).astype(np.int16)), "step": 7, "empty": np.zeros((0, 4), np.float64),
               "tiny": np.arange(3)}
    skeleton, arrays = split_arrays(payload, min_bytes=0)
    assert len(arrays) == 5 and skeleton["step"] == 7
    views = ArrayBundle.unpack(ArrayBundle.pack(arrays))
    back = join_arrays(skeleton, views)
    assert np.array_equal(back["layers"][0]["w"], payload["layers"][0]["w"]) and back["head"][0] == "bf16"
    assert np.array_equal(back["head"][1], payload["head"][1]) and back["empty"].shape == (0, 4) and back["tiny"].dtype == np.arange(3).dtype
    assert all((v.ctypes.data - views[0].ctypes.data) % 64 == 0 for v in views if v.nbytes)       # arrays start on 64-byte offsets
    # raw transfers: several sizes and stripe counts, several at once, wrong token, incomplete transfer
    rx = BulkReceiver(token="k3y")
    try:
        blobs = [os.urandom(n) for n in (0, 1, 300_000, 3_000_001)]
        handles = [None] * len(blobs)

        def send(i):
            handles[i] = send_bulk(rx.address, blobs[i], stripes=1 + i * 2, token="k3y")
        ts = [threading.Thread(target=send, args=(i,)) for i in range(len(blobs))]
        [t.start() for t in ts]
        [t.join() for t in ts]
        for h, blob in zip(handles, blobs):
            assert h.nbytes == len(blob) and bytes(rx.take(h.transfer_id, timeout=10)) == blob
        assert rx.bytes_received == sum(map(len, blobs))
        with pytest.raises(ConnectionError):
            send_bulk(rx.address, b"x" * 1000, token="wrong")
        with pytest.raises(TimeoutError):
            rx.take(b"\x00" * 16, timeout=0.05)
    finally:
        rx.close()
    # a remote worker: the weight payload goes over the bulk plane, small payloads and servers without one use the RPC
    got = {}

    class W(MockWorker):
        def _sync_weights(self, version, payload):
            got[version] = payload
    for bulk in (True, False):
        w = W("w0")
        with serve_worker(w, token="k3y") if bulk else __import__("tunix_b200.experimental.worker.remote_execution", fromlist=["WorkerServer"]).WorkerServer(w, token="k3y", bulk=False) as srv:
            rw = RemoteWorker(srv.address, token="k3y")
            rw.start()
            rw.sync_weights(1, payload)
            assert np.array_equal(got[1]["layers"][0]["w"], payload["layers"][0]["w"]) and got[1]["head"][0] == "bf16"
            assert np.array_equal(got[1]["head"][1], payload["head"][1]) and got[1]["step"] == 7 and np.array_equal(got[1]["tiny"], np.arange(3))
            assert (rw.bulk_bytes_sent > 700_000) == bulk                      # the arrays left the pickle, or could not
            rw.sync_weights(2, {"small": np.ones(8)})
            assert got[2]["small"].sum() == 8 and (rw.bulk_bytes_sent > 700_000) == bulk
            if bulk:                                        # a worker that copies its payload hands the buffer back
                w.releases_bulk_payloads = True
                rw.sync_weights(4, payload)
                rw.sync_weights(5, payload)
                assert srv.bulk.buffers_reused == 1 and np.array_equal(got[5]["layers"][0]["w"], payload["layers"][0]["w"])
            sent = rw.bulk_bytes_sent
            rw.sync_weights(3, None)
            assert got[3] is None and rw.bulk_bytes_sent == sent
            rw.close()


def test_async_sampler_adapter_over_server_and_batch_engines():
    import asyncio
    import torch
    from tests.test_sampler_cpu import CharTok, _FakeEngine
    from tunix_b200.common.configs import CacheConfig
    from tunix_b200.experimental.rollout.sampler import EngineSamplerAdapter, SamplingParams, SamplingRequest, SamplingResponse
    from tunix_b200.experimental.weight_sync.participants import EngineParticipant
    from tunix_b200.generate.engine import EngineServer
    from tunix_b200.generate.sampler import Sampler
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    with pytest.raises(ValueError):
        SamplingResponse("r", [1, 2], [0.0])

    async def server_case():
        srv = EngineServer(_FakeEngine(slots=3, fail_on=13), max_new_tokens=5, max_prompt_length=8, eos_tokens=[2])
        trainer, rollout = torch.nn.Linear(4, 4), torch.nn.Linear(4, 4)
        ad = EngineSamplerAdapter(srv, tokenizer=CharTok(), participant=EngineParticipant("r0", rollout, trainer.named_parameters, srv))
        await ad.start()
        reqs = [SamplingRequest(f"q{i}", [1, 20 + i], SamplingParams(max_tokens=1 + i % 3)) for i in range(6)]
        out = await ad.sample(reqs)
        assert [r.request_id for r in out] == [f"q{i}" for i in range(6)] and all(r.error is None for r in out)
        assert [r.token_ids for r in out] == [[20 + i + k + 1 for k in range(1 + i % 3)] for i in range(6)]
        assert out[0].text == CharTok().decode(out[0].token_ids) and out[0].finish_reason == "length"
        # a weight sync: sampling waits at the gate, then sees the new version
        await ad.pre_weight_sync(1)
        pending = asyncio.ensure_future(ad.sample([SamplingRequest("late", [1, 3], SamplingParams(max_tokens=1))]))
        await asyncio.sleep(0.05)
        assert not pending.done() and (await ad.get_load_info()).paused
        await ad.weight_sync(1)
        await ad.post_weight_sync(1)
        late = (await pending)[0]
        assert late.policy_version == 1 and torch.equal(rollout.weight, trainer.weight)
        # an aborted sync reopens the gate on the old version
        await ad.pre_weight_sync(2)
        await ad.abort_weight_sync()
        assert (await ad.sample([SamplingRequest("x", [1, 4], SamplingParams(max_tokens=1))]))[0].policy_version == 1
        info = await ad.get_load_info()
        assert info.served == 8 and info.inflight == 0 and not info.paused
        # the engine fails on one request: that response carries the error
        bad = await ad.sample([SamplingRequest("boom", [1, 13], SamplingParams(max_tokens=2))])
        assert isinstance(bad[0].error, RuntimeError) and bad[0].finish_reason == "error"
        await ad.stop()

    async def batch_case():
        cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16, num_kv_heads=1)
        model = create_model(cfg, seed=0)
        ad = EngineSamplerAdapter(Sampler(model, CharTok(), CacheConfig(32, 1, 1, 16)), tokenizer=CharTok(), eos_tokens=[2])
        out = await ad.sample([SamplingRequest("a", [1, 5, 6], SamplingParams(max_tokens=4, temperature=0.0)),
                               SamplingRequest("b", [1, 7], SamplingParams(max_tokens=3, temperature=0.0, return_logprobs=False))])
        assert len(out[0].token_ids) <= 4 and len(out[0].logprobs) == len(out[0].token_ids) and out[1].logprobs is None
        assert await ad.pause() and (await ad.get_load_info()).paused
        await ad.resume()
        await ad.stop()
    asyncio.run(server_case())
    asyncio.run(batch_case())


def test_orchestrator_streaming_overlaps_training_with_rollout():
    """With streaming, micro-batches reach the trainer while later prompts are still being generated; the set of
    trajectories, the last-micro-batch flag and the update are the same as without."""
    import threading
    import time
    import numpy as np
    from tunix_b200.experimental.common.datatypes import RolloutResponse
    from tunix_b200.experimental.orchestrator.algorithm_adapter import GRPOAdapter
    from tunix_b200.experimental.orchestrator.batch_assembly import BatchConfig, create_batch_assembler
    from tunix_b200.experimental.orchestrator.orchestrator import Orchestrator
    from tunix_b200.experimental.orchestrator.worker_registry import WorkerRegistry
    from tunix_b200.experimental.worker.mock_worker import MockWorker
    busy = {"n": 0}
    lock = threading.Lock()
    log = []

    def generate(req):
        slow = int(req.group_id[1:]) >= 2                   # the later prompts take much longer
        with lock:
            busy["n"] += 1
        time.sleep(0.25 if slow else 0.01)
        with lock:
            busy["n"] -= 1
        n = 2 + req.seed % 3
        return RolloutResponse(req.request_id, tokens=[10 + (req.seed + k) % 40 for k in range(n)], logprobs=[-0.3] * n,
                               group_id=req.group_id, policy_version=req.policy_version, metadata=dict(req.metadata))

    def train(req):
        if req["op"] == "fwd_bwd":
            log.append(("fwd_bwd", req["is_last_microbatch"], busy["n"], req["batch"]["input_tokens"].shape[0]))
            return {"loss": 0.5}
        log.append(("update",))
        return {"grad_norm": 1.0, "step": sum(1 for e in log if e[0] == "update")}

    def build(streaming):
        reg = WorkerRegistry()
        ws = [MockWorker(f"rollout-{i}", handler=generate, max_inflight=64) for i in range(2)] + [MockWorker("trainer-0", handler=train)]
        for w in ws:
            w.role = "trainer" if w.worker_id.startswith("trainer") else "rollout"
            w.start()
            reg.register(w)
        return Orchestrator(reg, create_batch_assembler(BatchConfig(rows_per_microbatch=4, max_prompt_length=4, max_response_length=4),
                                                        packed=False),
                            GRPOAdapter(lambda item, r: float(sum(r.tokens) % 7)), group_size=4, streaming=streaming,
                            rollout_params={"max_tokens": 4, "seed": 0})
    prompts = [{"prompt_id": f"p{i}", "prompt_ids": [1, 5 + i]} for i in range(4)]
    recs = {}
    for streaming in (False, True):
        log.clear()
        orch = build(streaming)
        recs[streaming] = orch.step(0, prompts)
        orch.close()
        steps = [e for e in log if e[0] == "fwd_bwd"]
        assert [e[1] for e in steps] == [False] * (len(steps) - 1) + [True] and log[-1] == ("update",)
        assert sum(e[3] for e in steps) == recs[streaming]["trajectories"]
        if streaming:
            assert any(e[2] > 0 for e in steps[:-1]), log            # a training pass ran while rollouts were in flight
            assert recs[True]["microbatches_overlapped_with_rollout"] >= 1
        else:
            assert all(e[2] == 0 for e in steps)
    for k in ("trajectories", "filtered_groups", "microbatches", "policy_version"):
        assert recs[True][k] == recs[False][k], k
    assert abs(recs[True]["reward_mean"] - recs[False]["reward_mean"]) < 1e-6


def test_prompt_dataset_prefetch_skip_errors_and_early_close():
    import asyncio
    import threading
    import time
    from tunix_b200.experimental.orchestrator.dataset_utils import PrefetchIterator, iter_dataset_async, total_prompt_groups
    assert total_prompt_groups(100, 8) == 800 and total_prompt_groups(100, 8, max_staleness=2) == (100 + 25) * 8
    assert total_prompt_groups(8, 4, max_staleness=1) == (8 + 6) * 4
    assert list(PrefetchIterator(["a", "b", "c"], skip_count=1)) == [(1, "b"), (2, "c")]
    produced, closed = [], threading.Event()

    def gen(n, fail_at=None):
        try:
            for i in range(n):
                if i == fail_at:
                    raise OSError("shard missing")
                produced.append(i)
                yield {"prompt": i}
        finally:
            closed.set()
    assert [(i, d["prompt"]) for i, d in PrefetchIterator(gen(6), skip_count=2, prefetch_size=2)] == [(i, i) for i in range(2, 6)]
    assert closed.is_set()
    # bounded look-ahead: the producer stays at most prefetch_size (+ the one in hand) ahead of the consumer
    produced.clear(); closed.clear()
    it = PrefetchIterator(gen(100), prefetch_size=3)
    assert next(it)[0] == 0
    time.sleep(0.2)
    assert len(produced) <= 1 + 3 + 1
    it.close()                                              # stopping early closes the generator
    assert closed.wait(2.0) and len(produced) < 100
    # the dataset's failure arrives at its position
    got = []
    with pytest.raises(OSError, match="shard missing"):
        for i, _ in PrefetchIterator(gen(10, fail_at=3)):
            got.append(i)
    assert got == [0, 1, 2]

    async def consume():
        out = []
        async for i, d in iter_dataset_async(gen(5), skip_count=1, prefetch_size=2):
            out.append(i)
            if i == 3:
                break
        return out
    closed.clear()
    assert asyncio.run(consume()) == [1, 2, 3]

    async def consume_list():
        return [i async for i, _ in iter_dataset_async([10, 11, 12], skip_count=2)]
    assert asyncio.run(consume_list()) == [2]
