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
