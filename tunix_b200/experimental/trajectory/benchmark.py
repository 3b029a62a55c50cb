"""Write and read throughput of the step-level trajectory stores
(tunix/experimental/trajectory/benchmarks/{benchmark_lib,data_generator,run_benchmark}.py).

    python -m tunix_b200.experimental.trajectory.benchmark --store file --root /tmp/traj_bench --trajectories 200 --turns 8

Synthetic trajectories with `turns` agent / environment step pairs of `tokens` token ids each are logged step by step
from `writers` producer threads (the way rollout workers call a store), flushed, then read back whole. Reported:
steps/s as seen by the producers (enqueue), steps/s including the flush (durable), trajectories/s read."""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import threading
import time
from typing import Optional

import numpy as np

from . import trajectory as T
from .file_store import FileTrajectoryStore
from .in_memory_store import InMemoryTrajectoryStore
from .sql_store import SqlTrajectoryStore


def generate_trajectory(trajectory_id: str, turns: int, tokens: int, seed: int = 0) -> T.TunixTrajectory:
    rng = np.random.default_rng(seed)
    steps: list = [T.TunixEnvStep(step_id=0, source="user", message="task " + "x" * 64)]
    for t in range(turns):
        steps.append(T.TunixAgentStep(step_id=len(steps), source="agent", message="y" * (4 * tokens), llm_call_count=1,
                                      assistant_tokens=rng.integers(0, 32000, tokens), assistant_masks=np.ones(tokens, np.int64),
                                      logprobs=-rng.random(tokens).astype(np.float32), policy_version=t // 4, mc_return=1.0,
                                      metrics=T.Metrics(completion_tokens=tokens)))
        steps.append(T.TunixEnvStep(step_id=len(steps), source="user", message="obs " + "z" * 128, reward=float(t == turns - 1),
                                    done=t == turns - 1, env_tokens=rng.integers(0, 32000, 32), env_masks=np.zeros(32, np.int64)))
    return T.TunixTrajectory(agent=T.Agent(name="bench", version="1"), trajectory_id=trajectory_id, prompt_id=f"p{seed // 8}",
                             group_index=seed % 8, status="SUCCEEDED", total_reward=1.0, steps=steps)


def run_benchmark(store, trajectories: int = 100, turns: int = 8, tokens: int = 256, writers: int = 4) -> dict:
    trajs = [generate_trajectory(f"bench-{i}", turns, tokens, i) for i in range(trajectories)]
    n_steps = sum(len(t.steps) for t in trajs)

    def produce(part) -> None:
        for t in part:
            meta = t.metadata()
            for s in t.steps:
                store.add_step(s, meta)
    threads = [threading.Thread(target=produce, args=(trajs[i::writers],)) for i in range(writers)]
    t0 = time.perf_counter()
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    t_enqueue = time.perf_counter() - t0
    store.flush()
    t_durable = time.perf_counter() - t0
    t1 = time.perf_counter()
    ids = [m.trajectory_id for m in store.get_trajectories_metadata()]
    got = store.get_trajectories(ids)
    t_read = time.perf_counter() - t1
    assert sum(len(t.steps) for t in got) == n_steps, "the store did not return every step"
    return {"trajectories": trajectories, "steps": n_steps, "writers": writers, "enqueue_steps_per_s": n_steps / t_enqueue,
            "durable_steps_per_s": n_steps / t_durable, "read_trajectories_per_s": trajectories / t_read,
            "write_errors": getattr(store, "write_errors", 0)}


def main(argv: Optional[list] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--store", choices=["memory", "file", "sql"], default="file")
    ap.add_argument("--root", default=None, help="directory for the file / SQL store (default: a temporary directory)")
    ap.add_argument("--trajectories", type=int, default=100)
    ap.add_argument("--turns", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--writers", type=int, default=4)
    a = ap.parse_args(argv)
    with tempfile.TemporaryDirectory() as tmp:
        root = a.root or tmp
        os.makedirs(root, exist_ok=True)
        store = {"memory": InMemoryTrajectoryStore, "file": lambda: FileTrajectoryStore(os.path.join(root, "atif")),
                 "sql": lambda: SqlTrajectoryStore(f"sqlite:///{os.path.join(os.path.abspath(root), 'bench.db')}")}[a.store]()
        try:
            print(json.dumps({"store": a.store, **run_benchmark(store, a.trajectories, a.turns, a.tokens, a.writers)}))
        finally:
            store.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
