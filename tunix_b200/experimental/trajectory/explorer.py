"""Command-line explorer of a trajectory store (the reference ships an explorer CLI with
tunix/experimental/trajectory/).

    python -m tunix_b200.experimental.trajectory.explorer runs/traj.db stats
    python -m tunix_b200.experimental.trajectory.explorer runs/traj.db list --min-reward 0.5 --limit 20
    python -m tunix_b200.experimental.trajectory.explorer runs/traj.jsonl show <trajectory_id>
    python -m tunix_b200.experimental.trajectory.explorer runs/traj.jsonl export out.db        (JSON lines -> SQL or back)
    python -m tunix_b200.experimental.trajectory.explorer runs/traj.db export-sft best.jsonl --min-reward 1.0 --best-of-group
                                                      (conversations of good trajectories as {"messages": [...]} rows for SFT)

Works on both store formats; a JSON-lines file is scanned, a SQL store is queried."""
from __future__ import annotations

import argparse
import json
import sys
from typing import Iterator, Optional

from .store import SqliteTrajectoryStore, open_store


def _records(path: str, group_id=None, min_version=None, min_reward=None, max_reward=None, limit=None) -> Iterator[dict]:
    store = open_store(path)
    try:
        if isinstance(store, SqliteTrajectoryStore):
            yield from store.query(group_id=group_id, min_policy_version=min_version, min_reward=min_reward,
                                   max_reward=max_reward, limit=limit)
            return
        n = 0
        for r in store.read():
            if group_id is not None and str(r.get("group_id")) != str(group_id):
                continue
            if min_version is not None and r.get("policy_version", 0) < min_version:
                continue
            if min_reward is not None and r.get("reward", 0.0) < min_reward:
                continue
            if max_reward is not None and r.get("reward", 0.0) > max_reward:
                continue
            yield r
            n += 1
            if limit is not None and n >= limit:
                return
    finally:
        store.close()


def _stats(path: str) -> dict:
    store = open_store(path)
    try:
        if isinstance(store, SqliteTrajectoryStore):
            return store.stats()
        acc: dict = {}
        for r in store.read():
            a = acc.setdefault(int(r.get("policy_version", 0)), [0, 0.0, float("inf"), float("-inf"), 0])
            rew = float(r.get("reward", 0.0))
            a[0] += 1
            a[1] += rew
            a[2], a[3] = min(a[2], rew), max(a[3], rew)
            a[4] += len(r.get("steps") or ())
        return {v: {"count": c, "reward_mean": s / c, "reward_min": lo, "reward_max": hi, "steps_mean": n / c}
                for v, (c, s, lo, hi, n) in sorted(acc.items())}
    finally:
        store.close()


def _short(text, n: int = 60) -> str:
    text = " ".join(str(text).split())
    return text if len(text) <= n else text[: n - 1] + "…"


def main(argv: Optional[list] = None, out=None) -> int:
    out = out or sys.stdout
    ap = argparse.ArgumentParser(prog="trajectory-explorer", description=__doc__.split("\n")[0])
    ap.add_argument("path")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("stats")
    ls = sub.add_parser("list")
    for flag, typ in (("--group", str), ("--min-version", int), ("--min-reward", float), ("--max-reward", float), ("--limit", int)):
        ls.add_argument(flag, type=typ, default=None)
    sh = sub.add_parser("show")
    sh.add_argument("trajectory_id")
    sh.add_argument("--json", action="store_true")
    ex = sub.add_parser("export")
    ex.add_argument("dest")
    sft = sub.add_parser("export-sft")
    sft.add_argument("dest")
    sft.add_argument("--min-reward", type=float, default=None)
    sft.add_argument("--best-of-group", action="store_true", help="keep only the highest-reward trajectory of each group")
    a = ap.parse_args(argv)

    if a.cmd == "stats":
        print(f"{'version':>8} {'count':>7} {'reward mean':>12} {'min':>8} {'max':>8} {'steps':>7}", file=out)
        for v, s in _stats(a.path).items():
            print(f"{v:>8} {s['count']:>7} {s['reward_mean']:>12.4f} {s['reward_min']:>8.3f} {s['reward_max']:>8.3f} "
                  f"{s['steps_mean']:>7.2f}", file=out)
        return 0
    if a.cmd == "list":
        for r in _records(a.path, a.group, a.min_version, a.min_reward, a.max_reward, a.limit):
            first = (r.get("steps") or [{}])[0]
            print(f"{r['trajectory_id']}  v{r.get('policy_version', 0):<4} group={r.get('group_id')}  reward={r.get('reward', 0.0):.3f}  "
                  f"steps={len(r.get('steps') or ())}  {_short(first.get('model_response', ''))}", file=out)
        return 0
    if a.cmd == "show":
        for r in _records(a.path):
            if r["trajectory_id"] == a.trajectory_id:
                if a.json:
                    print(json.dumps(r, indent=2), file=out)
                    return 0
                print(f"trajectory {r['trajectory_id']}  group={r.get('group_id')}  policy version {r.get('policy_version', 0)}  "
                      f"reward {r.get('reward', 0.0):.4f}", file=out)
                for k, v in (r.get("metadata") or {}).items():
                    print(f"  {k}: {_short(v, 100)}", file=out)
                for i, s in enumerate(r.get("steps") or ()):
                    print(f"  step {i}: reward={s.get('reward', 0.0):.3f} done={s.get('done', False)}", file=out)
                    for k in ("observation", "thought", "model_response", "action"):
                        if s.get(k) not in (None, ""):
                            print(f"    {k}: {_short(s[k], 100)}", file=out)
                return 0
        print(f"no trajectory {a.trajectory_id}", file=sys.stderr)
        return 1
    if a.cmd == "export-sft":
        rows = [r for r in _records(a.path, min_reward=a.min_reward) if (r.get("metadata") or {}).get("conversation")]
        if a.best_of_group:
            best: dict = {}
            for r in rows:
                key = r.get("group_id") if r.get("group_id") is not None else r["trajectory_id"]
                if key not in best or r.get("reward", 0.0) > best[key].get("reward", 0.0):
                    best[key] = r
            rows = list(best.values())
        with open(a.dest, "w", encoding="utf-8") as f:
            for r in rows:
                f.write(json.dumps({"messages": r["metadata"]["conversation"], "reward": r.get("reward", 0.0),
                                    "trajectory_id": r["trajectory_id"]}) + "\n")
        print(f"{len(rows)} conversations -> {a.dest}", file=out)
        return 0
    if a.cmd == "export":
        dest = open_store(a.dest)
        n = 0
        try:
            for r in _records(a.path):
                dest.put(r)
                n += 1
        finally:
            dest.close()
        print(f"{n} trajectories -> {a.dest}", file=out)
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
