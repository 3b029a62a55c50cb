"""FrozenLake as a multi-turn text environment (the reference trains on it in examples/frozenlake/: a grid world
rendered as text, one move per turn, reward 1 on reaching the goal).

The map is generated from a seed, so a task is just `{"seed": s, "size": n, "p": frozen_probability}`; maps with
no path from start to goal are re-drawn. The environment is deterministic by default (`is_slippery=False`); with
slipping, the move goes sideways with probability 2/3 as in the Gym original, from a per-episode generator, so that
an episode is reproducible from its task.

    P  player      _  frozen      O  hole      G  goal      X  player in a hole      *  player on the goal
"""
from __future__ import annotations

import random
import re
from typing import Any, Optional

from ..agents.agent_types import Action, Step
from ..agents.base_agent import ConversationAgentBase
from .base_environment import BaseTaskEnv

MOVES = {"left": (0, -1), "down": (1, 0), "right": (0, 1), "up": (-1, 0)}
_SIDEWAYS = {"left": ("up", "down"), "right": ("up", "down"), "up": ("left", "right"), "down": ("left", "right")}

SYSTEM_PROMPT = ("You are walking on a frozen lake. Reach the goal G without falling into a hole O. "
                 "Each turn, think briefly, then give exactly one move as ```Up```, ```Down```, ```Left``` or ```Right```.")


def _reachable(grid: list) -> bool:
    n = len(grid)
    seen, stack = {(0, 0)}, [(0, 0)]
    while stack:
        r, c = stack.pop()
        if grid[r][c] == "G":
            return True
        for dr, dc in MOVES.values():
            rr, cc = r + dr, c + dc
            if 0 <= rr < n and 0 <= cc < n and (rr, cc) not in seen and grid[rr][cc] != "O":
                seen.add((rr, cc))
                stack.append((rr, cc))
    return False


def generate_map(size: int = 4, p: float = 0.8, seed: Optional[int] = None) -> list:
    """A `size` x `size` grid with start in the top-left corner, the goal in the bottom-right one and holes with
    probability 1 - p elsewhere; always solvable."""
    rng = random.Random(seed)
    while True:
        grid = [["_" if rng.random() < p else "O" for _ in range(size)] for _ in range(size)]
        grid[0][0], grid[-1][-1] = "S", "G"
        if _reachable(grid):
            return grid


def parse_move(text: str) -> Optional[str]:
    """The last fenced move of a response, else the last bare direction word; None when there is none."""
    fenced = re.findall(r"```\s*(up|down|left|right)\s*```", text, flags=re.I)
    if fenced:
        return fenced[-1].lower()
    bare = re.findall(r"\b(up|down|left|right)\b", text, flags=re.I)
    return bare[-1].lower() if bare else None


class FrozenLakeEnv(BaseTaskEnv):
    def __init__(self, task: Any = None, max_steps: int = 8, is_slippery: bool = False, invalid_penalty: float = 0.0, **kwargs):
        task = dict(task or {})
        if "seed" not in task and "map" not in task and isinstance(task.get("question"), str):
            # a prompt dataset row: either the task as JSON, or any text, which then names the map through its checksum
            import json
            import zlib
            try:
                parsed = json.loads(task["question"])
            except ValueError:
                parsed = None
            task.update(parsed if isinstance(parsed, dict) else {"seed": zlib.crc32(task["question"].encode())})
        super().__init__(task=task, max_steps=int(task.get("max_steps", max_steps)), **kwargs)
        self.size, self.p, self.seed = int(task.get("size", 4)), float(task.get("p", 0.8)), task.get("seed", 0)
        self.is_slippery = bool(task.get("is_slippery", is_slippery))
        self.invalid_penalty = invalid_penalty
        self.grid = [list(row) for row in task["map"]] if task.get("map") else generate_map(self.size, self.p, self.seed)
        self.size = len(self.grid)
        self.pos = (0, 0)
        self._rng = random.Random(self.seed)

    def render(self) -> str:
        rows = []
        for r, row in enumerate(self.grid):
            cells = []
            for c, ch in enumerate(row):
                ch = "_" if ch == "S" else ch
                if (r, c) == self.pos:
                    ch = {"O": "X", "G": "*"}.get(ch, "P")
                cells.append(ch)
            rows.append(" ".join(cells))
        return "\n".join(rows)

    def _initial_observation(self):
        self.pos = (0, 0)
        self._rng = random.Random(self.seed)
        return f"Current map:\n{self.render()}\nYou have {self.max_steps} moves."

    def _step_impl(self, action):
        move = parse_move(action if isinstance(action, str) else str(getattr(action, "action", action)))
        left = self.max_steps - self.step_count
        if move is None:
            return (f"That was not a move. Answer with ```Up```, ```Down```, ```Left``` or ```Right```.\n"
                    f"Current map:\n{self.render()}\nMoves left: {left}."), -self.invalid_penalty, False, {"valid": False}
        if self.is_slippery and self._rng.random() < 2.0 / 3.0:
            move = self._rng.choice(_SIDEWAYS[move])
        dr, dc = MOVES[move]
        r, c = min(max(self.pos[0] + dr, 0), self.size - 1), min(max(self.pos[1] + dc, 0), self.size - 1)
        self.pos = (r, c)
        cell = self.grid[r][c]
        if cell == "G":
            return f"You reached the goal.\n{self.render()}", 1.0, True, {"valid": True, "won": True, "moved": move}
        if cell == "O":
            return f"You fell into a hole.\n{self.render()}", 0.0, True, {"valid": True, "won": False, "moved": move}
        return f"Current map:\n{self.render()}\nMoves left: {left}.", 0.0, False, {"valid": True, "moved": move}


class FrozenLakeAgent(ConversationAgentBase):
    """Keeps the whole conversation; the action handed to the environment is the parsed move (or the raw text when
    there is none, which the environment answers with a reminder)."""

    def __init__(self, system_prompt: str = SYSTEM_PROMPT):
        super().__init__(system_prompt)

    def update_from_model(self, response: str, **kwargs) -> Action:
        import copy
        move = parse_move(response)
        thought = response.split("```")[0].strip() if "```" in response else ""
        step = Step(chat_completions=copy.deepcopy(self._messages), model_response=response, thought=thought,
                    action=Action(action=move if move is not None else response))
        self._messages.append({"role": "assistant", "content": response})
        self._trajectory.steps.append(step)
        return step.action


def shortest_path(grid: list) -> Optional[list]:
    """Moves of a shortest safe path from the start to the goal (breadth first); used by tests and as an oracle
    for reward shaping experiments."""
    n = len(grid)
    prev = {(0, 0): None}
    queue = [(0, 0)]
    for r, c in queue:
        if grid[r][c] == "G":
            path, cur = [], (r, c)
            while prev[cur] is not None:
                cur, move = prev[cur]
                path.append(move)
            return path[::-1]
        for name, (dr, dc) in MOVES.items():
            nxt = (r + dr, c + dc)
            if 0 <= nxt[0] < n and 0 <= nxt[1] < n and nxt not in prev and grid[nxt[0]][nxt[1]] != "O":
                prev[nxt] = ((r, c), name)
                queue.append(nxt)
    return None
