"""Text environments for multi-turn agentic RL: FrozenLake, Sokoban and a minimal counting environment.

Interface (the one the reference's GEM-style envs expose, gpatch_v4/agentic/env/frozenlake/frozenlake_env.py:28-227,
sokoban/sokoban_env.py:29-203, simple_agentic_env.py:16-95): ``reset(seed) -> (observation_text, info)``,
``step(action_text) -> (observation_text, reward, terminated, truncated, info)``, ``get_instructions()``,
``parse_action(text)``.  Maps are generated here (no gym dependency): FrozenLake boards are random with a guaranteed
path from start to goal, Sokoban rooms are built by reverse play from a solved state so they are always solvable.
"""
from __future__ import annotations

import random
import re
from typing import Dict, List, Optional, Tuple

ACTION_RE = re.compile(r"<answer>\s*(.*?)\s*</answer>", re.S | re.I)


def parse_action_text(text: str, lookup: Dict[str, int]) -> Optional[int]:
    """``<answer>Left</answer>`` (or a bare action word) -> action id; None when nothing valid is found."""
    m = ACTION_RE.search(text or "")
    cand = (m.group(1) if m else (text or "")).strip().lower()
    for name, idx in lookup.items():
        if cand == name.lower():
            return idx
    for name, idx in lookup.items():
        if re.search(rf"\b{name.lower()}\b", cand):
            return idx
    return None


class TextEnv:
    max_steps = 20
    invalid_action_penalty = -0.1

    def get_instructions(self) -> str:
        raise NotImplementedError

    def reset(self, seed: Optional[int] = None):
        raise NotImplementedError

    def step(self, action_text: str):
        raise NotImplementedError

    def close(self):
        pass


# ------------------------------------------------------------------------------------------------ FrozenLake
def _has_path(board: List[List[str]]) -> bool:
    n = len(board)
    seen, stack = set(), [(0, 0)]
    while stack:
        r, c = stack.pop()
        if (r, c) in seen:
            continue
        seen.add((r, c))
        for dr, dc in ((1, 0), (0, 1), (-1, 0), (0, -1)):
            rr, cc = r + dr, c + dc
            if 0 <= rr < n and 0 <= cc < n and board[rr][cc] != "H":
                if board[rr][cc] == "G":
                    return True
                stack.append((rr, cc))
    return False


def generate_frozenlake_map(size: int = 4, p_frozen: float = 0.8, seed: Optional[int] = None) -> List[str]:
    rng = random.Random(seed)
    while True:
        board = [["F" if rng.random() < p_frozen else "H" for _ in range(size)] for _ in range(size)]
        board[0][0], board[-1][-1] = "S", "G"
        if _has_path(board):
            return ["".join(r) for r in board]


class FrozenLakeEnv(TextEnv):
    ACTIONS = {"Left": 0, "Down": 1, "Right": 2, "Up": 3}
    MOVES = {0: (0, -1), 1: (1, 0), 2: (0, 1), 3: (-1, 0)}
    SYMBOLS = {"S": "_", "F": "_", "H": "O", "G": "G"}

    def __init__(self, size: int = 4, p_frozen: float = 0.8, is_slippery: bool = False, max_steps: int = 20, **_):
        self.size, self.p, self.slippery, self.max_steps = size, p_frozen, is_slippery, max_steps
        self.map: List[str] = []
        self.pos = (0, 0)
        self.steps = 0
        self.rng = random.Random(0)

    def get_instructions(self) -> str:
        return ("You are walking on a frozen lake. Reach the goal (G) without falling into a hole (O). "
                "P is you, _ is ice. Reply with <answer>Left|Down|Right|Up</answer>.")

    def render(self) -> str:
        rows = []
        for r, line in enumerate(self.map):
            rows.append("".join("P" if (r, c) == self.pos else self.SYMBOLS[ch] for c, ch in enumerate(line)))
        return "\n".join(rows)

    def reset(self, seed: Optional[int] = None):
        self.rng = random.Random(seed)
        self.map = generate_frozenlake_map(self.size, self.p, seed)
        self.pos, self.steps = (0, 0), 0
        return self.render(), {"instructions": self.get_instructions()}

    def parse_action(self, text):
        return parse_action_text(text, self.ACTIONS)

    def step(self, action_text: str):
        self.steps += 1
        a = self.parse_action(action_text) if isinstance(action_text, str) else action_text
        info = {"action_is_valid": a is not None, "success": False}
        if a is None:
            return self.render(), self.invalid_action_penalty, False, self.steps >= self.max_steps, info
        if self.slippery and self.rng.random() < 2 / 3:
            a = (a + self.rng.choice((-1, 1))) % 4
        dr, dc = self.MOVES[a]
        r, c = min(max(self.pos[0] + dr, 0), self.size - 1), min(max(self.pos[1] + dc, 0), self.size - 1)
        self.pos = (r, c)
        cell = self.map[r][c]
        done = cell in "HG"
        info["success"] = cell == "G"
        return self.render(), 1.0 if cell == "G" else 0.0, done, (not done) and self.steps >= self.max_steps, info


# ------------------------------------------------------------------------------------------------ Sokoban
class SokobanEnv(TextEnv):
    """``#`` wall, ``_`` floor, ``O`` target, ``X`` box, ``√`` box on target, ``P`` player, ``S`` player on target."""
    ACTIONS = {"Up": 0, "Down": 1, "Left": 2, "Right": 3}
    MOVES = {0: (-1, 0), 1: (1, 0), 2: (0, -1), 3: (0, 1)}

    def __init__(self, dim: Tuple[int, int] = (6, 6), num_boxes: int = 1, max_steps: int = 30, scramble_steps: int = 12,
                 **_):
        self.dim, self.num_boxes, self.max_steps, self.scramble = dim, num_boxes, max_steps, scramble_steps
        self.walls, self.targets, self.boxes, self.player = set(), set(), set(), (1, 1)
        self.steps = 0

    def get_instructions(self) -> str:
        return ("Sokoban: push every box (X) onto a target (O). # wall, _ floor, P you. Boxes can only be pushed. "
                "Reply with <answer>Up|Down|Left|Right</answer>.")

    def _free(self, cell):
        return cell not in self.walls and 0 <= cell[0] < self.dim[0] and 0 <= cell[1] < self.dim[1]

    def reset(self, seed: Optional[int] = None):
        rng = random.Random(seed)
        H, W = self.dim
        self.walls = {(r, c) for r in range(H) for c in range(W) if r in (0, H - 1) or c in (0, W - 1)}
        interior = [(r, c) for r in range(1, H - 1) for c in range(1, W - 1)]
        for cell in rng.sample(interior, k=max(len(interior) // 8, 0)):
            self.walls.add(cell)
        floor = [c for c in interior if c not in self.walls]
        self.targets = set(rng.sample(floor, self.num_boxes))
        self.boxes = set(self.targets)  # solved state; reverse play (pulls) scrambles it, so it stays solvable
        spots = [c for c in floor if c not in self.boxes]
        self.player = rng.choice(spots)
        for _ in range(self.scramble):
            a = rng.randrange(4)
            dr, dc = self.MOVES[a]
            nxt = (self.player[0] + dr, self.player[1] + dc)
            behind = (self.player[0] - dr, self.player[1] - dc)
            if not self._free(nxt) or nxt in self.boxes:
                continue
            if behind in self.boxes and rng.random() < 0.7:   # pull the box that is behind the player
                self.boxes.remove(behind)
                self.boxes.add(self.player)
            self.player = nxt
        if self.boxes == self.targets:  # degenerate scramble: displace one box by a legal pull if possible
            return self.reset(None if seed is None else seed + 7919)
        self.steps = 0
        return self.render(), {"instructions": self.get_instructions()}

    def render(self) -> str:
        H, W = self.dim
        out = []
        for r in range(H):
            row = ""
            for c in range(W):
                cell = (r, c)
                if cell in self.walls:
                    row += "#"
                elif cell == self.player:
                    row += "S" if cell in self.targets else "P"
                elif cell in self.boxes:
                    row += "√" if cell in self.targets else "X"
                elif cell in self.targets:
                    row += "O"
                else:
                    row += "_"
            out.append(row)
        return "\n".join(out)

    def parse_action(self, text):
        return parse_action_text(text, self.ACTIONS)

    def step(self, action_text):
        self.steps += 1
        a = self.parse_action(action_text) if isinstance(action_text, str) else action_text
        info = {"action_is_valid": a is not None, "success": False}
        if a is None:
            return self.render(), self.invalid_action_penalty, False, self.steps >= self.max_steps, info
        dr, dc = self.MOVES[a]
        nxt = (self.player[0] + dr, self.player[1] + dc)
        reward = -0.1
        if self._free(nxt):
            if nxt in self.boxes:
                beyond = (nxt[0] + dr, nxt[1] + dc)
                if self._free(beyond) and beyond not in self.boxes:
                    was_on = nxt in self.targets
                    self.boxes.remove(nxt)
                    self.boxes.add(beyond)
                    self.player = nxt
                    reward += (1.0 if beyond in self.targets else 0.0) - (1.0 if was_on else 0.0)
            else:
                self.player = nxt
        done = self.boxes == self.targets
        if done:
            reward += 10.0
            info["success"] = True
        return self.render(), reward, done, (not done) and self.steps >= self.max_steps, info


# ------------------------------------------------------------------------------------------------ simple env
class SimpleAgenticEnv(TextEnv):
    """The agent must answer with the running step number; used by smoke tests of the multi-turn plumbing."""

    def __init__(self, max_steps: int = 3, **_):
        self.max_steps, self.steps = max_steps, 0

    def get_instructions(self):
        return "Reply with <answer>N</answer> where N is the number of the current turn, starting at 1."

    def reset(self, seed=None):
        self.steps = 0
        return "turn 1", {"instructions": self.get_instructions()}

    def step(self, action_text):
        self.steps += 1
        m = ACTION_RE.search(action_text or "")
        ok = bool(m) and m.group(1).strip() == str(self.steps)
        done = self.steps >= self.max_steps
        return f"turn {self.steps + 1}", 1.0 if ok else 0.0, done, False, {"action_is_valid": bool(m), "success": ok}


ENV_REGISTRY = {"frozen_lake": FrozenLakeEnv, "sokoban": SokobanEnv, "simple": SimpleAgenticEnv}


def make_env(name: str, **kw) -> TextEnv:
    return ENV_REGISTRY[name](**kw)
