"""Tool-call and reasoning parsers for agent turns (the reference vendors SGLang-style parsers under
gpatch_v4/agentic/tools and gpatch_v4/agentic/reasoning_parsers).  Two formats: Hermes / Qwen ``<tool_call>{json}
</tool_call>`` blocks and ``<think>...</think>`` reasoning spans."""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

TOOL_RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
THINK_RE = re.compile(r"<think>(.*?)</think>", re.S)


@dataclass
class ToolCall:
    name: str
    arguments: Dict[str, Any] = field(default_factory=dict)
    raw: str = ""


def split_reasoning(text: str) -> Tuple[str, str]:
    """-> (reasoning, answer).  An unterminated ``<think>`` makes the whole remainder reasoning."""
    m = THINK_RE.search(text)
    if m:
        return m.group(1).strip(), (text[:m.start()] + text[m.end():]).strip()
    if "<think>" in text:
        return text.split("<think>", 1)[1].strip(), ""
    return "", text.strip()


def parse_tool_calls(text: str) -> Tuple[str, List[ToolCall]]:
    """-> (text without the tool-call blocks, calls).  Malformed JSON blocks are kept in the text."""
    calls, keep, last = [], [], 0
    for m in TOOL_RE.finditer(text):
        try:
            obj = json.loads(m.group(1))
            calls.append(ToolCall(obj["name"], obj.get("arguments", obj.get("parameters", {})) or {}, m.group(0)))
            keep.append(text[last:m.start()])
            last = m.end()
        except (json.JSONDecodeError, KeyError):
            continue
    keep.append(text[last:])
    return "".join(keep).strip(), calls


class ToolRegistry:
    def __init__(self):
        self._tools: Dict[str, Callable[..., Any]] = {}

    def register(self, name: str, fn: Callable[..., Any]):
        self._tools[name] = fn

    def execute(self, call: ToolCall) -> str:
        if call.name not in self._tools:
            return json.dumps({"error": f"unknown tool {call.name}"})
        try:
            return json.dumps({"result": self._tools[call.name](**call.arguments)}, default=str)
        except Exception as e:  # tool errors go back to the model as observations
            return json.dumps({"error": f"{type(e).__name__}: {e}"})


class ToolReasonEnvWrapper:
    """Wraps a text env: strips reasoning, executes tool calls (their results become the observation) and forwards
    everything else to the env (gpatch_v4/agentic/env/tool_reason_env_wrapper.py)."""

    def __init__(self, env, tools: Optional[ToolRegistry] = None):
        self.env, self.tools = env, tools or ToolRegistry()

    def get_instructions(self):
        return self.env.get_instructions()

    def reset(self, seed=None):
        return self.env.reset(seed)

    def step(self, text: str):
        _, answer = split_reasoning(text)
        rest, calls = parse_tool_calls(answer)
        if calls:
            obs = "\n".join(f"<tool_response>{self.tools.execute(c)}</tool_response>" for c in calls)
            return obs, 0.0, False, False, {"action_is_valid": True, "tool_calls": len(calls), "success": False}
        return self.env.step(rest)
