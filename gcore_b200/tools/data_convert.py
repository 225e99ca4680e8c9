"""Data converters (the reference's data-conversion tools): bring text / chat records into the indexed-jsonl formats
the datasets read, tokenising once offline.

    python -m gcore_b200.tools.data_convert sft      --src chat.jsonl --dst sft.jsonl --tokenizer tok_dir
    python -m gcore_b200.tools.data_convert prompts  --src q.jsonl    --dst prompts.jsonl --tokenizer tok_dir
    python -m gcore_b200.tools.data_convert pretrain --src text.jsonl --dst tokens.jsonl --tokenizer tok_dir

``sft``: ``{"messages": [{"role", "content"}, ...]}``, the ShareGPT (``conversations``) and Alpaca (``instruction`` /
``input`` / ``output``) layouts of LLaMA-Factory datasets, or ``{"prompt", "response"}`` -> ``{"prompt": ids,
"response": ids}``; ``dpo``: preference records in the same layouts (``chosen`` / ``rejected``) -> ``{"prompt",
"chosen", "rejected"}`` ids; ``prompts``: ``{"prompt" | "question", "answer"}`` -> ``{"prompt": ids, "answer": ...}``; ``pretrain``:
``{"text"}`` -> ``{"tokens": ids}``.  Without ``--tokenizer`` a byte-level encoding (id = byte + 3) is used, which
keeps the tools usable in tests and for smoke runs.  The offset index (``.idx``) is written next to the output."""
from __future__ import annotations

import argparse
import json
from typing import Callable, List


def byte_tokenizer(text: str) -> List[int]:
    return [b + 3 for b in text.encode("utf-8")]


def load_tokenizer(path: str | None) -> Callable[[str], List[int]]:
    if not path:
        return byte_tokenizer
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(path)
    return lambda s: tok.encode(s, add_special_tokens=False)


_SHAREGPT_ROLES = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system",
                   "observation": "tool", "function_call": "assistant"}


def _messages(rec: dict) -> list:
    """Chat turns of a record in any of the accepted layouts: ``messages`` (role / content), the ShareGPT layout of
    LLaMA-Factory (``conversations`` of ``from`` / ``value``, optional ``system``), or the Alpaca layout
    (``instruction`` [+ ``input``] -> ``output``, optional ``system`` and ``history`` of [user, assistant] pairs)."""
    if "messages" in rec:
        return rec["messages"]
    if "conversations" in rec:
        msgs = [{"role": "system", "content": rec["system"]}] if rec.get("system") else []
        for t in rec["conversations"]:
            role = _SHAREGPT_ROLES.get(t.get("from", t.get("role")), "user")
            msgs.append({"role": role, "content": t.get("value", t.get("content", ""))})
        return msgs
    if "instruction" in rec:
        msgs = [{"role": "system", "content": rec["system"]}] if rec.get("system") else []
        for u, a in rec.get("history") or []:
            msgs += [{"role": "user", "content": u}, {"role": "assistant", "content": a}]
        q = rec["instruction"] + ("\n" + rec["input"] if rec.get("input") else "")
        msgs.append({"role": "user", "content": q})
        if "output" in rec and not isinstance(rec["output"], (list, tuple)):
            msgs.append({"role": "assistant", "content": rec["output"]})
        return msgs
    return None


def _render(msgs: list) -> str:
    return "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in msgs) + "<|assistant|>\n"


def _chat_to_pair(rec: dict) -> tuple:
    msgs = _messages(rec)
    if msgs is not None:
        last = max(i for i, m in enumerate(msgs) if m["role"] == "assistant")
        return _render(msgs[:last]), msgs[last]["content"]
    return rec["prompt"], rec["response"]


def _preference_triple(rec: dict) -> tuple:
    """(prompt, chosen, rejected) of a preference record: explicit ``prompt`` / ``chosen`` / ``rejected`` strings,
    ShareGPT / ``messages`` context with ``chosen`` / ``rejected`` turns ({"value" | "content"}), or the Alpaca layout
    with ``output = [chosen, rejected]``."""
    def text(x):
        return x if isinstance(x, str) else x.get("value", x.get("content", ""))
    if "instruction" in rec and isinstance(rec.get("output"), (list, tuple)):
        return _render(_messages(rec)), rec["output"][0], rec["output"][1]
    msgs = _messages(rec)
    prompt = _render(msgs) if msgs is not None else rec["prompt"]
    return prompt, text(rec["chosen"]), text(rec["rejected"])


def convert(kind: str, src: str, dst: str, encode: Callable[[str], List[int]], max_len: int | None = None) -> int:
    n = 0
    with open(src) as fi, open(dst, "w") as fo:
        for line in fi:
            if not line.strip():
                continue
            rec = json.loads(line)
            if kind == "sft":
                p, r = _chat_to_pair(rec)
                out = {"prompt": encode(p), "response": encode(r)}
                if max_len and len(out["prompt"]) + len(out["response"]) > max_len:
                    continue
            elif kind == "prompts":
                out = {"prompt": encode(rec.get("prompt") or rec["question"]), "answer": rec.get("answer")}
                if max_len and len(out["prompt"]) > max_len:
                    continue
            elif kind == "dpo":
                p, c, r = _preference_triple(rec)
                out = {"prompt": encode(p), "chosen": encode(c), "rejected": encode(r)}
                if max_len and len(out["prompt"]) + max(len(out["chosen"]), len(out["rejected"])) > max_len:
                    continue
            elif kind == "pretrain":
                out = {"tokens": encode(rec["text"])}
            else:
                raise ValueError(f"unknown conversion {kind}")
            fo.write(json.dumps(out) + "\n")
            n += 1
    from ..data.datasets import IndexedJsonlDataset
    IndexedJsonlDataset.build_index(dst, dst + ".idx")
    return n


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["sft", "prompts", "pretrain", "dpo"])
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--max-len", type=int, default=None)
    a = ap.parse_args(argv)
    n = convert(a.kind, a.src, a.dst, load_tokenizer(a.tokenizer), a.max_len)
    print(f"wrote {n} records to {a.dst}")
    return n


if __name__ == "__main__":
    main()
