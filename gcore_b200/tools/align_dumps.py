"""Working with the per-token dumps a GRPO / SFT run writes every ``training.ppo_dump_metrics_interval`` steps
(``token_dumps/step{N}_rank{R}.jsonl``: tokens, mask, trainer / reference / rollout log-probs, advantages, rewards).

* ``align``   - brings every field of one sample to the lengths the trainer uses: tokens ``[S]`` padded to the
  training pad multiple, everything that lives on the prediction axis ``[S - 1]`` (position t scores token t + 1), so
  that dumps of two frameworks can be laid side by side (the job of the reference's
  tools/align_dump_sample/align_sample.py:60-197).
* ``compare`` - two dump files (two runs, two back ends, two ranks of a replicated group): per field the number of
  compared samples, the largest absolute difference, and where the first difference above the tolerance sits.

    python -m gcore_b200.tools.align_dumps align --file step0000010_rank0.jsonl --sample 3 --pad-multiple 128
    python -m gcore_b200.tools.align_dumps compare --a run_a/step0000010_rank0.jsonl --b run_b/step0000010_rank0.jsonl
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List

PREDICTION_AXIS = ("mask", "logprobs", "ref_logprobs", "rollout_log_probs", "teacher_logprobs", "advantages", "values")


def read_dump(path: str) -> List[dict]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def _fit(xs: list, n: int, pad=0):
    return list(xs[:n]) + [pad] * max(0, n - len(xs))


def align_sample(row: dict, pad_multiple: int = 1, pad_token: int = 0) -> dict:
    """Tokens padded up to a multiple of ``pad_multiple`` (``S``); prediction-axis fields cut / zero-padded to
    ``S - 1``.  A field dumped on the token axis (length = number of tokens) drops its last, meaningless position."""
    n = len(row["tokens"])
    S = (n + pad_multiple - 1) // pad_multiple * pad_multiple
    out = {k: v for k, v in row.items() if not isinstance(v, list)}
    out["tokens"] = _fit(row["tokens"], S, pad_token)
    out["padded_seqlen"] = S
    for k in PREDICTION_AXIS:
        if k in row:
            out[k] = _fit(row[k], S - 1, 0.0)
    return out


def compare_dumps(a: List[dict], b: List[dict], atol: float = 1e-5) -> Dict[str, dict]:
    """Samples are matched by position in the file; a sample whose tokens differ is reported under ``tokens`` and its
    other fields are skipped (they would not be comparable)."""
    rep: Dict[str, dict] = {"samples": {"a": len(a), "b": len(b)}}

    def slot(k):
        return rep.setdefault(k, {"compared": 0, "max_abs_diff": 0.0, "first_difference": None})

    for i, (ra, rb) in enumerate(zip(a, b)):
        t = slot("tokens")
        t["compared"] += 1
        if ra["tokens"] != rb["tokens"]:
            if t["first_difference"] is None:
                n = min(len(ra["tokens"]), len(rb["tokens"]))
                pos = next((j for j in range(n) if ra["tokens"][j] != rb["tokens"][j]), n)
                t["first_difference"] = {"sample": i, "position": pos}
            t["max_abs_diff"] = float("inf")
            continue
        for k in PREDICTION_AXIS + ("reward",):
            if k not in ra or k not in rb:
                continue
            va = ra[k] if isinstance(ra[k], list) else [ra[k]]
            vb = rb[k] if isinstance(rb[k], list) else [rb[k]]
            s = slot(k)
            s["compared"] += 1
            if len(va) != len(vb):
                if s["first_difference"] is None:
                    s["first_difference"] = {"sample": i, "lengths": [len(va), len(vb)]}
                s["max_abs_diff"] = float("inf")
                continue
            for j, (x, y) in enumerate(zip(va, vb)):
                d = abs(float(x) - float(y))
                if d > s["max_abs_diff"]:
                    s["max_abs_diff"] = d
                if d > atol and s["first_difference"] is None:
                    s["first_difference"] = {"sample": i, "position": j, "a": x, "b": y}
    rep["equal"] = len(a) == len(b) and all(v["first_difference"] is None for k, v in rep.items()
                                            if isinstance(v, dict) and "first_difference" in v)
    return rep


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    al = sub.add_parser("align")
    al.add_argument("--file", required=True)
    al.add_argument("--sample", type=int, default=0)
    al.add_argument("--pad-multiple", type=int, default=128)
    cp = sub.add_parser("compare")
    cp.add_argument("--a", required=True)
    cp.add_argument("--b", required=True)
    cp.add_argument("--atol", type=float, default=1e-5)
    a = ap.parse_args(argv)
    if a.cmd == "align":
        print(json.dumps(align_sample(read_dump(a.file)[a.sample], a.pad_multiple)))
        return 0
    rep = compare_dumps(read_dump(a.a), read_dump(a.b), a.atol)
    print(json.dumps(rep, indent=1))
    return 0 if rep["equal"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
