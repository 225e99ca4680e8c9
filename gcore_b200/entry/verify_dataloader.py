"""Data-loader check (the reference's dataloader-verify main): walks the configured loader, reports batch / token
counts, and verifies that a loader resumed at ``consumed_batches = k`` yields exactly the batches the first one
yielded from ``k`` on, for every data-parallel rank.

``python -m gcore_b200.entry.verify_dataloader --config sft.yaml +verify.batches=8 +verify.dp_size=2``"""
import sys

import torch

from ..configs.config import FinetuneConfig, RlConfig
from ..data.datasets import default_dataset_fn
from ..configs.base import import_from_path
from ..utils.logging_utils import get_logger
from .common import load


def _fingerprint(batch) -> tuple:
    key = "tokens" if "tokens" in batch else "prompt_token_ids"
    rows = batch[key]
    out = []
    for r in rows:
        r = r["prompt_token_ids"] if isinstance(r, dict) else r
        t = torch.as_tensor(r)
        out.append((int(t.numel()), int(t.sum())))
    return tuple(out)


def verify(cfg, batches: int = 8, dp_size: int = 1, tokenizer=None) -> dict:
    fn = default_dataset_fn
    if cfg.data.py_path:
        fn = import_from_path(cfg.data.py_path, cfg.data.fn_name or "build_dataset")
    report = {"batches": batches, "dp_size": dp_size, "tokens": 0, "resume_ok": True, "disjoint_ok": True}
    seen_first = []
    for dp_rank in range(dp_size):
        full = fn(cfg, tokenizer, dp_rank, dp_size, None)
        it = iter(full["train_dataloader"])
        prints = []
        for _ in range(batches):
            try:
                prints.append(_fingerprint(next(it)))
            except StopIteration:
                break
        report["tokens"] += sum(n for b in prints for n, _ in b)
        k = len(prints) // 2
        resumed = fn(cfg, tokenizer, dp_rank, dp_size, {"consumed_batches": k, "resume_step": k})
        it2 = iter(resumed["train_dataloader"])
        again = [_fingerprint(next(it2)) for _ in range(len(prints) - k)]
        report["resume_ok"] &= again == prints[k:]
        seen_first.append(prints[0] if prints else ())
    report["disjoint_ok"] = len(set(seen_first)) == len(seen_first)
    return report


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    opts = {"batches": 8, "dp_size": 1, "kind": "sft"}
    for a in list(argv):
        if a.lstrip("+").startswith("verify."):
            k, v = a.lstrip("+")[len("verify."):].split("=", 1)
            opts[k] = v if k == "kind" else int(v)
            argv.remove(a)
    cfg = load(RlConfig if opts["kind"] == "rl" else FinetuneConfig, argv)
    rep = verify(cfg, opts["batches"], opts["dp_size"])
    get_logger("verify_dataloader").info(str(rep))
    print(rep)
    return rep


if __name__ == "__main__":
    r = main()
    sys.exit(0 if r["resume_ok"] and r["disjoint_ok"] else 1)
