"""Prompt dataset of the math recipe: a jsonl file with {"prompt": str | [token ids], "answer": str} lines, or a
synthetic stream when no file is configured (the counterpart of the reference's tasks/math_rl_v4/simple_dataset.py and
dapo_dataset.py).  Returns the dict contract of ``data.datasets.default_dataset_fn``."""
from gcore_b200.data.datasets import default_dataset_fn


def build_dataset(config, tokenizer, dp_rank, dp_size, meta_info=None):
    return default_dataset_fn(config, tokenizer, dp_rank, dp_size, meta_info)
