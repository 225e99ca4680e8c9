"""Datasets and samplers.

* ``ResumableDistributedSampler`` - DP-sharded, seeded shuffle per epoch, ``set_start_index`` to resume mid-epoch
  (the reference's resumable sampler, tasks/math_rl_v4/simple_dataset.py:104-188).
* ``IndexedJsonlDataset`` - jsonl with a byte-offset index file for O(1) random access and fast resume
  (megatron_datasets' indexed-jsonl datasets).
* ``SftDataset`` / ``PromptDataset`` - tokenise (or pass through pre-tokenised) SFT and RL-prompt records; collate
  functions produce the reference's batch contracts (``tokens, labels, sequence_lengths, prompt_lengths`` and
  ``prompt_token_ids, prompt_lens, gt_label``).
* ``PackedSftDataset`` - greedy packing of short samples up to ``seq_length`` tokens (pretrain-packed / SFT packing).
* ``SyntheticSftDataset`` / ``SyntheticPromptDataset`` - the benchmark recipes' random-token data.
* ``StreamingJsonlDataset`` - lazy multi-shard iterable dataset: DP / worker sharding, shuffle buffer, resume by
  consumed count.  ``PretrainTokenDataset`` - documents laid end to end and cut into fixed rows.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Callable, Dict, Iterator, List, Optional, Sequence

import torch
from torch.utils.data import Dataset, Sampler


class ResumableDistributedSampler(Sampler):
    def __init__(self, dataset_len: int, dp_rank: int = 0, dp_size: int = 1, shuffle: bool = True, seed: int = 42,
                 drop_last: bool = True):
        self.n, self.rank, self.size, self.shuffle, self.seed, self.drop_last = dataset_len, dp_rank, dp_size, shuffle, \
            seed, drop_last
        self.epoch = 0
        self.start_index = 0  # samples of this rank already consumed in the current epoch
        self.per_rank = self.n // self.size if drop_last else (self.n + self.size - 1) // self.size

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def set_start_index(self, idx: int):
        self.start_index = idx

    def state_dict(self):
        return {"epoch": self.epoch, "start_index": self.start_index}

    def load_state_dict(self, sd):
        self.epoch, self.start_index = sd["epoch"], sd["start_index"]

    def __len__(self):
        return max(self.per_rank - self.start_index, 0)

    def __iter__(self) -> Iterator[int]:
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            order = torch.randperm(self.n, generator=g).tolist()
        else:
            order = list(range(self.n))
        total = self.per_rank * self.size
        if len(order) < total:
            order += order[:total - len(order)]
        mine = order[self.rank:total:self.size]
        for i in mine[self.start_index:]:
            yield i
        self.start_index = 0


class IndexedJsonlDataset(Dataset):
    """``path`` + ``path.idx`` (little-endian uint64 byte offsets; built on first use)."""

    def __init__(self, path: str):
        self.path = path
        idx_path = path + ".idx"
        if not os.path.exists(idx_path) or os.path.getmtime(idx_path) < os.path.getmtime(path):
            self.build_index(path, idx_path)
        with open(idx_path, "rb") as f:
            raw = f.read()
        self.offsets = struct.unpack(f"<{len(raw) // 8}Q", raw)
        self._fh = None

    @staticmethod
    def build_index(path: str, idx_path: str):
        offs = []
        with open(path, "rb") as f:
            pos = 0
            for line in f:
                if line.strip():
                    offs.append(pos)
                pos += len(line)
        tmp = idx_path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(struct.pack(f"<{len(offs)}Q", *offs))
        os.replace(tmp, idx_path)

    def __len__(self):
        return len(self.offsets)

    def __getitem__(self, i):
        if self._fh is None:
            self._fh = open(self.path, "rb")
        self._fh.seek(self.offsets[i])
        return json.loads(self._fh.readline())


class StreamingJsonlDataset(torch.utils.data.IterableDataset):
    """Iterable dataset over several jsonl shards, read lazily: record ``k`` of the (epoch-shuffled) shard sequence
    belongs to data-parallel rank ``k % dp_size`` (and, inside a rank, to loader worker ``(k // dp_size) % workers``),
    records pass through a seeded shuffle buffer, an optional ``transform`` maps a raw record to a sample, and
    ``state_dict()`` records how many records this rank has handed out, so a resumed job skips exactly those and
    continues with the same stream (the reference's iterable dataset with shuffle buffer, DP sharding and
    consumed-offset resume: ``gdataset/``)."""

    def __init__(self, paths: Sequence[str], dp_rank: int = 0, dp_size: int = 1, shuffle_buffer: int = 0,
                 seed: int = 0, transform: Optional[Callable[[dict], dict]] = None, epochs: Optional[int] = 1):
        self.paths, self.rank, self.size = list(paths), dp_rank, dp_size
        self.buffer, self.seed, self.transform, self.epochs = shuffle_buffer, seed, transform, epochs
        self.consumed = 0   # records handed out by this rank since the beginning of training
        self._skip = 0

    def state_dict(self):
        return {"consumed": self.consumed}

    def load_state_dict(self, sd):
        self.consumed = self._skip = int(sd["consumed"])

    def _records(self, worker: int, workers: int):
        epoch = 0
        while self.epochs is None or epoch < self.epochs:
            order = list(range(len(self.paths)))
            if self.buffer:
                g = torch.Generator().manual_seed(self.seed + epoch)
                order = torch.randperm(len(order), generator=g).tolist()
            k = 0
            for pi in order:
                with open(self.paths[pi], "rb") as f:
                    for line in f:
                        if not line.strip():
                            continue
                        mine = k % self.size == self.rank and (k // self.size) % workers == worker
                        k += 1
                        if mine:
                            yield json.loads(line)
            epoch += 1

    def __iter__(self):
        info = torch.utils.data.get_worker_info()
        worker, workers = (info.id, info.num_workers) if info is not None else (0, 1)
        import random
        rng = random.Random(self.seed * 1000003 + self.rank * 1009 + worker)
        buf: List[dict] = []

        def shuffled():
            for rec in self._records(worker, workers):
                if not self.buffer:
                    yield rec
                    continue
                buf.append(rec)
                if len(buf) >= self.buffer:
                    yield buf.pop(rng.randrange(len(buf)))
            while buf:
                yield buf.pop(rng.randrange(len(buf)))

        skip = self._skip // workers + (1 if worker < self._skip % workers else 0)
        for n, rec in enumerate(shuffled()):
            if n < skip:      # replay the stream up to the resume point: same buffer state as the interrupted run
                continue
            self.consumed += 1
            yield self.transform(rec) if self.transform is not None else rec


def _encode(tokenizer, text_or_ids) -> List[int]:
    if isinstance(text_or_ids, (list, tuple)):
        return list(text_or_ids)
    if tokenizer is None:
        raise ValueError("text sample but no tokenizer")
    return tokenizer.encode(text_or_ids, add_special_tokens=False)


class SftDataset(Dataset):
    """Records: ``{"prompt": str | [ids], "response": str | [ids]}``; loss on the response only."""

    def __init__(self, records, tokenizer=None, max_len: int = 2048, prompt_key="prompt", response_key="response"):
        self.records, self.tok, self.max_len, self.pk, self.rk = records, tokenizer, max_len, prompt_key, response_key

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        r = self.records[i]
        p, a = _encode(self.tok, r[self.pk]), _encode(self.tok, r[self.rk])
        ids = (p + a)[:self.max_len]
        pl = min(len(p), len(ids))
        toks = torch.tensor(ids, dtype=torch.int64)
        labels = toks.clone()
        labels[:pl] = -100
        return {"tokens": toks, "labels": labels, "prompt_length": pl, "sequence_length": len(ids)}


def sft_collate(batch: Sequence[dict]) -> Dict[str, list]:
    return {"tokens": [b["tokens"] for b in batch], "labels": [b["labels"] for b in batch],
            "sequence_lengths": [b["sequence_length"] for b in batch],
            "prompt_lengths": [b["prompt_length"] for b in batch]}


class PromptDataset(Dataset):
    """RL prompts: ``{"prompt": str | [ids], "answer": any}``."""

    def __init__(self, records, tokenizer=None, max_prompt_length: int = 1024, prompt_key="prompt", label_key="answer"):
        self.records, self.tok, self.max_len, self.pk, self.lk = records, tokenizer, max_prompt_length, prompt_key, label_key

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        r = self.records[i]
        ids = _encode(self.tok, r[self.pk])[-self.max_len:]
        return {"prompt_token_ids": ids, "gt_label": r.get(self.lk), "index": i}


def prompt_collate(batch: Sequence[dict]) -> Dict[str, list]:
    return {"prompt_token_ids": [{"prompt_token_ids": b["prompt_token_ids"]} for b in batch],
            "prompt_lens": [len(b["prompt_token_ids"]) for b in batch], "gt_label": [b["gt_label"] for b in batch]}


class PackedSftDataset(Dataset):
    """Greedy first-fit packing of an SFT dataset into rows of at most ``seq_length`` tokens; every row keeps the
    boundaries of its members so attention stays block-diagonal (``cu_seqlens``)."""

    def __init__(self, base: Dataset, seq_length: int):
        self.base, self.seq_length = base, seq_length
        lens = [min(int(base[i]["sequence_length"]), seq_length) for i in range(len(base))]
        from ..core.packing import ffd_pack
        self.rows = ffd_pack(lens, seq_length)

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        members = [self.base[j] for j in self.rows[i]]
        return {"members": members, "num_tokens": sum(m["sequence_length"] for m in members)}


class PretrainTokenDataset(Dataset):
    """Pre-training rows: the documents of an indexed jsonl file (``{"tokens": [...]}`` or ``{"text": ...}`` lines) are
    laid end to end (an optional separator id between them) and cut into rows of ``seq_length`` tokens; the loss covers
    every token.  The (document, offset) of each row start is computed once from the document lengths, so a resumed
    job seeks straight to its row (the reference's indexed-jsonl pretrain datasets with an offset index:
    ``megatron_datasets/``)."""

    def __init__(self, base: Dataset, tokenizer, seq_length: int, eod_id: Optional[int] = None, key: str = "tokens"):
        self.base, self.tokenizer, self.seq_length, self.eod, self.key = base, tokenizer, seq_length, eod_id, key
        lens = [len(self._doc(i)) for i in range(len(base))]
        self.starts, pos = [], 0                       # global token offset of every document
        for n in lens:
            self.starts.append(pos)
            pos += n
        self.total = pos
        self.n_rows = self.total // seq_length

    def _doc(self, i) -> List[int]:
        row = self.base[i]
        ids = _encode(self.tokenizer, row[self.key] if self.key in row else row.get("text"))
        return ids + ([self.eod] if self.eod is not None else [])

    def __len__(self):
        return self.n_rows

    def __getitem__(self, r):
        import bisect
        lo = r * self.seq_length
        d = bisect.bisect_right(self.starts, lo) - 1
        out: List[int] = []
        off = lo - self.starts[d]
        while len(out) < self.seq_length:
            doc = self._doc(d)
            out += doc[off:off + self.seq_length - len(out)]
            d, off = d + 1, 0
        t = torch.tensor(out, dtype=torch.int64)
        return {"tokens": t, "labels": t.clone(), "prompt_length": 0, "sequence_length": t.numel()}


def pretrain_dataset_fn(config, tokenizer, dp_rank: int, dp_size: int, meta_info: Optional[dict] = None) -> dict:
    """``default_dataset_fn`` for pre-training: token-stream rows (or synthetic rows) with the loss on all tokens."""
    d, t = config.data, config.training
    syn = dict(d.synthetic or {})
    if d.train_data_path:
        ds = PretrainTokenDataset(IndexedJsonlDataset(d.train_data_path), tokenizer, t.seq_length,
                                  syn.get("eod_id"), syn.get("key", "tokens"))
    else:
        L = syn.get("seq_len", t.seq_length)
        ds = SyntheticSftDataset(syn.get("num_samples", 1024), L, syn.get("lo", 3), syn.get("hi", 1024), L, seed=d.seed)
    bs = t.train_gbs // max(dp_size, 1)
    sampler = ResumableDistributedSampler(len(ds), dp_rank, dp_size, d.shuffle, d.seed)
    if meta_info and meta_info.get("consumed_batches"):
        per_epoch = max(sampler.per_rank // bs, 1)
        sampler.set_epoch(meta_info["consumed_batches"] // per_epoch)
        sampler.set_start_index((meta_info["consumed_batches"] % per_epoch) * bs)
    dl = build_dataloader(ds, sampler, bs, sft_collate, d.num_workers)
    return {"train_dataset": ds, "train_sampler": sampler, "train_dataloader": dl, "eval_dataset": None,
            "eval_dataloader": None}


class SyntheticSftDataset(Dataset):
    """Sequences of ``seq_len`` token ids uniform in [lo, hi); the loss mask covers the last ``loss_tokens`` tokens."""

    def __init__(self, n: int, seq_len: int = 512, lo: int = 3, hi: int = 1024, loss_tokens: int = 256, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.tokens = torch.randint(lo, hi, (n, seq_len), generator=g)
        self.prompt_len = seq_len - loss_tokens

    def __len__(self):
        return self.tokens.shape[0]

    def __getitem__(self, i):
        t = self.tokens[i]
        labels = t.clone()
        labels[:self.prompt_len] = -100
        return {"tokens": t, "labels": labels, "prompt_length": self.prompt_len, "sequence_length": t.numel()}


class SyntheticPromptDataset(Dataset):
    def __init__(self, n: int, prompt_len: int = 256, lo: int = 100, hi: int = 150000, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.tokens = torch.randint(lo, hi, (n, prompt_len), generator=g)

    def __len__(self):
        return self.tokens.shape[0]

    def __getitem__(self, i):
        return {"prompt_token_ids": self.tokens[i].tolist(), "gt_label": None, "index": i}


def build_dataloader(dataset: Dataset, sampler: Sampler, batch_size: int, collate_fn: Callable, num_workers: int = 0):
    return torch.utils.data.DataLoader(dataset, batch_size=batch_size, sampler=sampler, collate_fn=collate_fn,
                                       num_workers=num_workers, drop_last=True)


def default_dataset_fn(config, tokenizer, dp_rank: int, dp_size: int, meta_info: Optional[dict] = None) -> dict:
    """The plug-in contract of ``data.py_path`` / ``data.fn_name``: returns ``{train_dataset, train_sampler,
    train_dataloader, eval_dataset, eval_dataloader}``; resumes from ``meta_info["consumed_batches"]``."""
    d = config.data
    rl = hasattr(config, "ppo")
    syn = dict(d.synthetic or {})
    if d.train_data_path:
        raw = IndexedJsonlDataset(d.train_data_path)
        ds = (PromptDataset(raw, tokenizer, d.max_prompt_length, d.prompt_key, d.label_key) if rl
              else SftDataset(raw, tokenizer, config.training.seq_length, d.prompt_key, "response"))
    elif rl:
        ds = SyntheticPromptDataset(syn.get("num_samples", 1024), syn.get("prompt_len", 256), syn.get("lo", 100),
                                    syn.get("hi", 150000), seed=d.seed)
    else:
        ds = SyntheticSftDataset(syn.get("num_samples", 1024), syn.get("seq_len", 512), syn.get("lo", 3),
                                 syn.get("hi", 1024), syn.get("loss_tokens", 256), seed=d.seed)
    t = config.training
    bs = (t.rollout_gbs if rl else t.train_gbs) // max(dp_size, 1)
    sampler = ResumableDistributedSampler(len(ds), dp_rank, dp_size, d.shuffle, d.seed)
    if meta_info and meta_info.get("consumed_batches"):
        per_epoch = max(sampler.per_rank // bs, 1)
        sampler.set_epoch(meta_info["consumed_batches"] // per_epoch)
        sampler.set_start_index((meta_info["consumed_batches"] % per_epoch) * bs)
    dl = build_dataloader(ds, sampler, bs, prompt_collate if rl else sft_collate, d.num_workers)
    eval_ds = eval_dl = None
    if rl and (d.eval_data_path or syn.get("eval_num_samples")):
        # held-out prompts for the periodic evaluation: fixed order, sharded over the data-parallel ranks
        if d.eval_data_path:
            eval_ds = PromptDataset(IndexedJsonlDataset(d.eval_data_path), tokenizer, d.max_prompt_length,
                                    d.prompt_key, d.label_key)
        else:
            eval_ds = SyntheticPromptDataset(int(syn["eval_num_samples"]), syn.get("prompt_len", 256),
                                             syn.get("lo", 100), syn.get("hi", 150000), seed=d.seed + 7919)
        eval_sampler = ResumableDistributedSampler(len(eval_ds), dp_rank, dp_size, False, d.seed)
        eval_dl = build_dataloader(eval_ds, eval_sampler, bs, prompt_collate, 0)
    return {"train_dataset": ds, "train_sampler": sampler, "train_dataloader": dl, "eval_dataset": eval_ds,
            "eval_dataloader": eval_dl}
