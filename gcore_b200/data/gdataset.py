"""Record stores, field decoders ("feats"), collators and the vision-language datasets built on the streaming jsonl
dataset (``data/datasets.py::StreamingJsonlDataset``: shuffle buffer, data-parallel + worker sharding,
consumed-offset resume).

The pieces follow the reference's ``gdataset`` package: a *store* fetches the bytes a record points to
(gdataset/store/*: local files, LMDB, key-value services, object storage, chosen by ``store_cli_provider``); a *feat*
turns one field of a record into its decoded form, lazily, inside the loader worker (gdataset/feat/*: JSON, PIL / cv2
images, video frames); ``GDataset`` applies a feat map to a record stream (gdataset/gdataset_v4.py:31); collators
assemble model inputs (gdataset/collate.py, data_loader/collator).  Remote object stores need credentials and SDKs
that are not on this machine: ``RemoteObjectStore`` takes the fetch function from the caller.
"""
from __future__ import annotations

import io
import json
import math
import os
from typing import Any, Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from .datasets import StreamingJsonlDataset, _encode


# ---------------------------------------------------------------------------------------------------- stores
class StoreClient:
    def get(self, url: str, **kw) -> bytes:
        raise NotImplementedError


class LocalFileStore(StoreClient):
    """Bytes of a file below ``root`` (the reference's local-file-system client)."""

    def __init__(self, metadata=None, root: str = "", **kw):
        self.root = root

    def get(self, url: str, **kw) -> bytes:
        with open(os.path.join(self.root, url) if self.root else url, "rb") as f:
            return f.read()


class DictStore(StoreClient):
    """In-memory key -> bytes (stands where a key-value service would; also what tests use)."""

    def __init__(self, metadata=None, table: Optional[Dict[str, bytes]] = None, **kw):
        self.table = dict(table or {})

    def get(self, url: str, **kw) -> bytes:
        return self.table[url]


class PackedFileStore(StoreClient):
    """One large file of concatenated blobs plus an index ``{key: (offset, length)}`` (a json file beside it): random
    access without one inode per sample, the access pattern an LMDB / union-db shard gives the reference."""

    def __init__(self, metadata=None, path: str = "", **kw):
        self.path = path
        self.index = {k: tuple(v) for k, v in json.load(open(path + ".index.json")).items()}
        self._f = None

    @staticmethod
    def build(path: str, blobs: Dict[str, bytes]):
        index, at = {}, 0
        with open(path, "wb") as f:
            for k, b in blobs.items():
                f.write(b)
                index[k] = (at, len(b))
                at += len(b)
        json.dump(index, open(path + ".index.json", "w"))

    def get(self, url: str, **kw) -> bytes:
        if self._f is None:          # opened lazily: one handle per loader worker
            self._f = open(self.path, "rb")
        off, n = self.index[url]
        self._f.seek(off)
        return self._f.read(n)


class RemoteObjectStore(StoreClient):
    """Object storage behind a caller-supplied ``fetch(url) -> bytes`` with retries (SDK and credentials are the
    caller's: none ship with this package)."""

    def __init__(self, metadata=None, fetch: Optional[Callable[[str], bytes]] = None, retries: int = 3, **kw):
        if fetch is None:
            raise ValueError("RemoteObjectStore needs a fetch(url) -> bytes function")
        self.fetch, self.retries = fetch, retries

    def get(self, url: str, **kw) -> bytes:
        err = None
        for _ in range(max(self.retries, 1)):
            try:
                return self.fetch(url)
            except Exception as e:  # noqa: BLE001
                err = e
        raise IOError(f"could not fetch {url!r} after {self.retries} attempts: {err}")


def store_provider(metadata=None, **kw) -> StoreClient:
    """Chooses the store from flags, in the reference's order of precedence (object store, packed shard, key-value,
    local files)."""
    if kw.get("remote"):
        return RemoteObjectStore(metadata, **kw)
    if kw.get("packed"):
        return PackedFileStore(metadata, **kw)
    if kw.get("table") is not None:
        return DictStore(metadata, **kw)
    return LocalFileStore(metadata, **kw)


# ---------------------------------------------------------------------------------------------------- feats
class Feat:
    """Decoder of one record field; ``post_init`` receives the dataset metadata once, ``encode_example`` runs per
    record inside the loader worker."""

    def post_init(self, metadata):
        pass

    def encode_example(self, key: str, value) -> Any:
        return value


class JsonFeat(Feat):
    """A field that holds JSON text (``nest``: strings inside the parsed object that are JSON themselves are parsed
    too, one level)."""

    def __init__(self, nest: bool = True):
        self.nest = nest

    def encode_example(self, key, value):
        obj = json.loads(value) if isinstance(value, (str, bytes)) else value
        if self.nest and isinstance(obj, dict):
            for k, v in list(obj.items()):
                if isinstance(v, str) and v[:1] in "[{":
                    try:
                        obj[k] = json.loads(v)
                    except ValueError:
                        pass
        return obj


class ImageFeat(Feat):
    """A field that names an image (path / key in a store, or a JSON string holding ``{"url": ...}``) -> float32
    array ``[H, W, 3]`` in [0, 1], optionally resized so that both sides are multiples of ``multiple`` and the pixel
    count stays within ``[min_pixels, max_pixels]`` (the smart-resize rule of the Qwen-VL processors)."""

    def __init__(self, field_value_is_json_str: bool = False, multiple: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 1280 * 28 * 28, **store_kw):
        self.json_str, self.multiple = field_value_is_json_str, multiple
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.store_kw, self.store = store_kw, None

    def post_init(self, metadata):
        self.store = store_provider(metadata, **self.store_kw)

    def target_size(self, h: int, w: int):
        m = self.multiple
        hh, ww = max(m, round(h / m) * m), max(m, round(w / m) * m)
        if hh * ww > self.max_pixels:
            beta = math.sqrt(h * w / self.max_pixels)
            hh, ww = max(m, math.floor(h / beta / m) * m), max(m, math.floor(w / beta / m) * m)
        elif hh * ww < self.min_pixels:
            beta = math.sqrt(self.min_pixels / (h * w))
            hh, ww = math.ceil(h * beta / m) * m, math.ceil(w * beta / m) * m
        return hh, ww

    def encode_example(self, key, value):
        from PIL import Image
        if self.store is None:
            self.post_init(None)
        url = json.loads(value)["url"] if self.json_str else value
        img = Image.open(io.BytesIO(self.store.get(url=url))).convert("RGB")
        hh, ww = self.target_size(img.height, img.width)
        if (hh, ww) != (img.height, img.width):
            img = img.resize((ww, hh), Image.BICUBIC)
        return np.asarray(img, dtype=np.float32) / 255.0


class VideoFramesFeat(ImageFeat):
    """A field that lists frame images (``[url, ...]``) -> ``[F, H, W, 3]``; every frame is resized like the first."""

    def encode_example(self, key, value):
        urls = json.loads(value) if isinstance(value, str) else list(value)
        first = super().encode_example(key, urls[0])
        frames = [first]
        from PIL import Image
        for u in urls[1:]:
            img = Image.open(io.BytesIO(self.store.get(url=u))).convert("RGB").resize((first.shape[1], first.shape[0]),
                                                                                    Image.BICUBIC)
            frames.append(np.asarray(img, dtype=np.float32) / 255.0)
        return np.stack(frames)


class TokenFeat(Feat):
    """Text (or ready token ids) -> token ids through the job's tokenizer."""

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer

    def encode_example(self, key, value):
        return _encode(self.tokenizer, value)


# ---------------------------------------------------------------------------------------------------- dataset
class GDataset(StreamingJsonlDataset):
    """Streaming records with a feat per field: ``feats = {"image": ImageFeat(root=...), "meta": JsonFeat()}``.
    Fields without a feat pass through; ``post`` (optional) maps the decoded record to the training sample."""

    def __init__(self, paths: Sequence[str], feats: Optional[Dict[str, Feat]] = None, metadata=None,
                 post: Optional[Callable[[dict], dict]] = None, **kw):
        self.feats = dict(feats or {})
        for f in self.feats.values():
            f.post_init(metadata)
        self.post = post
        super().__init__(paths, transform=self._decode, **kw)

    def _decode(self, rec: dict) -> dict:
        out = dict(rec)
        for k, f in self.feats.items():
            if k in rec and rec[k] is not None:
                out[k] = f.encode_example(k, rec[k])
        return self.post(out) if self.post is not None else out


# ---------------------------------------------------------------------------------------------------- vision-language
def patchify(image: np.ndarray, patch: int, merge: int = 2, temporal: int = 1, order: str = "raster"):
    """``[H, W, C]`` (or ``[F, H, W, C]``) in [0, 1] -> ``(patches [n, C * temporal * patch * patch], grid (t, h, w))``.
    ``order="raster"``: row-major over the patch grid (what ``models/vlm.py`` takes; its merger gathers the blocks
    itself).  ``order="merged"``: the patches of every ``merge x merge`` block adjacent (the order the Qwen-VL
    processors emit)."""
    x = torch.as_tensor(image, dtype=torch.float32)
    if x.dim() == 3:
        x = x[None]
    F, H, W, C = x.shape
    if F % temporal:
        x = torch.cat([x, x[-1:].expand(temporal - F % temporal, -1, -1, -1)])
        F = x.shape[0]
    gh, gw, gt = H // patch, W // patch, F // temporal
    assert gh % merge == 0 and gw % merge == 0, "image sides must be multiples of patch x merge"
    x = x[:, :gh * patch, :gw * patch].permute(0, 3, 1, 2)                                  # [F, C, H, W]
    if order == "merged":
        x = x.reshape(gt, temporal, C, gh // merge, merge, patch, gw // merge, merge, patch)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                 # t, h/m, w/m, m, m, C, temporal, p, p
    else:
        x = x.reshape(gt, temporal, C, gh, patch, gw, patch).permute(0, 3, 5, 2, 1, 4, 6)   # t, h, w, C, temporal, p, p
    return x.reshape(gt * gh * gw, C * temporal * patch * patch).contiguous(), (gt, gh, gw)


def build_vlm_sample(rec: dict, tokenizer, image_token_id: int, patch: int = 14, merge: int = 2,
                     image_field: str = "image", prompt_field: str = "prompt", response_field: str = "response",
                     placeholder: str = "<image>") -> dict:
    """Record with a decoded image and a prompt / response pair -> a training sample of the vision-language engine:
    the placeholder in the prompt expands to one image token per merged patch; loss on the response tokens."""
    patches, (gt, gh, gw) = patchify(rec[image_field], patch, merge)
    n_img = gt * gh * gw // (merge * merge)
    prompt = rec[prompt_field]
    if isinstance(prompt, str):
        before, _, after = prompt.partition(placeholder)
        ids = _encode(tokenizer, before) + [image_token_id] * n_img + _encode(tokenizer, after)
    else:   # token ids with one placeholder id marking the image position
        ids = []
        for t in prompt:
            ids += [image_token_id] * n_img if t == image_token_id else [int(t)]
    resp = _encode(tokenizer, rec[response_field])
    toks = torch.tensor(ids + resp, dtype=torch.int64)
    mask = torch.zeros(toks.numel(), dtype=torch.float32)
    mask[len(ids) - 1:toks.numel() - 1] = 1.0
    return {"tokens": toks, "loss_mask": mask, "prompt_length": len(ids), "pixel_patches": patches,
            "image_grid": (gh, gw) if gt == 1 else (gt, gh, gw)}


class VlmSftDataset(GDataset):
    """jsonl records ``{"image": <path or key>, "prompt": "... <image> ...", "response": "..."}`` -> samples with
    ``pixel_patches`` / ``image_grid`` that ``TrainingEngine.finetune_step`` and the GRPO trainer take (the role of the
    reference's Qwen2-VL / InternVL / Gemma-3 SFT datasets, megatron_datasets/)."""

    def __init__(self, paths, tokenizer, image_token_id: int, patch: int = 14, merge: int = 2, image_kw=None, **kw):
        feat = ImageFeat(multiple=patch * merge, **(image_kw or {}))
        super().__init__(paths, feats={"image": feat},
                         post=lambda r: build_vlm_sample(r, tokenizer, image_token_id, patch, merge), **kw)


# ---------------------------------------------------------------------------------------------------- collators
def pad_collate(batch: Sequence[dict], pad_id: int = 0, multiple: int = 1) -> Dict[str, torch.Tensor]:
    """Right-pads ``tokens`` / ``loss_mask`` to the longest sample (rounded up to ``multiple``); returns dense
    ``[B, L]`` tensors plus ``lengths`` (for consumers that do not pack)."""
    L = max(int(b["tokens"].numel()) for b in batch)
    L = (L + multiple - 1) // multiple * multiple
    toks = torch.full((len(batch), L), pad_id, dtype=torch.int64)
    mask = torch.zeros(len(batch), L, dtype=torch.float32)
    for i, b in enumerate(batch):
        n = b["tokens"].numel()
        toks[i, :n] = b["tokens"]
        if "loss_mask" in b:
            mask[i, :n] = b["loss_mask"]
    return {"tokens": toks, "loss_mask": mask, "lengths": torch.tensor([b["tokens"].numel() for b in batch])}


def list_collate(batch: Sequence[dict]) -> List[dict]:
    """Samples stay a list of dicts (what the packing engine consumes; images keep their own shapes)."""
    return list(batch)


def vlm_collate(batch: Sequence[dict]) -> Dict[str, Any]:
    """Tokens as a list (packed later), all images' patches concatenated, their grids in sample order."""
    out = {"tokens": [b["tokens"] for b in batch], "loss_mask": [b["loss_mask"] for b in batch],
           "prompt_lengths": [b["prompt_length"] for b in batch],
           "pixel_patches": torch.cat([b["pixel_patches"] for b in batch]) if batch else None,
           "image_grid": [b["image_grid"] for b in batch]}
    return out
