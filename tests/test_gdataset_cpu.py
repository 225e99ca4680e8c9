"""Stores, feats, the streaming feat dataset, collators and the vision-language SFT dataset."""
import io
import json

import numpy as np
import torch

from gcore_b200.data.gdataset import (DictStore, GDataset, ImageFeat, JsonFeat, LocalFileStore, PackedFileStore,
                                      RemoteObjectStore, VideoFramesFeat, VlmSftDataset, pad_collate, patchify,
                                      store_provider, vlm_collate)


def _png(h, w, seed):
    from PIL import Image
    rng = np.random.RandomState(seed)
    buf = io.BytesIO()
    Image.fromarray(rng.randint(0, 255, (h, w, 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


def test_stores(tmp_path):
    (tmp_path / "a.bin").write_bytes(b"hello")
    assert LocalFileStore(root=str(tmp_path)).get(url="a.bin") == b"hello"
    assert isinstance(store_provider(root=str(tmp_path)), LocalFileStore)
    PackedFileStore.build(str(tmp_path / "pack"), {"x": b"12345", "y": b"abc"})
    st = store_provider(packed=True, path=str(tmp_path / "pack"))
    assert st.get(url="y") == b"abc" and st.get(url="x") == b"12345"
    assert store_provider(table={"k": b"v"}).get(url="k") == b"v"
    calls = []

    def flaky(url):
        calls.append(url)
        if len(calls) < 3:
            raise IOError("transient")
        return b"ok"

    assert RemoteObjectStore(fetch=flaky, retries=3).get(url="u") == b"ok" and len(calls) == 3


def test_feats_and_streaming_dataset_with_resume(tmp_path):
    table = {f"img{i}": _png(30 + i, 61, i) for i in range(6)}
    shards = []
    for s in range(2):
        p = tmp_path / f"s{s}.jsonl"
        with open(p, "w") as f:
            for i in range(3):
                k = s * 3 + i
                f.write(json.dumps({"id": k, "image": f"img{k}", "meta": json.dumps({"a": 1, "b": "[1, 2]"})}) + "\n")
        shards.append(str(p))
    feats = {"image": ImageFeat(table=table, multiple=28, min_pixels=28 * 28), "meta": JsonFeat()}
    ds = GDataset(shards, feats=feats, shuffle_buffer=4, seed=1)
    recs = list(ds)
    assert sorted(r["id"] for r in recs) == list(range(6))
    for r in recs:
        assert r["image"].dtype == np.float32 and r["image"].shape[0] % 28 == 0 and r["image"].shape[1] % 28 == 0
        assert r["meta"] == {"a": 1, "b": [1, 2]}
    # two data-parallel ranks split the stream; a resumed rank continues where it stopped
    a = [r["id"] for r in GDataset(shards, feats=feats, dp_rank=0, dp_size=2, shuffle_buffer=4, seed=1)]
    b = [r["id"] for r in GDataset(shards, feats=feats, dp_rank=1, dp_size=2, shuffle_buffer=4, seed=1)]
    assert sorted(a + b) == list(range(6)) and not set(a) & set(b)
    d1 = GDataset(shards, feats=feats, shuffle_buffer=4, seed=1)
    it = iter(d1)
    head = [next(it)["id"] for _ in range(2)]
    d2 = GDataset(shards, feats=feats, shuffle_buffer=4, seed=1)
    d2.load_state_dict(d1.state_dict())
    assert head + [r["id"] for r in d2] == [r["id"] for r in recs]


def test_image_resize_rule_and_video_frames():
    f = ImageFeat(table={}, multiple=28, min_pixels=56 * 56, max_pixels=28 * 28 * 16)
    assert f.target_size(100, 100) == (112, 112)
    h, w = f.target_size(1000, 500)                                   # capped by max_pixels, aspect kept
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 28 * 28 * 16 and h > w
    assert f.target_size(10, 10)[0] * f.target_size(10, 10)[1] >= 56 * 56
    table = {f"f{i}": _png(56, 84, 10 + i) for i in range(3)}
    v = VideoFramesFeat(table=table, multiple=28, min_pixels=28 * 28)
    v.post_init(None)
    frames = v.encode_example("video", ["f0", "f1", "f2"])
    assert frames.shape == (3, 56, 84, 3)
    patches, grid = patchify(frames, patch=14, merge=2, temporal=2)
    assert grid == (2, 4, 6) and patches.shape == (2 * 4 * 6, 3 * 2 * 14 * 14)   # the odd frame is repeated


def test_patch_orders_agree_up_to_permutation():
    img = np.random.RandomState(0).rand(56, 84, 3).astype(np.float32)
    raster, g = patchify(img, 14, 2, order="raster")
    merged, g2 = patchify(img, 14, 2, order="merged")
    assert g == g2 == (1, 4, 6)
    # raster patch (r, c) is the merged patch at block (r // 2, c // 2), position (r % 2, c % 2)
    for r in range(4):
        for c in range(6):
            j = ((r // 2) * 3 + c // 2) * 4 + (r % 2) * 2 + c % 2
            assert torch.equal(raster[r * 6 + c], merged[j])
    # a patch holds its pixels channel-major
    p00 = torch.as_tensor(img[:14, :14]).permute(2, 0, 1).reshape(-1)
    assert torch.equal(raster[0], p00)


def test_vlm_sft_dataset_feeds_the_vision_language_engine(tmp_path):
    from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
    from gcore_b200.engine.train_engine import TrainingEngine
    from gcore_b200.models.config import get_preset
    from gcore_b200.models.vlm import VisionConfig
    for i in range(4):
        (tmp_path / f"im{i}.png").write_bytes(_png(40 + 4 * i, 50, i))
    p = tmp_path / "vlm.jsonl"
    with open(p, "w") as f:
        for i in range(4):
            f.write(json.dumps({"image": f"im{i}.png", "prompt": [5, 6, 1023, 7], "response": [9 + i, 10, 11]}) + "\n")
    vc = VisionConfig(patch_size=14, hidden_size=64, num_layers=1, num_heads=2, ffn_hidden_size=128)
    ds = VlmSftDataset([str(p)], tokenizer=None, image_token_id=1023, patch=14, merge=2,
                       image_kw=dict(root=str(tmp_path), min_pixels=28 * 28))
    samples = list(ds)
    assert len(samples) == 4
    for s in samples:
        gh, gw = s["image_grid"]
        assert s["pixel_patches"].shape == (gh * gw, vc.patch_dim)
        assert int((s["tokens"] == 1023).sum()) == gh * gw // 4
        assert s["loss_mask"].sum() == 3
    batch = vlm_collate(samples)
    assert batch["pixel_patches"].shape[0] == sum(g[0] * g[1] for g in batch["image_grid"])
    dense = pad_collate(samples, multiple=8)
    assert dense["tokens"].shape[1] % 8 == 0 and dense["loss_mask"].sum() == 12
    pc = PolicyConfig(recompute="none", without_ref=True)
    eng = TrainingEngine(pc, OptimizerConfig(lr=1e-3, lr_decay_style="constant"), TrainingConfig(train_mbs=2, train_gbs=4),
                         model_cfg=get_preset("tiny_llama", dtype="float32"), vision_cfg=vc, image_token_id=1023)
    eng.setup_model_and_get_optimizer(seed=3)
    l0 = eng.finetune_step(samples)["lm_loss"]
    for _ in range(5):
        l1 = eng.finetune_step(samples)["lm_loss"]
    assert l1 < l0
