"""Dataset plug-in of the vision-language SFT recipe: jsonl records ``{"image": path, "prompt": "... <image> ...",
"response": "..."}`` streamed through ``VlmSftDataset`` (shuffle buffer, data-parallel sharding, resume by consumed
count)."""
import glob
import os

from gcore_b200.data.gdataset import VlmSftDataset, list_collate


def build_dataset(config, tokenizer, dp_rank, dp_size, meta_info=None):
    import torch
    path = config.data.train_data_path
    shards = sorted(glob.glob(os.path.join(path, "*.jsonl"))) if os.path.isdir(path) else [path]
    vc = config.policy.vision_config or {}
    ds = VlmSftDataset(shards, tokenizer, config.policy.image_token_id, patch=vc.get("patch_size", 14),
                       merge=vc.get("spatial_merge", 2), image_kw={"root": os.path.dirname(shards[0])},
                       dp_rank=dp_rank, dp_size=dp_size, shuffle_buffer=1024, seed=config.training.seed, epochs=None)
    if meta_info and "consumed_batches" in meta_info:
        per_rank = max(config.training.train_gbs // max(dp_size, 1), 1)
        ds.load_state_dict({"consumed": meta_info["consumed_batches"] * per_rank})
    loader = torch.utils.data.DataLoader(ds, batch_size=max(config.training.train_gbs // max(dp_size, 1), 1),
                                         collate_fn=list_collate, num_workers=0)
    return {"train_dataloader": loader, "train_sampler": None, "dataset": ds}
