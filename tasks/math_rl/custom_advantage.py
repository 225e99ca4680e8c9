"""Example of a user-supplied advantage function (``ppo.custom_advantage_py_path`` / ``custom_advantage_py_name``):
leave-one-out baseline inside each prompt group, broadcast over the response tokens (the role of the reference's
tasks/math_rl_v4/custom_advantage.py).  Called as ``fn(samples, ppo_cfg, dp_group)``; sets ``advantages`` (and
``returns``) on every sample and returns the list."""
from collections import defaultdict

import torch


def leave_one_out_advantage(samples, ppo_cfg, dp_group=None):
    groups = defaultdict(list)
    for s in samples:
        groups[s.get("group_id", 0)].append(s)
    for members in groups.values():
        r = torch.stack([torch.as_tensor(s["rewards"], dtype=torch.float32).sum() for s in members])
        n = r.numel()
        for i, s in enumerate(members):
            base = (r.sum() - r[i]) / (n - 1) if n > 1 else r.new_zeros(())
            mask = torch.as_tensor(s["mask"], dtype=torch.float32)
            s["advantages"] = (r[i] - base) * mask
            s["returns"] = s["advantages"].clone()
    return samples
