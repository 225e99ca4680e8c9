"""Start-up sanity checks (gpatch_v4/gdebug/ppo_padding_check.py, utils/training_utils.py:187-231): combinations of
settings that train but silently misalign tensors, and structural checks of rollout samples.  Mode ``off | warn |
abort``."""
from __future__ import annotations

from typing import List, Sequence

import torch

VALID_MODES = ("off", "warn", "abort")


def find_risky_settings(config) -> List[str]:
    risks: List[str] = []
    t, ppo = config.training, config.ppo
    critic = getattr(config, "critic", None)
    if ppo.advantage_type == "ppo" and critic is not None:
        p = config.policy
        if getattr(critic, "smart_pad_infer", False) and not getattr(p, "smart_pad_infer", False):
            risks.append("critic.smart_pad_infer=True with policy.smart_pad_infer=False: values and log-probs are "
                         "grouped differently and can end up with different padded lengths")
        if (getattr(p, "smart_pad_infer", False) and getattr(critic, "smart_pad_infer", False)
                and p.forward_only_mbs != critic.forward_only_mbs):
            risks.append(f"policy.forward_only_mbs={p.forward_only_mbs} != critic.forward_only_mbs="
                         f"{critic.forward_only_mbs} with smart_pad_infer on both")
    if getattr(ppo, "skip_prev_logps", False):
        keep = getattr(t, "sampling_keep_n", None) or t.sampling_repeat_n
        if t.train_gbs != t.rollout_gbs * keep:
            risks.append("skip_prev_logps=True needs strictly on-policy updates: train_gbs must equal rollout_gbs * "
                         "sampling_keep_n")
    if ppo.offpolicy_correction != "none" and t.rollout_max_staleness == 0 and not getattr(ppo, "use_rollout_logprobs",
                                                                                          True):
        risks.append("offpolicy_correction is set but rollout log-probs are not kept")
    return risks


def run_config_checks(config, mode: str = "warn", log=None) -> List[str]:
    assert mode in VALID_MODES, mode
    if mode == "off":
        return []
    risks = find_risky_settings(config)
    for r in risks:
        (log.warning if log else print)(f"[config check] {r}")
    if risks and mode == "abort":
        raise ValueError("risky configuration:\n" + "\n".join(risks))
    return risks


def check_rollout_batches(samples: Sequence[dict]) -> None:
    """Every sample: 1-D integer tokens, prompt_length inside the sequence, per-token fields as long as the tokens,
    mask zero on the prompt and on the last position."""
    for i, s in enumerate(samples):
        tok = torch.as_tensor(s["tokens"])
        assert tok.dim() == 1 and not tok.is_floating_point(), f"sample {i}: tokens must be a 1-D integer tensor"
        S, P = tok.numel(), int(s.get("prompt_length", 0))
        assert 0 < P <= S, f"sample {i}: prompt_length {P} outside (0, {S}]"
        for k in ("mask", "loss_mask", "logprobs", "ref_logprobs", "rollout_log_probs", "advantages"):
            if k in s and s[k] is not None:
                n = torch.as_tensor(s[k]).numel()
                assert n in (S, S - 1), f"sample {i}: field {k} has {n} entries for {S} tokens"
        if "mask" in s:
            m = torch.as_tensor(s["mask"]).float()
            assert float(m[:max(P - 1, 0)].sum()) == 0, f"sample {i}: mask covers prompt positions"
            if m.numel() == S:
                assert float(m[-1]) == 0, f"sample {i}: the last position has no target and must be masked"
