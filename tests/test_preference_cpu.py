"""DPO, Bradley-Terry reward-model training and teacher log-prob attachment on a tiny CPU model."""
import torch

from gcore_b200.configs.config import OptimizerConfig, PolicyConfig, TrainingConfig
from gcore_b200.engine.train_engine import TrainingEngine
from gcore_b200.models.config import get_preset
from gcore_b200.trainer.preference_trainers import attach_teacher_logprobs, dpo_step, rm_step


def _engine(value_head=False, with_ref=False, lr=2e-3, seed=3):
    e = TrainingEngine(PolicyConfig(recompute="none", without_ref=not with_ref),
                       OptimizerConfig(lr=lr, lr_decay_style="constant", weight_decay=0.0), TrainingConfig(train_mbs=4),
                       model_cfg=get_preset("tiny_llama", dtype="float32"), value_head=value_head)
    e.setup_model_and_get_optimizer(seed=seed, with_ref=with_ref)
    return e


def _pairs(n, seed):
    g = torch.Generator().manual_seed(seed)
    chosen, rejected = [], []
    for _ in range(n):
        prompt = torch.randint(3, 1024, (6,), generator=g)
        # chosen answers live in the low half of the vocabulary, rejected ones in the high half: learnable preference
        c = torch.randint(3, 400, (8,), generator=g)
        r = torch.randint(600, 1024, (8,), generator=g)
        chosen.append({"tokens": torch.cat([prompt, c]), "prompt_length": 6})
        rejected.append({"tokens": torch.cat([prompt, r]), "prompt_length": 6})
    return chosen, rejected


def test_dpo_lowers_loss_and_raises_reward_accuracy():
    e = _engine(with_ref=True)
    first = last = None
    for step in range(12):
        c, r = _pairs(8, 100 + step % 3)
        m = dpo_step(e, c, r, beta=0.5)
        first = first or m
        last = m
    loss_key = [k for k in last if "loss" in k][0]
    assert last[loss_key] < first[loss_key]
    acc_key = [k for k in last if "acc" in k]
    if acc_key:
        assert last[acc_key[0]] >= first[acc_key[0]]


def test_reward_model_learns_to_rank():
    e = _engine(value_head=True)
    first = last = None
    for step in range(15):
        c, r = _pairs(8, 200 + step % 3)
        m = rm_step(e, c, r)
        first = first or m
        last = m
    loss_key = [k for k in last if "loss" in k][0]
    assert last[loss_key] < first[loss_key]


def test_teacher_logprobs_are_attached_per_token():
    teacher = _engine(seed=9)
    c, _ = _pairs(3, 5)
    out = attach_teacher_logprobs(teacher, c)
    for s in out:
        key = [k for k in s if "teacher" in k][0]
        assert s[key].numel() == s["tokens"].numel() and bool((s[key][:-1] <= 0).all())
