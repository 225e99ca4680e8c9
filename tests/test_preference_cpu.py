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


def test_embedding_step_with_gradient_cache_equals_direct_step():
    from gcore_b200.trainer.preference_trainers import embed, embedding_step
    g = torch.Generator().manual_seed(2)
    topics = torch.randint(3, 1000, (6, 5), generator=g)
    mk = lambda t: {"tokens": torch.cat([t, torch.randint(3, 1000, (3,), generator=g)])}  # noqa: E731
    q, p = [mk(t) for t in topics], [mk(t) for t in topics]
    outs = []
    for cached in (False, True):
        e = _engine(seed=4)
        e.train_cfg.train_mbs = 2          # several micro-batches, so the cache actually splits the work
        m = embedding_step(e, q, p, temperature=0.1, grad_cache=cached)
        outs.append((m, [b.grad_data.detach().clone() for b in e.ddp.buffers]))   # the reduced gradients
    (ma, pa), (mb, pb) = outs
    assert abs(ma["embedding/loss"] - mb["embedding/loss"]) < 1e-5
    assert abs(ma["grad_norm"] - mb["grad_norm"]) < 1e-4 * max(1.0, ma["grad_norm"])
    for a, b in zip(pa, pb):
        assert float(a.abs().max()) > 0 and torch.allclose(a, b, atol=1e-5 * float(a.abs().max()))
    v = embed(_engine(seed=4), q)
    assert v.shape[0] == 6 and torch.allclose(v.norm(dim=-1), torch.ones(6), atol=1e-5)
