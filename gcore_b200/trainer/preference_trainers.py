"""Preference / reward-model / distillation steps built on ``TrainingEngine`` primitives.

* ``dpo_step``      - DPO on (chosen, rejected) pairs with a frozen reference (``DpoTrainer`` / ``DpoActor``,
  gpatch_v4/training_backend/loss_factory.py DPO losses): sequence log-probs from the packed forward.
* ``rm_step``       - Bradley-Terry reward-model training with a value-head engine (``RewardTrainer``).
* ``distill_step``  - on-policy distillation: student rollouts scored by a teacher engine; the per-token advantage is
  the teacher-student log-prob gap (``advantage_type=on_policy_distill``); off-policy distillation is SFT on teacher
  samples with an optional reverse-KL term on top-k teacher log-probs.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch
import torch.distributed as dist

from ..core import parallel_state as ps
from ..engine.train_engine import TrainingEngine, backend_scope
from ..loss import policy_loss as PL


def _whole_stream(x: torch.Tensor, mb) -> torch.Tensor:
    """Per-token outputs of a context-parallel shard -> the whole packed stream on every rank of the group (sequence
    ends and pooled means index global positions).  Every rank then computes the same loss; the gather's backward adds
    the ranks' copies up, which the gradient reduction's division by the group size undoes."""
    if mb.cp_ctx is None:
        return x
    from ..parallel.cp import gather_from_cp
    return gather_from_cp(x.contiguous(), mb.cp_ctx.group)


def _seq_logps(engine: TrainingEngine, model, samples: Sequence[dict], grad: bool) -> torch.Tensor:
    """Sum of masked token log-probs per sample, differentiable when ``grad``."""
    out = []
    ctx = torch.enable_grad() if grad else torch.no_grad()
    with ctx, backend_scope(engine.backend):
        for idx in engine._microbatches(samples, forward_only=not grad):
            mb = engine._pack(samples, idx)
            hidden, _ = engine._hidden(model, mb)
            lp, _ = engine._logprob_entropy(model, hidden, mb.targets, False, mb.loss_mask)
            seg = torch.zeros(mb.num_seqs + 1, dtype=lp.dtype, device=lp.device).index_add(0, mb.seq_ids.long(),
                                                                                           lp * mb.loss_mask)
            if mb.cp_ctx is not None:
                # a sequence's tokens are spread over the context-parallel ranks: every rank needs the whole sum for the
                # (non-linear) preference loss, and sends gradient back only into its own tokens
                from ..parallel.cp import all_reduce_cp
                seg = all_reduce_cp(seg, mb.cp_ctx.group)
            out.append((idx, seg[:len(idx)]))
    res = [None] * len(samples)
    for idx, seg in out:
        for j, i in enumerate(idx):
            res[i] = seg[j]
    return torch.stack(res)


def dpo_step(engine: TrainingEngine, chosen: List[dict], rejected: List[dict], beta: float = 0.1,
             label_smoothing: float = 0.0, reference_free: bool = False, sft_coef: float = 0.0) -> Dict[str, float]:
    assert len(chosen) == len(rejected)
    engine.model.train()
    engine.ddp.zero_grad_buffer()
    allc = list(chosen) + list(rejected)
    if reference_free or engine.ref_model is None:
        ref = torch.zeros(len(allc), device=engine.device)
    else:
        ref = _seq_logps(engine, engine.ref_model, allc, grad=False)
    pol = _seq_logps(engine, engine.model, allc, grad=True)
    n = len(chosen)
    loss, m = PL.dpo_loss(pol[:n], pol[n:], ref[:n], ref[n:], beta, label_smoothing, reference_free)
    if sft_coef:
        def resp_tokens(s):
            m = s.get("loss_mask", s.get("mask"))
            if m is not None:
                return float(torch.as_tensor(m).sum())
            return float(len(s["tokens"]) - int(s.get("prompt_length", 0)))
        ntok = sum(resp_tokens(s) for s in chosen)
        dpw = ps.get_data_parallel_world_size()
        if dpw > 1:
            # token mean over the global batch: (sum of all replicas' tokens) / dp is what the gradient average needs
            t = torch.tensor([ntok], dtype=torch.float64, device=engine.device)
            dist.all_reduce(t, group=ps.get_data_parallel_group())
            ntok = float(t) / dpw
        loss = loss - sft_coef * pol[:n].sum() / max(ntok, 1.0)
    loss.backward()
    # the loss is the mean over this data-parallel rank's pairs (averaged over the replicas by the reduction); the
    # context-parallel ranks of one replica hold parts of the same gradient, which add up
    engine.ddp.finish_grad_sync(extra_scale=float(ps.get_context_parallel_world_size()))
    lr = engine.optimizer.step()
    engine.step += 1
    shown = loss.detach().clone()
    if ps.get_data_parallel_world_size() > 1:
        dist.all_reduce(shown, group=ps.get_data_parallel_group())
        shown /= ps.get_data_parallel_world_size()
    out = {"dpo/loss": float(shown), "lr": lr, "grad_norm": float(engine.optimizer.last_grad_norm)}
    out.update({k: float(v) for k, v in m.items()})
    return out


def rm_step(engine: TrainingEngine, chosen: List[dict], rejected: List[dict], margin: float = 0.0) -> Dict[str, float]:
    """``engine`` has a value head; the score of a sequence is the head's output at its last token."""
    assert engine.value_head
    engine.model.train()
    engine.ddp.zero_grad_buffer()
    allc = list(chosen) + list(rejected)
    scores = []
    with backend_scope(engine.backend):
        for idx in engine._microbatches(allc):
            mb = engine._pack(allc, idx)
            v, _ = engine._hidden(engine.model, mb)
            v = _whole_stream(v, mb)
            last = (mb.cu_seqlens[1:len(idx) + 1] - 1).long()
            scores.append((idx, v[last]))
    s = [None] * len(allc)
    for idx, sc in scores:
        for j, i in enumerate(idx):
            s[i] = sc[j]
    s = torch.stack(s)
    n = len(chosen)
    loss, m = PL.rm_bt_loss(s[:n], s[n:], margin)
    loss.backward()
    engine.ddp.finish_grad_sync(extra_scale=1.0)
    lr = engine.optimizer.step()
    engine.step += 1
    return {"rm/loss": float(loss.detach()), "rm/acc": float(m["rm/acc"]), "lr": lr}


def attach_teacher_logprobs(teacher: TrainingEngine, samples: List[dict]) -> List[dict]:
    """Scores student samples under the teacher (forward only) -> ``teacher_logprobs`` for ``on_policy_distill``."""
    teacher.compute_log_probs(samples, use_ref=False, with_entropy=False, out_key="teacher_logprobs")
    return samples


def _pooled(engine: TrainingEngine, samples: Sequence[dict], grad: bool, pooling: str = "last") -> torch.Tensor:
    """One unit-norm vector per sequence: the final hidden state of its last token, or the mean over its tokens."""
    out = []
    ctx = torch.enable_grad() if grad else torch.no_grad()
    with ctx, backend_scope(engine.backend):
        for idx in engine._microbatches(samples, forward_only=not grad):
            mb = engine._pack(samples, idx)
            h, _ = engine._hidden(engine.model, mb)
            h = _whole_stream(h, mb)
            if grad and getattr(engine.model, "sequence_parallel", False):
                # pooling and the contrastive loss are repeated in full on every TP rank, so every rank back-propagates
                # the whole gradient into the gathered hidden states
                from ..core import parallel_state as ps
                from ..parallel.tp_ops import replicated_consumer_of_gathered
                h = replicated_consumer_of_gathered(h, ps.get_tensor_model_parallel_group())
            if pooling == "mean":
                n = mb.num_seqs + 1
                sid = _whole_stream(mb.seq_ids, mb).long()
                seg = torch.zeros(n, h.shape[1], dtype=torch.float32, device=h.device).index_add(
                    0, sid, h.float())
                cnt = torch.zeros(n, dtype=torch.float32, device=h.device).index_add(
                    0, sid, torch.ones(h.shape[0], device=h.device))
                vec = seg[:len(idx)] / cnt[:len(idx), None].clamp_min(1.0)
            else:
                vec = h[(mb.cu_seqlens[1:len(idx) + 1] - 1).long()].float()
            out.append((idx, torch.nn.functional.normalize(vec, dim=-1)))
    res = [None] * len(samples)
    for idx, v in out:
        for j, i in enumerate(idx):
            res[i] = v[j]
    return torch.stack(res)


def _info_nce(vec: torch.Tensor, n: int, temperature: float):
    sim = vec[:n] @ vec[n:].t() / temperature
    tgt = torch.arange(n, device=sim.device)
    loss = 0.5 * (torch.nn.functional.cross_entropy(sim, tgt) + torch.nn.functional.cross_entropy(sim.t(), tgt))
    return loss, sim, tgt


def embedding_step(engine: TrainingEngine, queries: List[dict], positives: List[dict], temperature: float = 0.05,
                   pooling: str = "last", grad_cache: bool = False) -> Dict[str, float]:
    """Contrastive embedding training (the reference's embedding main): query ``i`` must pick ``positives[i]`` among
    all positives of the batch (in-batch negatives, symmetric InfoNCE on cosine similarity / ``temperature``).

    ``grad_cache``: the batch of negatives can be much larger than what fits in memory with activations kept.  All
    vectors are first computed without a graph, the loss is differentiated with respect to the vectors only, and each
    micro-batch is then run again with a graph and back-propagated through ``sum(vector * cached gradient)``; the
    parameter gradients are the same as those of the direct computation."""
    assert len(queries) == len(positives)
    engine.model.train()
    engine.ddp.zero_grad_buffer()
    n = len(queries)
    allc = list(queries) + list(positives)
    if grad_cache:
        vec = _pooled(engine, allc, False, pooling).detach().requires_grad_(True)
        loss, sim, tgt = _info_nce(vec, n, temperature)
        loss.backward()
        g = vec.grad
        with backend_scope(engine.backend):
            for idx in engine._microbatches(allc):
                part = _pooled(engine, [allc[i] for i in idx], True, pooling)
                (part * g[torch.tensor(idx, device=g.device)]).sum().backward()
    else:
        vec = _pooled(engine, allc, True, pooling)
        loss, sim, tgt = _info_nce(vec, n, temperature)
        loss.backward()
    engine.ddp.finish_grad_sync(extra_scale=1.0)
    lr = engine.optimizer.step()
    engine.step += 1
    return {"embedding/loss": float(loss.detach()), "embedding/acc": float((sim.argmax(1) == tgt).float().mean()),
            "lr": lr, "grad_norm": float(engine.optimizer.last_grad_norm)}


@torch.no_grad()
def embed(engine: TrainingEngine, samples: List[dict], pooling: str = "last") -> torch.Tensor:
    engine.model.eval()
    return _pooled(engine, samples, False, pooling)
