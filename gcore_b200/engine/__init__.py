"""Training engines.  ``get_training_engine`` is the factory the trainers use (the role of
``TrainingEngineFactory.get_training_engine``, gpatch_v4/training_backend/__init__.py:58-117): ``training_backend``
selects the ZeRO-1 engine (``native``; ``nccl_eager`` is the same engine on library ops) or the ZeRO-3 engine
(``fsdp2``)."""
from __future__ import annotations


def get_training_engine(policy_cfg, optimizer_cfg, training_cfg, ppo_cfg=None, **kw):
    backend = getattr(training_cfg, "training_backend", "native")
    if backend == "fsdp2":
        from .fsdp2_engine import Fsdp2Engine
        return Fsdp2Engine(policy_cfg, optimizer_cfg, training_cfg, ppo_cfg, **kw)
    from .train_engine import TrainingEngine
    return TrainingEngine(policy_cfg, optimizer_cfg, training_cfg, ppo_cfg, **kw)
