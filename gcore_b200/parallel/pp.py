"""Pipeline parallelism: stage layout and the 1F1B schedule over point-to-point sends.

Every pipeline rank of a (tp, cp, dp) coordinate receives the same samples and packs the same micro-batches, so the
shape of every inter-stage activation is known locally and only the activation itself ([tokens, hidden] of the stage's
sequence-parallel / context-parallel shard) crosses the stage boundary; gradients travel the other way.  Sends are
asynchronous (`isend`), receives blocking, which is deadlock-free for the one-forward-one-backward order.  Transport
is `torch.distributed` p2p on the pipeline group (NCCL between GPUs, gloo on CPU): pipeline traffic is point-to-point
by nature and stays on the library path, as in the reference (mcore ``get_forward_backward_func`` configured in
gpatch_v4/training_backend/megatron_backend/mixin.py:411-414,2783-2794; stage p2p helpers in
gpatch_v4/utils/communication_utils.py:69-126).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def stage_layer_range(num_layers: int, pp: int, stage: int, first_stage_layers: Optional[int] = None,
                      last_stage_layers: Optional[int] = None) -> Tuple[int, int]:
    """Layers [lo, hi) of ``stage``.  Uneven first / last stages (embedding and head make them heavier) follow the
    reference's ``num_layers_in_first/last_pipeline_stage`` knobs; the rest is split evenly."""
    if pp == 1:
        return 0, num_layers
    first = first_stage_layers
    last = last_stage_layers
    middle_stages = pp - (first is not None) - (last is not None)
    remaining = num_layers - (first or 0) - (last or 0)
    assert middle_stages == 0 or remaining % middle_stages == 0, "layers do not divide over the pipeline stages"
    per = remaining // middle_stages if middle_stages else 0
    sizes = []
    for s in range(pp):
        if s == 0 and first is not None:
            sizes.append(first)
        elif s == pp - 1 and last is not None:
            sizes.append(last)
        else:
            sizes.append(per)
    assert sum(sizes) == num_layers
    lo = sum(sizes[:stage])
    return lo, lo + sizes[stage]


class PipelineComm:
    """Point-to-point plumbing of one pipeline.  Activations travel on ``group`` and gradients on ``bwd_group`` (a
    second communicator over the same ranks when given): with two stages the next and the previous stage are the
    same peer, and an interleaved schedule would otherwise mix both kinds of message in one FIFO."""

    def __init__(self, group, bwd_group=None, wrap_group=None, bwd_wrap_group=None):
        self.group = group
        self.bwd_group = bwd_group if bwd_group is not None else group
        # last stage -> first stage (interleaved chunks) and the gradients coming back
        self.wrap_group = wrap_group if wrap_group is not None else group
        self.bwd_wrap_group = bwd_wrap_group if bwd_wrap_group is not None else self.bwd_group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ranks = dist.get_process_group_ranks(group)
        self._pending = []

    @property
    def is_first(self):
        return self.rank == 0

    @property
    def is_last(self):
        return self.rank == self.size - 1

    def _peer(self, delta):
        return self.ranks[(self.rank + delta) % self.size]  # the ring closes for interleaved stages

    def send_forward(self, t):
        g = self.wrap_group if self.is_last else self.group
        self._pending.append((dist.isend(t.contiguous(), self._peer(+1), group=g), t))

    def send_backward(self, t):
        g = self.bwd_wrap_group if self.is_first else self.bwd_group
        self._pending.append((dist.isend(t.contiguous(), self._peer(-1), group=g), t))

    def recv_forward(self, shape, dtype, device):
        t = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(t, self._peer(-1), group=self.wrap_group if self.is_first else self.group)
        return t

    def recv_backward(self, shape, dtype, device):
        t = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(t, self._peer(+1), group=self.bwd_wrap_group if self.is_last else self.bwd_group)
        return t

    def drain(self):
        for h, _ in self._pending:
            h.wait()
        self._pending.clear()


def forward_backward_1f1b(comm: PipelineComm, num_microbatches: int,
                          forward_step: Callable[[int, Optional[torch.Tensor]], Tuple[torch.Tensor, object]],
                          loss_step: Callable[[int, torch.Tensor, object], torch.Tensor],
                          act_shape: Callable[[int], Tuple[Sequence[int], torch.dtype, torch.device]],
                          forward_only: bool = False) -> List[object]:
    """Runs ``num_microbatches`` through this stage.

    ``forward_step(i, hidden_in)`` -> (stage output, aux); ``loss_step(i, output, aux)`` -> scalar loss (last stage;
    in forward-only mode its return value is collected and returned); ``act_shape(i)`` -> shape / dtype / device of
    the activation entering and leaving middle stages for micro-batch ``i``.
    """
    P, s, M = comm.size, comm.rank, num_microbatches
    inputs: List[Optional[torch.Tensor]] = [None] * M
    outputs: List[Optional[torch.Tensor]] = [None] * M
    results: List[object] = []

    def fwd(i):
        x = None
        if not comm.is_first:
            x = comm.recv_forward(*act_shape(i))
            if not forward_only:
                x.requires_grad_(True)
        with torch.set_grad_enabled(not forward_only):
            out, aux = forward_step(i, x)
            if comm.is_last:
                out = loss_step(i, out, aux)
                if forward_only:
                    results.append(out)
            else:
                comm.send_forward(out.detach())
                if aux is not None and not forward_only:
                    out = (out, aux)
        inputs[i], outputs[i] = x, (None if forward_only else out)

    def bwd(i):
        out, x = outputs[i], inputs[i]
        if comm.is_last:
            out.backward()
        else:
            shape, dtype, dev = act_shape(i)
            g = comm.recv_backward(shape, dtype, dev)
            if isinstance(out, tuple):  # a stage-local auxiliary loss (MoE balance) joins the backward here
                torch.autograd.backward([out[0], out[1]], [g, torch.ones_like(out[1])])
            else:
                out.backward(g)
        if not comm.is_first:
            comm.send_backward(x.grad)
        inputs[i] = outputs[i] = None

    if forward_only:
        for i in range(M):
            fwd(i)
        comm.drain()
        return results
    warm = min(P - s - 1, M)
    for i in range(warm):
        fwd(i)
    for i in range(M - warm):
        fwd(warm + i)
        bwd(i)
    for i in range(M - warm, M):
        bwd(i)
    comm.drain()
    return results


def interleaved_order(num_microbatches: int, pp: int, vpp: int) -> List[Tuple[int, int]]:
    """Forward order of (chunk, micro-batch) pairs of the interleaved schedule, identical on every stage:
    micro-batches go in groups of ``pp``; a group passes through chunk 0 on all stages, then chunk 1, ...  The
    backward order is the same list with the chunks mirrored."""
    order = []
    for g0 in range(0, num_microbatches, pp):
        group = range(g0, min(g0 + pp, num_microbatches))
        for v in range(vpp):
            order += [(v, i) for i in group]
    return order


def forward_backward_interleaved(comm: PipelineComm, num_microbatches: int, num_chunks: int,
                                 forward_step: Callable[[int, int, Optional[torch.Tensor]], Tuple[torch.Tensor, object]],
                                 loss_step: Callable[[int, torch.Tensor, object], torch.Tensor],
                                 act_shape: Callable[[int], Tuple[Sequence[int], torch.dtype, torch.device]],
                                 forward_only: bool = False) -> List[object]:
    """Interleaved 1F1B (virtual pipeline stages): stage ``s`` holds model chunks ``v = 0 .. V-1``, chunk ``v`` being
    virtual stage ``v * P + s``; the bubble shrinks by a factor ``V`` for ``V`` times as many (smaller) messages.
    ``forward_step(i, v, hidden_in)`` runs chunk ``v`` on micro-batch ``i``.  The steady state needs the number of
    micro-batches to be a multiple of ``P``; otherwise (and when it equals ``P``) all forwards run before all
    backwards, which is always consistent.  (The schedule the reference gets from Megatron-Core's
    ``get_forward_backward_func`` when ``virtual_pipeline_model_parallel_size`` is set:
    gpatch_v4/training_backend/megatron_backend/mixin.py:411-414.)"""
    P, s, M, V = comm.size, comm.rank, num_microbatches, num_chunks
    order_f = interleaved_order(M, P, V)
    order_b = [(V - 1 - v, i) for v, i in order_f]
    total = len(order_f)
    inputs, outputs = {}, {}
    results: List[object] = []

    def fwd(k):
        v, i = order_f[k]
        x = None
        if not (s == 0 and v == 0):
            x = comm.recv_forward(*act_shape(i))
            if not forward_only:
                x.requires_grad_(True)
        with torch.set_grad_enabled(not forward_only):
            out, aux = forward_step(i, v, x)
            if s == P - 1 and v == V - 1:
                out = loss_step(i, out, aux)
                if forward_only:
                    results.append(out)
            else:
                comm.send_forward(out.detach())
                if aux is not None and not forward_only:
                    out = (out, aux)
        if not forward_only:
            inputs[(v, i)], outputs[(v, i)] = x, out

    def bwd(k):
        v, i = order_b[k]
        out, x = outputs.pop((v, i)), inputs.pop((v, i))
        if s == P - 1 and v == V - 1:
            out.backward()
        else:
            g = comm.recv_backward(*act_shape(i))
            if isinstance(out, tuple):
                torch.autograd.backward([out[0], out[1]], [g, torch.ones_like(out[1])])
            else:
                out.backward(g)
        if x is not None:
            comm.send_backward(x.grad)

    if forward_only:
        for k in range(total):
            fwd(k)
        comm.drain()
        return results
    if M % P != 0 or M == P:
        warm = total
    else:
        warm = min((P - s - 1) * 2 + (V - 1) * P, total)
    for k in range(warm):
        fwd(k)
    for k in range(total - warm):
        fwd(warm + k)
        bwd(k)
    for k in range(total - warm, total):
        bwd(k)
    comm.drain()
    return results


def broadcast_from_last_stage(t: Optional[torch.Tensor], shape, dtype, device, group) -> torch.Tensor:
    """Last pipeline stage -> every stage (log-probs / values computed at the end of the pipeline;
    gpatch_v4/utils/communication_utils.py:367-453)."""
    n = dist.get_world_size(group)
    if n == 1:
        return t
    if dist.get_rank(group) != n - 1:
        t = torch.empty(shape, dtype=dtype, device=device)
    dist.broadcast(t, dist.get_process_group_ranks(group)[-1], group=group)
    return t
