"""Pipeline parallelism: contiguous blocks per stage, 1F1B micro-batch schedule, activations and their gradients
exchanged with point-to-point sends between neighbouring stages.

The reference builds PP from ``torch.distributed.pipelining`` schedules patched for dynamic sequence lengths
(cosmos_rl/utils/pipelining/pipelining_utils.py:36-260, cosmos_rl/patch/__init__.py:226-446). Here the schedule is
explicit: packed micro-batches have different token counts, but every stage holds the same batch description, so
receive shapes are known without a shape exchange. Sends are asynchronous (``isend``) and complete behind the
next micro-batch's compute; on GPUs they are NCCL p2p on the stage group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass
class MicroBatch:
    """What every stage knows about a micro-batch (built from the same rollouts on every pipeline rank)."""
    input_ids: torch.Tensor
    position_ids: torch.Tensor
    cu_seqlens: torch.Tensor
    max_seqlen: int
    extra: Any = None            # labels, advantages ... consumed by the loss on the last stage

    @property
    def tokens(self) -> int:
        return int(self.input_ids.numel())


def schedule_1f1b(stage: int, n_stages: int, n_micro: int) -> List[tuple]:
    """Order of ('F', i) / ('B', i) steps of one stage under the one-forward-one-backward schedule."""
    warm = min(n_stages - stage - 1, n_micro)
    steps: List[tuple] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < n_micro:
        steps.append(("F", f))
        steps.append(("B", b))
        f, b = f + 1, b + 1
    while b < n_micro:
        steps.append(("B", b))
        b += 1
    return steps


def schedule_gpipe(stage: int, n_stages: int, n_micro: int) -> List[tuple]:
    """Fill-drain: every forward, then every backward (more activations alive than 1F1B, same bubble)."""
    return [("F", i) for i in range(n_micro)] + [("B", i) for i in range(n_micro)]


def interleaved_order(n_stages: int, n_chunks: int, n_micro: int, backward: bool = False) -> List[tuple]:
    """(micro-batch, chunk) in the order a rank visits them under the interleaved schedule: micro-batches go in
    groups of ``n_stages``; a group runs through chunk 0, then chunk 1, ... (backward: last chunk first)."""
    out: List[tuple] = []
    for g0 in range(0, n_micro, n_stages):
        group = range(g0, min(g0 + n_stages, n_micro))
        chunks = range(n_chunks - 1, -1, -1) if backward else range(n_chunks)
        for c in chunks:
            out.extend((i, c) for i in group)
    return out


def _interleaved_steps(stage: int, n_stages: int, n_micro: int, n_chunks: int, extra_warm: int) -> List[tuple]:
    fwd = interleaved_order(n_stages, n_chunks, n_micro)
    bwd = interleaved_order(n_stages, n_chunks, n_micro, backward=True)
    total = len(fwd)
    warm = min(total, (n_stages - stage - 1) * 2 + (n_chunks - 1) * n_stages + extra_warm)
    steps: List[tuple] = [("F",) + fwd[k] for k in range(warm)]
    f, b = warm, 0
    while f < total:
        steps.append(("F",) + fwd[f])
        steps.append(("B",) + bwd[b])
        f, b = f + 1, b + 1
    while b < total:
        steps.append(("B",) + bwd[b])
        b += 1
    return steps


_EXTRA_WARM: Dict[tuple, int] = {}


def schedule_interleaved_1f1b(stage: int, n_stages: int, n_micro: int, n_chunks: int = 1) -> List[tuple]:
    """Interleaved one-forward-one-backward: every rank holds ``n_chunks`` model chunks (virtual stage
    ``chunk * n_stages + stage``), which divides the pipeline bubble by about ``n_chunks`` at the price of
    ``n_chunks`` times the point-to-point messages (the reference selects torch's ``ScheduleInterleaved1F1B`` for
    multi-stage ranks, cosmos_rl/utils/pipelining/pipelining_utils.py:170-260). Steps are ('F' | 'B', micro-batch,
    chunk). A rank warms up with ``2 (P - stage - 1) + (chunks - 1) P`` forwards; when the number of micro-batches is
    not a multiple of the stages the last group is short and that warm-up can be too small, so the smallest extra
    warm-up (the same on every rank) with which the schedule completes in a dry run is added."""
    if n_chunks == 1:
        return [(k, i, 0) for k, i in schedule_1f1b(stage, n_stages, n_micro)]
    key = (n_stages, n_micro, n_chunks)
    if key not in _EXTRA_WARM:
        for extra in range(n_micro * n_chunks + 1):
            try:
                simulate_schedule(lambda r: _interleaved_steps(r, n_stages, n_micro, n_chunks, extra),
                                  n_stages, n_micro, n_chunks)
            except RuntimeError:
                continue
            _EXTRA_WARM[key] = extra
            break
    return _interleaved_steps(stage, n_stages, n_micro, n_chunks, _EXTRA_WARM[key])


def simulate_schedule(make, n_stages: int, n_micro: int, n_chunks: int = 1) -> Dict[str, float]:
    """Dry-run a schedule with asynchronous sends and blocking receives (what ``PipelineStage.run`` does): every rank
    executes its steps in order; a forward step of virtual stage s > 0 needs the forward of (micro-batch, s - 1), a
    backward step of s < last needs the backward of (micro-batch, s + 1) and its own forward. Raises on a deadlock;
    returns the makespan in units of one chunk-forward (backward = 2) and the bubble fraction."""
    S = n_stages * n_chunks
    plans = [make(r) for r in range(n_stages)]
    pos = [0] * n_stages
    clock = [0.0] * n_stages
    done: Dict[tuple, float] = {}
    remaining = sum(len(p) for p in plans)
    while remaining:
        progressed = False
        for r in range(n_stages):
            while pos[r] < len(plans[r]):
                kind, i, c = plans[r][pos[r]]
                s = c * n_stages + r
                deps = []
                if kind == "F" and s > 0:
                    deps.append(("F", i, s - 1))
                if kind == "B":
                    deps.append(("F", i, s))
                    if s < S - 1:
                        deps.append(("B", i, s + 1))
                if any(d not in done for d in deps):
                    break
                start = max([clock[r]] + [done[d] for d in deps])
                clock[r] = start + (1.0 if kind == "F" else 2.0)
                done[(kind, i, s)] = clock[r]
                pos[r] += 1
                remaining -= 1
                progressed = True
        if not progressed:
            raise RuntimeError(f"schedule deadlocks at positions {pos} (stages {n_stages}, chunks {n_chunks}, "
                               f"micro-batches {n_micro})")
    span = max(clock)
    work = 3.0 * n_micro * n_chunks
    return {"makespan": span, "bubble": 1.0 - work / span}


SCHEDULES = {"1F1B": schedule_1f1b, "GPipe": schedule_gpipe, "Interleaved1F1B": schedule_interleaved_1f1b}


class PipelineStage:
    """Runs this rank's part of a pipelined model over a list of micro-batches.

    ``model`` is one stage module (built with ``pp_size`` / ``pp_rank``) or, for the interleaved schedule, a list of
    chunk modules: chunk ``c`` of rank ``stage`` is virtual stage ``c * n_stages + stage`` of a model built with
    ``pp_size = n_stages * len(chunks)``. Activations travel to the next rank (wrapping from the last rank to the next
    chunk of the first) on ``group``; gradients travel the other way on ``back_group`` when one is given, so that the
    two kinds of traffic between a pair of ranks never share a communicator's message order.

    ``loss_fn(hidden, micro_batch) -> scalar`` is evaluated on the last virtual stage only; its value is already
    scaled for accumulation over micro-batches by the caller. Returns the list of losses there, ``[]`` elsewhere."""

    def __init__(self, model, group, stage: int, n_stages: int, hidden_dim: int, dtype: torch.dtype,
                 device: torch.device, schedule: str = "1F1B", back_group=None):
        if schedule not in SCHEDULES:
            raise ValueError(f"pp_schedule must be one of {sorted(SCHEDULES)}, got {schedule!r}")
        self.chunks = list(model) if isinstance(model, (list, tuple, torch.nn.ModuleList)) else [model]
        self.model = self.chunks[0]
        self.n_chunks = len(self.chunks)
        if self.n_chunks > 1 and schedule != "Interleaved1F1B":
            raise ValueError("several model chunks per rank need pp_schedule = 'Interleaved1F1B'")
        self.schedule_name = schedule
        self.group, self.stage, self.n = group, stage, n_stages
        self.back_group = back_group if back_group is not None else group
        self.hidden_dim, self.dtype, self.device = hidden_dim, dtype, device
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(n_stages))
        self.prev = ranks[(stage - 1) % n_stages]
        self.next = ranks[(stage + 1) % n_stages]
        self.n_virtual = n_stages * self.n_chunks

    def steps(self, n_micro: int) -> List[tuple]:
        fn = SCHEDULES[self.schedule_name]
        if fn is schedule_interleaved_1f1b:
            return fn(self.stage, self.n, n_micro, self.n_chunks)
        return [(k, i, 0) for k, i in fn(self.stage, self.n, n_micro)]

    def _tag(self, micro: int, virtual_stage: int) -> int:
        return micro * self.n_virtual + virtual_stage        # honoured by gloo; NCCL matches by order

    def _recv(self, tokens: int, src: int, group, tag: int) -> torch.Tensor:
        buf = torch.empty(tokens, self.hidden_dim, dtype=self.dtype, device=self.device)
        dist.recv(buf, src=src, group=group, tag=tag)
        return buf

    def run(self, micro_batches: Sequence[MicroBatch], loss_fn: Optional[Callable] = None) -> List[torch.Tensor]:
        inputs: Dict[tuple, torch.Tensor] = {}
        outputs: Dict[tuple, torch.Tensor] = {}
        pending: List[Any] = []
        keep: List[torch.Tensor] = []          # buffers of sends in flight
        losses: List[torch.Tensor] = []
        for kind, i, c in self.steps(len(micro_batches)):
            mb = micro_batches[i]
            s = c * self.n + self.stage
            first, last = s == 0, s == self.n_virtual - 1
            if kind == "F":
                if first:
                    x = mb.input_ids
                else:
                    x = self._recv(mb.tokens, self.prev, self.group, self._tag(i, s)).requires_grad_(True)
                    inputs[(i, c)] = x
                out = self.chunks[c](x, mb.position_ids, mb.cu_seqlens, mb.max_seqlen)
                if last:
                    loss = loss_fn(out, mb)
                    outputs[(i, c)] = loss
                    losses.append(loss.detach())
                else:
                    outputs[(i, c)] = out
                    send = out.detach().contiguous()
                    keep.append(send)
                    pending.append(dist.isend(send, dst=self.next, group=self.group, tag=self._tag(i, s + 1)))
            else:
                out = outputs.pop((i, c))
                if last:
                    out.backward()
                else:
                    out.backward(self._recv(mb.tokens, self.next, self.back_group, self._tag(i, s)))
                if not first:
                    gin = inputs.pop((i, c)).grad.contiguous()
                    keep.append(gin)
                    pending.append(dist.isend(gin, dst=self.prev, group=self.back_group, tag=self._tag(i, s - 1)))
        for w in pending:
            w.wait()
        return losses

    @torch.no_grad()
    def forward_only(self, micro_batches: Sequence[MicroBatch], fn: Optional[Callable] = None) -> List[Any]:
        """Fill-drain forward pass without gradients (old / reference log-probs, validation: the reference uses a
        GPipe schedule there). Returns ``fn(hidden, micro_batch)`` per micro-batch on the last virtual stage, ``[]``
        elsewhere. With several chunks per rank the micro-batches run in the interleaved forward order."""
        outs: List[Any] = []
        pending: List[Any] = []
        keep: List[torch.Tensor] = []
        order = interleaved_order(self.n, self.n_chunks, len(micro_batches))
        for i, c in order:
            mb = micro_batches[i]
            s = c * self.n + self.stage
            first, last = s == 0, s == self.n_virtual - 1
            x = mb.input_ids if first else self._recv(mb.tokens, self.prev, self.group, self._tag(i, s))
            out = self.chunks[c](x, mb.position_ids, mb.cu_seqlens, mb.max_seqlen)
            if last:
                outs.append((i, fn(out, mb) if fn is not None else out))
            else:
                send = out.contiguous()
                keep.append(send)
                pending.append(dist.isend(send, dst=self.next, group=self.group, tag=self._tag(i, s + 1)))
        for w in pending:
            w.wait()
        return [o for _, o in sorted(outs, key=lambda t: t[0])]
