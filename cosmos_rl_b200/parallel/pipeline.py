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


SCHEDULES = {"1F1B": schedule_1f1b, "GPipe": schedule_gpipe,
             # one stage per rank here: the multi-stage name of the reference's default selects plain 1F1B
             "Interleaved1F1B": schedule_1f1b}


class PipelineStage:
    """Runs one stage of ``model`` (built with ``pp_size`` / ``pp_rank``) over a list of micro-batches.

    ``loss_fn(hidden, micro_batch) -> scalar`` is evaluated on the last stage only; its value is already scaled
    for accumulation over micro-batches by the caller. Returns the list of losses (last stage) or ``[]``."""

    def __init__(self, model, group, stage: int, n_stages: int, hidden_dim: int, dtype: torch.dtype,
                 device: torch.device, schedule: str = "1F1B"):
        if schedule not in SCHEDULES:
            raise ValueError(f"pp_schedule must be one of {sorted(SCHEDULES)}, got {schedule!r}")
        self.schedule = SCHEDULES[schedule]
        self.model, self.group, self.stage, self.n = model, group, stage, n_stages
        self.hidden_dim, self.dtype, self.device = hidden_dim, dtype, device
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(n_stages))
        self.prev = ranks[stage - 1] if stage > 0 else None
        self.next = ranks[stage + 1] if stage < n_stages - 1 else None

    def _recv(self, tokens: int, src: int) -> torch.Tensor:
        buf = torch.empty(tokens, self.hidden_dim, dtype=self.dtype, device=self.device)
        dist.recv(buf, src=src, group=self.group)
        return buf

    def run(self, micro_batches: Sequence[MicroBatch], loss_fn: Optional[Callable] = None) -> List[torch.Tensor]:
        first, last = self.stage == 0, self.stage == self.n - 1
        inputs: Dict[int, torch.Tensor] = {}
        outputs: Dict[int, torch.Tensor] = {}
        pending: List[Any] = []
        keep: List[torch.Tensor] = []          # buffers of sends in flight
        losses: List[torch.Tensor] = []
        for kind, i in self.schedule(self.stage, self.n, len(micro_batches)):
            mb = micro_batches[i]
            if kind == "F":
                if first:
                    x = mb.input_ids
                else:
                    x = self._recv(mb.tokens, self.prev).requires_grad_(True)
                    inputs[i] = x
                out = self.model(x, mb.position_ids, mb.cu_seqlens, mb.max_seqlen)
                if last:
                    loss = loss_fn(out, mb)
                    outputs[i] = loss
                    losses.append(loss.detach())
                else:
                    outputs[i] = out
                    send = out.detach().contiguous()
                    keep.append(send)
                    pending.append(dist.isend(send, dst=self.next, group=self.group))
            else:
                out = outputs.pop(i)
                if last:
                    out.backward()
                else:
                    g = self._recv(mb.tokens, self.next)
                    out.backward(g)
                if not first:
                    gin = inputs.pop(i).grad.contiguous()
                    keep.append(gin)
                    pending.append(dist.isend(gin, dst=self.prev, group=self.group))
        for w in pending:
            w.wait()
        return losses

    @torch.no_grad()
    def forward_only(self, micro_batches: Sequence[MicroBatch], fn: Optional[Callable] = None) -> List[Any]:
        """Fill-drain forward pass without gradients (old / reference log-probs, validation: the reference uses a
        GPipe schedule there). Returns ``fn(hidden, micro_batch)`` per micro-batch on the last stage, ``[]`` elsewhere."""
        first, last = self.stage == 0, self.stage == self.n - 1
        outs: List[Any] = []
        pending: List[Any] = []
        keep: List[torch.Tensor] = []
        for mb in micro_batches:
            x = mb.input_ids if first else self._recv(mb.tokens, self.prev)
            out = self.model(x, mb.position_ids, mb.cu_seqlens, mb.max_seqlen)
            if last:
                outs.append(fn(out, mb) if fn is not None else out)
            else:
                send = out.contiguous()
                keep.append(send)
                pending.append(dist.isend(send, dst=self.next, group=self.group))
        for w in pending:
            w.wait()
        return outs
