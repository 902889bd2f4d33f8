"""Wire schemas of RL samples (field names of cosmos_rl/dispatcher/data/schema.py:47-250).

``RLPayload`` travels rollout -> controller (one prompt, n completions); the controller splits it into
``Rollout`` items (one completion each) that travel controller -> policy.
``completion_token_ids[c][p][k]``: completion c, position p, k-th most likely id (index 0 = sampled token);
``completion_logprobs`` mirrors it.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple, Union

from pydantic import BaseModel, Field

ConversationType = List[Dict[str, Any]]


class RLPayload(BaseModel):
    prompt: Optional[Any] = None
    prompt_idx: int = -1
    conversation: Optional[ConversationType] = None
    reference_answer: Optional[str] = None
    weight_version: int = 0
    completions: Optional[Any] = None
    completed_conversations: Optional[List[ConversationType]] = None
    n_ignore_prefix_tokens: Optional[List[int]] = None
    rewards: Optional[List[float]] = None
    advantages: Optional[List[float]] = None
    valid: Optional[bool] = True
    filter_rewards: Optional[List[float]] = None
    completion_token_ids: Optional[List[List[List[int]]]] = None
    completion_logprobs: Optional[List[List[List[float]]]] = None
    prompt_logprobs: Optional[List[List[float]]] = None
    prompt_token_ids: Optional[List[List[int]]] = None
    cumulative_logprob: Optional[List[float]] = None
    extra_info: Optional[Dict[str, Any]] = None
    report_metrics: Optional[List[Dict[str, Any]]] = None
    teacher_result_uuids: Optional[List[str]] = None
    payload_refs: Optional[List[str]] = None        # per completion: reference to token ids + log-probs parked with a
                                                    # payload transport (they then do not travel in this message)

    @staticmethod
    def collate_fn(batch: List["IdxAndRLPayload"]):
        return [b[0] for b in batch], [b[1] for b in batch]


IdxAndRLPayload = Tuple[int, RLPayload]


class Rollout(BaseModel):
    prompt: Optional[Any] = None
    prompt_idx: int = -1
    conversation: Optional[ConversationType] = None
    completion: Any = ""
    teacher_result_uuid: str = ""
    teacher_logprobs: Optional[List[List[float]]] = None
    teacher_topk_ids: Optional[List[List[int]]] = None        # per completion token: the teacher's k most likely ids
    teacher_topk_logprobs: Optional[List[List[float]]] = None
    completed_conversation: Optional[ConversationType] = None
    is_end: bool = False
    reward: float = 0.0
    advantage: float = 0.0
    n_ignore_prefix_tokens: int = 0
    filter_reward: float = 0.0
    completion_token_ids: Optional[List[List[int]]] = None
    completion_logprobs: Optional[List[List[float]]] = None
    prompt_logprobs: Optional[List[List[float]]] = None
    prompt_token_ids: Optional[List[List[int]]] = None
    extra_info: Optional[Dict[str, Any]] = None
    weight_version: int = 0
    report_metrics: Optional[Dict[str, Any]] = None
    payload_ref: str = ""


def payload_to_rollouts(p: RLPayload) -> List[Rollout]:
    """Split one prompt's payload into per-completion rollouts."""
    out: List[Rollout] = []
    n = len(p.completions or [])
    for i in range(n):
        out.append(Rollout(
            prompt=p.prompt, prompt_idx=p.prompt_idx, conversation=p.conversation,
            completion=p.completions[i],
            completed_conversation=(p.completed_conversations[i] if p.completed_conversations else None),
            reward=(p.rewards[i] if p.rewards else 0.0),
            advantage=(p.advantages[i] if p.advantages else 0.0),
            n_ignore_prefix_tokens=(p.n_ignore_prefix_tokens[i] if p.n_ignore_prefix_tokens else 0),
            filter_reward=(p.filter_rewards[i] if p.filter_rewards else 0.0),
            completion_token_ids=(p.completion_token_ids[i] if p.completion_token_ids else None),
            completion_logprobs=(p.completion_logprobs[i] if p.completion_logprobs else None),
            prompt_logprobs=p.prompt_logprobs, prompt_token_ids=p.prompt_token_ids, extra_info=p.extra_info,
            weight_version=p.weight_version,
            report_metrics=(p.report_metrics[i] if p.report_metrics else None),
            teacher_result_uuid=(p.teacher_result_uuids[i] if p.teacher_result_uuids else ""),
            payload_ref=(p.payload_refs[i] if p.payload_refs else ""),
        ))
    return out
