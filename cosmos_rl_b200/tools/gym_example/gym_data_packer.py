"""Data packer for tensor trajectories: the "prompt" is an initial condition (a seed), the "completion" a whole
episode. Also the trajectory-iteration view (transitions / chunks / rollouts) that trainers over long trajectories
walk instead of materialising everything at once (cosmos_rl/tools/gym_example/gym_data_packer.py and the
TrajectoryPacker protocol of cosmos_rl/dispatcher/data/packer/trajectory_packer.py)."""
from __future__ import annotations

import json
from typing import Any, Dict, Iterator, List, Optional

import torch

from ...data.packer import BaseDataPacker


@BaseDataPacker.register("gym_mlp")
class GymDataPacker(BaseDataPacker):
    def get_rollout_input(self, item: Any) -> int:
        """Prompt -> episode seed. Accepts an int, a JSON string ``{"seed": n}`` or a dict."""
        if isinstance(item, dict) and "prompt" in item:       # a whole dataset row
            item = item["prompt"]
        if isinstance(item, str):
            item = json.loads(item)
        return int(item["seed"] if isinstance(item, dict) else item)

    def get_policy_input(self, sample: Any, rollout_output: Any, n_ignore_prefix_tokens: int = 0, **kw) -> Dict[str, torch.Tensor]:
        t = rollout_output
        return {"observations": torch.tensor(t["observations"], dtype=torch.float32),
                "actions": torch.tensor(t["actions"], dtype=torch.float32),
                "rewards": torch.tensor(t["rewards"], dtype=torch.float32),
                "logprobs": torch.tensor(t["logprobs"], dtype=torch.float32)}

    def policy_compute_max_len(self, processed: List[Any]) -> int:
        return max((int(p["rewards"].numel()) for p in processed), default=0)

    def policy_collate_fn(self, processed: List[Any], computed_max_len: int) -> Dict[str, Any]:
        return {"trajectories": processed, "max_len": computed_max_len}

    # ------------------------------------------------------------------ trajectory iteration
    def num_transitions(self, rollout) -> int:
        return int(rollout.completion["episode_length"])

    def iter_transitions(self, rollout) -> Iterator[Dict[str, Any]]:
        t = rollout.completion
        for o, a, r in zip(t["observations"], t["actions"], t["rewards"]):
            yield {"observation": o, "action": a, "reward": r}

    def iter_chunks(self, rollouts, chunk_size: int) -> Iterator[List[Dict[str, Any]]]:
        buf: List[Dict[str, Any]] = []
        for ro in rollouts:
            for tr in self.iter_transitions(ro):
                buf.append(tr)
                if len(buf) == chunk_size:
                    yield buf
                    buf = []
        if buf:
            yield buf

    def iter_rollouts(self, rollouts) -> Iterator[Any]:
        yield from rollouts
