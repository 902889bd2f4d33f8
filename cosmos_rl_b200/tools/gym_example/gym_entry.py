"""Launch entry of the control example: `cosmos-rl --config .../cartpole_colocated.toml .../gym_entry.py`
(cosmos_rl/tools/gym_example/gym_entry.py). The dataset is a stream of initial conditions, not training data."""
from __future__ import annotations

import json
import os

from cosmos_rl_b200.tools.gym_example import GymDataPacker, gym_episode_reward  # noqa: F401  (registers trainer/backend)


class GymSeedDataset:
    def __init__(self, n: int = 4096, base: int = 0):
        self.n, self.base = n, base

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, i: int):
        return {"prompt": json.dumps({"seed": self.base + i}), "reference_answer": ""}


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=GymSeedDataset(int(os.environ.get("GYM_EXAMPLE_EPISODE_SEEDS", "4096"))), data_packer=GymDataPacker(), reward_fns=[gym_episode_reward])
