"""User script of the disaggregated diffusion job test: text-embedding prompts and a reward that reads the generated
latent out of the trajectory store (a file system folder both workers see)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from cosmos_rl_b200.launcher.worker_entry import main  # noqa: E402
from cosmos_rl_b200.rollout.diffusion_rollout import LatentStore  # noqa: E402


class Prompts:
    def __init__(self, n):
        g = torch.Generator().manual_seed(5)
        self.rows = [{"text_embeds": torch.randn(3, 64, generator=g).tolist(), "seed": i} for i in range(n)]

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]

    def get_reference_answer(self, i):
        return ""


def brightness_reward(completion, reference=None, **kw) -> float:
    return float(LatentStore.get(completion)["x0"].float().mean())


if __name__ == "__main__":
    main(dataset=Prompts(int(os.environ.get("N_PROMPTS", "16"))), reward_fns=[brightness_reward])
