"""User script of the end-to-end test job: a synthetic dataset of token-id prompts (uniform ids from a seeded
RNG) launched for every role through the public ``worker_entry.main``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from cosmos_rl_b200.dispatcher.data import SyntheticTokenDataset  # noqa: E402
from cosmos_rl_b200.launcher.worker_entry import main  # noqa: E402

if __name__ == "__main__":
    n = int(os.environ.get("E2E_N_PROMPTS", "16"))
    main(dataset=SyntheticTokenDataset(n, 64, 32000, seed=3))
