"""Entry script of the launcher-layout benchmark job: every role of the job (controller, policy, rollout or the
colocated worker) starts here with a synthetic data set of uniform random token-id prompts, the shape of which comes
from the environment (``B200RL_BENCH_PROMPTS``, ``B200RL_BENCH_PROMPT_LEN``, ``B200RL_BENCH_VOCAB``)."""
import os

from cosmos_rl_b200.dispatcher.data import SyntheticTokenDataset
from cosmos_rl_b200.launcher.worker_entry import main

if __name__ == "__main__":
    main(dataset=SyntheticTokenDataset(int(os.environ.get("B200RL_BENCH_PROMPTS", "64")),
                                       int(os.environ.get("B200RL_BENCH_PROMPT_LEN", "512")),
                                       int(os.environ.get("B200RL_BENCH_VOCAB", "32000")), seed=11))
