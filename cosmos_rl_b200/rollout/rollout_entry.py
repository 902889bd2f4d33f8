"""``python -m cosmos_rl_b200.rollout.rollout_entry``: a rollout replica without a user script."""
from ..launcher.worker_entry import rollout_entry

if __name__ == "__main__":
    rollout_entry()
