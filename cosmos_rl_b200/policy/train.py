"""``python -m cosmos_rl_b200.policy.train``: a policy replica without a user script (built-in datasets only)."""
from ..launcher.worker_entry import policy_entry

if __name__ == "__main__":
    policy_entry()
