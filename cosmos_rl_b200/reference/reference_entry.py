"""``python -m cosmos_rl_b200.reference.reference_entry``: a teacher replica."""
from ..launcher.worker_entry import reference_entry

if __name__ == "__main__":
    reference_entry()
