"""Example of a custom GRPO flow: a trainer registered under its own ``train_policy.trainer_type``
(cosmos_rl/tools/custom_example/)."""
from .custom_grpo_trainer import CustomGRPOTrainer  # noqa: F401
