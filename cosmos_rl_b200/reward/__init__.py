from .dispatcher import RewardDispatcher  # noqa: F401
