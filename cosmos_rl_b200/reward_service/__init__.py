"""Stand-alone reward service: an HTTP front end that accepts media tensors (images / video latents) or text with
metadata, scores them asynchronously with registered reward handlers and keeps the scores in a key-value store until
the trainer pulls them (reward_service/cosmos_rl_reward/: launcher/reward_serve.py, handler/reward_base.py,
utils/protocol.py)."""
from .handler import BaseRewardHandler, RewardHandlerRegistry  # noqa: F401
from .protocol import decode_request, encode_request  # noqa: F401
