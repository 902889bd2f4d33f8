"""Control-task example of the custom trainer / rollout-backend / data-packer extension API, runnable on CPU
(cosmos_rl/tools/gym_example/). Importing the package registers trainer type ``gym_pg``, rollout backend ``gym`` and
the ``gym_mlp`` data packer."""
from .gym_algo import compute_returns, pg_loss  # noqa: F401
from .gym_data_packer import GymDataPacker  # noqa: F401
from .gym_policy import GymMLPConfig, GymPolicy  # noqa: F401
from .gym_rollout import GymRolloutEngine  # noqa: F401
from .gym_rollout_backend import GymRolloutBackend  # noqa: F401
from .gym_trainer import GymTrainer  # noqa: F401


def gym_episode_reward(completion, reference=None, **kw) -> float:
    """Reward of one "completion" = undiscounted return of the episode."""
    return float(sum(completion["rewards"]))
