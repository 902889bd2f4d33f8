"""Environment-tunable constants (names follow cosmos_rl/utils/constant.py:20-121)."""
from .misc import env_float, env_int

COSMOS_HEARTBEAT_SEND_INTERVAL = env_float("COSMOS_HEARTBEAT_SEND_INTERVAL", 60.0)
COSMOS_HEARTBEAT_PROCESS = env_int("COSMOS_HEARTBEAT_PROCESS", 0)     # 1: heartbeats from a child process
COSMOS_HEARTBEAT_TIMEOUT = env_float("COSMOS_HEARTBEAT_TIMEOUT", 200.0)
COSMOS_ROLLOUT_SCAN_INTERVAL = env_float("COSMOS_ROLLOUT_SCAN_INTERVAL", 10.0)
# an RL job whose rollout replicas are all gone ends (final checkpoint, failure status) after this long without one
COSMOS_NO_ROLLOUT_GRACE_S = env_float("COSMOS_NO_ROLLOUT_GRACE_S", 600.0)
COSMOS_NCCL_TIMEOUT_MS = env_int("COSMOS_NCCL_TIMEOUT_MS", 600_000)
COSMOS_NCCL_ERROR_CLEAN_REPLICA_DELAY = env_float("COSMOS_NCCL_ERROR_CLEAN_REPLICA_DELAY", 10.0)
COSMOS_GLOO_TIMEOUT = env_int("COSMOS_GLOO_TIMEOUT", 600)
COSMOS_P2R_NCCL_GROUP_SIZE = env_int("COSMOS_P2R_NCCL_GROUP_SIZE", 0)
COSMOS_HTTP_RETRY_MAX = env_int("COSMOS_HTTP_RETRY_CONFIG_MAX_RETRY", 8)
COSMOS_HTTP_RETRY_INITIAL_DELAY = env_float("COSMOS_HTTP_RETRY_CONFIG_INITIAL_DELAY", 0.25)
COSMOS_HTTP_RETRY_MAX_DELAY = env_float("COSMOS_HTTP_RETRY_CONFIG_MAX_DELAY", 8.0)
COSMOS_ROLLOUT_PROMPT_QUEUE_MAX_SIZE = env_int("COSMOS_ROLLOUT_PROMPT_QUEUE_MAX_SIZE", 2048)
COSMOS_WEIGHT_GATE_SLEEP = env_float("COSMOS_WEIGHT_GATE_SLEEP", 0.05)
COSMOS_WEIGHT_SYNC_CHECK = env_int("COSMOS_WEIGHT_SYNC_CHECK", 0)   # verify the first policy-to-rollout transfer
COSMOS_DEFAULT_MODEL_TYPE = "hfmodel"
import os as _os  # noqa: E402
CACHE_DIR = _os.environ.get("COSMOS_CACHE", _os.path.join(_os.path.expanduser("~"), ".cache", "cosmos"))

RedisStreamConstant = type("RedisStreamConstant", (), {
    "CMD_FETCH_SIZE": 5, "ROLLOUT_FETCH_SIZE": 8, "STREAM_MAXLEN": 10000, "CMD_READING_TIMEOUT_MS": 500,
    "ROLLOUT_READING_TIMEOUT_MS": 500,
})
