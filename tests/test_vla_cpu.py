"""Action-token policy in closed loop: tokenizers, episode expansion, and GRPO on cart-pole with a tiny language
model through the colocated worker."""
import torch

from cosmos_rl_b200.config import Config
from cosmos_rl_b200.dispatcher.data.schema import Rollout
from cosmos_rl_b200.rollout.vla_rollout import ActionTokenizer, ObservationTokenizer, episode_return


def test_tokenizers_and_expansion():
    from cosmos_rl_b200.policy.trainer.vla_trainer import expand_episode
    a = ActionTokenizer([-2.0, 0.0], [2.0, 1.0], 256)
    x = a.decode([0, 255])
    assert abs(x[0] + 2.0) < 0.01 and abs(x[1] - 1.0) < 0.01 and a.decode([256 + 7, 3])[0] == a.decode([7, 3])[0]
    assert a.encode(a.decode([17, 200])) == [17, 200]
    assert ActionTokenizer([0], [1], discrete=True).decode([31999]) == 1
    o = ObservationTokenizer([-1, -1], [1, 1], 256, offset=1024)
    assert o.encode([-5.0, 1.0]) == [1024, 1024 + 256 + 255]
    ep = {"steps": [{"obs_tokens": [1, 2], "action_tokens": [i], "logprobs": [-0.5]} for i in range(10)], "rewards": [1.0] * 10}
    out = expand_episode(Rollout(prompt="{}", completion=ep, advantage=0.7, reward=10.0), 4)
    assert [r.completion for r in out] == [[0], [2], [5], [7]] and all(r.advantage == 0.7 for r in out)
    assert episode_return(ep) == 10.0


class _Seeds:
    def __init__(self, n):
        self.n = n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        return {"seed": i}

    def get_reference_answer(self, i):
        return ""


def test_vla_grpo_on_cartpole(tmp_path):
    from cosmos_rl_b200.colocated.worker import ColocatedRLControlWorker
    c = Config.from_dict({
        "mode": "colocated", "custom": {"vla": {"env_name": "cartpole", "max_steps": 40, "num_envs": 16}},
        "policy": {"model_name_or_path": "tiny-qwen2", "model_max_length": 64, "model_gradient_checkpointing": False},
        "rollout": {"backend": "vla", "batch_size": 4, "n_generation": 4, "seed": 0,
                    "sampling_config": {"temperature": 1.0, "top_p": 1.0, "top_k": -1}},
        "train": {"seed": 0, "optm_lr": 3e-4, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_batch_per_replica": 16, "epoch": 1,
                  "train_policy": {"type": "grpo", "trainer_type": "vla_grpo", "mini_batch": 64, "rollout_as_token_ids": True},
                  "ckpt": {"enable_checkpoint": False}}})
    w = ColocatedRLControlWorker(c, _Seeds(48), reward_fns=[episode_return], device=torch.device("cpu"))
    assert type(w.rollout).__name__ == "VLARollout" and type(w.trainer).__name__ == "VLATrainer"
    reports = w.run(max_iterations=300)
    rets = [r["train/episode_return"] for r in reports]
    assert len(rets) == 12 and all(r["train/transitions"] > 16 for r in reports)
    assert sum(rets[-4:]) > sum(rets[:4]), rets                   # the policy balances longer than at the start
