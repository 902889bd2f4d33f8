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


def test_flow_matching_vla_behaviour_cloning_and_flow_grpo():
    """A vision-language-action policy with a flow-matching action expert (the construction of PI0.5): a decoder
    backbone reads the instruction, a DiT over the action chunk cross-attends to its hidden states and to the
    proprioceptive state. Behaviour cloning by flow matching reproduces instruction- and state-dependent action chunks;
    SDE exploration records transitions whose log-probabilities the current policy reproduces exactly (ratio 1 before
    any update); clipped-ratio updates on group-normalised advantages raise the reward."""
    import torch
    from cosmos_rl_b200.models.gpt import GPT, GPTArgs
    from cosmos_rl_b200.models.vla_flow import FlowVLA, FlowVLAArgs, denormalize_actions, normalize_actions
    torch.manual_seed(0)
    backbone = GPT(GPTArgs(vocab_size=64, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=128, qkv_bias=True,
                           model_type="qwen2"))
    pol = FlowVLA(backbone, FlowVLAArgs(action_dim=3, horizon=4, state_dim=2, expert_dim=64, expert_layers=2,
                                        expert_heads=2, expert_head_dim=32, expert_ffn=128))
    pol.init_weights(0)
    g = torch.Generator().manual_seed(1)
    patterns = torch.rand(4, 4, 3, generator=g) * 1.6 - 0.8               # one action chunk per instruction

    def batch(n):
        goal = torch.randint(0, 4, (n,), generator=g)
        state = torch.rand(n, 2, generator=g) * 2 - 1
        prompts = [[1, 10 + int(k), 2] + [3] * int(k) for k in goal]       # different lengths: padded context
        target = (patterns[goal] + 0.3 * state[:, :1, None]).clamp(-1, 1)
        return prompts, state, target
    opt = torch.optim.Adam([p for p in pol.parameters() if p.requires_grad], lr=2e-3)
    first = None
    for _ in range(180):
        prompts, state, target = batch(32)
        loss = pol.bc_loss(prompts, target, state)
        opt.zero_grad()
        loss.backward()
        opt.step()
        first = first if first is not None else float(loss)
    assert float(loss) < 0.45 * first, (first, float(loss))
    prompts, state, target = batch(64)
    acts = pol.act(prompts, state, steps=12, solver="heun", generator=torch.Generator().manual_seed(2))
    err = (acts - target).abs().mean()
    assert acts.shape == (64, 4, 3) and err < 0.3, err
    base = (torch.zeros_like(target) - target).abs().mean()
    assert err < 0.5 * base                                                # far better than ignoring the instruction
    # exploration: the recorded behaviour log-probabilities are reproduced by the unchanged policy
    ro = pol.explore(prompts, state, steps=6, noise_level=0.7, generator=torch.Generator().manual_seed(3))
    assert ro["states"].shape == (64, 5, 4, 3) and ro["logprobs"].shape == (64, 5)
    l0, m0 = pol.flow_grpo_loss(prompts, ro, torch.ones(64), state)
    assert abs(float(l0) + 1.0) < 1e-3 and m0["clip_frac"] == 0.0           # ratio 1 everywhere: loss = -mean(adv)
    # RL: the reward wants the first action dimension at 0.8, which is not what behaviour cloning taught
    def reward(a):
        return -((a[:, :, 0] - 0.8) ** 2).mean(1)
    opt = torch.optim.Adam([p for p in pol.expert.parameters()], lr=3e-4)
    fixed = batch(16)
    before = float(reward(pol.act(fixed[0], fixed[1], steps=8, generator=torch.Generator().manual_seed(5))).mean())
    for it in range(15):
        prompts16, state16, _ = fixed
        pr = [p for p in prompts16 for _ in range(8)]                       # groups of 8 samples per observation
        st = state16.repeat_interleave(8, 0)
        ro = pol.explore(pr, st, steps=6, noise_level=0.9, generator=torch.Generator().manual_seed(100 + it))
        r = reward(ro["x0"]).view(16, 8)
        adv = ((r - r.mean(1, keepdim=True)) / (r.std(1, keepdim=True) + 1e-6)).flatten()
        loss, _ = pol.flow_grpo_loss(pr, ro, adv, st, noise_level=0.9)
        opt.zero_grad()
        loss.backward()
        opt.step()
    after = float(reward(pol.act(fixed[0], fixed[1], steps=8, generator=torch.Generator().manual_seed(5))).mean())
    assert after > 0.4 * before and after > before + 0.1, (before, after)        # e.g. -0.55 -> -0.02
    lo, hi = torch.tensor([-2.0, 0.0, 10.0]), torch.tensor([2.0, 1.0, 20.0])
    a = torch.tensor([[1.0, 0.25, 12.0]])
    assert torch.allclose(denormalize_actions(normalize_actions(a, lo, hi), lo, hi), a)


def torque_reward(completion, reference=None, **kw) -> float:
    a = torch.tensor(completion["actions"])
    return float(-((a - 1.0) ** 2).mean())


def test_flow_vla_job_on_pendulum_through_the_colocated_worker(tmp_path):
    """The flow-matching action policy as a JOB: model type ``flow_vla`` built from its named architecture by the
    model registry, rollout backend ``flow_vla`` (closed loop with the pendulum, action chunks explored by the SDE
    sampler, transitions parked in the latent store), trainer ``flow_vla_grpo`` (clipped ratios of the recorded
    transitions, episode advantage on every chunk), all driven by the controller inside the colocated worker. The
    reward reads the executed torques out of the completion; evaluation episodes (deterministic flow, fixed starts)
    score better after training, and every parked trace was released."""
    from cosmos_rl_b200.colocated.worker import ColocatedRLControlWorker
    from cosmos_rl_b200.dispatcher.data.schema import RLPayload
    from cosmos_rl_b200.rollout.diffusion_rollout import LatentStore
    c = Config.from_dict({
        "mode": "colocated", "custom": {"vla": {"env_name": "pendulum", "max_steps": 16, "num_envs": 32, "flow_steps": 4,
                                                "noise_level": 0.7}},
        "policy": {"model_name_or_path": "tiny-flow-vla", "model_max_length": 64, "model_gradient_checkpointing": False},
        "rollout": {"backend": "flow_vla", "batch_size": 4, "n_generation": 8, "seed": 0},
        "validation": {"n_generation": 1},
        "train": {"seed": 0, "optm_lr": 1e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_batch_per_replica": 32, "epoch": 1,
                  "train_policy": {"type": "grpo", "trainer_type": "flow_vla_grpo", "mini_batch": 128,
                                   "epsilon_high": 0.2},
                  "ckpt": {"enable_checkpoint": False}}})
    torch.manual_seed(0)
    w = ColocatedRLControlWorker(c, _Seeds(96), reward_fns=[torque_reward], device=torch.device("cpu"))
    assert type(w.rollout).__name__ == "FlowVLARollout" and type(w.trainer).__name__ == "FlowVLAGRPOTrainer"
    assert type(w.trainer.model).__name__ == "FlowVLA"

    def evaluate():
        pl = [RLPayload(prompt={"seed": 5000 + i}, prompt_idx=i) for i in range(32)]
        res = w.rollout.rollout_generation(pl, None, is_validation=True)
        assert all(len(r.completions[0]["actions"]) == 16 and len(r.completions[0]["rewards"]) == 4 for r in res)
        return sum(torque_reward(r.completions[0]) for r in res) / len(res)

    before = evaluate()
    LatentStore._items.clear()                                       # evaluation parks empty traces
    reports = w.run(max_iterations=600)
    assert len(reports) == 24 and all(r["train/transitions"] == 32 * 4 for r in reports)
    assert not LatentStore._items
    after = evaluate()
    assert after > before + 1.0, (before, after)


def test_flow_vla_sft_trainer_clones_action_chunks(tmp_path):
    from cosmos_rl_b200.parallel.dims import ParallelDims
    from cosmos_rl_b200.policy.trainer.vla_flow_trainer import FlowVLASFTTrainer
    c = Config.from_dict({
        "policy": {"model_name_or_path": "tiny-flow-vla", "model_max_length": 64, "model_gradient_checkpointing": False},
        "train": {"seed": 0, "optm_lr": 2e-3, "optm_warmup_steps": 0, "output_dir": str(tmp_path),
                  "train_batch_per_replica": 8,
                  "train_policy": {"type": "sft", "trainer_type": "flow_vla_sft", "mini_batch": 8},
                  "ckpt": {"enable_checkpoint": False}}})
    tr = FlowVLASFTTrainer(c, ParallelDims(world_size=1, device=torch.device("cpu")), device=torch.device("cpu"))
    tr.model_load_from_hf()
    g = torch.Generator().manual_seed(0)
    batch = [{"obs_tokens": [1024 + i, 1300 + i, 1600 + i], "state": [0.1 * i, -0.1 * i, 0.0],
              "actions": [[0.5 if i % 2 else -0.5]] * 4} for i in range(8)]
    prompts, state = [b["obs_tokens"] for b in batch], torch.tensor([b["state"] for b in batch])
    target = torch.tensor([b["actions"] for b in batch])
    t_fix, n_fix = torch.linspace(0.1, 0.9, 8), torch.randn(8, 4, 1, generator=g)
    with torch.no_grad():
        first = float(tr.model.bc_loss(prompts, target, state, t=t_fix, noise=n_fix))
    torch.manual_seed(0)
    reports = [tr.step_training(batch, total_steps=150, train_step=i + 1) for i in range(150)]
    assert tr.train_step == 150 and all(r["train/grad_norm"] > 0 for r in reports)
    with torch.no_grad():
        last = float(tr.model.bc_loss(prompts, target, state, t=t_fix, noise=n_fix))
    assert last < 0.5 * first, (first, last)
    acts = tr.model.eval().act(prompts, state, steps=8, generator=g)
    means = torch.stack([acts[i].mean() for i in range(8)])
    want = target.mean(dim=(1, 2))
    assert sum(int((m > 0) == (t > 0)) for m, t in zip(means, want)) >= 7, means.tolist()
    assert float(torch.corrcoef(torch.stack([means, want]))[0, 1]) > 0.8, means.tolist()
