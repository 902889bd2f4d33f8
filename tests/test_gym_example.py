"""The control-task example: environment physics, the env manager in a child process, the trajectory-iteration
contract, and the whole colocated loop (controller, custom rollout backend, reward, custom trainer) learning to
balance the pole on CPU."""
import math
import os

import torch

from cosmos_rl_b200.config import Config, load_toml
from cosmos_rl_b200.dispatcher.data.schema import Rollout
from cosmos_rl_b200.parallel.dims import ParallelDims
from cosmos_rl_b200.simulators import BatchedControlEnv, CartPoleEnv, EnvManager, PendulumEnv, SimulatorUnavailable, get_env_cls
from cosmos_rl_b200.tools import gym_example as G
from cosmos_rl_b200.tools.gym_example.gym_entry import GymSeedDataset

CFG_DIR = os.path.join(os.path.dirname(G.__file__), "configs")


def test_environment_physics_and_termination():
    env = CartPoleEnv(max_steps=500)
    obs, _ = env.reset(seed=1)
    assert len(obs) == 4 and all(abs(v) <= 0.05 for v in obs)
    steps, term = 0, False
    while not term and steps < 500:                # always pushing right tips the pole over quickly
        obs, r, term, trunc, _ = env.step(1)
        steps += 1
        assert r == 1.0
    assert term and steps < 60 and abs(obs[2]) > CartPoleEnv.theta_limit
    p = PendulumEnv(max_steps=5)
    o, _ = p.reset(seed=2)
    assert abs(o[0] ** 2 + o[1] ** 2 - 1.0) < 1e-9
    th, thd = p.th, p.thd
    o, r, term, trunc, _ = p.step([0.0])
    want = thd + 3 * 10.0 / 2 * math.sin(th) * 0.05              # one Euler step without torque
    assert abs(p.thd - want) < 1e-9 and r <= 0 and not term
    for _ in range(4):
        _, _, _, trunc, _ = p.step([5.0])                          # torque is clipped to 2
    assert trunc


def test_env_manager_subprocess_keeps_state_across_restart():
    m = EnvManager({"num_envs": 2, "env_name": "cartpole", "max_steps": 50}, 0, get_env_cls("cartpole"),
                   use_subprocess=True)
    m.start_simulator()
    m.reset([0, 1], [11, 12])
    for _ in range(3):
        out = m.step([0, 1], [0, 1])
    assert out["rewards"] == [1.0, 1.0]
    before = m.get_env_states([0, 1])
    m.stop_simulator()
    assert m.process is None and m.state_buffer
    m.start_simulator()
    assert m.get_env_states([0, 1]) == before and before[0]["length"] == 3
    m.stop_simulator()
    try:
        get_env_cls("libero")
        assert False
    except SimulatorUnavailable as e:
        assert "graphics" in str(e)


def test_trajectory_contract_and_chunk_mode():
    from cosmos_rl_b200.policy.trainer.trajectory_mixin import TrajectoryExpansionMixin
    packer = G.GymDataPacker()
    traj = {"observations": [[0.0] * 4] * 5, "actions": [0, 1, 0, 1, 1], "rewards": [1.0] * 5, "logprobs": [-0.7] * 5,
            "episode_length": 5}
    ros = [Rollout(prompt='{"seed": 1}', completion=traj), Rollout(prompt='{"seed": 2}', completion=traj)]
    assert packer.get_rollout_input('{"seed": 7}') == 7 and packer.num_transitions(ros[0]) == 5
    assert [len(c) for c in packer.iter_chunks(ros[:1], 2)] == [2, 2, 1]

    class Chunked(TrajectoryExpansionMixin):
        chunk_size = 2
        data_packer = packer

        def _begin_training_step(self, rollouts, *a, **kw):
            return {"chunks": []}

        def _train_one_chunk(self, rollout, chunk, state, *a, **kw):
            state["chunks"].append(len(chunk))

        def _finalize_training_step(self, rollouts, state, *a, **kw):
            return {"chunks": state["chunks"]}

    assert Chunked().step_training(ros)["chunks"] == [2, 2, 1, 2, 2, 1]      # chunks never span two rollouts
    assert torch.allclose(G.compute_returns(torch.tensor([1.0, 1.0, 1.0]), 0.5), torch.tensor([1.75, 1.5, 1.0]))


def test_cartpole_learns_through_the_colocated_worker(tmp_path):
    from cosmos_rl_b200.colocated.worker import ColocatedRLControlWorker
    c = Config.from_dict(load_toml(os.path.join(CFG_DIR, "cartpole_colocated.toml")))
    c.train.output_dir = str(tmp_path)
    c.train.train_batch_per_replica = 32
    c.rollout.batch_size, c.rollout.n_generation = 8, 4
    w = ColocatedRLControlWorker(c, GymSeedDataset(n=480), reward_fns=[G.gym_episode_reward],
                                 data_packer=G.GymDataPacker(), device=torch.device("cpu"))
    assert type(w.trainer).__name__ == "GymTrainer" and type(w.rollout).__name__ == "GymRolloutBackend"
    assert w.rollout.model is w.trainer.model                       # colocated: one set of weights
    reports = w.run(max_iterations=500)
    rets = [r["train/episode_return"] for r in reports]
    assert len(rets) == 60 and sum(rets[-5:]) / 5 > 2.0 * sum(rets[:5]) / 5, (rets[:5], rets[-5:])
    # a second, continuous-action config resolves and plays an episode
    p = Config.from_dict(load_toml(os.path.join(CFG_DIR, "pendulum_colocated.toml")))
    pol = G.GymPolicy(G.GymMLPConfig.from_dict(p.custom["gym"]))
    eng = G.GymRolloutEngine(pol, env_name="pendulum", num_envs=2, max_steps=20)
    t = eng.run([1, 2, 3])
    assert len(t) == 3 and t[0]["episode_length"] == 20 and isinstance(t[0]["actions"][0], list)


def test_launcher_runs_the_colocated_example_as_one_process(tmp_path):
    """`cosmos-rl --config cartpole_colocated.toml gym_entry.py`: the launcher starts one colocated process."""
    import subprocess
    import sys
    raw = load_toml(os.path.join(CFG_DIR, "cartpole_colocated.toml"))
    raw["train"]["output_dir"] = str(tmp_path / "out")
    from cosmos_rl_b200.config import dump_toml
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml(raw))
    entry = os.path.join(os.path.dirname(G.__file__), "gym_entry.py")
    env = dict(os.environ, GYM_EXAMPLE_EPISODE_SEEDS="64", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", str(cfg), "--cpu",
                        "--log-dir", str(tmp_path / "logs"), entry], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    log = open(tmp_path / "logs" / "logs_latest" / "colocated_0.log").read()
    assert "[Colocated] finished after" in log
