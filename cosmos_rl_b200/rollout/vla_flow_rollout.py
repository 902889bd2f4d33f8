"""Rollout backend ``flow_vla``: a policy with a flow-matching action expert in closed loop with an environment
(the role of cosmos_rl/rollout/vla_rollout/ for PI0.5-style policies: continuous action chunks, explored by sampling
the flow as an SDE).

One "prompt" is an initial condition (``{"seed": n}``), one "completion" a whole episode. At every decision point the
observation becomes the backbone's prompt tokens and the proprioceptive state, the policy draws one chunk of
``horizon`` actions by integrating its flow with noise injected at every step, and the batched environment executes
the first ``exec_horizon`` actions of the chunk. For every chunk the episode keeps what the trainer needs to score it
again: prompt tokens, state, and the SDE transitions (states, next states, behaviour log-probabilities). Those tensors
stay in ``LatentStore`` on the worker; the completion that travels through the controller carries their key, the
per-chunk rewards and the executed actions (environment units), which is what reward functions see."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

import torch

from ..models import hf_io
from ..models.base import ModelRegistry
from ..models.vla_flow import denormalize_actions
from ..parallel.flat import FlatParams
from ..simulators import EnvManager, get_env_cls
from .base import RolloutBase, RolloutRegistry, RolloutResult
from .diffusion_rollout import LatentStore
from .vla_rollout import ENV_SPECS, ObservationTokenizer


def flow_vla_options(config) -> Dict[str, Any]:
    d = dict(env_name="pendulum", max_steps=48, num_envs=16, n_bins=256, subprocess_env=False, flow_steps=4,
             noise_level=0.7, exec_horizon=0, eval_solver="euler")
    d.update(config.custom.get("vla", {}))
    return d


@RolloutRegistry.register("flow_vla")
class FlowVLARollout(RolloutBase):
    def __init__(self, config, parallel_dims, device, tokenizer=None, **kw):
        super().__init__(config, parallel_dims, device)
        self.opts = flow_vla_options(config)
        LatentStore.configure(config)
        self.model = None

    def init_engine(self, load_format: str = "dummy", shared_model=None, seed: Optional[int] = None, **kw) -> None:
        if shared_model is not None:
            self.model = shared_model
        else:
            hf_config = hf_io.load_hf_config(self.config.policy.model_name_or_path, self.config.custom.get("model_config"))
            with torch.device("meta"):
                self.model = ModelRegistry.build_model(hf_config)
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            self.flat = FlatParams(self.model, dtype, self.device, with_grad=False)
            self.model.init_weights(self.config.rollout.seed or 0)
        o = self.opts
        spec = ENV_SPECS[o["env_name"]]
        if spec["discrete"]:
            raise ValueError(f"environment {o['env_name']!r} has discrete actions; the flow policy acts in a continuous space")
        a = self.model.args
        if a.action_dim != len(spec["act_low"]) or a.state_dim not in (0, len(spec["obs_low"])):
            raise ValueError(f"the policy acts in {a.action_dim} dimensions with a {a.state_dim}-dimensional state; "
                             f"{o['env_name']} has {len(spec['act_low'])} and {len(spec['obs_low'])}")
        self.observations = ObservationTokenizer(spec["obs_low"], spec["obs_high"], o["n_bins"])
        self.act_low = torch.tensor(spec["act_low"], dtype=torch.float32)
        self.act_high = torch.tensor(spec["act_high"], dtype=torch.float32)
        self.env = EnvManager({"num_envs": o["num_envs"], "env_name": o["env_name"], "max_steps": o["max_steps"]},
                              0, get_env_cls(o["env_name"]), use_subprocess=bool(o["subprocess_env"]))

    def get_underlying_model(self):
        return self.model

    def _seed_of(self, prompt) -> int:
        p = prompt["prompt"] if isinstance(prompt, dict) and "prompt" in prompt else prompt
        p = json.loads(p) if isinstance(p, str) else p
        return int(p["seed"] if isinstance(p, dict) else p)

    @torch.no_grad()
    def rollout_generation(self, payloads, data_packer, data_fetcher=None, is_validation: bool = False, **kw
                           ) -> List[RolloutResult]:
        o, a = self.opts, self.model.args
        n = self.config.validation.n_generation if is_validation else self.config.rollout.n_generation
        # the members of a group start from the SAME initial condition and differ only in the exploration noise, so
        # the group-relative advantage measures the actions, not the luck of the start
        seeds = [self._seed_of(p.prompt) for p in payloads for _ in range(n)]
        H = a.horizon
        exec_h = int(o["exec_horizon"]) or H
        episodes: List[Dict[str, Any]] = []
        was_training = self.model.training
        self.model.eval()
        self.env.start_simulator()
        E = o["num_envs"]
        gen = torch.Generator(device="cpu").manual_seed(1000003 * (seeds[0] + 1) + int(self.config.rollout.seed or 0))
        for s0 in range(0, len(seeds), E):
            chunk_seeds = seeds[s0:s0 + E]
            ids = list(range(len(chunk_seeds)))
            obs = self.env.reset(ids, chunk_seeds)
            eps = [{"rewards": [], "chunks": [], "actions": []} for _ in ids]
            live = list(ids)
            steps_left = o["max_steps"]
            while live and steps_left > 0:
                prompts = [self.observations.encode(obs[i]) for i in live]
                state = torch.tensor([obs[i] for i in live], dtype=torch.float32, device=self.device) \
                    if a.state_dim else None
                if is_validation:
                    x0 = self.model.act(prompts, state, steps=o["flow_steps"], solver=o["eval_solver"], generator=gen)
                    trace = None
                else:
                    trace = self.model.explore(prompts, state, steps=o["flow_steps"], noise_level=o["noise_level"],
                                               generator=gen)
                    x0 = trace["x0"]
                acts = denormalize_actions(x0.float().cpu(), self.act_low, self.act_high)      # [B, H, A]
                k = min(exec_h, steps_left)
                res = self.env.chunk_step(live, [[acts[j, t].tolist() for t in range(k)] for j in range(len(live))])
                steps_left -= k
                nxt = []
                for j, i in enumerate(live):
                    eps[i]["rewards"].append(res["rewards"][j])
                    eps[i]["actions"].extend(acts[j, :k].tolist())
                    if trace is not None:
                        eps[i]["chunks"].append({"obs_tokens": prompts[j],
                                                 "state": state[j].cpu() if state is not None else None,
                                                 "states": trace["states"][j].cpu(), "next_states": trace["next_states"][j].cpu(),
                                                 "logprobs": trace["logprobs"][j].cpu(), "timesteps": trace["timesteps"].cpu()})
                    obs[i] = res["observations"][j]
                    if not (res["terminated"][j] or res["truncated"][j]):
                        nxt.append(i)
                live = nxt
            episodes.extend(eps)
        self.env.stop_simulator()
        self.model.train(was_training)
        results = []
        for i, p in enumerate(payloads):
            comps = []
            for e in episodes[i * n:(i + 1) * n]:
                comps.append({"latent_id": LatentStore.put({"chunks": e["chunks"]}), "rewards": e["rewards"],
                              "actions": e["actions"], "n_chunks": len(e["rewards"])})
            results.append(RolloutResult(prompt=p.prompt, completions=comps))
        return results
