"""Rollout backend ``openvla``: the image-conditioned action-token policy (``models/openvla.py``) in closed loop with an
environment (cosmos_rl/rollout/vla_rollout/ drives the published model against LIBERO / RoboTwin the same way:
observation image + instruction in, ``action_dim`` tokens out, un-normalised, stepped).

One "prompt" is an initial condition (``{"seed": n}``), one "completion" a whole episode. At every control step the
state is drawn by the software rasteriser (``simulators/render.py``; the rendered simulators need a graphics stack),
normalised once per featurizer, and spliced into the prompt; the policy samples ``action_dim`` tokens one after the
other from the softmax over the ACTION BINS only (re-running the packed forward: no KV cache, as the other families
without a paged-attention path), the tokens decode to an action, the batched environment steps. Per step the episode
keeps prompt ids, pixels, action tokens and their behaviour log-probabilities in the trajectory store; the completion
that travels through the controller carries the key, the rewards and the executed actions."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

import torch

from ..models import hf_io
from ..models.base import ModelRegistry
from ..models.openvla import build_prompt
from ..parallel.flat import FlatParams
from ..simulators import EnvManager, get_env_cls
from ..simulators.render import render_state
from ..tools.dataset.robot_records import PROMPT, HashTokenizer, featurizer_pixels
from .base import RolloutBase, RolloutRegistry, RolloutResult
from .diffusion_rollout import LatentStore
from .vla_rollout import ENV_SPECS

INSTRUCTIONS = {"cartpole": "keep the pole upright", "pendulum": "swing the pendulum up"}


def openvla_options(config) -> Dict[str, Any]:
    d = dict(env_name="cartpole", max_steps=40, num_envs=16, subprocess_env=False, instruction=None)
    d.update(config.custom.get("vla", {}))
    return d


@RolloutRegistry.register("openvla")
class OpenVLARollout(RolloutBase):
    def __init__(self, config, parallel_dims, device, tokenizer=None, **kw):
        super().__init__(config, parallel_dims, device)
        self.opts = openvla_options(config)
        self.tokenizer = tokenizer
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
        self.discrete = bool(spec["discrete"])
        self.n_actions = int(spec["act_high"][0]) + 1 if self.discrete else 0
        self.act_dim = 1 if self.discrete else len(spec["act_low"])
        self.act_low = torch.tensor(spec["act_low"], dtype=torch.float32)
        self.act_high = torch.tensor(spec["act_high"], dtype=torch.float32)
        tok = self.tokenizer or HashTokenizer()
        text = PROMPT.format(instruction=str(o["instruction"] or INSTRUCTIONS.get(o["env_name"], o["env_name"])))
        ids = tok.encode(text) if not hasattr(tok, "bos_token_id") else tok(text, add_special_tokens=True)["input_ids"]
        self.prompt_ids = build_prompt(list(ids), self.model.n_patches, self.model.args.image_token_id)
        self.image_size = self.model.args.towers[0].image_size
        self.n_feat = len(self.model.args.towers)
        self.env = EnvManager({"num_envs": o["num_envs"], "env_name": o["env_name"], "max_steps": o["max_steps"]},
                              0, get_env_cls(o["env_name"]), use_subprocess=bool(o["subprocess_env"]))

    def get_underlying_model(self):
        return self.model

    def _seed_of(self, prompt) -> int:
        p = prompt["prompt"] if isinstance(prompt, dict) and "prompt" in prompt else prompt
        p = json.loads(p) if isinstance(p, str) else p
        return int(p["seed"] if isinstance(p, dict) else p)

    def _action_of(self, tokens: List[int]):
        lo, _ = self.model.action_token_range
        if self.discrete:
            return (tokens[0] - lo) % self.n_actions
        n = self.model.args.n_action_bins
        frac = torch.tensor([(t - lo + 0.5) / n for t in tokens])
        return (self.act_low + frac * (self.act_high - self.act_low)).tolist()

    @torch.no_grad()
    def _sample_actions(self, pixels: torch.Tensor, temperature: float, greedy: bool, gen) -> tuple:
        """``pixels [B, 3 * featurizers, S, S]`` -> action tokens ``[B, act_dim]`` and their log-probs under the softmax
        over the action bins."""
        m, dev = self.model, self.device
        B = pixels.shape[0]
        lo, _ = m.action_token_range
        seqs = [list(self.prompt_ids) for _ in range(B)]
        toks = torch.zeros(B, self.act_dim, dtype=torch.long)
        lps = torch.zeros(B, self.act_dim)
        m.mm_inputs = {"pixel_values": pixels.to(dev)}
        for d in range(self.act_dim):
            L = len(seqs[0])
            ids = torch.tensor([t for s in seqs for t in s], dtype=torch.long, device=dev)
            cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=dev)
            h = m(ids, m.get_position_ids(cu, int(ids.numel())), cu, L)
            lsm = torch.log_softmax(m.action_logits(h[(cu[1:] - 1).long()]) / max(temperature, 1e-6), dim=-1).cpu()
            pick = lsm.argmax(-1) if greedy else torch.multinomial(lsm.exp(), 1, generator=gen)[:, 0]
            toks[:, d] = pick + lo
            lps[:, d] = lsm.gather(1, pick[:, None])[:, 0]
            for b in range(B):
                seqs[b].append(int(toks[b, d]))
        return toks, lps

    @torch.no_grad()
    def rollout_generation(self, payloads, data_packer, data_fetcher=None, is_validation: bool = False, **kw
                           ) -> List[RolloutResult]:
        o = self.opts
        n = self.config.validation.n_generation if is_validation else self.config.rollout.n_generation
        temperature = float(self.config.rollout.sampling_config.temperature)
        seeds = [self._seed_of(p.prompt) for p in payloads for _ in range(n)]     # a group shares its initial condition
        gen = torch.Generator(device="cpu").manual_seed(1000003 * (seeds[0] + 1) + int(self.config.rollout.seed or 0))
        was_training = self.model.training
        self.model.eval()
        self.env.start_simulator()
        E = o["num_envs"]
        episodes: List[Dict[str, Any]] = []
        for s0 in range(0, len(seeds), E):
            chunk = seeds[s0:s0 + E]
            ids = list(range(len(chunk)))
            obs = self.env.reset(ids, chunk)
            eps = [{"rewards": [], "actions": [], "steps": []} for _ in ids]
            live = list(ids)
            for _ in range(o["max_steps"]):
                if not live:
                    break
                pixels = torch.stack([featurizer_pixels(render_state(o["env_name"], obs[i], self.image_size),
                                                        self.image_size, self.n_feat) for i in live])
                toks, lps = self._sample_actions(pixels, temperature, is_validation, gen)
                acts = [self._action_of(toks[j].tolist()) for j in range(len(live))]
                res = self.env.step(live, acts)
                nxt = []
                for j, i in enumerate(live):
                    eps[i]["rewards"].append(res["rewards"][j])
                    eps[i]["actions"].append(acts[j])
                    if not is_validation:
                        eps[i]["steps"].append({"pixel_values": pixels[j].to(torch.float16), "action_tokens": toks[j].tolist(),
                                                "logprobs": lps[j].tolist()})
                    obs[i] = res["observations"][j]
                    if not (res["terminated"][j] or res["truncated"][j]):
                        nxt.append(i)
                live = nxt
            episodes.extend(eps)
        self.env.stop_simulator()
        self.model.train(was_training)
        results = []
        for i, p in enumerate(payloads):
            comps = [{"latent_id": LatentStore.put({"prompt_ids": self.prompt_ids, "steps": e["steps"]}),
                      "rewards": e["rewards"], "actions": e["actions"], "episode_length": len(e["rewards"])}
                     for e in episodes[i * n:(i + 1) * n]]
            results.append(RolloutResult(prompt=p.prompt, completions=comps))
        return results
