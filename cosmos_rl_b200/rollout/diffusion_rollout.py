"""Rollout backend ``diffusion``: a prompt is a text embedding (``{"text_embeds": [[...]], "seed": n}``), a
completion is one generated latent (cosmos_rl/rollout/diffuers_rollout/nft_rollout.py, rollout/wfm_rollout). Latents
never travel through the controller: they stay in ``LatentStore`` on the worker and the completion only carries
their key (what the reference's payload transport does for large trajectories). ``sampler = "sde"`` additionally
records the per-step states and behaviour log-probabilities FlowGRPO trains on."""
from __future__ import annotations

import threading
import uuid
from typing import Any, Dict, List, Optional

import torch

from ..models import hf_io
from ..models.base import ModelRegistry
from ..parallel.flat import FlatParams
from ..policy import diffusion as D
from .base import RolloutBase, RolloutRegistry, RolloutResult
from .generation_mixin import RolloutGenerationMixin


class LatentStore:
    """Store of generated latents and sampler traces, keyed by the id carried in the completion. Process-local by
    default (colocated jobs); with a replay-buffer folder (``configure``: ``[custom] replay_buffer_dir``) every item is a
    file on a file system the rollout and policy workers share, so the two can be separate processes or nodes."""
    _items: Dict[str, Dict[str, torch.Tensor]] = {}
    _lock = threading.Lock()
    _fs = None                                   # utils.replay_buffer.ReplayBuffer when configured

    @classmethod
    def configure(cls, config=None, buffer_dir: Optional[str] = None) -> None:
        from ..utils.replay_buffer import ReplayBuffer, buffer_dir_of
        d = buffer_dir or buffer_dir_of(config)
        if d and (cls._fs is None or cls._fs.dir != d):
            cls._fs = ReplayBuffer(d)
        elif not d:
            cls._fs = None

    @staticmethod
    def _key(c: Any) -> str:
        return c["latent_id"] if isinstance(c, dict) else c

    @classmethod
    def put(cls, item: Dict[str, torch.Tensor]) -> str:
        if cls._fs is not None:
            return cls._fs.save(item)
        key = uuid.uuid4().hex
        with cls._lock:
            cls._items[key] = item
        return key

    @classmethod
    def get(cls, completion: Any) -> Dict[str, torch.Tensor]:
        key = cls._key(completion)
        with cls._lock:
            if key in cls._items:
                return cls._items[key]
        if cls._fs is not None:
            return cls._fs.load(key, wait_s=30.0)
        raise KeyError(f"latent {key} is not in this process; separate rollout and policy processes need "
                       f"[custom] replay_buffer_dir on a file system they share")

    @classmethod
    def release(cls, completions) -> None:
        keys = [cls._key(c) for c in completions]
        with cls._lock:
            for k in keys:
                cls._items.pop(k, None)
        if cls._fs is not None:
            cls._fs.delete(keys)

    @classmethod
    def __len__(cls) -> int:
        return len(cls._items)


def diffusion_options(config) -> Dict[str, Any]:
    d = dict(sample_steps=10, sampler="ode", solver="euler", noise_level=0.7, shift=1.0, guidance=1.0, latent_shape=[4, 8, 8],
             nft_beta=1.0, train_timesteps=4, old_decay="ramp", timestep_scheme="logit_normal")
    d.update(config.custom.get("diffusion", {}))
    return d


@RolloutRegistry.register("diffusion")
class DiffusionRollout(RolloutGenerationMixin, RolloutBase):
    def __init__(self, config, parallel_dims, device, tokenizer=None, **kw):
        super().__init__(config, parallel_dims, device)
        self.opts = diffusion_options(config)
        LatentStore.configure(config)
        self.model = None
        self.behaviour = None      # set by the NFT trainer: samples come from the trailing "old" weights

    def init_engine(self, load_format: str = "dummy", shared_model=None, **kw) -> None:
        if shared_model is not None:
            self.model = shared_model
            return
        hf_config = hf_io.load_hf_config(self.config.policy.model_name_or_path, self.config.custom.get("model_config"))
        with torch.device("meta"):
            self.model = ModelRegistry.build_model(hf_config)
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.flat = FlatParams(self.model, dtype, self.device, with_grad=False)
        self.model.init_weights(self.config.rollout.seed or 0)

    def get_underlying_model(self):
        return self.model

    def _prepare_sample(self, payload, data_packer, is_validation: bool):
        p = payload.prompt
        p = p["prompt"] if isinstance(p, dict) and "prompt" in p else p
        emb = torch.tensor(p["text_embeds"], dtype=torch.float32)
        return emb, int(p.get("seed", payload.prompt_idx if payload.prompt_idx >= 0 else 0))

    def _collate_batch(self, samples, is_validation: bool):
        n = self.config.validation.n_generation if is_validation else self.config.rollout.n_generation
        L = max(e.shape[0] for e, _ in samples)
        text = torch.zeros(len(samples), L, samples[0][0].shape[1])
        mask = torch.zeros(len(samples), L, dtype=torch.bool)
        for i, (e, _) in enumerate(samples):
            text[i, : e.shape[0]], mask[i, : e.shape[0]] = e, True
        return text.repeat_interleave(n, 0), mask.repeat_interleave(n, 0), [s for _, s in samples], n

    @torch.no_grad()
    def _generate(self, batch, is_validation: bool):
        text, mask, seeds, n = batch
        o = self.opts
        model = self.behaviour if (self.behaviour is not None and not is_validation) else self.model
        dtype = next(model.parameters()).dtype
        g = torch.Generator(device="cpu").manual_seed(1000003 * (seeds[0] + 1) + int(self.config.rollout.seed or 0))
        noise = torch.randn(text.shape[0], *o["latent_shape"], generator=g).to(self.device, dtype)
        text, mask = text.to(self.device, dtype), mask.to(self.device)
        was_training = model.training
        model.eval()
        def sample(rows: slice):
            if o["sampler"] == "sde" and not is_validation:
                return D.sde_sample(model, noise[rows], text[rows], mask[rows], o["sample_steps"], o["shift"],
                                    o["noise_level"])
            if o.get("solver", "euler") != "euler":       # higher-order / multistep ODE solvers (policy/diffusion_solvers.py)
                from ..policy.diffusion_solvers import sample
                return {"x0": sample(model, noise[rows], text[rows], mask[rows], o["sample_steps"], o["shift"],
                                     solver=o["solver"])}
            return {"x0": D.euler_sample(model, noise[rows], text[rows], mask[rows], o["sample_steps"], o["shift"])}

        # rollout.n_generation_mini_batch: the sampler sees that many latents at a time (activation memory of a large
        # group). The starting noise of every row is drawn up front, so the ODE sampler returns the same latents as in
        # one pass; the SDE sampler draws its per-step noise chunk by chunk
        mb = int(getattr(self.config.rollout, "n_generation_mini_batch", None) or 0)
        rows = text.shape[0]
        if mb > 0 and rows > mb:
            parts = [sample(slice(s_, min(s_ + mb, rows))) for s_ in range(0, rows, mb)]
            out = {k: (parts[0][k] if k == "timesteps" else torch.cat([p[k] for p in parts], 0)) for k in parts[0]}
        else:
            out = sample(slice(0, rows))
        model.train(was_training)
        out["text"], out["text_mask"] = text, mask
        return out, n

    def _postprocess(self, payloads, raw, is_validation: bool) -> List[RolloutResult]:
        out, n = raw
        results = []
        for i, p in enumerate(payloads):
            comps = []
            for j in range(i * n, (i + 1) * n):
                item = {k: v[j] for k, v in out.items() if k != "timesteps"}
                if "timesteps" in out:
                    item["timesteps"] = out["timesteps"]
                comps.append({"latent_id": LatentStore.put(item), "shape": list(out["x0"][j].shape)})
            results.append(RolloutResult(prompt=p.prompt, completions=comps))
        return results
