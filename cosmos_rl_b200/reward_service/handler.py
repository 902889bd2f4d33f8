"""Reward handlers: ``calculate_reward(tensor, metadata) -> {"scores": {...}, "duration": s, "type": name}``
(reward_service/cosmos_rl_reward/handler/reward_base.py, handler/registry.py). Model-backed handlers load their
weights from a local path in ``set_up``; the built-in ones need no weights and serve as reference-free signals and
as the test surface of the service."""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, List, Optional, Type

import torch


class RewardHandlerRegistry:
    _handlers: Dict[str, Type["BaseRewardHandler"]] = {}

    @classmethod
    def register(cls, name: str):
        def deco(c):
            c.reward_name = name
            cls._handlers[name] = c
            return c
        return deco

    @classmethod
    def create(cls, name: str, **kw) -> "BaseRewardHandler":
        if name not in cls._handlers:
            raise KeyError(f"unknown reward {name!r}; known: {sorted(cls._handlers)}")
        h = cls._handlers[name](**kw)
        h.set_up()
        return h

    @classmethod
    def known(cls) -> List[str]:
        return sorted(cls._handlers)


class BaseRewardHandler:
    reward_name = "base"

    def __init__(self, device: str = "cpu", **kw):
        self.device = torch.device(device)
        self.options = kw

    def set_up(self) -> None:
        """Load models / tokenizers. Called once in the scoring worker."""

    def score(self, media: Optional[torch.Tensor], metadata: Dict[str, Any]) -> Dict[str, List[float]]:
        raise NotImplementedError

    def calculate_reward(self, media: Optional[torch.Tensor], metadata: Dict[str, Any]) -> Dict[str, Any]:
        t0 = time.perf_counter()
        info = None
        if media is not None:
            m = media.float()
            info = {"shape": list(media.shape), "min": float(m.min()), "max": float(m.max())}
        scores = self.score(media, metadata)
        return {"scores": scores, "input_info": info, "duration": time.perf_counter() - t0, "type": self.reward_name}


def _as_video(media: torch.Tensor) -> torch.Tensor:
    """[B, C, H, W] or [B, C, T, H, W] -> float [B, C, T, H, W] in 0..1."""
    x = media.float()
    if media.dtype == torch.uint8:
        x = x / 255.0
    return x.unsqueeze(2) if x.dim() == 4 else x


@RewardHandlerRegistry.register("sharpness")
class SharpnessReward(BaseRewardHandler):
    """Mean Laplacian energy per sample: a reference-free focus measure."""

    def score(self, media, metadata):
        x = _as_video(media).to(self.device).mean(1)                         # luminance [B, T, H, W]
        k = torch.tensor([[0.0, 1.0, 0.0], [1.0, -4.0, 1.0], [0.0, 1.0, 0.0]], device=self.device)[None, None]
        B, T, H, W = x.shape
        lap = torch.nn.functional.conv2d(torch.nn.functional.pad(x.reshape(B * T, 1, H, W), (1, 1, 1, 1), mode="replicate"), k)
        return {"sharpness": lap.pow(2).mean(dim=(1, 2, 3)).view(B, T).mean(1).tolist()}


@RewardHandlerRegistry.register("temporal_smoothness")
class TemporalSmoothnessReward(BaseRewardHandler):
    """Negative mean squared frame difference of a video (0 for a still image)."""

    def score(self, media, metadata):
        x = _as_video(media).to(self.device)
        if x.shape[2] < 2:
            return {"temporal_smoothness": [0.0] * x.shape[0]}
        return {"temporal_smoothness": (-(x[:, :, 1:] - x[:, :, :-1]).pow(2).mean(dim=(1, 2, 3, 4))).tolist()}


@RewardHandlerRegistry.register("prompt_keyword")
class PromptKeywordReward(BaseRewardHandler):
    """Text-side reward: fraction of ``metadata["keywords"]`` found in each of ``metadata["texts"]``."""

    def score(self, media, metadata):
        kws = [k.lower() for k in metadata.get("keywords", [])]
        out = []
        for t in metadata.get("texts", []):
            low = str(t).lower()
            out.append(sum(k in low for k in kws) / max(1, len(kws)))
        return {"prompt_keyword": out}


@RewardHandlerRegistry.register("torchscript")
class TorchScriptReward(BaseRewardHandler):
    """A scoring network exported with ``torch.jit.save`` (``model_path`` option): called on the media batch, must
    return one score per sample. This is how learned image / video reward models are plugged in offline."""

    def set_up(self) -> None:
        self.model = torch.jit.load(self.options["model_path"], map_location=self.device).eval()

    @torch.no_grad()
    def score(self, media, metadata):
        return {self.options.get("score_name", "model_score"): self.model(_as_video(media).to(self.device)).flatten().tolist()}
