"""Exponential moving average of the flat parameter buffer (cosmos_rl/utils/ema.py:21-130)."""
from __future__ import annotations

import contextlib

import torch


class FlatEMA:
    def __init__(self, flat_data: torch.Tensor, decay: float = 0.999, update_interval: int = 1):
        self.src = flat_data
        self.decay = decay
        self.interval = max(1, update_interval)
        self.shadow = flat_data.detach().to(torch.float32).clone()
        self.n = 0

    @torch.no_grad()
    def update(self) -> None:
        self.n += 1
        if self.n % self.interval:
            return
        d = self.decay ** self.interval
        self.shadow.mul_(d).add_(self.src.to(torch.float32), alpha=1.0 - d)

    @contextlib.contextmanager
    def swapped_in(self):
        """Temporarily evaluate / export with the averaged weights."""
        backup = self.src.clone()
        self.src.copy_(self.shadow.to(self.src.dtype))
        try:
            yield
        finally:
            self.src.copy_(backup)

    def state_dict(self):
        return {"shadow": self.shadow, "n": self.n}

    def load_state_dict(self, sd):
        self.shadow.copy_(sd["shadow"])
        self.n = int(sd["n"])
