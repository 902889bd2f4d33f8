"""SFT smoke job on generated conversations (no files needed): `cosmos-rl --config <sft toml> .../dummy_sft.py`
(cosmos_rl/tools/dataset/dummy_sft.py)."""
from __future__ import annotations

import random


class DummySFTDataset:
    def __init__(self, n: int = 512, seed: int = 0):
        self.n, self.seed = n, seed

    def setup(self, config, tokenizer=None, *a, **kw):
        self.config, self.tokenizer = config, tokenizer

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, i: int):
        rng = random.Random(self.seed * 7919 + i)
        a, b = rng.randint(0, 999), rng.randint(0, 999)
        if self.tokenizer is None:          # token-id form for tokenizer-less runs
            ids = [rng.randrange(1000) for _ in range(rng.randint(8, 48))]
            return {"input_ids": ids}
        return [{"role": "user", "content": f"What is {a} + {b}?"}, {"role": "assistant", "content": str(a + b)}]


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=DummySFTDataset(), val_dataset=DummySFTDataset(64, seed=1))
