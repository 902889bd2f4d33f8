"""Datasets of the diffusion trainers (cosmos_rl/tools/dataset/diffusers_dataset.py, diffusion_nft.py).

SFT: a folder of paired files with a common basename, ``0001.json`` (metadata: caption, optional ``text_embeds``) and
``0001.pt`` / ``0001.npy`` (the latent ``[C, H, W]`` or ``[C, T, H, W]`` already encoded by the tokenizer / VAE; the
encoders themselves are not part of this package). RL: one prompt per row, carrying the text embedding.

`cosmos-rl --config <toml> cosmos_rl_b200/tools/dataset/diffusion_dataset.py` launches either, by
``train.train_policy.type``."""
from __future__ import annotations

import glob
import json
import os
from typing import Any, Dict, List

import torch


def _embed(meta: Dict[str, Any], text_dim: int, length: int = 8) -> List[List[float]]:
    """Text conditioning of a sample: precomputed ``text_embeds`` when present, else a deterministic hash embedding of
    the caption (lets jobs run without a text encoder; replace with real encoder outputs for actual training)."""
    if "text_embeds" in meta:
        if "pooled_embeds" in meta:                 # SD3-style networks read the pooled vector from row 0
            return with_pooled(meta["text_embeds"], meta["pooled_embeds"])
        return meta["text_embeds"]
    words = str(meta.get("caption", meta.get("prompt", ""))).lower().split()[:length] or ["<empty>"]
    out = []
    for w in words:
        g = torch.Generator().manual_seed(int.from_bytes(w.encode()[:8].ljust(8, b"\0"), "little") % (2 ** 31))
        out.append(torch.randn(text_dim, generator=g).tolist())
    return out


def with_pooled(text_embeds: List[List[float]], pooled: List[float]) -> List[List[float]]:
    """Put the pooled text embedding in front of the token embeddings as row 0, zero-padded to their width: the layout
    two-stream networks with a pooled conditioning input expect (``models/mmdit.py``)."""
    width = len(text_embeds[0])
    if len(pooled) > width:
        raise ValueError(f"pooled embedding of {len(pooled)} values does not fit the text width {width}")
    return [list(pooled) + [0.0] * (width - len(pooled))] + [list(r) for r in text_embeds]


class LatentFolderDataset:
    def __init__(self, folder: str = "", text_dim: int = 1024):
        self.folder, self.text_dim = folder, text_dim
        self.names: List[str] = []

    def setup(self, config, tokenizer=None, *a, **kw):
        d = config.train.train_policy.dataset
        self.folder = self.folder or getattr(d, "local_dir", None) or d.name
        self.names = sorted(os.path.splitext(f)[0] for f in glob.glob(os.path.join(self.folder, "*.json")))

    def __len__(self) -> int:
        return len(self.names)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        base = self.names[i]
        with open(base + ".json") as f:
            meta = json.load(f)
        if os.path.exists(base + ".pt"):
            z = torch.load(base + ".pt", map_location="cpu")
        else:
            import numpy as np
            z = torch.from_numpy(np.load(base + ".npy"))
        return {"latents": z.float(), "text_embeds": _embed(meta, self.text_dim)}


class PromptEmbeddingDataset:
    """RL prompts: rows of a jsonl file with ``prompt`` (and optionally ``text_embeds``)."""

    def __init__(self, path: str = "", text_dim: int = 1024):
        self.path, self.text_dim, self.rows = path, text_dim, []

    def setup(self, config, tokenizer=None, *a, **kw):
        path = self.path or config.train.train_policy.dataset.name
        with open(path) as f:
            self.rows = [json.loads(ln) for ln in f if ln.strip()]

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        return {"text_embeds": _embed(self.rows[i], self.text_dim), "seed": i, "prompt": self.rows[i].get("prompt", "")}

    def get_reference_answer(self, i: int):
        return self.rows[i].get("prompt", "")


def latent_norm_reward(completion, reference=None, **kw) -> float:
    """Reference-free placeholder reward (keeps latents near unit scale); real jobs score decoded media through the
    reward service."""
    from cosmos_rl_b200.rollout.diffusion_rollout import LatentStore
    x = LatentStore.get(completion)["x0"].float()
    return -abs(float(x.pow(2).mean()) - 1.0)


if __name__ == "__main__":
    from cosmos_rl_b200.config import Config, load_toml
    from cosmos_rl_b200.launcher.worker_entry import main
    cfg_path = os.environ.get("COSMOS_CONFIG")
    is_sft = bool(cfg_path) and Config.from_dict(load_toml(cfg_path)).train.train_policy.type == "sft"
    if is_sft:
        main(dataset=LatentFolderDataset())
    else:
        main(dataset=PromptEmbeddingDataset(), reward_fns=[latent_norm_reward])
