"""Robot demonstration data for the OpenVLA family: episodes -> per-step training records.

The reference's robot data scripts wrap simulator-specific loaders (cosmos_rl/tools/dataset/b1k_sft.py for BEHAVIOR
demonstrations, ``libero_grpo.py`` / ``robotwin2_grpo.py`` for simulator rollouts). What is independent of a simulator
is written out here:

* an episode is a dict ``{"instruction": str, "images": uint8 [T, H, W, 3], "actions": [T, A], "proprio": [T, P]
  (optional)}``, stored one per sample in tar shards (member ``episode.pt``) or ``.pt`` files of a folder;
* every (episode, step) pair is one record in the form ``data/packer.py: OpenVLADataPacker`` takes: the instruction in
  the published prompt wording, tokenised; the camera image letter-boxed to the featurizers' input size and normalised
  once per featurizer (ImageNet statistics for the first, 0.5 / 0.5 for the second), channel-stacked; the next
  ``action_chunk`` actions; the robot state;
* ``action_statistics`` computes the 1st / 99th percentiles (and the mask that leaves the last, gripper, dimension
  un-normalised) that the action bins un-normalise with: the ``norm_stats`` entry of the model config.
"""
from __future__ import annotations

import glob
import os
import zlib
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .tar_shards import expand_shards, iter_tar_samples

PROMPT = "In: What action should the robot take to {instruction}?\nOut:"
IMAGENET = ((0.485, 0.456, 0.406), (0.229, 0.224, 0.225))
HALF = ((0.5, 0.5, 0.5), (0.5, 0.5, 0.5))


def resize_with_pad(img: torch.Tensor, height: int, width: int, fill: float = 0.0) -> torch.Tensor:
    """``[C, H, W]`` float image scaled to fit ``height x width`` without distortion, centred, the rest filled."""
    C, H, W = img.shape
    ratio = max(W / width, H / height)
    nh, nw = max(1, int(H / ratio)), max(1, int(W / ratio))
    small = torch.nn.functional.interpolate(img[None], size=(nh, nw), mode="bilinear", align_corners=False,
                                            antialias=ratio > 1)[0]
    out = img.new_full((C, height, width), fill)
    top, left = (height - nh) // 2, (width - nw) // 2
    out[:, top:top + nh, left:left + nw] = small
    return out


def featurizer_pixels(image: torch.Tensor, size: int, n_featurizers: int = 2) -> torch.Tensor:
    """uint8 ``[H, W, 3]`` camera frame -> ``[3 * n, size, size]``: one normalised copy per featurizer."""
    x = image.permute(2, 0, 1).float() / 255.0
    x = resize_with_pad(x, size, size)
    outs = []
    for mean, std in (IMAGENET, HALF)[:n_featurizers]:
        m, s = torch.tensor(mean)[:, None, None], torch.tensor(std)[:, None, None]
        outs.append((x - m) / s)
    return torch.cat(outs, dim=0)


def action_statistics(episodes: Sequence[Dict[str, Any]], gripper_last: bool = True) -> Dict[str, Any]:
    """``{"action": {"q01", "q99", "mask", "mean", "std"}, "num_transitions", "num_trajectories"}`` over the episodes."""
    acts = torch.cat([torch.as_tensor(e["actions"], dtype=torch.float32) for e in episodes])
    q = torch.quantile(acts, torch.tensor([0.01, 0.99]), dim=0)
    mask = [True] * acts.shape[1]
    if gripper_last and acts.shape[1] > 1:
        mask[-1] = False                      # the gripper command is binary: kept in its own units
    return {"action": {"q01": q[0].tolist(), "q99": q[1].tolist(), "mask": mask, "mean": acts.mean(0).tolist(),
                       "std": acts.std(0).tolist()},
            "num_transitions": int(acts.shape[0]), "num_trajectories": len(episodes)}


class HashTokenizer:
    """Stand-in for jobs without a text tokenizer (tests, smoke runs): words map to stable ids in
    ``[first_id, first_id + buckets)``; id 1 opens every prompt."""

    def __init__(self, first_id: int = 1000, buckets: int = 20000):
        self.first_id, self.buckets = first_id, buckets

    def encode(self, text: str) -> List[int]:
        return [1] + [self.first_id + zlib.crc32(w.encode()) % self.buckets for w in text.split()]


def episode_bytes(ep: Dict[str, Any]) -> bytes:
    """Serialised form of one episode for ``tar_shards.write_shard`` (member ``episode.pt``)."""
    import io
    buf = io.BytesIO()
    torch.save(ep, buf)
    return buf.getvalue()


def load_episodes(source) -> List[Dict[str, Any]]:
    """Episodes from tar shards (brace pattern, glob or list; member ``episode.pt`` / ``pt``) or a folder of ``.pt``."""
    if isinstance(source, str) and os.path.isdir(source):
        return [torch.load(f, map_location="cpu", weights_only=True) for f in sorted(glob.glob(os.path.join(source, "*.pt")))]
    eps = []
    for shard in expand_shards(source):
        for s in iter_tar_samples(shard):
            ep = s.get("episode.pt", s.get("pt"))
            if isinstance(ep, (bytes, bytearray)):          # a member whose extension has no decoder arrives raw
                import io
                ep = torch.load(io.BytesIO(ep), map_location="cpu", weights_only=True)
            if isinstance(ep, dict) and "actions" in ep:
                eps.append(ep)
    return eps


class RobotStepDataset:
    """One record per (episode, step). ``setup(config, tokenizer)`` reads the image size, the number of featurizers and
    the action chunk length from the model's config."""

    def __init__(self, source=None, episodes: Optional[List[Dict[str, Any]]] = None, unnorm_key: Optional[str] = None,
                 image_size: int = 224, n_featurizers: int = 2, action_chunk: int = 1, tokenizer=None):
        self.episodes = episodes if episodes is not None else (load_episodes(source) if source is not None else [])
        self.unnorm_key, self.image_size, self.n_feat, self.chunk = unnorm_key, image_size, n_featurizers, action_chunk
        self.tokenizer = tokenizer
        self._index()

    def _index(self) -> None:
        self.index: List[Tuple[int, int]] = []
        for e, ep in enumerate(self.episodes):
            T = len(ep["actions"])
            self.index += [(e, t) for t in range(max(0, T - self.chunk + 1))]

    def setup(self, config=None, tokenizer=None, *a, **kw):
        if tokenizer is not None:
            self.tokenizer = tokenizer
        if config is not None:
            from ...models import hf_io
            from ...models.openvla import OpenVLAArgs
            d = getattr(config.train.train_policy, "dataset", None)
            if not self.episodes and d is not None and (getattr(d, "local_dir", None) or d.name):
                self.episodes = load_episodes(getattr(d, "local_dir", None) or d.name)
            args = OpenVLAArgs.from_hf_config(hf_io.load_hf_config(config.policy.model_name_or_path,
                                                                   config.custom.get("model_config")))
            self.image_size, self.n_feat = args.towers[0].image_size, len(args.towers)
            self.chunk = max(1, args.action_chunk)
            if self.unnorm_key is None and len(args.norm_stats) == 1:
                self.unnorm_key = next(iter(args.norm_stats))
            self._index()

    def __len__(self) -> int:
        return len(self.index)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        e, t = self.index[i]
        ep = self.episodes[e]
        tok = self.tokenizer or HashTokenizer()
        text = PROMPT.format(instruction=str(ep.get("instruction", "")).lower().strip())
        ids = tok.encode(text) if not hasattr(tok, "bos_token_id") else tok(text, add_special_tokens=True)["input_ids"]
        rec = {"instruction_ids": list(ids),
               "image": featurizer_pixels(torch.as_tensor(ep["images"][t]), self.image_size, self.n_feat),
               "actions": torch.as_tensor(ep["actions"][t:t + self.chunk], dtype=torch.float32).tolist()}
        if ep.get("proprio") is not None:
            rec["proprio"] = torch.as_tensor(ep["proprio"][t], dtype=torch.float32).tolist()
        if self.unnorm_key:
            rec["unnorm_key"] = self.unnorm_key
        return rec

    def get_reference_answer(self, i: int):
        return ""
