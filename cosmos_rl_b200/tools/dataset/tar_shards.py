"""Streaming data sets over tar shards (the "webdataset" layout) with an augmentation pipeline.

Image / video training sets of the world-model trainers are published as many tar files in which consecutive members
that share a basename form one sample (``0001.json`` + ``0001.pt`` + ``0001.txt`` ...). The reference reads them with
the ``webdataset`` package and its own augmentor classes (cosmos_rl/tools/dataset/wfm/webdataset/webdataset.py:200-340,
``augmentors/``); that package is not a dependency here, so the reader is written out:

* shard lists from brace patterns (``data/shard-{000..127}.tar``), globs or explicit lists;
* shards are dealt out to ``rank`` of ``world`` (data-parallel ranks) and again to data-loader workers, re-shuffled every
  epoch from ``seed + epoch``; samples pass through a bounded shuffle buffer;
* members are decoded by extension (``json``, ``txt``, ``pt`` / ``pth``, ``npy``; further ones can be registered), a
  member that fails to decode skips its sample (a corrupt file must not end a training run);
* augmentors are callables ``sample -> sample | None`` applied in order; the ones the latent / pixel pipelines need are
  here (resize-crop, horizontal flip, normalise, frame sampling, caption drop-out for classifier-free guidance).
"""
from __future__ import annotations

import glob
import io
import json
import random
import re
import tarfile
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch

from ...utils.logging import logger


# ---------------------------------------------------------------------------------------------------
# shard lists
# ---------------------------------------------------------------------------------------------------
def expand_shards(spec) -> List[str]:
    """``"a-{00..03}.tar"`` -> four names (several brace ranges multiply); a glob -> its matches, sorted; a list ->
    every entry expanded."""
    if isinstance(spec, (list, tuple)):
        return [s for x in spec for s in expand_shards(x)]
    m = re.search(r"\{(\d+)\.\.(\d+)\}", spec)
    if m:
        lo, hi, width = int(m.group(1)), int(m.group(2)), len(m.group(1))
        return [s for i in range(lo, hi + 1) for s in expand_shards(spec[:m.start()] + str(i).zfill(width) + spec[m.end():])]
    if any(c in spec for c in "*?["):
        return sorted(glob.glob(spec))
    return [spec]


# ---------------------------------------------------------------------------------------------------
# decoding
# ---------------------------------------------------------------------------------------------------
def _npy(b: bytes):
    import numpy as np
    return torch.from_numpy(np.load(io.BytesIO(b), allow_pickle=False))


DECODERS: Dict[str, Callable[[bytes], Any]] = {
    "json": lambda b: json.loads(b.decode("utf-8")),
    "txt": lambda b: b.decode("utf-8").strip(),
    "pt": lambda b: torch.load(io.BytesIO(b), map_location="cpu", weights_only=True),
    "pth": lambda b: torch.load(io.BytesIO(b), map_location="cpu", weights_only=True),
    "npy": _npy,
}


def iter_tar_samples(path: str, decoders: Optional[Dict[str, Callable]] = None) -> Iterator[Dict[str, Any]]:
    """Samples of one shard: ``{"__key__": basename, "__shard__": path, <extension>: decoded member, ...}``."""
    dec = DECODERS if decoders is None else decoders
    cur: Dict[str, Any] = {}
    with tarfile.open(path, "r:*") as tf:
        for m in tf:
            if not m.isfile():
                continue
            base = m.name.rsplit("/", 1)[-1]
            key, _, ext = base.partition(".")
            key = m.name[: len(m.name) - len(base)] + key
            if cur and cur["__key__"] != key:
                if "__bad__" not in cur:
                    yield cur
                cur = {}
            if not cur:
                cur = {"__key__": key, "__shard__": path}
            raw = tf.extractfile(m).read()
            try:
                cur[ext] = dec[ext](raw) if ext in dec else raw
            except Exception as e:  # noqa: BLE001
                logger.warning("[tar shards] %s in %s does not decode (%s): sample skipped", m.name, path, e)
                cur["__bad__"] = True
    if cur and "__bad__" not in cur:
        yield cur


# ---------------------------------------------------------------------------------------------------
# augmentors
# ---------------------------------------------------------------------------------------------------
class ResizeCrop:
    """Scale the pixel tensor ``[..., H, W]`` under ``key`` so that it covers ``size`` and cut the centre (or a random
    window when ``random_crop``)."""

    def __init__(self, key: str, size: Tuple[int, int], random_crop: bool = False, seed: int = 0):
        self.key, self.size, self.random_crop, self.rng = key, size, random_crop, random.Random(seed)

    def __call__(self, s):
        x = s[self.key].float()
        lead = x.shape[:-2]
        H, W = x.shape[-2:]
        th, tw = self.size
        f = max(th / H, tw / W)
        nh, nw = max(th, round(H * f)), max(tw, round(W * f))
        x = torch.nn.functional.interpolate(x.reshape(-1, 1, H, W), size=(nh, nw), mode="bilinear", align_corners=False,
                                            antialias=f < 1)
        y0 = self.rng.randint(0, nh - th) if self.random_crop else (nh - th) // 2
        x0 = self.rng.randint(0, nw - tw) if self.random_crop else (nw - tw) // 2
        s[self.key] = x[..., y0:y0 + th, x0:x0 + tw].reshape(*lead, th, tw)
        return s


class HorizontalFlip:
    def __init__(self, keys: Sequence[str], p: float = 0.5, seed: int = 0):
        self.keys, self.p, self.rng = list(keys), p, random.Random(seed)

    def __call__(self, s):
        if self.rng.random() < self.p:
            for k in self.keys:
                s[k] = s[k].flip(-1)
        return s


class Normalize:
    """``(x / scale - mean) / std`` per channel; the channel axis is ``channel_dim`` (0 for ``[C, H, W]`` and
    ``[C, T, H, W]``)."""

    def __init__(self, key: str, mean: Sequence[float], std: Sequence[float], scale: float = 255.0, channel_dim: int = 0):
        self.key, self.mean, self.std, self.scale, self.cd = key, list(mean), list(std), scale, channel_dim

    def __call__(self, s):
        x = s[self.key].float() / self.scale
        shape = [1] * x.dim()
        shape[self.cd] = -1
        s[self.key] = (x - torch.tensor(self.mean).view(shape)) / torch.tensor(self.std).view(shape)
        return s


class SampleFrames:
    """Keep ``n`` frames of a video ``[C, T, H, W]`` at a fixed stride from a random start; shorter clips are dropped."""

    def __init__(self, key: str, n: int, stride: int = 1, seed: int = 0):
        self.key, self.n, self.stride, self.rng = key, n, stride, random.Random(seed)

    def __call__(self, s):
        x = s[self.key]
        span = (self.n - 1) * self.stride + 1
        if x.shape[1] < span:
            return None
        t0 = self.rng.randint(0, x.shape[1] - span)
        s[self.key] = x[:, t0:t0 + span:self.stride]
        return s


class CaptionDropout:
    """Replace the caption by the empty string with probability ``p`` (the unconditional branch of classifier-free
    guidance is trained on those samples)."""

    def __init__(self, key: str = "txt", p: float = 0.1, seed: int = 0):
        self.key, self.p, self.rng = key, p, random.Random(seed)

    def __call__(self, s):
        if self.key in s and self.rng.random() < self.p:
            s[self.key] = ""
        return s


# ---------------------------------------------------------------------------------------------------
# the data set
# ---------------------------------------------------------------------------------------------------
class TarShardDataset(torch.utils.data.IterableDataset):
    def __init__(self, shards, rank: int = 0, world: int = 1, shuffle_buffer: int = 0, seed: int = 0,
                 augmentors: Sequence[Callable] = (), decoders: Optional[Dict[str, Callable]] = None,
                 repeat: bool = False, required: Sequence[str] = ()):
        """``required``: member extensions a sample must have (others are skipped and counted in ``n_skipped``)."""
        self.shards = expand_shards(shards)
        if not self.shards:
            raise FileNotFoundError(f"no shard matches {shards!r}")
        self.rank, self.world, self.buffer, self.seed = rank, world, shuffle_buffer, seed
        self.augmentors, self.decoders, self.repeat, self.required = list(augmentors), decoders, repeat, list(required)
        self.epoch = 0
        self.n_skipped = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def my_shards(self, epoch: int) -> List[str]:
        """Shards of this rank (and of this data-loader worker) for ``epoch``: one shuffle shared by all ranks, dealt
        round-robin, so every shard is read exactly once per epoch across the job."""
        order = list(self.shards)
        random.Random(self.seed + epoch).shuffle(order)
        info = torch.utils.data.get_worker_info()
        nw, wid = (info.num_workers, info.id) if info is not None else (1, 0)
        return order[self.rank * nw + wid::self.world * nw]

    def _raw(self, epoch: int) -> Iterator[Dict[str, Any]]:
        for shard in self.my_shards(epoch):
            try:
                yield from iter_tar_samples(shard, self.decoders)
            except (tarfile.TarError, OSError) as e:
                logger.warning("[tar shards] %s cannot be read (%s): shard skipped", shard, e)

    def _shuffled(self, it: Iterable, rng: random.Random) -> Iterator:
        if self.buffer <= 1:
            yield from it
            return
        buf: List[Any] = []
        for x in it:
            if len(buf) < self.buffer:
                buf.append(x)
                continue
            i = rng.randrange(self.buffer)
            buf[i], x = x, buf[i]
            yield x
        rng.shuffle(buf)
        yield from buf

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        epoch = self.epoch
        while True:
            rng = random.Random((self.seed + epoch) * 1000003 + self.rank)
            for s in self._shuffled(self._raw(epoch), rng):
                if any(k not in s for k in self.required):
                    self.n_skipped += 1
                    continue
                for aug in self.augmentors:
                    s = aug(s)
                    if s is None:
                        break
                if s is None:
                    self.n_skipped += 1
                    continue
                yield s
            if not self.repeat:
                return
            epoch += 1


def write_shard(path: str, samples: Iterable[Dict[str, Any]]) -> int:
    """Write samples (``{"__key__": ..., ext: value}``; tensors as ``pt``, dicts / lists as ``json``, strings as
    ``txt``, bytes as they are) into one tar shard. Returns the number of samples."""
    n = 0
    with tarfile.open(path, "w") as tf:
        for i, s in enumerate(samples):
            key = s.get("__key__", f"{i:08d}")
            for ext, v in s.items():
                if ext.startswith("__"):
                    continue
                if isinstance(v, torch.Tensor):
                    buf = io.BytesIO()
                    torch.save(v, buf)
                    raw = buf.getvalue()
                elif isinstance(v, (dict, list)):
                    raw = json.dumps(v).encode()
                elif isinstance(v, str):
                    raw = v.encode()
                else:
                    raw = bytes(v)
                ti = tarfile.TarInfo(f"{key}.{ext}")
                ti.size = len(raw)
                tf.addfile(ti, io.BytesIO(raw))
            n += 1
    return n
