"""Dataset contract and controller/worker data fetchers.

User datasets implement ``setup(config, *a)``, ``__len__``, ``__getitem__(idx)`` (a prompt string or a
conversation list) and ``get_reference_answer(idx)`` (cosmos_rl/dispatcher/data/__init__.py:83-170,
docs/quickstart/customization.rst). The controller iterates over prompt *indices* only; workers resolve an
index to the sample locally when ``train.local_dataset`` is set.
"""
from __future__ import annotations

import random
from typing import Any, Callable, Dict, Iterator, List, Optional, Tuple

from .schema import RLPayload, Rollout  # noqa: F401


class CosmosDataset:
    """Wraps a user dataset (or a factory returning one) and applies the ``setup`` hook once."""

    def __init__(self, dataset_or_factory, config=None, tokenizer=None):
        ds = dataset_or_factory
        if callable(ds) and not hasattr(ds, "__getitem__"):
            ds = ds(config)
        if hasattr(ds, "setup"):
            try:
                ds.setup(config, tokenizer)
            except TypeError:
                ds.setup(config)
        self.dataset = ds

    @classmethod
    def wrap(cls, dataset_or_factory, config=None, tokenizer=None) -> Optional["CosmosDataset"]:
        """None stays None, and so does a factory that finds nothing to load (a config without ``dataset.name``)."""
        if dataset_or_factory is None:
            return None
        if isinstance(dataset_or_factory, cls):
            return dataset_or_factory
        if callable(dataset_or_factory) and not hasattr(dataset_or_factory, "__getitem__"):
            dataset_or_factory = dataset_or_factory(config)
            if dataset_or_factory is None:
                return None
        return cls(dataset_or_factory, config, tokenizer)

    def __len__(self):
        return len(self.dataset)

    def __getitem__(self, idx):
        return self.dataset[idx]

    def get_reference_answer(self, idx):
        if hasattr(self.dataset, "get_reference_answer"):
            return self.dataset.get_reference_answer(idx)
        return None


class SyntheticTokenDataset:
    """Prompts of ``prompt_len`` token ids drawn uniformly from a seeded RNG; used by the benchmark
    configurations (random-init weights, synthetic prompts, even-token reward)."""

    def __init__(self, n_prompts: int, prompt_len: int, vocab_size: int, seed: int = 0):
        self.n, self.prompt_len, self.vocab, self.seed = n_prompts, prompt_len, vocab_size, seed

    def setup(self, config=None, tokenizer=None):
        pass

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        rng = random.Random(self.seed * 1_000_003 + idx)
        return [rng.randrange(self.vocab) for _ in range(self.prompt_len)]

    def get_reference_answer(self, idx):
        return ""


class ControllerDataFetcher:
    """Hands out prompt indices epoch by epoch (cosmos_rl/dispatcher/data/data_fetcher.py:93-665).

    ``remain_samples_num`` (prompts not yet handed out, over all remaining epochs) is stored in checkpoints
    and restores the position on resume.
    """

    def __init__(self, config, dataset: Optional[CosmosDataset], val_dataset: Optional[CosmosDataset] = None,
                 sampler: Optional[Callable] = None, is_rl: bool = True):
        self.config = config
        self.dataset = dataset
        self.val_dataset = val_dataset
        tp = config.train.train_policy
        self.shuffle = bool(getattr(tp, "dataloader_shuffle", True))
        self.seed = int(getattr(tp, "dataloader_seed", 0))
        self.epochs = max(1, int(config.train.epoch))
        self.sampler = sampler
        self.local_dataset = bool(config.train.local_dataset)
        self.n = len(dataset) if dataset is not None else 0
        self.epoch = 0
        self.pos = 0
        self._order = self._make_order(0)
        self.ckpt_extra_info: Dict[str, Any] = {}
        self._val_iters: Dict[int, int] = {}

    # ------------------------------------------------------------------
    def _make_order(self, epoch: int) -> List[int]:
        if self.sampler is not None:
            return list(self.sampler(self.n, epoch))
        order = list(range(self.n))
        if self.shuffle:
            random.Random(self.seed + epoch).shuffle(order)
        return order

    @property
    def total_samples(self) -> int:
        return self.n * self.epochs

    @property
    def remain_samples_num(self) -> int:
        return (self.epochs - self.epoch) * self.n - self.pos if self.epoch < self.epochs else 0

    def restore(self, remain_samples_num: int) -> None:
        consumed = self.total_samples - remain_samples_num
        self.epoch, self.pos = divmod(consumed, max(self.n, 1))
        self._order = self._make_order(self.epoch)

    def _payload(self, ds: CosmosDataset, idx: int) -> RLPayload:
        if self.local_dataset:
            return RLPayload(prompt_idx=idx)
        return RLPayload(prompt=ds[idx], prompt_idx=idx, reference_answer=ds.get_reference_answer(idx))

    def get_batched_prompt(self, n: int) -> Tuple[List[Tuple[int, RLPayload]], bool]:
        out: List[Tuple[int, RLPayload]] = []
        while len(out) < n and self.epoch < self.epochs:
            if self.pos >= self.n:
                self.epoch += 1
                self.pos = 0
                if self.epoch < self.epochs:
                    self._order = self._make_order(self.epoch)
                continue
            idx = self._order[self.pos]
            self.pos += 1
            out.append((idx, self._payload(self.dataset, idx)))
        is_end = self.epoch >= self.epochs or (self.epoch == self.epochs - 1 and self.pos >= self.n)
        return out, is_end

    def get_validation_prompts(self, n: int, validation_step: int) -> Tuple[List[Tuple[int, RLPayload]], bool]:
        if self.val_dataset is None:
            return [], True
        pos = self._val_iters.get(validation_step, 0)
        total = len(self.val_dataset)
        idxs = list(range(pos, min(pos + n, total)))
        self._val_iters[validation_step] = pos + len(idxs)
        return [(i, self._payload(self.val_dataset, i)) for i in idxs], pos + len(idxs) >= total


class WorkerDataFetcher:
    """Worker-side index -> sample lookup (cosmos_rl/dispatcher/data/data_fetcher.py:667-744)."""

    def __init__(self, config, dataset: Optional[CosmosDataset], val_dataset: Optional[CosmosDataset] = None):
        self.config = config
        self.dataset = dataset
        self.val_dataset = val_dataset

    def fill(self, payload, validation: bool = False):
        ds = self.val_dataset if validation else self.dataset
        if ds is not None and payload.prompt is None and payload.prompt_idx >= 0:
            payload.prompt = ds[payload.prompt_idx]
            if hasattr(payload, "reference_answer") and payload.reference_answer is None:
                payload.reference_answer = ds.get_reference_answer(payload.prompt_idx)
        return payload

    def get_reference_answer(self, idx: int, validation: bool = False):
        ds = self.val_dataset if validation else self.dataset
        return ds.get_reference_answer(idx) if ds is not None else None
