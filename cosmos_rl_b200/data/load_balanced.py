"""Token-balanced dynamic batching for SFT over data-parallel ranks.

Every data-parallel rank walks its own shard of the (shuffled) sample order, keeps a small pool of tokenised samples
and cuts batches that fill a token budget instead of a fixed sample count, so that ranks do comparable work per
optimizer step whatever the length distribution is. The behaviour follows the reference's pool batcher
(cosmos_rl/dispatcher/data/load_balanced_dataset.py:149-672, wired in cosmos_rl/policy/worker/sft_worker.py:455-497):

* the oldest sample of the pool seeds a batch; a sample at least as long as ``max_tokens_len`` or the budget goes
  out alone;
* padded cost model (``packed=False``): a batch of n samples costs ``n * longest``; ``prefer_first`` adds the
  candidate with the smallest new cost (first in pool order on ties), ``prefer_closest`` breaks ties by the length
  closest to the current longest;
* packed cost model (``packed=True``, what the trainers here use: sequences are concatenated, not padded): a batch
  costs the sum of its lengths and the first candidate in pool order that still fits is added;
* ``accumulate_steps`` batches form one optimizer step; the stream restarts with a new shuffle when the shard is
  exhausted, so every rank can serve any number of steps (ranks need the same step count, not the same samples).

The stream is a pure function of (seed, rank, world, step), which makes resume a replay: ``skip_steps(k)``.
"""
from __future__ import annotations

import random
from collections import deque
from typing import Any, Callable, Deque, Dict, Iterator, List, Optional, Sequence

STRATEGIES = ("prefer_first", "prefer_closest")


def sample_length(sample: Any, length_key: str = "input_ids") -> int:
    if isinstance(sample, dict):
        if length_key in sample:
            return len(sample[length_key])
        for v in sample.values():
            if hasattr(v, "__len__") and not isinstance(v, (str, bytes)):
                return len(v)
        raise ValueError(f"no sequence field in sample with keys {sorted(sample)}")
    return len(sample)


class LoadBalancedBatcher:
    def __init__(self, dataset: Sequence[Any], *, pool_size: int = 32, max_tokens_for_batch: int = 32768,
                 batching_strategy: str = "prefer_closest", max_tokens_len: Optional[int] = None, packed: bool = True,
                 seed: int = 0, shuffle: bool = True, dp_rank: int = 0, dp_world_size: int = 1,
                 accumulate_steps: int = 1, process_fn: Optional[Callable[[Any], Any]] = None,
                 length_key: str = "input_ids"):
        if batching_strategy not in STRATEGIES:
            raise ValueError(f"batching_strategy must be one of {STRATEGIES}, got {batching_strategy!r}")
        if accumulate_steps < 1 or pool_size < 1 or max_tokens_for_batch < 1:
            raise ValueError("accumulate_steps, pool_size and max_tokens_for_batch must be positive")
        if not 0 <= dp_rank < dp_world_size:
            raise ValueError(f"dp_rank {dp_rank} outside [0, {dp_world_size})")
        if len(dataset) < dp_world_size:
            raise ValueError(f"{len(dataset)} samples cannot be sharded over {dp_world_size} ranks")
        self.dataset, self.pool_size, self.budget = dataset, pool_size, max_tokens_for_batch
        self.strategy, self.packed = batching_strategy, packed
        self.max_len = max_tokens_len or max_tokens_for_batch
        self.seed, self.shuffle, self.rank, self.world = seed, shuffle, dp_rank, dp_world_size
        self.accumulate, self.process_fn, self.length_key = accumulate_steps, process_fn, length_key
        self.reset()

    # ------------------------------------------------------------------ the sample stream of this rank
    def reset(self) -> None:
        self.epoch = 0
        self._order: List[int] = self._shard(0)
        self._cursor = 0
        self._pool: Deque[Any] = deque()
        self.tokens_served = self.samples_served = self.batches_served = 0

    def _shard(self, epoch: int) -> List[int]:
        order = list(range(len(self.dataset)))
        if self.shuffle:
            random.Random(self.seed + epoch).shuffle(order)
        return order[self.rank::self.world]

    def _next_sample(self) -> Any:
        if self._cursor >= len(self._order):
            self.epoch += 1
            self._order, self._cursor = self._shard(self.epoch), 0
        s = self.dataset[self._order[self._cursor]]
        self._cursor += 1
        return self.process_fn(s) if self.process_fn is not None else s

    def _len(self, s: Any) -> int:
        return sample_length(s, self.length_key)

    # ------------------------------------------------------------------ batch building
    def _candidate(self, chosen: List[Any], cur_max: int, total: int) -> Optional[int]:
        if self.packed:
            for i, c in enumerate(self._pool):
                if total + self._len(c) <= self.budget:
                    return i
            return None
        best, best_cost, best_diff = None, None, None
        for i, c in enumerate(self._pool):
            n = self._len(c)
            cost = max(cur_max, n) * (len(chosen) + 1)
            if cost > self.budget:
                continue
            diff = abs(n - cur_max)
            better = best_cost is None or cost < best_cost or (
                self.strategy == "prefer_closest" and cost == best_cost and diff < best_diff)
            if better:
                best, best_cost, best_diff = i, cost, diff
        return best

    def _take(self, i: int) -> Any:
        self._pool.rotate(-i)
        s = self._pool.popleft()
        self._pool.rotate(i)
        return s

    def next_batch(self) -> List[Any]:
        while len(self._pool) < self.pool_size:
            self._pool.append(self._next_sample())
        first = self._pool.popleft()
        n = self._len(first)
        chosen, cur_max, total = [first], n, n
        if n < self.max_len and n < self.budget:
            while True:
                i = self._candidate(chosen, cur_max, total)
                if i is None:
                    break
                s = self._take(i)
                chosen.append(s)
                cur_max, total = max(cur_max, self._len(s)), total + self._len(s)
                while len(self._pool) < self.pool_size:      # keep the choice as wide as the pool allows
                    self._pool.append(self._next_sample())
        self.tokens_served += total
        self.samples_served += len(chosen)
        self.batches_served += 1
        return chosen

    def next_step(self) -> List[List[Any]]:
        """The ``accumulate_steps`` batches of one optimizer step."""
        return [self.next_batch() for _ in range(self.accumulate)]

    def skip_steps(self, n_steps: int) -> None:
        """Resume: replay the stream from the start up to optimizer step ``n_steps``."""
        self.reset()
        for _ in range(n_steps):
            self.next_step()

    def __iter__(self) -> Iterator[List[List[Any]]]:
        while True:
            yield self.next_step()

    def stats(self) -> Dict[str, float]:
        b = max(1, self.batches_served)
        return {"batches": self.batches_served, "samples": self.samples_served, "tokens": self.tokens_served,
                "tokens_per_batch": self.tokens_served / b, "budget_fill": self.tokens_served / (b * self.budget)}
