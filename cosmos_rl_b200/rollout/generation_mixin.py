"""Four-hook skeleton for custom rollout backends: per-sample preparation (optionally overlapped with generation on a
background thread), batch collation, generation, post-processing into ``RolloutResult``s
(cosmos_rl/rollout/generation_mixin.py). Backends override the hooks instead of writing ``rollout_generation``."""
from __future__ import annotations

import concurrent.futures
from typing import Any, List

from .base import RolloutResult


class RolloutGenerationMixin:
    prefetch_workers: int = 2

    def rollout_generation(self, payloads, data_packer, data_fetcher=None, is_validation: bool = False, **kw
                           ) -> List[RolloutResult]:
        prefetch = bool(getattr(self.config.rollout, "prefetch_rollout", False))
        if prefetch and len(payloads) > 1:
            pool = self.__dict__.setdefault("_prep_pool", concurrent.futures.ThreadPoolExecutor(
                max_workers=max(1, int(getattr(self.config.rollout, "prefetch_queue_maxsize", self.prefetch_workers))),
                thread_name_prefix="rollout-prep"))
            samples = list(pool.map(lambda p: self._prepare_sample(p, data_packer, is_validation), payloads))
        else:
            samples = [self._prepare_sample(p, data_packer, is_validation) for p in payloads]
        batch = self._collate_batch(samples, is_validation)
        raw = self._generate(batch, is_validation)
        return self._postprocess(payloads, raw, is_validation)

    def _prepare_sample(self, payload, data_packer, is_validation: bool) -> Any:
        return data_packer.get_rollout_input(payload.prompt)

    def _collate_batch(self, samples: List[Any], is_validation: bool) -> Any:
        return samples

    def _generate(self, batch: Any, is_validation: bool) -> Any:
        raise NotImplementedError

    def _postprocess(self, payloads, raw: Any, is_validation: bool) -> List[RolloutResult]:
        raise NotImplementedError
