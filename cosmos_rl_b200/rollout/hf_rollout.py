"""Rollout backend for models served by the generic transformers wrapper (``models/hf_model.py``): plain
``generate`` with sampling, one prompt group at a time. Native models use the paged engine (``b200_rollout.py``);
this backend exists so that every family the trainer accepts can also produce rollouts
(cosmos_rl/rollout/rollout_base.py:29-274 registry; the reference serves such models through vLLM)."""
from __future__ import annotations

from typing import List

import torch

from ..models import hf_io
from ..models.base import ModelRegistry
from ..parallel.flat import FlatParams
from .base import RolloutBase, RolloutRegistry, RolloutResult
from .engine import SamplingParams


@RolloutRegistry.register("hf")
class HFRollout(RolloutBase):
    def __init__(self, config, parallel_dims, device, tokenizer=None, **kw):
        super().__init__(config, parallel_dims, device)
        self.tokenizer = tokenizer

    def init_engine(self, load_format: str = "dummy", shared_model=None, **kw) -> None:
        if shared_model is not None:
            self.model = shared_model
            return
        cfg = self.config
        hf_config = hf_io.load_hf_config(cfg.policy.model_name_or_path, cfg.custom.get("model_config"))
        with torch.device("meta"):
            self.model = ModelRegistry.build_model(hf_config)
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.flat = FlatParams(self.model, dtype, self.device, with_grad=False)
        self.model.init_weights(cfg.rollout.seed or 0)

    def get_underlying_model(self):
        return self.model

    @torch.no_grad()
    def rollout_generation(self, payloads, data_packer, data_fetcher=None, is_validation: bool = False, **kw
                           ) -> List[RolloutResult]:
        sp = SamplingParams.from_config(self.config, validation=is_validation)
        inner = self.model.inner
        results = []
        for p in payloads:
            ids = torch.tensor([data_packer.get_rollout_input(p.prompt)], dtype=torch.long, device=self.device)
            out = inner.generate(ids.expand(sp.n, -1), attention_mask=torch.ones_like(ids).expand(sp.n, -1),
                                 do_sample=sp.temperature > 0, temperature=max(sp.temperature, 1e-5),
                                 top_p=sp.top_p, top_k=sp.top_k if sp.top_k > 0 else None,
                                 max_new_tokens=sp.max_tokens, output_scores=True, return_dict_in_generate=True,
                                 pad_token_id=0, eos_token_id=list(sp.stop_token_ids) or None)
            gen = out.sequences[:, ids.shape[1]:]
            lps = torch.stack([torch.log_softmax(s.float(), -1) for s in out.scores], 1)      # [n, steps, V]
            tok_lp = lps.gather(-1, gen.unsqueeze(-1)).squeeze(-1)
            toks, logps = [], []
            for i in range(sp.n):
                t = gen[i].tolist()
                stop = next((j + 1 for j, x in enumerate(t) if x in sp.stop_token_ids), len(t))
                toks.append(t[:stop])
                logps.append(tok_lp[i, :stop].tolist())
            texts = toks if self.tokenizer is None or self.config.train.train_policy.rollout_as_token_ids else \
                [self.tokenizer.decode(t, skip_special_tokens=True) for t in toks]
            results.append(RolloutResult(prompt=p.prompt, completions=texts, completion_token_ids=toks,
                                         completion_logprobs=logps, cumulative_logprob=[sum(l) for l in logps]))
        return results
