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
            item = data_packer.get_rollout_input(p.prompt)
            mm = {}
            if isinstance(item, dict):              # vision-language sample: ids + pixel inputs, repeated per sample
                mm = {k: torch.cat([torch.as_tensor(v)] * sp.n, dim=0).to(self.device) for k, v in item["mm"].items()}
                item = item["input_ids"]
            ids = torch.tensor([item], dtype=torch.long, device=self.device)
            out = inner.generate(ids.expand(sp.n, -1), attention_mask=torch.ones_like(ids).expand(sp.n, -1), **mm,
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


@RolloutRegistry.register("recompute")
class RecomputeRollout(HFRollout):
    """Generation for native families the paged engine has no path for (DeepSeek-V3's latent attention; the native
    vision-language models, whose prompts carry pixels and multimodal positions): every step re-runs the packed forward
    over all live sequences and samples with the engine's sampling kernel. No KV cache, so a step costs O(length); it
    keeps such families usable end to end (rollouts, weight sync, validation) at small scale. Pixel inputs of the live
    sequences are handed to the model before every step. The reference serves them through vLLM (cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:262-326)."""

    @torch.no_grad()
    def rollout_generation(self, payloads, data_packer, data_fetcher=None, is_validation: bool = False, **kw
                           ) -> List[RolloutResult]:
        from ..ops import functional as F
        sp = SamplingParams.from_config(self.config, validation=is_validation)
        model, dev = self.model, self.device
        items = [data_packer.get_rollout_input(p.prompt) for p in payloads]
        prompts = [list(it["input_ids"]) if isinstance(it, dict) else list(it) for it in items]
        mms = [it.get("mm") if isinstance(it, dict) else None for it in items for _ in range(sp.n)]
        seqs = [list(pr) for pr in prompts for _ in range(sp.n)]
        plen = [len(s) for s in seqs]
        logps: List[List[float]] = [[] for _ in seqs]
        live = list(range(len(seqs)))
        gen = torch.Generator(device="cpu").manual_seed(int(sp.seed or 0)) if dev.type != "cuda" else None
        w = model.lm_head_weight
        for step in range(sp.max_tokens):
            if not live:
                break
            lens = [len(seqs[i]) for i in live]
            ids = torch.tensor([t for i in live for t in seqs[i]], dtype=torch.long, device=dev)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32, device=dev)
            if getattr(model, "is_vlm", False):
                from ..data.packer import merge_mm
                model.mm_inputs = {k: v.to(dev) if k.startswith("pixel") else v
                                   for k, v in merge_mm([mms[i] for i in live]).items()}
            h = model(ids, model.get_position_ids(cu, int(ids.numel())), cu, max(lens))
            last = h[(cu[1:] - 1).long()]
            logits = torch.nn.functional.linear(last, w).float().contiguous()
            B = len(live)
            t = torch.full((B,), float(sp.temperature), dtype=torch.float32, device=dev)
            tp = torch.full((B,), float(sp.top_p), dtype=torch.float32, device=dev)
            tk = torch.full((B,), int(sp.top_k), dtype=torch.int32, device=dev)
            toks, lps = F.sample(logits, t, tp, tk, seed=int(sp.seed or 0), offset=step, generator=gen)
            nxt = []
            for j, i in enumerate(live):
                tok = int(toks[j])
                seqs[i].append(tok)
                logps[i].append(float(lps[j]))
                if tok not in sp.stop_token_ids and len(seqs[i]) < self.config.policy.model_max_length:
                    nxt.append(i)
            live = nxt
        results = []
        for pi, p in enumerate(payloads):
            rng = range(pi * sp.n, (pi + 1) * sp.n)
            toks = [seqs[i][plen[i]:] for i in rng]
            texts = toks if self.tokenizer is None or self.config.train.train_policy.rollout_as_token_ids else \
                [self.tokenizer.decode(t, skip_special_tokens=True) for t in toks]
            lp = [logps[i] for i in rng]
            results.append(RolloutResult(prompt=p.prompt, completions=texts, completion_token_ids=toks,
                                         completion_logprobs=lp, cumulative_logprob=[sum(l) for l in lp]))
        return results
