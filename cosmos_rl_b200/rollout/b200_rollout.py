"""The built-in rollout backend: this framework's own sm_100a generation engine behind the
``RolloutBase`` interface. The names ``vllm``, ``vllm_async`` and ``trtllm`` are accepted as aliases so job
files written for the reference run unchanged (cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:145-1128)."""
from __future__ import annotations

import copy
from typing import Any, List, Optional

import torch

from ..models import hf_io
from ..models.base import ModelRegistry
from ..parallel.flat import FlatParams
from .base import RolloutBase, RolloutRegistry, RolloutResult
from .engine import RolloutEngine, SamplingParams


@RolloutRegistry.register("b200")
class B200Rollout(RolloutBase):
    def __init__(self, config, parallel_dims, device, tokenizer=None, **kw):
        super().__init__(config, parallel_dims, device)
        self.tokenizer = tokenizer
        self.engine: Optional[RolloutEngine] = None
        self.model = None
        self.flat: Optional[FlatParams] = None

    def init_engine(self, load_format: str = "dummy", shared_model=None, seed: Optional[int] = None, **kw) -> None:
        cfg = self.config
        if shared_model is not None:
            self.model = shared_model          # colocated: generate on the policy's own tensors
        else:
            hf_config = hf_io.load_hf_config(cfg.policy.model_name_or_path, cfg.custom.get("model_config"))
            tp = self.parallel_dims.tp
            with torch.device("meta"):
                self.model = ModelRegistry.build_model(hf_config, tp_size=tp, tp_rank=self.parallel_dims.tp_coord)
            dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            self.flat = FlatParams(self.model, dtype, self.device, with_grad=False)
            if tp > 1:
                from ..parallel.tp import TensorParallel
                self.model.tp = TensorParallel(self.parallel_dims.group("tp"), tp, self.parallel_dims.tp_coord)
            path = cfg.policy.model_name_or_path
            import os
            if load_format != "dummy" and os.path.isdir(path) and hf_io.has_safetensors(path):
                hf_io.load_hf_weights(self.model, path, self.parallel_dims)
        self.fp8 = None
        if cfg.rollout.quantization == "fp8" and shared_model is None and self.device.type == "cuda":
            # linear weights are served from block-scaled fp8 copies; the weight sync writes them directly
            from .weight_sync import Fp8WeightStore
            self.fp8 = Fp8WeightStore(self.flat)
            self.fp8.attach(self.model)
            self.fp8.quantize_local()
        r = cfg.rollout
        self.engine = RolloutEngine(
            self.model, max_num_seqs=max(8, r.batch_size * r.n_generation),
            max_model_len=cfg.policy.model_max_length, page_size=cfg.b200.rollout_page_size,
            use_cuda_graph=cfg.b200.cuda_graph_decode and not r.enforce_eager or cfg.b200.cuda_graph_decode,
            seed=seed if seed is not None else (r.seed or 0),
            shared_prefix_decode=cfg.b200.shared_prefix_decode, gpu_memory_utilization=r.gpu_memory_utilization)

    def get_underlying_model(self):
        return self.model

    def rollout_generation_multi_turn(self, payloads, data_packer, sp: SamplingParams) -> List[RolloutResult]:
        """Every (prompt, sample) pair is its own conversation path; all live paths of a turn are generated in one
        engine call, then each response is appended and its tool calls are executed
        (cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:768-955 walks one conversation at a time)."""
        mt = self.config.rollout.multi_turn_config
        if self.tokenizer is None:
            raise RuntimeError("multi-turn rollouts need a tokenizer with a chat template")
        n = max(1, sp.n)
        one = copy.copy(sp)
        one.n = 1
        paths = []
        for pi, p in enumerate(payloads):
            conv = p.conversation if p.conversation is not None else p.prompt
            if isinstance(conv, str):
                conv = [{"role": "user", "content": conv}]
            for _ in range(n):
                paths.append({"payload": pi, "conv": list(conv), "done": False, "turns": 0, "last": ""})
        for _ in range(mt.max_assistant_turns):
            live = [q for q in paths if not q["done"]]
            if not live:
                break
            prompts = [data_packer.get_rollout_input(q["conv"]) for q in live]
            outs = self.engine.generate(prompts, one)
            for q, comps in zip(live, outs):
                text = self.tokenizer.decode(comps[0].token_ids, skip_special_tokens=True)
                q["conv"], q["done"] = data_packer.extend_conversation(q["conv"], text, payloads[q["payload"]].reference_answer)
                q["turns"] += 1
                q["last"] = text
        results = []
        for pi, p in enumerate(payloads):
            mine = [q for q in paths if q["payload"] == pi]
            results.append(RolloutResult(prompt=p.prompt, completions=[q["last"] for q in mine],
                                         completed_conversations=[q["conv"] for q in mine],
                                         extra_info={"assistant_turns": [q["turns"] for q in mine]}))
        return results

    def rollout_generation(self, payloads, data_packer, data_fetcher=None, is_validation: bool = False, **kw
                           ) -> List[RolloutResult]:
        sp = SamplingParams.from_config(self.config, validation=is_validation)
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if eos is not None:
            sp.stop_token_ids = (eos,)
        if self.config.rollout.multi_turn_config.enable:
            return self.rollout_generation_multi_turn(payloads, data_packer, sp)
        prompts = [data_packer.get_rollout_input(p.prompt) for p in payloads]
        outs = self.engine.generate(prompts, sp)
        results = []
        for p, comps in zip(payloads, outs):
            if self.tokenizer is not None and not self.config.train.train_policy.rollout_as_token_ids:
                texts = [self.tokenizer.decode(c.token_ids, skip_special_tokens=True) for c in comps]
            else:
                texts = [c.token_ids for c in comps]
            results.append(RolloutResult(
                prompt=p.prompt, completions=texts,
                completion_token_ids=[c.token_ids for c in comps],
                completion_logprobs=[c.logprobs for c in comps],
                cumulative_logprob=[c.cumulative_logprob for c in comps]))
        return results


for _alias in ("vllm", "vllm_async", "trtllm"):
    RolloutRegistry._backends[_alias] = B200Rollout
