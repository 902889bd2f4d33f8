"""Shared machinery of the LLM trainers: model construction, flat parameter storage, optimizer, LR schedule,
checkpointing and HF export (cosmos_rl/policy/trainer/llm_trainer/llm_trainer.py:51-790)."""
from __future__ import annotations

import json
import os
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ...config import Config
from ...data.packer import BaseDataPacker
from ...models.base import ModelRegistry
from ...parallel.dims import ParallelDims
from ...parallel.flat import FlatParams
from ...utils import checkpoint as ckpt_util
from ...utils.logging import logger
from ...utils.misc import seed_everything, str2dtype
from ..optim import FlatAdamW, lr_factor
from .base import Trainer


def resolve_hf_config(config: Config):
    """Model architecture: a named built-in architecture, a local HF folder, or a dict under [custom]."""
    from ...models import hf_io
    return hf_io.load_hf_config(config.policy.model_name_or_path, config.custom.get("model_config"))


class LLMTrainer(Trainer):
    def __init__(self, config: Config, parallel_dims: ParallelDims, device: Optional[torch.device] = None,
                 data_packer: Optional[BaseDataPacker] = None, val_data_packer=None, hook_fns=None, **kw):
        self.config = config
        self.parallel_dims = parallel_dims
        self.device = device or parallel_dims.device
        self.hook_fns = hook_fns or {}
        seed_everything(config.train.seed)
        if config.train.deterministic and self.device.type == "cuda":
            torch.use_deterministic_algorithms(True, warn_only=True)
        self.param_dtype = str2dtype(config.train.param_dtype) if self.device.type == "cuda" else torch.float32
        self.hf_config = resolve_hf_config(config)
        mt = self.hf_config.get("model_type") if isinstance(self.hf_config, dict) else self.hf_config.model_type
        self.model_type = mt
        tp = parallel_dims.tp
        ep = getattr(parallel_dims, "ep", 1)
        build_kw = {}
        if ep > 1:
            # experts are spread over the dp_shard ranks (the layout of the reference's Qwen3-MoE plan,
            # cosmos_rl/policy/model/qwen3_moe/parallelize.py:120-190, with ep == dp_shard)
            # with ep < dp_shard the dp_shard axis splits into blocks of ep ranks that exchange tokens; ranks at the
            # same position of different blocks replicate the experts and sum their gradients
            if parallel_dims.dp_shard % ep or parallel_dims.cp > 1:
                raise NotImplementedError("expert parallelism needs ep_size to divide dp_shard_size, and cp_size == 1")
            if parallel_dims.group("ep") is None and parallel_dims.dp_shard > 1:
                parallel_dims.build_ep_groups()
            build_kw = dict(ep_size=ep, ep_rank=parallel_dims.ep_coord)
        self.pp_chunks = 1
        if parallel_dims.pp > 1:
            build_kw.update(pp_size=parallel_dims.pp, pp_rank=parallel_dims.pp_coord)
            par = config.policy.parallelism
            if par.pp_schedule == "Interleaved1F1B":
                # several model chunks per rank: asked for directly, or through the reference's layers-per-stage key
                chunks = config.b200.pp_chunks
                n_layers = (self.hf_config.get("num_hidden_layers") if isinstance(self.hf_config, dict)
                            else getattr(self.hf_config, "num_hidden_layers", 0)) or 0
                if chunks <= 0 or (chunks == 1 and par.pp_layers_per_stage > 0):
                    chunks = max(1, -(-n_layers // max(1, par.pp_layers_per_stage)) // parallel_dims.pp) \
                        if par.pp_layers_per_stage > 0 else 1
                if chunks > 1:
                    if n_layers < chunks * parallel_dims.pp:
                        raise ValueError(f"{n_layers} blocks cannot fill {chunks} chunks on each of "
                                         f"{parallel_dims.pp} pipeline ranks")
                    self.pp_chunks = chunks
                    build_kw.update(pp_chunks=chunks)
            if config.b200.pp_head_weight or config.b200.pp_embed_weight:
                build_kw.update(pp_head_weight=config.b200.pp_head_weight, pp_embed_weight=config.b200.pp_embed_weight)
        with torch.device("meta"):
            if config.train.force_use_hf:
                if tp > 1 or build_kw:
                    raise NotImplementedError("train.force_use_hf: the generic wrapper trains with data parallelism only")
                model = ModelRegistry.build_model(self.hf_config, force_hf=True)
            else:
                model = ModelRegistry.build_model(self.hf_config, tp_size=tp, tp_rank=parallel_dims.tp_coord, **build_kw)
        if ep > 1 and not hasattr(model, "set_ep_group"):
            raise NotImplementedError(f"model type {mt} has no expert-parallel plan")
        # the model stays on the meta device here: FlatParams materialises every parameter as a view of
        # one flat buffer, so no second copy of the weights is ever allocated
        self.model = model
        self.lora_targets: List[str] = []
        if config.policy.lora is not None:
            # adapters become parameters of the projections before the flat buffer is laid out; the base is frozen
            from .. import lora
            if tp > 1 or not hasattr(model, "layers"):
                raise NotImplementedError("policy.lora needs a native model and tp_size == 1")
            self.lora_targets = lora.attach_lora(model, config.policy.lora)
        else:
            self._apply_trainable_patterns()
        dp = parallel_dims.dp_shard
        is_expert = (lambda n: n.endswith("w_gate_up") or n.endswith("w_down")) if ep > 1 else None
        # parameter-sharded data parallelism (``fsdp_reshard_after_forward = "always"`` or ``b200.shard_params``):
        # weights, gradients and optimizer state are all 1/dp_shard per rank, gathered unit by unit around their use
        self._allocator = kw.get("allocator")
        self._sync_full = None
        self.shard_params = bool(config.b200.shard_params or config.train.fsdp_reshard_after_forward == "always")
        if self.shard_params:
            if (tp > 1 or ep > 1 or parallel_dims.pp > 1 or parallel_dims.cp > 1 or self.lora_targets
                    or config.train.fp8.enable_fp8 or not hasattr(model, "param_sharder")):
                raise NotImplementedError("parameter sharding runs native dense models under dp_shard x dp_replicate "
                                          "only (no tp / cp / pp / ep, no adapters, no fp8 weights)")
            from ...parallel.sharded_params import ShardedFlatParams
            rd = str2dtype(config.train.fsdp_reduce_dtype) if self.device.type == "cuda" else None
            self.flat = ShardedFlatParams(model, self.param_dtype, self.device,
                                          parallel_dims.group("dp_shard") if dp > 1 else None, reduce_dtype=rd)
            model.param_sharder = self.flat
            logger.info("[Policy] parameter sharding over %d ranks: %s", dp,
                        {k: round(v, 2) for k, v in self.flat.memory_report().items()})
        else:
            self.flat = FlatParams(model, self.param_dtype, self.device, shard_multiple=dp,
                                   allocator=kw.get("allocator"), local_filter=is_expert)
        if ep > 1:
            model.set_ep_group(parallel_dims.group("ep") or parallel_dims.group("dp_shard"))
        if self.lora_targets:
            from .. import lora
            lora.bind_lora(model)
        self.n_fp8_weights = 0
        if config.train.fp8.enable_fp8:
            # every projection of the blocks runs its three GEMMs on the block-scaled fp8 kernel; embeddings, norms and
            # lm_head stay in bf16 (cosmos_rl/policy/model/gpt/__init__.py:795-797 excludes lm_head too). All recipes
            # of the reference map to block scaling here: 1 x 128 activations, 128 x 128 weights.
            from ...ops.functional import fp8_train_supported
            for name, p in model.named_parameters():
                if name.startswith("layers.") and name.endswith("_proj.weight") and fp8_train_supported(p):
                    p._fp8_train = True
                    self.n_fp8_weights += 1
        rc = config.b200.recompute if config.policy.model_gradient_checkpointing else "none"
        self._recompute_auto = rc == "auto"
        model.gradient_checkpointing = {"none": False, "auto": "selective"}.get(rc, rc)
        if tp > 1:
            from ...parallel.tp import TensorParallel
            model.tp = TensorParallel(parallel_dims.group("tp"), tp, parallel_dims.tp_coord)
            from ...models.gpt import GPT
            model.tp.sequence_parallel = bool(config.b200.sequence_parallel and type(model) is GPT
                                              and parallel_dims.pp == 1 and parallel_dims.cp == 1)
            model.tp.keep_gathered = bool(config.b200.sp_keep_gathered)
        if parallel_dims.cp > 1:
            # context parallelism composes with tp (the exchange moves this rank's heads between the cp ranks that
            # share its tp coordinate) and with pp (every stage's attention layers exchange inside the stage)
            if not hasattr(model, "attach_context_parallel"):
                raise NotImplementedError("cp_size > 1 needs a native model")
            from ...parallel.context_parallel import ContextParallel
            model.attach_context_parallel(ContextParallel(parallel_dims.group("cp"), parallel_dims.cp,
                                                          parallel_dims.cp_coord, config.b200.cp_mode))
        self.pipeline = None
        if parallel_dims.pp > 1:
            # stages exchange the full [T, H] hidden states between ranks of equal tp / cp coordinates (tensor
            # parallelism without sequence sharding keeps them replicated inside a stage)
            if not hasattr(getattr(model, "args", None), "pp_size"):
                raise NotImplementedError("pp_size > 1 needs a native model")
            from ...parallel.pipeline import PipelineStage
            stage = model
            if self.pp_chunks > 1:
                if not hasattr(model, "forward_chunk"):
                    raise NotImplementedError("several model chunks per pipeline rank need a model of the GPT family")
                stage = [(lambda *a, c=c: model.forward_chunk(c, *a)) for c in range(self.pp_chunks)]
            self.pipeline = PipelineStage(stage, parallel_dims.group("pp"), parallel_dims.pp_coord, parallel_dims.pp,
                                          model.args.dim, self.param_dtype, self.device,
                                          schedule=config.policy.parallelism.pp_schedule,
                                          back_group=parallel_dims.group("pp_back"))
        from ...utils.extension import parallelism_strategy
        custom_plan = parallelism_strategy(mt)
        if custom_plan is not None:
            custom_plan(model, parallel_dims, config)
        lr = config.train.optm_lr if isinstance(config.train.optm_lr, float) else float(
            list(config.train.optm_lr.values())[0] if isinstance(config.train.optm_lr, dict) else config.train.optm_lr[0])
        if config.train.optm_name not in ("AdamW", "Adam", "AdamW8bit", "Adam8bit"):
            raise NotImplementedError(f"optimizer {config.train.optm_name!r}: the flat sharded optimizer implements AdamW "
                                      f"(Adam = AdamW without decoupled weight decay; the 8bit names keep block-quantised moments)")
        tp_mask = None
        if tp > 1:
            # parameters every tensor-parallel rank holds in full (norm weights): counted once in the gradient norm
            tp_mask = torch.zeros(self.flat.total, dtype=torch.bool, device=self.device)
            for slot in self.flat.slots:
                if "norm" in slot.name or slot.name.startswith(("visual.", "projector.", "proprio_projector.", "action_head.")):   # towers and heads beside the decoder are replicated too
                    tp_mask[slot.offset:slot.offset + slot.numel] = True
        sharded_norm = [parallel_dims.group("dp_shard")] if (self.shard_params and dp > 1) else []
        self.optimizer = FlatAdamW(
            self.flat.optimizer_view() if self.shard_params else self.flat, lr=lr, betas=tuple(config.train.optm_betas), eps=config.train.epsilon,
            weight_decay=config.train.optm_weight_decay if config.train.optm_name.startswith("AdamW") else 0.0,
            state_bits=8 if config.train.optm_name.endswith("8bit") else 32,
            max_grad_norm=config.train.optm_grad_norm_clip,
            tp_group=parallel_dims.group("tp") if tp > 1 else None, tp_replicated=tp_mask,
            norm_groups=([parallel_dims.group("pp")] if parallel_dims.pp > 1 else []) + sharded_norm,
            sum_groups=[parallel_dims.group("cp")] if parallel_dims.cp > 1 else [],
            dp_group=parallel_dims.group("dp_shard") if (dp > 1 and not self.shard_params) else None,
            collective=kw.get("collective"),
            tail_replica_group=parallel_dims.group("ep_replica") if ep > 1 else None,
            replicate_group=parallel_dims.group("dp_replicate") if parallel_dims.dp_replicate > 1 else None)
        self.data_packer = data_packer or BaseDataPacker.get_default(mt)()
        self.tokenizer = kw.get("tokenizer")
        self.data_packer.setup(config, self.tokenizer)
        self.ckpt_manager = ckpt_util.CheckpointManager(config, parallel_dims.global_rank)
        self.train_step = 0
        self.total_steps = 0
        self.weights_ready = False
        self.reference_state: Optional[torch.Tensor] = None   # host copy of the frozen anchor policy (KL term, DPO)
        self.reference_step = 0                               # step at which the anchor was last (re)set
        self._ref_ship = None
        self.ema = None          # ShardEMA when train.ema_enable (created once the weights are in place)

    # ------------------------------------------------------------------
    def resolve_recompute(self, max_tokens: int) -> None:
        """``recompute = "auto"``: decide once, before the first backward pass, from the memory that is actually
        free. Activations kept per token and block without recomputation: the two norm inputs and residuals (4 H),
        q/k/v and the attention output, the gate/up product (2 I) and the SwiGLU output (I), all bf16."""
        tpo = getattr(self.model, "tp", None)
        if (tpo is not None and tpo.sequence_parallel and self.config.b200.sp_fused_kernels
                and self.device.type == "cuda" and tpo.fused_ag is None and hasattr(self.model, "args")):
            # peer-memory workspaces of the fused all-gather -> GEMM and GEMM -> reduce-scatter kernels, sized for the
            # largest packed micro-batch (padded to whole 128-row blocks per rank)
            rows = (max_tokens + 128 * tpo.size - 1) // (128 * tpo.size) * (128 * tpo.size)
            tpo.attach_fused(self.device, rows, self.model.args.dim, all_gather_k=self.model.args.dim)
        if not self._recompute_auto:
            return
        self._recompute_auto = False
        a = getattr(self.model, "args", None)
        if self.device.type != "cuda" or a is None or not hasattr(a, "ffn_dim"):
            return
        tp = max(1, getattr(a, "tp_size", 1))
        attn = 4 * a.dim + ((2 * a.n_heads + 2 * a.n_kv_heads) * a.head_dim) // tp     # elements per token and block
        fixed = self.config.b200.dlogits_chunk * (a.vocab_size // tp) * 6 + (6 << 30)     # lm_head backward, slack
        n = max_tokens * len(self.model.layers) * 2 * 1.15
        need_none = int(n * (attn + 3 * a.ffn_dim // tp)) + fixed
        need_swiglu = int(n * (attn + 2 * a.ffn_dim // tp)) + fixed                    # SwiGLU output recomputed
        free, _ = torch.cuda.mem_get_info(self.device)
        free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        choice = False if need_none < free else ("swiglu" if need_swiglu < free else "selective")
        self.model.gradient_checkpointing = choice
        logger.info("[Policy] recompute=auto -> %s (no recomputation needs %.1f GB, SwiGLU-only %.1f GB, %.1f GB free)",
                    choice or "none", need_none / 2**30, need_swiglu / 2**30, free / 2**30)

    def _apply_trainable_patterns(self) -> None:
        import re
        pc = self.config.policy
        for name, p in self.model.named_parameters():
            if pc.freeze_pattern and any(re.search(pat, name) for pat in pc.freeze_pattern):
                p.requires_grad_(False)
            if pc.trainable_pattern:
                p.requires_grad_(any(re.search(pat, name) for pat in pc.trainable_pattern))
            if pc.trainable_map and name in pc.trainable_map:
                p.requires_grad_(bool(pc.trainable_map[name]))

    def _weights_changed(self) -> None:
        """Call after writing ``flat.data`` directly (weights swapped in or out): under parameter sharding the
        gathered copies of the units have to be fetched again."""
        if self.shard_params:
            self.flat.invalidate()

    def optimizer_step(self) -> torch.Tensor:
        """One optimizer step plus what rides on it (the router bias of DeepSeek-style MoE blocks, moved from the
        expert load of the batch summed over the data-parallel ranks). Returns the gradient norm."""
        norm = self.optimizer.step(self.lr_scale(self.train_step))
        if self.shard_params:
            self.flat.invalidate()               # the gathered copies of the units are stale now
        if self.ema is not None:
            self.ema.step(self.optimizer.step_count - 1)
        rate = self.config.b200.router_bias_update_rate
        if rate > 0 and hasattr(self.model, "update_router_bias"):
            dims = self.parallel_dims
            self.model.update_router_bias(rate, dims.group("dp_shard") if dims.dp_shard > 1 else None)
        return norm

    # ------------------------------------------------------------------ running packed batches (with or without pp)
    def _micro(self, batches):
        from ...parallel.pipeline import MicroBatch
        return [MicroBatch(b["input_ids"], b["position_ids"], b["cu_seqlens"], b["max_seqlen"], extra=(i, b))
                for i, b in enumerate(batches)]

    def run_batches_train(self, batches, loss_of) -> List[torch.Tensor]:
        """Forward + backward over packed batches; ``loss_of(hidden, index, batch) -> scalar`` (already scaled for
        accumulation). With pipeline stages the batches are the micro-batches of a 1F1B schedule and the loss is
        evaluated on the last stage only; the returned (detached) losses are empty on the other stages."""
        if self.pipeline is not None:
            return self.pipeline.run(self._micro(batches), lambda h, mb: loss_of(h, mb.extra[0], mb.extra[1]))
        from ...utils.activation_offloading import maybe_offload
        losses = []
        for i, b in enumerate(batches):
            self._set_mm(b)
            # train.activation_offload: saved activations of at least 1 MiB wait in pinned host memory for backward
            with maybe_offload(self.config.train.activation_offload, self.model):
                loss = loss_of(self.model(b["input_ids"], b["position_ids"], b["cu_seqlens"], b["max_seqlen"]), i, b)
            loss.backward()
            if self.shard_params:
                self.flat.finish_backward()
            losses.append(loss.detach())
        return losses

    @torch.no_grad()
    def run_batches_nograd(self, batches, fn) -> List[Any]:
        """``fn(hidden, index, batch)`` per packed batch without gradients (last stage only under pp)."""
        if self.pipeline is not None:
            return self.pipeline.forward_only(self._micro(batches), lambda h, mb: fn(h, mb.extra[0], mb.extra[1]))
        out = []
        for i, b in enumerate(batches):
            self._set_mm(b)
            out.append(fn(self.model(b["input_ids"], b["position_ids"], b["cu_seqlens"], b["max_seqlen"]), i, b))
        return out

    def _set_mm(self, b) -> None:
        """Vision-language wrapper models read the pixel inputs of the batch they are about to run from here."""
        if getattr(self.model, "is_vlm", False):
            self.model.mm_inputs = b.get("mm") or {}

    def pp_sum(self, value: torch.Tensor) -> torch.Tensor:
        """A value only the last stage has (losses, metrics): summed over the stages so every rank reports it."""
        if self.pipeline is not None:
            dist.all_reduce(value, group=self.parallel_dims.group("pp"))
        return value

    def cp_shard(self, b: Dict[str, Any]) -> Dict[str, Any]:
        """Under context parallelism: keep this rank's chunk of every sequence of a packed batch; the number of scored
        tokens of the whole batch is kept for the loss normalisation (gradients are summed over the cp ranks)."""
        b["n_scored"] = int((b["label_ids"] >= 0).sum())
        dims = self.parallel_dims
        if dims.cp == 1:
            return b
        from ...utils.sequence_packing import shard_packed
        return shard_packed(b, dims.cp, dims.cp_coord, zigzag=self.config.b200.cp_mode == "ring-zigzag")

    def pack_multiple(self) -> int:
        """Sequences of a packed batch are padded to multiples of this (context-parallel chunks, twice as many for the
        zig-zag layout, times the tensor-parallel row split)."""
        dims = self.parallel_dims
        cp = dims.cp * (2 if (dims.cp > 1 and self.config.b200.cp_mode == "ring-zigzag") else 1)
        return max(1, cp * dims.tp)

    def lr_scale(self, step: int) -> float:
        t = self.config.train
        return lr_factor(step, self.total_steps, t.optm_warmup_steps, t.optm_warmup_start_factor, t.optm_decay_ratio,
                         t.optm_decay_type, t.optm_min_lr_factor)

    # ------------------------------------------------------------------ weights in
    def model_load_from_hf(self) -> None:
        from ...models import hf_io
        path = self.config.policy.model_safetensor_path or self.config.policy.model_name_or_path
        import contextlib
        # sharded parameters: load into a transient full copy (device memory if it fits, else host) and keep the shard
        whole = self.flat.materialized(fill=False, writeback=True) if self.shard_params else contextlib.nullcontext()
        with whole as full:
            if path and os.path.isdir(path) and hf_io.has_safetensors(path):
                hf_io.load_hf_weights(self.model, path, self.parallel_dims)
            else:
                seed = self.config.train.seed if self.config.train.seed is not None else 0
                if self.device.type == "cuda" and (full is None or full.is_cuda):
                    self.model.init_weights_on_device(seed)
                else:
                    self.model.init_weights(seed)
                logger.info("[Policy] no checkpoint at %r: random-init weights from seed %d", path, seed)
        if self.lora_targets:
            from .. import lora
            lora.reset_lora_parameters(self.model, self.config.train.seed or 0,
                                       init=self.config.policy.lora.init_lora_weights)
        self.optimizer.refresh_master_from_params()
        self._init_ema()
        self.weights_ready = True

    def _init_ema(self) -> None:
        """``train.ema_enable``: a moving average of the trained weights on the optimizer shard; exports and
        validation read it (cosmos_rl/policy/trainer/diffusers_trainer/diffusers_trainer.py:130-146)."""
        t = self.config.train
        if t.ema_enable:
            from ...utils.ema import ShardEMA
            self.ema = ShardEMA(self.optimizer, t.ema_decay, t.ema_update_step_interval)

    # ------------------------------------------------------------------ adapters around weight hand-over
    def before_weight_sync(self) -> None:
        """Rollout replicas receive plain dense weights: adapters are folded into the base weights for the duration of
        a policy-to-rollout transfer (cosmos_rl/policy/worker/rl_worker.py:455-466, 548-551)."""
        if self.lora_targets:
            from .. import lora
            lora.merge_native(self.model)
        if self.shard_params:
            self.flat.gather_full(out=self.sync_buffer())

    def sync_buffer(self) -> torch.Tensor:
        """The buffer rollout replicas read the weights from (its layout is what ``flat.slots`` index). With resident
        weights that is the flat buffer itself. Under parameter sharding it is a full copy that exists for weight
        synchronisation only; it is allocated once (peer-visible where the flat buffer would be) so that its exported
        handle stays valid, and refilled by ``before_weight_sync``."""
        if not self.shard_params:
            return self.flat.data
        if self._sync_full is None:
            alloc = self._allocator or (lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev))
            self._sync_full = alloc(self.flat.total, self.flat.dtype, self.device)
        return self._sync_full

    def after_weight_sync(self) -> None:
        if self.lora_targets:
            from .. import lora
            lora.unmerge_native(self.model)

    def model_resume_from_checkpoint(self) -> bool:
        state = self.ckpt_manager.load_latest(self.device)
        if state is None:
            return False
        ref = state["model"].get("reference")
        if ref is not None:
            self.reference_state = ref.to("cpu", self.flat.dtype, copy=True)
            self.reference_step = int(state["model"].get("reference_step", 0))
        elif self.needs_reference():
            # a checkpoint written without the reference weights: the anchor is the model the run started from
            # (cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:2041-2051 reloads the HF weights the same way)
            self.model_load_from_hf()
            self.reference_state = self.flat.data.to("cpu", copy=True)
            self.reference_step = 0
        self.flat.data.copy_(state["model"]["flat"].to(self.flat.dtype))
        if self.shard_params:
            self.flat.invalidate()
        self.optimizer.load_state_dict(state["optimizer"])
        self._init_ema()
        if self.ema is not None and state["model"].get("ema") is not None:
            self.ema.load_state_dict(state["model"]["ema"])
        extra = state["extra_info"]
        self.train_step = int(extra.get("step", 0))
        self.total_steps = int(extra.get("total_steps", 0))
        ckpt_util.restore_rng(extra)
        self.resume_extra_info = extra
        self.weights_ready = True
        logger.info("[Policy] resumed from checkpoint at step %d", self.train_step)
        return True

    def weight_resume(self) -> bool:
        """Load the latest valid checkpoint when resuming, else the HF weights. Returns True if resumed."""
        if self.config.train.resume and self.model_resume_from_checkpoint():
            return True
        self.model_load_from_hf()
        return False

    # ------------------------------------------------------------------ weights out
    def save_checkpoint(self, step: int, total_steps: int, remain_samples_num: int = 0, is_final: bool = False,
                        **kw) -> None:
        extra = {"step": step, "total_steps": total_steps, "remain_samples_num": remain_samples_num,
                 "is_final": is_final}
        model_state = {"flat": self.flat.data, "slots": [s.__dict__ for s in self.flat.slots]}
        if self.ema is not None:
            model_state["ema"] = self.ema.state_dict()
        if self.reference_state is not None:
            # the KL / DPO anchor is part of the run's state: a resume must not re-anchor to the resumed policy
            model_state["reference"] = self.reference_state
            model_state["reference_step"] = self.reference_step
        self.ckpt_manager.save(step, model_state=model_state,
                               optimizer_state=self.optimizer.state_dict(), scheduler_state={"step": step},
                               extra_info=extra, is_final=is_final)
        if self.config.train.ckpt.export_safetensors:
            out = os.path.join(self.config.train.output_dir, "safetensors", f"step_{step}")
            if self.ema is not None:            # the exported model is the averaged one; training resumes from the raw one
                with self.ema.swapped_in():
                    self.export_safetensors(out)
            else:
                self.export_safetensors(out)
        hook = self.hook_fns.get("save_checkpoint_hook")
        if hook:
            hook(step=step, trainer=self)

    def export_safetensors(self, output_dir: str, **kw) -> None:
        from ...models import hf_io
        if self.lora_targets:
            # LoRA run: the export is the adapter in PEFT layout (adapter_model.safetensors + adapter_config.json)
            import json
            from safetensors.torch import save_file
            from .. import lora
            if self.parallel_dims.global_rank == 0:
                os.makedirs(output_dir, exist_ok=True)
                save_file(lora.native_adapter_state_dict(self.model), os.path.join(output_dir, "adapter_model.safetensors"))
                with open(os.path.join(output_dir, "adapter_config.json"), "w") as f:
                    json.dump(lora.adapter_config(self.config.policy.lora, self.lora_targets), f, indent=1)
            return
        import contextlib
        with (self.flat.materialized() if self.shard_params else contextlib.nullcontext()):
            hf_io.export_safetensors(self.model, self.hf_config, output_dir, self.parallel_dims,
                                     source_dir=self.config.policy.model_name_or_path)
        ck = self.config.train.ckpt
        if self.parallel_dims.global_rank == 0 and (ck.upload_hf or ck.upload_s3):
            from ...utils import upload
            if ck.upload_hf:
                upload.upload_folder_to_hub(output_dir, ck.hf_repo_name)
            if upload.wants_s3(ck, bool(kw.get("is_final", False))):
                rel = os.path.relpath(output_dir, self.config.train.output_dir)
                upload.upload_folder_to_s3(output_dir, ck.s3_bucket, os.path.join(ck.s3_prefix, rel),
                                           client=self.ckpt_manager.s3_client)

    # ------------------------------------------------------------------ state shipping (elastic scale-up)
    def state_tensors(self) -> List[Tuple[str, torch.Tensor]]:
        """Every tensor a new policy replica needs to continue identically: weights, optimizer state, step."""
        meta = torch.tensor([self.train_step, self.total_steps, self.optimizer.step_count], dtype=torch.int64,
                            device=self.device)
        if self.ema is None:
            self._init_ema()                    # a receiving replica has not loaded weights yet
        ema = [("ema.shard", self.ema.shard)] if self.ema is not None else []
        if ema and self.ema.tail is not None:
            ema.append(("ema.tail", self.ema.tail))
        ref = []
        if self.needs_reference():
            # every replica must score against the same anchor: the sender stages its host copy on the device (its
            # current weights when no step has run yet), the receiver a buffer of the same size
            src = self.reference_state if self.reference_state is not None else self.flat.data
            self._ref_ship = src.to(self.device, copy=True) if self.weights_ready else torch.empty_like(self.flat.data)
            ref = [("reference", self._ref_ship)]
        return [("flat.data", self.flat.data), *self.optimizer.state_tensors(), *ema, *ref, ("meta", meta)]

    def needs_reference(self) -> bool:
        """Trainers that score against a frozen copy of the initial policy (KL term, DPO) return True."""
        return False

    def after_state_received(self, meta: torch.Tensor) -> None:
        self.train_step, self.total_steps, self.optimizer.step_count = (int(x) for x in meta.tolist())
        if getattr(self, "_ref_ship", None) is not None:
            self.reference_state = self._ref_ship.to("cpu", copy=True)
        self._ref_ship = None
        self.weights_ready = True
