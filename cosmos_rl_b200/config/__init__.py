"""TOML -> typed configuration.

One TOML file describes a whole job; the controller parses it and is the single source of configuration for
every worker (workers fetch it over ``GET /api/meta``). Section and key names are those of the reference
(cosmos_rl/policy/config/__init__.py:73-2045) so existing job files load unchanged; keys this framework does
not know are kept (``extra="allow"``) rather than rejected.

Additions that have no counterpart in the reference are grouped under ``[b200]`` (kernel / peer-memory
switches of this implementation).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field, model_validator

try:  # py311+: stdlib
    import tomllib as _toml_reader
except Exception:  # pragma: no cover
    _toml_reader = None


class _Section(BaseModel):
    model_config = ConfigDict(extra="allow", validate_assignment=False, protected_namespaces=())


# --------------------------------------------------------------------------------------------------
# data / reward
# --------------------------------------------------------------------------------------------------
class DatasetConfig(_Section):
    name: str = ""
    subset: Optional[str] = ""
    revision: Optional[str] = ""
    split: Union[str, List[str]] = ""
    test_size: Optional[Union[float, int]] = None
    local_dir: str = ""


class OverlongRewardConfig(_Section):
    enable_overlong_penalty: bool = False
    buffer_length: int = 4096
    penalty_factor: float = 1.0


class RewardFunctionConfig(_Section):
    name: str = ""
    weight: float = 1.0
    score_key: Optional[str] = None
    clip_min: float = float("-inf")
    clip_max: float = float("inf")


class RemoteRewardConfig(_Section):
    scale: float = 1.0
    reward_fns: List[RewardFunctionConfig] = Field(default_factory=list)
    reward_clip_min: float = -5.0
    reward_clip_max: float = 5.0
    batch_size: int = 1


class SFTDataConfig(_Section):
    type: Literal["sft"] = "sft"
    trainer_type: str = "sft"
    dataset: DatasetConfig = Field(default_factory=DatasetConfig)
    mini_batch: int = 2
    dataloader_shuffle: bool = True
    dataloader_seed: int = 0
    dataloader_batch_size: Optional[int] = None
    enable_dataset_cache: bool = False
    dataloader_num_workers: int = 0
    dataloader_prefetch_factor: Optional[int] = None
    dataloader_drop_last: bool = True
    data_dispatch_as_rank_in_mesh: bool = False
    conversation_column_name: str = "conversations"
    system_prompt: str = ""
    balance_dp_token: bool = True
    enable_dp_load_balancing: bool = False
    load_balanced_pool_size: int = 32
    load_balanced_max_tokens_for_batch: Optional[int] = None
    load_balanced_batching_strategy: str = "prefer_closest"
    load_balanced_batches_per_optimizer_step: int = 1
    dataloader_broadcast: bool = False


class GrpoConfig(_Section):
    type: Literal["grpo"] = "grpo"
    trainer_type: str = "grpo"
    variant: str = "grpo"  # grpo | dapo | gspo
    dataset: DatasetConfig = Field(default_factory=DatasetConfig)
    dataloader_shuffle: bool = True
    dataloader_seed: int = 0
    data_dispatch_as_rank_in_mesh: bool = False
    enable_dataset_cache: bool = False
    dataloader_num_workers: int = 0
    dataloader_prefetch_factor: Optional[int] = None
    dataloader_batch_size: Optional[int] = None
    prompt_column_name: str = ""
    response_column_name: str = ""
    reward_function: Union[str, List[str], Dict[str, float]] = Field(default_factory=lambda: ["single_choice"])
    use_remote_reward: bool = False
    remote_reward: RemoteRewardConfig = Field(default_factory=RemoteRewardConfig)
    filter_reward_metric: Union[str, List[str]] = Field(default_factory=list)
    bypass_reward: bool = False
    group_reward_calculation: bool = False
    temperature: float = 1.0
    epsilon_low: float = 0.2
    epsilon_high: float = 0.2
    advantage_low: float = -1e9
    advantage_high: float = 1e9
    positive_nll_coef: Optional[float] = None
    lower_bound_ratio: float = 3.0
    loss_type: str = "token-mean"
    unbiased_loss_max_tokens: Optional[int] = None
    unbiased_advantage: bool = False
    algo: str = "grpo"
    overlong_reward: OverlongRewardConfig = Field(default_factory=OverlongRewardConfig)
    kl_beta: float = 0.0
    unbiased_kl_estimate: bool = False
    off_policy_masking_delta: Optional[float] = None
    aipo_rho: Optional[float] = None
    mu_iterations: int = 1
    mini_batch: int = 2
    batch_size_per_optimize: Optional[int] = None
    max_token_len_per_mini_batch: Optional[int] = None
    entropy_coeff: float = 0.0
    allowed_outdated_steps: int = 4
    on_policy: bool = False
    uncentralized_training: bool = False
    outdated_rollout_fetch_batch_size: int = 8
    max_inflight_steps: Optional[int] = None
    min_filter_prefix_tokens: Optional[int] = None
    max_retry_for_on_policy: int = 10
    reference_reset_interval: Optional[int] = None
    reset_optimizer_with_reference: bool = True
    balance_dp_token: bool = True
    use_decoupled_loss: bool = False
    behav_imp_weight_cap: Optional[float] = None
    rollout_as_token_ids: bool = False
    collect_rollout_logprobs: bool = False
    use_rollout_logprobs_for_loss: bool = False


# --------------------------------------------------------------------------------------------------
# training
# --------------------------------------------------------------------------------------------------
class CheckpointConfig(_Section):
    enable_checkpoint: bool = False
    save_freq: int = 20
    save_freq_in_epoch: int = 0
    save_mode: str = "async"  # sync | async
    max_keep: int = 5
    export_safetensors: bool = True
    upload_hf: bool = False
    hf_repo_name: str = "Comos-Reason1"
    upload_s3: Union[bool, str] = False
    s3_bucket: Optional[str] = None
    s3_prefix: str = "outputs"


class SubProfilerConfig(_Section):
    do_profile: bool = False
    active_steps: int = 1
    warmup_steps: int = 1
    wait_steps: int = 1
    rank_filter: List[int] = Field(default_factory=lambda: [0])
    record_shape: bool = False
    profile_memory: bool = False
    with_stack: bool = False
    with_modules: bool = False


class ProfilerConfig(_Section):
    enable_profiler: bool = False
    enable_nsys: bool = False
    sub_profiler_config: SubProfilerConfig = Field(default_factory=SubProfilerConfig)


class FP8Config(_Section):
    enable_fp8: bool = False
    fp8_recipe: str = "dynamic_scaling"
    quant_recipe: str = "rowwise"  # rowwise | tensorwise | blockwise (128x128 weights, 1x128 activations)


class FP4Config(_Section):
    enable_fp4: bool = False
    fp4_recipe: str = "dynamic_scaling"
    quant_recipe: str = "rowwise"


class TrainingConfig(_Section):
    train_policy: Union[SFTDataConfig, GrpoConfig] = Field(default_factory=GrpoConfig, discriminator="type")
    optm_name: str = "AdamW"
    optm_lr: Union[float, List[float], Dict[str, float]] = 1e-6
    optm_impl: Union[str, List[str]] = "fused"
    optm_weight_decay: float = 0.01
    optm_betas: tuple[float, float] = (0.9, 0.999)
    optm_warmup_steps: Union[int, float] = 20
    optm_warmup_start_factor: float = 0.0
    optm_decay_ratio: Optional[float] = None
    optm_decay_type: Optional[str] = None
    optm_min_lr_factor: float = 0.0
    optm_grad_norm_clip: float = 1.0
    ema_enable: bool = False
    ema_decay: float = 0.999
    ema_update_step_interval: int = 1
    master_dtype: str = "float32"
    param_dtype: str = "bfloat16"
    transfer_dtype: Optional[str] = None
    logprob_dtype: str = "float32"
    fsdp_reduce_dtype: str = "float32"
    fsdp_offload: bool = False
    fsdp_reshard_after_forward: str = "default"
    train_batch_per_replica: int = 8
    fp8: FP8Config = Field(default_factory=FP8Config)
    fp4: FP4Config = Field(default_factory=FP4Config)
    ckpt: CheckpointConfig = Field(default_factory=CheckpointConfig)
    resume: Union[bool, str] = False
    epoch: int = 1
    output_dir: str = "./outputs"
    timestamp: str = ""
    epsilon: float = 1e-6
    async_tp_enabled: bool = False
    compile: bool = True
    sync_weight_interval: int = 1
    coalesce_weight_sync: bool = False
    deterministic: bool = False
    activation_offload: bool = False
    fa_version: Optional[int] = None
    seed: Optional[int] = None
    local_dataset: Optional[bool] = True
    force_use_hf: Optional[bool] = False
    non_text: bool = False
    max_num_steps: Optional[int] = None
    sequence_packing: bool = False
    save_ckpt_at_exit: bool = False
    signal_to_handle: List[str] = Field(default_factory=lambda: ["SIGUSR1"])

    @property
    def param_torch_dtype(self):
        from ..utils.misc import str2dtype
        return str2dtype(self.param_dtype)

    @property
    def master_torch_dtype(self):
        from ..utils.misc import str2dtype
        return str2dtype(self.master_dtype)


class ParallelismConfig(_Section):
    n_init_replicas: int = 1
    tp_size: int = 2
    cp_size: int = 1
    ep_size: int = 1
    dp_shard_size: int = -1
    pp_size: int = 1
    pp_dynamic_shape: bool = False
    pp_micro_batch_size: int = 1
    dp_replicate_size: int = 1
    pp_schedule: str = "1F1B"
    pp_layers_per_stage: int = 0

    @property
    def world_size(self) -> int:
        shard = max(self.dp_shard_size, 1)
        return self.tp_size * self.cp_size * self.pp_size * shard * self.dp_replicate_size


class RolloutParallelismConfig(ParallelismConfig):
    tp_size: int = 2


class LoraConfig(_Section):
    r: int = 8
    lora_names: List[str] = Field(default_factory=list)
    lora_path: Optional[str] = None
    lora_alpha: float = 8.0
    lora_dropout: float = 0.0
    target_modules: Union[List[str], str] = Field(default_factory=list)
    primary_adapter: Optional[str] = None
    use_rslora: bool = False
    modules_to_save: Optional[List[str]] = None
    alpha_pattern: Optional[Dict[str, float]] = None
    r_pattern: Optional[Dict[str, int]] = None
    init_lora_weights: Union[bool, str] = True


class PolicyConfig(_Section):
    parallelism: ParallelismConfig = Field(default_factory=ParallelismConfig)
    diffusers: Optional[Dict[str, Any]] = None
    is_diffusers: bool = False
    model_name_or_path: str = "Qwen/Qwen2.5-VL-7B-Instruct"
    model_safetensor_path: Optional[str] = None
    model_revision: Optional[str] = None
    model_max_length: int = 4096
    model_gradient_checkpointing: bool = True
    lora: Optional[LoraConfig] = None
    trainable_map: Optional[Dict[str, bool]] = None
    freeze_pattern: Optional[List[str]] = None
    trainable_pattern: Optional[List[str]] = None
    enable_liger_kernel: bool = False
    enable_liger_cross_entropy: bool = False
    enable_liger_fused_cross_entropy: bool = False
    aux_loss_coeff: float = 0.0


class SamplingConfig(_Section):
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    repetition_penalty: float = 1.0
    use_flashinfer: bool = False


class MultiTurnRolloutConfig(_Section):
    enable: bool = False
    enable_tools: bool = False
    enable_thinking: bool = False
    custom_chat_template_path: Optional[str] = None
    max_assistant_turns: int = 5
    add_generation_prompt: bool = True
    continue_final_message: bool = False


class RolloutAsyncConfig(_Section):
    max_concurrent_requests: int = 10


class ValidationConfig(_Section):
    enable: bool = False
    val_before_train: bool = False
    freq: int = 20
    batch_size: Optional[int] = None
    dataset: DatasetConfig = Field(default_factory=DatasetConfig)
    temperature: float = 0.0
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    repetition_penalty: float = 1.0
    n_generation: int = 1
    max_response_length: Optional[int] = None
    reward_function: Union[str, List[str], Dict[str, float]] = Field(default_factory=list)
    use_remote_reward: Optional[bool] = None
    remote_reward: Optional[RemoteRewardConfig] = None


class RolloutConfig(_Section):
    parallelism: RolloutParallelismConfig = Field(default_factory=RolloutParallelismConfig)
    enforce_eager: bool = True
    include_stop_str_in_output: bool = False
    gpu_memory_utilization: float = 0.8
    enable_chunked_prefill: bool = False
    max_response_length: int = 2048
    n_generation: int = 16
    n_generation_to_batch: bool = False
    n_generation_mini_batch: Optional[int] = None
    batch_size: int = 1
    quantization: str = "none"  # none | fp8 | mxfp4
    seed: Optional[int] = None
    sampling_config: SamplingConfig = Field(default_factory=SamplingConfig)
    vllm_use_flashinfer: bool = False
    backend: str = "b200"  # the built-in sm_100a engine; "vllm"/"trtllm" names are accepted as aliases
    multi_turn_config: MultiTurnRolloutConfig = Field(default_factory=MultiTurnRolloutConfig)
    mode: str = "sync"
    async_config: RolloutAsyncConfig = Field(default_factory=RolloutAsyncConfig)
    async_r2r_sync: Literal["disabled", "generation", "inference"] = "disabled"
    prefetch_rollout: bool = False
    prefetch_queue_maxsize: int = 2
    broadcast_all_params: bool = False


class LoggingConfig(_Section):
    logger: List[str] = Field(default_factory=lambda: ["console"])
    log_interval: int = 1
    multi_modal_log_interval: Optional[int] = None
    project_name: str = "cosmos_rl"
    group_name: Optional[str] = None
    experiment_name: Optional[str] = None
    report_mfu: bool = False


class VLAConfig(_Section):
    vla_type: str = "openvla-oft"
    num_envs: int = 8
    use_proprio: bool = False
    proprio_dim: int = 7
    num_images_in_input: int = 1
    training_chunk_size: int = 16
    save_video: bool = False
    continuous: bool = False
    trace_verbosity: int = 0
    unnorm_key: str = ""
    max_steps: Optional[int] = None
    use_subprocess: Optional[bool] = True


class DistillationConfig(_Section):
    enable: bool = False
    parallelism: ParallelismConfig = Field(default_factory=ParallelismConfig)
    model_name_or_path: str = ""
    model_revision: Optional[str] = None
    compile: bool = False
    master_dtype: str = "float32"
    param_dtype: str = "bfloat16"
    logprob_dtype: str = "float32"
    fsdp_reduce_dtype: str = "float32"
    fsdp_offload: bool = False
    fsdp_reshard_after_forward: str = "default"
    batch_size_per_replica: int = 8
    max_token_len_per_mini_batch: Optional[int] = None
    sequence_packing: bool = False
    mini_batch: int = 1
    seed: Optional[int] = None
    kl_penalty_coef: float = 1.0
    kl_discount_factor: float = 0.0
    include_prompt: bool = False
    top_k: int = 0
    jsd_beta: float = 0.5
    trainer_token_ids_from_teacher: bool = False
    rollout_top_k_recompute: bool = False


class B200Config(_Section):
    """Switches of this implementation (no counterpart in the reference)."""

    peer_weight_sync: bool = True        # pull policy shards over NVLink peer memory instead of NCCL send/recv
    rollout_page_size: int = 128         # tokens per KV-cache page
    cuda_graph_decode: bool = True       # capture the decode step in a CUDA graph
    shared_prefix_decode: bool = False   # read a group's shared prompt pages once per group in decode attention
                                         # (correct, but slower than the plain kernel at 8 x 512-token prompts:
                                         # three launches per layer instead of one)
    fused_logprob: bool = True           # tcgen05 fused lm_head + log-prob kernel
    nvls: bool = True                    # allow multimem (NVSwitch) reductions where available
    dlogits_chunk: int = 16384
    pp_head_weight: float = 0.0          # pipeline layer split: cost of final norm + lm_head / of the embedding in
    pp_embed_weight: float = 0.0         # block-equivalents (the last / first stage get fewer blocks); -1 = from shapes
    cp_mode: str = "kv-gather"           # context-parallel attention exchange: kv-gather | ring | ring-zigzag
                                         # (ring on a layout that balances the causal work) | ulysses
    sequence_parallel: bool = False      # with tp_size > 1 (dense models, no pp / cp): residual stream and norms hold
                                         # T / tp rows (the reference's plan; halves activation memory at tp 2).
                                         # Off by default: one 7B block fwd+bwd at tp 2 takes 6.57 ms without it,
                                         # 7.17 ms with it (library collectives), 8.14 ms with the fused kernels
    sp_keep_gathered: bool = True        # keep the gathered inputs of column-parallel projections for their weight
                                         # gradients (one all-gather less per projection in backward)
    sp_fused_kernels: bool = False       # sequence-parallel projections through the all-gather -> GEMM and
                                         # GEMM -> reduce-scatter kernels instead of library collectives + cuBLAS
    pp_chunks: int = 1                   # model chunks per pipeline rank under pp_schedule = "Interleaved1F1B" (dense
                                         # GPT family); 0 = derive from policy.parallelism.pp_layers_per_stage
    shard_params: bool = False           # parameter-sharded data parallelism: weights and gradients are 1/dp_shard
                                         # per rank too, gathered block by block around their use (same switch as
                                         # train.fsdp_reshard_after_forward = "always"). Off by default: models whose
                                         # bf16 weights fit stay resident and skip the gathers
    router_bias_update_rate: float = 1e-3  # DeepSeek-V3 load-balancing bias step per optimizer step (0 = frozen)
    recompute: str = "auto"              # with policy.model_gradient_checkpointing: "selective" (attention half +
                                         # SwiGLU only), "full" (whole block, least memory), "none", or "auto":
                                         # no recomputation when the activations of one micro-batch fit in the
                                         # memory that is free after weights and optimizer state, else selective


class Config(_Section):
    custom: Dict[str, Any] = Field(default_factory=dict)
    train: TrainingConfig = Field(default_factory=TrainingConfig)
    rollout: RolloutConfig = Field(default_factory=RolloutConfig)
    policy: PolicyConfig = Field(default_factory=PolicyConfig)
    logging: LoggingConfig = Field(default_factory=LoggingConfig)
    profiler: ProfilerConfig = Field(default_factory=ProfilerConfig)
    validation: ValidationConfig = Field(default_factory=ValidationConfig)
    distillation: DistillationConfig = Field(default_factory=DistillationConfig)
    vla: VLAConfig = Field(default_factory=VLAConfig)
    b200: B200Config = Field(default_factory=B200Config)
    redis: str = ""
    eth_ips: str = ""
    mode: str = "disaggregated"  # disaggregated | colocated | colocated_separated

    # ------------------------------------------------------------------ validators
    @model_validator(mode="before")
    @classmethod
    def _infer_policy_type(cls, data):
        """Legacy job files omit ``train.train_policy.type``: infer it from GRPO-only keys
        (cosmos_rl/policy/config/__init__.py:1901-1938)."""
        if not isinstance(data, dict) or not data:
            return data
        tp = data.get("train", {}).get("train_policy") if isinstance(data.get("train"), dict) else None
        if isinstance(tp, dict) and "type" not in tp:
            grpo_keys = ("temperature", "epsilon_low", "epsilon_high", "kl_beta", "use_remote_reward")
            tp["type"] = "grpo" if any(k in tp for k in grpo_keys) else "sft"
        return data

    @model_validator(mode="after")
    def _cross_checks(self):
        pp = self.policy.parallelism
        tp = self.train.train_policy
        if pp.pp_size > 1:
            if pp.pp_micro_batch_size <= 0:
                raise ValueError("pp_micro_batch_size must be greater than 0")
            if self.train.train_batch_per_replica % pp.pp_micro_batch_size:
                raise ValueError("train_batch_per_replica must be divisible by pp_micro_batch_size")
            if self.train.fsdp_offload:
                raise ValueError("fsdp_offload is not supported together with pp_size > 1")
        if tp.type == "grpo":
            if self.policy.lora is not None and pp.tp_size != 1:
                raise ValueError("GRPO with LoRA requires policy.parallelism.tp_size == 1")
            if pp.dp_replicate_size > 1:
                raise ValueError("GRPO scales by adding policy replicas; dp_replicate_size must be 1")
            if tp.allowed_outdated_steps + 1 < self.train.sync_weight_interval:
                tp.allowed_outdated_steps = self.train.sync_weight_interval - 1
            if tp.max_inflight_steps is not None and tp.max_inflight_steps < tp.allowed_outdated_steps + 1:
                tp.max_inflight_steps = tp.allowed_outdated_steps + 1
            if tp.on_policy and self.train.sync_weight_interval != 1:
                raise ValueError("on_policy training requires sync_weight_interval == 1")
            if self.validation.use_remote_reward is None:
                self.validation.use_remote_reward = tp.use_remote_reward
            if self.validation.remote_reward is None:
                self.validation.remote_reward = tp.remote_reward
        if isinstance(self.validation.dataset.split, str):
            self.validation.dataset.split = [self.validation.dataset.split]
        if self.train.transfer_dtype is None:
            self.train.transfer_dtype = self.train.master_dtype
        if self.train.async_tp_enabled and not self.train.compile:
            # the reference ties async TP to torch.compile; here the fused AG-GEMM / GEMM-RS kernels need no compiler
            pass
        if self.distillation.enable and tp.type == "grpo":
            tp.rollout_as_token_ids = True
            tp.bypass_reward = True
        elif not self.distillation.enable:
            self.distillation.top_k = 0
        if self.mode not in ("disaggregated", "colocated", "colocated_separated"):
            raise ValueError(f"unknown mode {self.mode!r}")
        return self

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "Config":
        return cls.model_validate(data)

    @classmethod
    def from_toml(cls, path: str) -> "Config":
        return cls.from_dict(load_toml(path))

    def to_dict(self) -> Dict[str, Any]:
        return json.loads(self.model_dump_json())

    @classmethod
    def json_schema(cls) -> Dict[str, Any]:
        return cls.model_json_schema()


def load_toml(path: str) -> Dict[str, Any]:
    with open(path, "rb") as f:
        return _toml_reader.load(f)


def dump_toml(data: Dict[str, Any]) -> str:
    """Minimal TOML writer (tables, scalars, lists) for the launcher's patched job file."""
    lines: List[str] = []

    def fmt(v):
        if isinstance(v, bool):
            return "true" if v else "false"
        if isinstance(v, (int, float)):
            if isinstance(v, float) and v in (float("inf"), float("-inf")):
                return "inf" if v > 0 else "-inf"
            return repr(v)
        if isinstance(v, str):
            return json.dumps(v)
        if isinstance(v, (list, tuple)):
            return "[" + ", ".join(fmt(x) for x in v) + "]"
        if isinstance(v, dict):
            return "{" + ", ".join(f"{k} = {fmt(x)}" for k, x in v.items() if x is not None) + "}"
        raise TypeError(f"cannot write {type(v)} to TOML")

    def emit(table: Dict[str, Any], prefix: str):
        scalars = {k: v for k, v in table.items() if not isinstance(v, dict) and v is not None}
        tables = {k: v for k, v in table.items() if isinstance(v, dict)}
        if prefix and (scalars or not tables):
            lines.append(f"[{prefix}]")
        for k, v in scalars.items():
            lines.append(f"{k} = {fmt(v)}")
        if scalars:
            lines.append("")
        for k, v in tables.items():
            emit(v, f"{prefix}.{k}" if prefix else k)

    emit(data, "")
    return "\n".join(lines) + "\n"
