"""API-surface contracts: what user scripts, job files and operators of the reference rely on must keep its name and
shape here (entry point signature, data-packer and dataset contracts, registries, HTTP routes, command fields, wire
schemas, configuration defaults)."""
import inspect

import pytest

from cosmos_rl_b200.config import Config


def test_entry_point_signature_and_import_paths():
    from cosmos_rl.launcher.worker_entry import main as launch_worker          # the reference's import path
    params = inspect.signature(launch_worker).parameters
    for name in ("dataset", "val_dataset", "data_packer", "val_data_packer", "reward_fns", "filter_reward_fns",
                 "val_reward_fns", "custom_logger_fns", "hook_fns", "sampler", "batch_sampler", "args"):
        assert name in params, name
    from cosmos_rl.dispatcher.data.packer import BaseDataPacker, DecoderOnlyLLMDataPacker  # noqa: F401
    from cosmos_rl.policy.config import Config as C2
    assert C2 is Config


def test_data_packer_contract_and_mask_convention():
    from cosmos_rl_b200.data.packer import BaseDataPacker, DecoderOnlyLLMDataPacker
    for m in ("get_rollout_input", "rollout_collate_fn", "get_rollout_output", "get_policy_input",
              "policy_compute_max_len", "policy_collate_fn", "sft_process_sample", "sft_compute_max_len",
              "sft_collate_fn", "batch_size", "slice_batch", "save_state"):
        assert callable(getattr(BaseDataPacker, m)), m
    p = DecoderOnlyLLMDataPacker()
    p.setup(Config.from_dict({}), None)
    pi = p.get_policy_input([1, 2, 3], [7, 8, 9, 10], n_ignore_prefix_tokens=1)
    # mask[i] == 1 <=> token i + 1 is a scored completion token
    assert pi.input_ids == [1, 2, 3, 7, 8, 9, 10] and pi.logprob_masks == [0, 0, 0, 1, 1, 1, 0]
    b = p.policy_collate_fn([pi], 8)
    assert b["input_ids"].shape == (1, 8) and b["logprob_masks"].dtype.is_floating_point is False


def test_registries():
    from cosmos_rl_b200.colocated import worker  # noqa: F401  (imports every built-in trainer and backend)
    from cosmos_rl_b200.dispatcher.algo.grpo import register_rule_based_algo  # noqa: F401
    from cosmos_rl_b200.models.base import ModelRegistry
    from cosmos_rl_b200.policy.trainer import dpo_trainer, sft_trainer  # noqa: F401
    from cosmos_rl_b200.policy.trainer.base import TrainerRegistry
    from cosmos_rl_b200.rollout.base import RolloutRegistry
    from cosmos_rl_b200.utils import constant
    for t in ("grpo", "sft", "dpo", "diffusion_sft", "diffusion_nft", "flow_grpo", "vla_grpo"):
        assert t in TrainerRegistry.known(), t
    for b in ("vllm", "vllm_async", "trtllm", "b200", "hf", "recompute", "diffusion", "vla"):
        assert b in RolloutRegistry.known(), b
    for mt in ("qwen2", "qwen3", "llama", "qwen3_moe", "deepseek_v3", "dit"):
        assert ModelRegistry.get(mt).__name__ != "HFModel", mt
    assert ModelRegistry.get("some_future_family").__name__ == "HFModel" and constant.COSMOS_DEFAULT_MODEL_TYPE == "hfmodel"


def test_http_routes(tmp_path):
    from cosmos_rl_b200.dispatcher.controller import Controller
    from cosmos_rl_b200.dispatcher.run_web_panel import create_app
    app = create_app(Controller(Config.from_dict({"train": {"output_dir": str(tmp_path)}})))
    routes = {(m, r.path) for r in app.routes for m in getattr(r, "methods", [])}
    for path in ("/panel", "/api/status", "/api/meta", "/api/next_prompt", "/api/nccl/comm_all", "/api/get_trainable_params"):
        assert ("GET", path) in routes, path
    for path in ("/api/register", "/api/unregister", "/api/heartbeat", "/api/set_profile", "/api/set_trace_path",
                 "/api/nccl/comm_initiator", "/api/nccl/comm_acceptor", "/api/nccl/comm_error", "/api/nccl/comm_store_clear",
                 "/api/rollout", "/api/validation_report", "/api/policy/train_ack", "/api/policy/shard_infos",
                 "/api/rollout/shard_infos", "/api/policy_shard_send_insts", "/api/shard_recv_insts", "/api/resume_info"):
        assert ("POST", path) in routes, path


def test_command_and_wire_schemas():
    from cosmos_rl_b200.dispatcher import command as cmd
    from cosmos_rl_b200.dispatcher.data.schema import RLPayload, Rollout
    c = cmd.DataFetchCommand(replica_name="p", items_count=4, global_step=3, total_steps=3, remain_samples_num=0)
    d = cmd.Command.depack(c.pack())
    assert type(d) is cmd.DataFetchCommand and d.replica_should_stop() and d.items_count == 4
    u = cmd.PolicyToRolloutUnicastCommand("p", "r", 4, 2, weight_step=7, total_steps=9, do_weight_sync_check=True)
    d = cmd.Command.depack(u.pack())
    assert (d.src_replica_name, d.dst_replica_size, d.weight_step, d.do_weight_sync_check) == ("p", 2, 7, True)
    for f in ("prompt", "prompt_idx", "conversation", "reference_answer", "weight_version", "completions",
              "completed_conversations", "n_ignore_prefix_tokens", "rewards", "advantages", "valid", "filter_rewards",
              "completion_token_ids", "completion_logprobs", "cumulative_logprob", "extra_info", "report_metrics",
              "teacher_result_uuids"):
        assert f in RLPayload.model_fields, f
    for f in ("prompt", "completion", "completed_conversation", "reward", "advantage", "n_ignore_prefix_tokens",
              "filter_reward", "completion_token_ids", "completion_logprobs", "weight_version", "teacher_result_uuid"):
        assert f in Rollout.model_fields, f
    p = RLPayload(prompt="q", completions=["a"], completion_token_ids=[[[5, 9], [6, 2]]], completion_logprobs=[[[-0.1, -3.0], [-0.2, -2.0]]])
    assert p.completion_token_ids[0][1][0] == 6            # [completion][position][rank], rank 0 = sampled token


def test_configuration_defaults_match_the_reference():
    c = Config.from_dict({})
    tp = c.train.train_policy
    assert c.policy.parallelism.tp_size == 2 and c.train.sync_weight_interval == 1 and c.train.optm_grad_norm_clip == 1.0
    assert c.train.param_dtype == "bfloat16" and c.train.master_dtype == "float32"
    assert c.rollout.n_generation == 16 and c.rollout.max_response_length == 2048 and c.rollout.batch_size == 1
    s = c.rollout.sampling_config
    assert (s.temperature, s.top_p, s.top_k) == (1.0, 1.0, -1)
    g = Config.from_dict({"train": {"train_policy": {"type": "grpo"}}}).train.train_policy
    assert (g.mini_batch, g.mu_iterations, g.epsilon_low, g.epsilon_high, g.lower_bound_ratio, g.kl_beta,
            g.loss_type, g.allowed_outdated_steps) == (2, 1, 0.2, 0.2, 3.0, 0.0, "token-mean", 4)
    with pytest.raises(ValueError):
        Config.from_dict({"mode": "somewhere"})
