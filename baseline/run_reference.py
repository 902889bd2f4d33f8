"""Reference arm of the benchmark: the unmodified reference tree under ``baseline/_ref`` on the benchmark's config.

    python baseline/run_reference.py --half rollout|train --steps K --warmup W [--prompts-per-gpu 16 ...]

What runs is the reference's own code: its ``vLLMRollout`` backend (``init_engine(load_format="dummy")`` +
``rollout_generation_single_turn``, cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:249-339, 593-730) for the
generation half and its ``GRPOTrainer`` (``step_training``, cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:977-1931:
its GPT model, FSDP2 plan, flash-attn, per-token log-prob and loss code, fused AdamW) for the training half, with
the settings of its shipped Qwen2.5-7B GRPO job file (configs/qwen2-5/qwen2-5-7b-p-fsdp4-r-tp2-pp1-grpo.toml:
compile, gradient checkpointing, mini_batch 8, fp32 reduce). Nothing of this repository's package is imported.

What does NOT run is the reference's controller / worker glue: its controller process needs a ``redis-server``
binary and the python ``redis`` client (cosmos_rl/dispatcher/controller.py:172-232), neither of which exists on this
machine, and its colocated mode still registers with that controller over HTTP and Redis
(cosmos_rl/policy/policy_entry.py:32-39, cosmos_rl/policy/worker/colocated/policy_control.py:43-61). The two halves
are therefore driven directly, one after the other (a colocated step is exactly that sequence), each in its own
process so that each owns the GPU's memory while it runs; weight hand-over between them is not performed (work the
reference would additionally do, so the figure is an upper bound of its throughput).

Model: a directory with the Qwen2.5-7B ``config.json``, a synthetic whitespace tokenizer of the same vocabulary size
(every token id has the surface form ``<t{id}>``) and no weights; both halves start from random weights. Prompts are
strings of 512 such tokens, completions 1024 tokens, 8 per prompt.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 152064, "hidden_size": 3584,
    "num_hidden_layers": 28, "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 32768, "hidden_act": "silu",
    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "attention_dropout": 0.0, "initializer_range": 0.02,
    "use_cache": True, "use_sliding_window": False, "sliding_window": 131072, "max_window_layers": 28,
    "bos_token_id": 151643, "eos_token_id": 151645,
}


def make_model_dir(path: str, cfg: dict) -> str:
    """config.json + generation_config.json + a tokenizer whose ids are spelled ``<t{id}>`` (no weights)."""
    marker = os.path.join(path, ".complete")
    if os.path.exists(marker):
        return path
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    with open(os.path.join(path, "generation_config.json"), "w") as f:
        json.dump({"bos_token_id": cfg["bos_token_id"], "eos_token_id": [cfg["eos_token_id"], cfg["bos_token_id"]],
                   "do_sample": True, "temperature": 1.0, "top_p": 1.0}, f)
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    V = cfg["vocab_size"]
    tok = Tokenizer(models.WordLevel({f"<t{i}>": i for i in range(V)}, unk_token="<t0>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, eos_token=f"<t{cfg['eos_token_id']}>",
                                   pad_token=f"<t{cfg['bos_token_id']}>", bos_token=f"<t{cfg['bos_token_id']}>")
    fast.chat_template = "{% for m in messages %}{{ m['content'] }}{% endfor %}"
    fast.save_pretrained(path)
    # The reference reads the vocabulary size from the SHAPE of lm_head.weight in the checkpoint's safetensors header
    # (cosmos_rl/utils/util.py:640-697). A header that declares that one tensor, followed by a sparse (never
    # written, never read) data section of the declared size, answers it; no weights are loaded from it.
    import struct
    nbytes = cfg["vocab_size"] * cfg["hidden_size"] * 2
    header = json.dumps({"lm_head.weight": {"dtype": "BF16", "shape": [cfg["vocab_size"], cfg["hidden_size"]],
                                            "data_offsets": [0, nbytes]}}).encode()
    header += b" " * ((8 - len(header) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        f.truncate(8 + len(header) + nbytes)
    open(marker, "w").close()
    return path


def reference_config(a, model_dir: str, world: int):
    """The shipped 7B GRPO job file's settings on the benchmark's shapes."""
    from cosmos_rl.policy.config import Config
    n_seq = a.prompts_per_gpu * a.group
    return Config.from_dict({
        "redis": "12800",
        "train": {
            "resume": False, "epoch": 1, "output_dir": a.output_dir, "epsilon": 1e-6, "optm_name": "AdamW",
            "optm_lr": 1e-6, "optm_impl": "fused", "optm_weight_decay": 0.01, "optm_betas": [0.9, 0.999],
            "optm_warmup_steps": 20, "optm_grad_norm_clip": 1.0, "async_tp_enabled": False,
            "compile": not a.no_compile, "param_dtype": "bfloat16", "fsdp_reduce_dtype": "float32",
            "fsdp_offload": False, "fsdp_reshard_after_forward": "default",
            "train_batch_per_replica": n_seq * world, "sync_weight_interval": 1,
            "train_policy": {"type": "grpo", "temperature": 1.0, "epsilon_low": 0.2, "epsilon_high": 0.2,
                             "kl_beta": 0.0, "mu_iterations": 1, "mini_batch": a.mini_batch,
                             "rollout_as_token_ids": True, "dataset": {"name": "synthetic", "split": "train"},
                             "reward_function": "gsm8k"},
            "ckpt": {"enable_checkpoint": False},
        },
        "rollout": {"gpu_memory_utilization": 0.7, "enable_chunked_prefill": True, "n_generation": a.group,
                    "batch_size": a.prompts_per_gpu, "quantization": "none", "max_response_length": a.max_response,
                    "enforce_eager": False, "sampling_config": {"temperature": 1.0, "top_p": 1.0, "top_k": -1},
                    "parallelism": {"n_init_replicas": 1, "tp_size": 1, "pp_size": 1}},
        "policy": {"model_name_or_path": model_dir, "model_max_length": a.prompt_len + a.max_response,
                   "model_gradient_checkpointing": True,
                   "parallelism": {"n_init_replicas": 1, "tp_size": 1, "cp_size": 1, "dp_shard_size": world,
                                   "pp_size": 1, "dp_replicate_size": 1}},
        "logging": {"logger": ["console"]},
        "validation": {"enable": False},
    })


def prompt_strings(n: int, length: int, vocab: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (n, length), generator=g)
    return [" ".join(f"<t{t}>" for t in row.tolist()) for row in ids], ids


def run_rollout(a) -> dict:
    import torch
    from cosmos_rl.dispatcher.data.packer.decoder_only_llm_data_packer import DecoderOnlyLLMDataPacker
    from cosmos_rl.dispatcher.data.schema import RLPayload
    from cosmos_rl.rollout.vllm_rollout.vllm_rollout import vLLMRollout
    from cosmos_rl.utils.distributed import init_distributed
    from cosmos_rl.utils.parallelism import ParallelDims
    model_dir = make_model_dir(a.model_dir, QWEN25_7B)
    cfg = reference_config(a, model_dir, 1)
    init_distributed()
    dims = ParallelDims.from_config(cfg.rollout.parallelism)
    dims.build_mesh(device_type="cuda")
    dev = torch.device("cuda", torch.cuda.current_device())
    packer = DecoderOnlyLLMDataPacker()
    packer.setup(cfg)
    rollout = vLLMRollout(cfg, dims, dev)
    rollout.init_engine(quantization=None, seed=42, load_format="dummy")
    times = []
    n_tok = 0
    for it in range(a.warmup + a.steps):
        prompts, _ = prompt_strings(a.prompts_per_gpu, a.prompt_len, QWEN25_7B["vocab_size"], 1000 + it)
        payloads = [RLPayload(prompt=p, prompt_idx=i) for i, p in enumerate(prompts)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        res = rollout.rollout_generation_single_turn(payloads, torch.cuda.current_stream(), packer, False)
        e1.record()
        torch.cuda.synchronize()
        if len(res) != len(payloads):
            raise RuntimeError("the reference's rollout backend returned no results (see its traceback above)")
        if it >= a.warmup:
            times.append(e0.elapsed_time(e1) / 1e3)
            n_tok += sum(len(t) for r in res for t in r.completion_token_ids) if res[0].completion_token_ids and \
                res[0].completion_token_ids[0] else a.prompts_per_gpu * a.group * a.max_response
    return {"half": "rollout", "seconds_per_step": sum(times) / len(times), "steps": len(times),
            "generated_tokens_per_step": n_tok / max(len(times), 1)}


def run_train(a) -> dict:
    import torch
    import torch.distributed as dist
    from cosmos_rl.dispatcher.data.packer.decoder_only_llm_data_packer import DecoderOnlyLLMDataPacker
    from cosmos_rl.dispatcher.data.schema import Rollout
    from cosmos_rl.policy.trainer.llm_trainer.grpo_trainer import GRPOTrainer
    from cosmos_rl.utils.distributed import HighAvailabilitylNccl, init_distributed
    from cosmos_rl.utils.parallelism import ParallelDims
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False      # as policy_entry does
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    model_dir = make_model_dir(a.model_dir, QWEN25_7B) if rank == 0 else a.model_dir
    init_distributed()
    if world > 1:
        dist.barrier()
    cfg = reference_config(a, model_dir, world)
    dims = ParallelDims.from_config(cfg.policy.parallelism)
    dims.build_mesh(device_type="cuda")
    packer = DecoderOnlyLLMDataPacker()
    packer.setup(cfg)
    stream = torch.cuda.current_stream()
    trainer = GRPOTrainer(cfg, dims, train_stream=stream, data_packer=packer, val_data_packer=packer)
    # no checkpoint exists for this architecture here: random weights in place of load_hf_weights
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    with torch.no_grad():
        for name, p in trainer.model.named_parameters():
            t = p.to_local() if hasattr(p, "to_local") else p
            if t.dim() >= 2:
                t.normal_(0.0, 0.02, generator=g)
            elif "norm" in name:
                t.fill_(1.0)
            else:
                t.zero_()
    trainer.model.train()
    # one policy replica: the controller would send it a BuildMesh command that names only itself, after which the
    # cross-replica gradient reduction is the identity (cosmos_rl/utils/distributed.py:637-647)
    from cosmos_rl.dispatcher.command import BuildMeshCommand
    ha = HighAvailabilitylNccl(replica_name="bench-policy-0", global_rank=rank, api_client=None)
    ha.push_cmd(BuildMeshCommand({"bench-policy-0": 0}))
    ha.wait_comm_ready(timeout=60)
    n_seq = a.prompts_per_gpu * a.group
    V = QWEN25_7B["vocab_size"]
    times = []
    for it in range(a.warmup + a.steps):
        prompts, _ = prompt_strings(a.prompts_per_gpu, a.prompt_len, V, 2000 + it * world + rank)
        gen = torch.Generator().manual_seed(3000 + it * world + rank)
        rollouts = []
        for pi, p in enumerate(prompts):
            comp = torch.randint(0, V, (a.group, a.max_response), generator=gen)
            rew = (comp % 2 == 0).float().mean(1)
            adv = (rew - rew.mean()) / (rew.std() + 1e-6)
            for j in range(a.group):
                rollouts.append(Rollout(prompt=p, prompt_idx=pi, completion="",
                                        completion_token_ids=[[t] for t in comp[j].tolist()],
                                        reward=float(rew[j]), advantage=float(adv[j]), n_ignore_prefix_tokens=0))
        assert len(rollouts) == n_seq
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rep = trainer.step_training(rollouts, it + 1, 1 << 20, 1 << 20, ha, True, False)
        e1.record()
        torch.cuda.synchronize()
        dt = torch.tensor([e0.elapsed_time(e1) / 1e3], device="cuda")
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        if it >= a.warmup:
            times.append(float(dt))
        if rank == 0:
            print(f"[reference train] step {it}: {float(dt):.2f} s {({k: v for k, v in rep.items() if 'loss' in k})}",
                  file=sys.stderr, flush=True)
    ha.shutdown()
    return {"half": "train", "seconds_per_step": sum(times) / len(times), "steps": len(times), "world": world}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--half", required=True, choices=["rollout", "train"])
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--prompts-per-gpu", type=int, default=16)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--max-response", type=int, default=1024)
    ap.add_argument("--mini-batch", type=int, default=8)
    ap.add_argument("--no-compile", action="store_true")
    ap.add_argument("--model-dir", default="/tmp/b200rl_ref_model/qwen2.5-7b-arch")
    ap.add_argument("--output-dir", default="/tmp/b200rl_ref_out")
    ap.add_argument("--result", default=None, help="write the result JSON here as well")
    ap.add_argument("--dump-stacks-after", type=float, default=0.0,
                    help="seconds after which every thread's Python stack is written to stderr (diagnosis of a stall)")
    a = ap.parse_args(argv)
    if a.dump_stacks_after > 0:
        import faulthandler
        faulthandler.dump_traceback_later(a.dump_stacks_after, repeat=False, file=sys.stderr)
    sys.path.insert(0, HERE)
    sys.path.insert(0, REF)
    import ref_shims
    ref_shims.install()
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29641")
    import torch
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    t0 = time.time()
    out = run_rollout(a) if a.half == "rollout" else run_train(a)
    out["wall_s"] = time.time() - t0
    if int(os.environ.get("RANK", "0")) == 0:
        line = json.dumps(out)
        print("REFERENCE_RESULT " + line, flush=True)
        if a.result:
            with open(a.result, "w") as f:
                f.write(line)
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
