"""GRPO step benchmark driver used by ``bench.py`` (kept in the package so the layouts it builds are the
public ones: ``ColocatedGRPO`` at one GPU, policy/rollout roles over peer memory at several)."""
from __future__ import annotations

import os
import sys
import time
from typing import Any, Dict, List

import torch
import torch.distributed as dist

from .config import Config
from .models import named_architectures
from .ops import native


def make_config(args, n_policy_gpus: int, rollout_tp: int, colocated: bool) -> Config:
    arch = named_architectures()[args.model]
    max_len = args.prompt_len + args.max_response
    return Config.from_dict({
        "mode": "colocated" if colocated else "disaggregated",
        "policy": {"model_name_or_path": args.model, "model_max_length": max_len,
                   "model_gradient_checkpointing": True,
                   "parallelism": {"tp_size": 1, "dp_shard_size": n_policy_gpus, "n_init_replicas": 1}},
        "rollout": {"n_generation": args.group, "batch_size": args.prompts_per_gpu,
                    "max_response_length": args.max_response, "seed": 1234,
                    "parallelism": {"tp_size": rollout_tp, "n_init_replicas": 1},
                    "sampling_config": {"temperature": 1.0, "top_p": 1.0, "top_k": -1}},
        "train": {"seed": 0, "optm_lr": 1e-6, "optm_warmup_steps": 20, "output_dir": "/tmp/b200rl_bench",
                  "train_batch_per_replica": args.prompts_per_gpu * args.group,
                  "train_policy": {"type": "grpo", "reward_function": ["even_token_fraction"],
                                   "max_token_len_per_mini_batch": args.mb_tokens, "temperature": 1.0}},
        "logging": {"logger": ["console"]},
    })


class GRPOBench:
    def __init__(self, args, rank: int, world: int, local_rank: int):
        self.args, self.rank, self.world, self.local_rank = args, rank, world, local_rank
        self.device = torch.device("cuda", local_rank)
        self.vocab = named_architectures()[args.model].vocab_size

    # ------------------------------------------------------------------ synthetic prompts
    def host_prompts(self, step: int, n_prompts: int) -> torch.Tensor:
        g = torch.Generator().manual_seed(1000 + step)
        return torch.randint(0, self.vocab, (n_prompts, self.args.prompt_len), generator=g, dtype=torch.int64).pin_memory()

    # ------------------------------------------------------------------
    def run(self) -> Dict[str, Any]:
        if self.world == 1:
            return self.run_colocated()
        from .bench_multi import run_disaggregated
        return run_disaggregated(self)

    def run_colocated(self) -> Dict[str, Any]:
        from bench import ClockSampler
        from .colocated import ColocatedGRPO
        a = self.args
        cfg = make_config(a, 1, 1, colocated=True)
        job = ColocatedGRPO(cfg, device=self.device, max_num_seqs=a.prompts_per_gpu * a.group)
        n_prompts = a.prompts_per_gpu
        tokens_per_step = n_prompts * a.group * (a.prompt_len + a.max_response)

        def one_step(i: int, from_host: bool):
            hp = self.host_prompts(i, n_prompts)
            dp = hp.to(self.device, non_blocking=True)
            rep = job.step([dp[j] for j in range(n_prompts)])
            return rep

        for i in range(a.warmup):
            one_step(i, True)
        native.read_status(self.device)
        # ---- device-timed region: K steps between CUDA events
        clocks = ClockSampler(self.local_rank)
        torch.cuda.synchronize()
        clocks.start()
        launches0 = native.LAUNCHES[0]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        reports = [one_step(a.warmup + i, True) for i in range(a.steps)]
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = native.LAUNCHES[0] - launches0
        clk = clocks.stop()
        native.read_status(self.device)
        value = tokens_per_step * a.steps / (ms / 1e3)
        out = {
            "metric": "GRPO step tokens/s (prompt+response tokens generated and trained per second)",
            "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic prompts (uniform random token ids), random-init weights, "
                                     "even-token-fraction reward",
            "config": {"model": f"{a.model}-arch", "global_batch": n_prompts * a.group, "seq_len": a.prompt_len + a.max_response,
                       "prompts": n_prompts, "group": a.group, "prompt_len": a.prompt_len,
                       "max_response": a.max_response, "parallelism": "colocated policy+rollout on 1 GPU (dp1,tp1)",
                       "l2": "inputs larger than L2 (15 GB of weights streamed every decode step and every layer)",
                       "optimizer": "AdamW fp32 master + moments, 1 optimizer step per GRPO step",
                       "weight_sync": "shared tensors (colocated): version bump"},
            "clocks": clk, "gpu_launches": launches,
            "breakdown": {"rollout_s": sum(r["rollout/time"] for r in reports) / a.steps,
                          "train_s": sum(r["train/time"] for r in reports) / a.steps,
                          "weight_sync_ms": 0.0, "loss": reports[-1]["train/loss_avg"],
                          "grad_norm": reports[-1]["train/grad_norm"],
                          "reward_mean": reports[-1]["rollout/reward_mean"]},
        }
        if not a.no_e2e:
            # ---- end-to-end: the same public call, wall clock, inputs start in pinned host memory and the
            # step's loss is read back to the host
            h2d = d2h = 0
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for i in range(a.steps):
                hp = self.host_prompts(10_000 + i, n_prompts)
                dp = hp.to(self.device, non_blocking=True)
                rep = job.step([dp[j] for j in range(n_prompts)])
                loss_host = float(rep["train/loss_avg"])
                h2d += hp.numel() * hp.element_size() + int(rep["train/n_tokens"]) * 8 * 3
                d2h += n_prompts * a.group * a.max_response * 12 + 64
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            out["e2e"] = {"value": tokens_per_step * a.steps / dt, "unit": "tokens/s",
                          "h2d_bytes_per_step": h2d // a.steps, "d2h_bytes_per_step": d2h // a.steps,
                          "api": "cosmos_rl_b200.colocated.ColocatedGRPO.step"}
        return out
