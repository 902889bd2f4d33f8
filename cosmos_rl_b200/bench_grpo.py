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
        layout = getattr(self.args, "layout", "auto")
        if layout == "auto":
            layout = "disaggregated" if self.world == 8 else "colocated"
        if self.world == 1 or layout == "colocated":
            return self.run_colocated()
        from .bench_multi import run_disaggregated
        return run_disaggregated(self)

    def run_colocated(self) -> Dict[str, Any]:
        from bench import ClockSampler
        from .colocated import ColocatedGRPO
        a = self.args
        W = self.world
        cfg = make_config(a, W, 1, colocated=True)
        grp = None
        if W > 1:
            # data-parallel colocated replicas: every GPU generates and trains its own prompts; gradients meet in
            # the fused peer-memory reduce-scatter, the sharded AdamW publishes the new weights to every GPU
            from .parallel.dims import ParallelDims
            from .parallel.fsdp import PeerCollective
            from .parallel.peer import peer_allocator
            gloo = dist.new_group(backend="gloo")
            grp = dist.new_group(list(range(W)))
            dims = ParallelDims(dp_shard=W, world_size=W, global_rank=self.rank, device=self.device)
            dims.set_group("dp_shard", grp)
            job = ColocatedGRPO(cfg, dims, device=self.device, max_num_seqs=a.prompts_per_gpu * a.group,
                                allocator=peer_allocator(self.device))
            job.trainer.optimizer.collective = PeerCollective(job.trainer.flat, grp, object_group=gloo)
        else:
            job = ColocatedGRPO(cfg, device=self.device, max_num_seqs=a.prompts_per_gpu * a.group)
        n_prompts = a.prompts_per_gpu
        tokens_per_step = W * n_prompts * a.group * (a.prompt_len + a.max_response)

        def sync_all():
            torch.cuda.synchronize()
            if grp is not None:
                dist.barrier(group=grp)
                torch.cuda.synchronize()

        def one_step(i: int, from_host: bool):
            hp = self.host_prompts(i * W + self.rank, n_prompts)
            dp = hp.to(self.device, non_blocking=True)
            rep = job.step([dp[j] for j in range(n_prompts)])
            return rep

        for i in range(a.warmup):
            one_step(i, True)
        native.read_status(self.device)
        # ---- device-timed region: K steps between CUDA events
        clocks = ClockSampler(self.local_rank)
        sync_all()
        clocks.start()
        launches0 = native.LAUNCHES[0]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        reports = [one_step(a.warmup + i, True) for i in range(a.steps)]
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        launches = native.LAUNCHES[0] - launches0
        clk = clocks.stop()
        native.read_status(self.device)
        if grp is not None:                         # device time: max over ranks; launches: sum over ranks
            t = torch.tensor([ms, float(launches)], device=self.device, dtype=torch.float64)
            tmax = t.clone()
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX, group=grp)
            dist.all_reduce(t, group=grp)
            ms, launches = tmax[0].item(), int(t[1].item())
        value = tokens_per_step * a.steps / (ms / 1e3)
        out = {
            "metric": "GRPO step tokens/s (prompt+response tokens generated and trained per second)",
            "value": value, "unit": "tokens/s", "n_gpus": W, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic prompts (uniform random token ids), random-init weights, "
                                     "even-token-fraction reward",
            "config": {"model": f"{a.model}-arch", "global_batch": W * n_prompts * a.group,
                       "seq_len": a.prompt_len + a.max_response,
                       "prompts": W * n_prompts, "group": a.group, "prompt_len": a.prompt_len,
                       "max_response": a.max_response,
                       "parallelism": f"colocated policy+rollout on every GPU (dp{W}, tp1; optimizer state sharded over "
                                      f"{W} GPUs)" if W > 1 else "colocated policy+rollout on 1 GPU (dp1,tp1)",
                       "l2": "inputs larger than L2 (15 GB of weights streamed every decode step and every layer)",
                       "optimizer": "AdamW fp32 master + moments, 1 optimizer step per GRPO step",
                       "weight_sync": "shared tensors (colocated): version bump" + (
                           "; new weights reach every GPU through the fused AdamW + peer publish kernel" if W > 1 else "")},
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
            sync_all()
            t0 = time.perf_counter()
            for i in range(a.steps):
                hp = self.host_prompts(10_000 + i * W + self.rank, n_prompts)
                dp = hp.to(self.device, non_blocking=True)
                rep = job.step([dp[j] for j in range(n_prompts)])
                loss_host = float(rep["train/loss_avg"])
                h2d += hp.numel() * hp.element_size() + int(rep["train/n_tokens"]) * 8 * 3
                d2h += n_prompts * a.group * a.max_response * 12 + 64
            sync_all()
            dt = time.perf_counter() - t0
            if grp is not None:
                t = torch.tensor([dt], device=self.device, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=grp)
                dt = t.item()
                h2d, d2h = h2d * W, d2h * W
            out["e2e"] = {"value": tokens_per_step * a.steps / dt, "unit": "tokens/s",
                          "h2d_bytes_per_step": h2d // a.steps, "d2h_bytes_per_step": d2h // a.steps,
                          "api": "cosmos_rl_b200.colocated.ColocatedGRPO.step"}
        return out
