"""GRPO step benchmark THROUGH the framework's own job stack (``bench.py --layout launcher``): the job is started by
``launcher.launch_all`` exactly as a user's job is (controller, broker, policy and rollout workers as separate
processes, or the colocated worker with the controller in its process at one GPU), on the same model, prompt shape,
group size and reward as the direct loop of ``bench_grpo`` / ``bench_multi``.

The number comes from the controller's own step reports: the ``jsonl`` report sink stamps every finished step with
the wall clock, so tokens/s = (prompt + response tokens trained per step) x K / (stamp of step W + K - stamp of step
W). This is a host-clock figure of the whole control path (prompt hand-out, JSON rollouts through the broker, reward
dispatch, step scheduling, weight-sync commands); the device-timed direct loop beside it shows what that path costs.

Layout by GPU count: 1 = colocated worker; 2 = policy 1 GPU + rollout 1 GPU; 4 = policy FSDP2 + rollout TP1 x 2;
8 = policy FSDP4 + rollout TP2 x 2 (the same split as the direct disaggregated loop).
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
import time
from typing import Any, Dict, List, Tuple

from .config import dump_toml
from .models import named_architectures

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def job_layout(n_gpus: int) -> Tuple[str, int, int, int]:
    """(mode, policy dp_shard, rollout tp, rollout replicas)."""
    if n_gpus == 1:
        return "colocated", 1, 1, 1
    from .bench_multi import layout
    p, tp, r = layout(n_gpus)
    return "disaggregated", p, tp, r


def job_config(args, n_gpus: int, output_dir: str) -> Dict[str, Any]:
    mode, p, tp, r = job_layout(n_gpus)
    prompts_per_step = args.prompts_per_gpu * n_gpus
    return {
        "mode": mode,
        "policy": {"model_name_or_path": args.model, "model_max_length": args.prompt_len + args.max_response,
                   "model_gradient_checkpointing": True,
                   "parallelism": {"tp_size": 1, "dp_shard_size": p, "n_init_replicas": 1}},
        "rollout": {"n_generation": args.group, "batch_size": prompts_per_step // r,
                    "max_response_length": args.max_response, "seed": 1234, "gpu_memory_utilization": 0.9,
                    "parallelism": {"tp_size": tp, "n_init_replicas": r},
                    "sampling_config": {"temperature": 1.0, "top_p": 1.0, "top_k": -1}},
        "train": {"seed": 0, "epoch": 1, "optm_lr": 1e-6, "optm_warmup_steps": 20, "output_dir": output_dir,
                  "train_batch_per_replica": prompts_per_step * args.group, "sync_weight_interval": 1,
                  "ckpt": {"enable_checkpoint": False},
                  "train_policy": {"type": "grpo", "reward_function": ["even_token_fraction"],
                                   "rollout_as_token_ids": True, "dataloader_shuffle": False,
                                   "max_token_len_per_mini_batch": args.mb_tokens, "temperature": 1.0,
                                   # generation of step n + 1 overlaps the update of step n, as in the direct loop
                                   "allowed_outdated_steps": 0 if mode == "colocated" else 1}},
        "logging": {"logger": ["console", "jsonl"]},
    }


def read_steps(path: str) -> List[Dict[str, Any]]:
    if not os.path.exists(path):
        return []
    rows = []
    for ln in open(path):
        try:
            rows.append(json.loads(ln))
        except ValueError:
            pass
    return rows


def throughput(rows: List[Dict[str, Any]], warmup: int, steps: int, tokens_per_step: int) -> Dict[str, float]:
    """Tokens/s over the K steps that follow step ``warmup`` (the stamp of step W closes the warm-up)."""
    by = {int(r["step"]): r for r in rows}
    if warmup < 1 or warmup not in by or warmup + steps not in by:
        raise ValueError(f"step reports {sorted(by)} do not cover steps {warmup}..{warmup + steps}")
    dt = float(by[warmup + steps]["time"]) - float(by[warmup]["time"])
    return {"seconds": dt, "ms_per_step": dt / steps * 1e3, "value": tokens_per_step * steps / dt}


def run(args, cpu: bool = False, timeout_s: float = 0.0) -> Dict[str, Any]:
    """Start the job, wait for it, and turn the controller's step reports into the benchmark record. The job is
    stopped (its whole process group) after ``timeout_s`` seconds, ``B200RL_JOB_TIMEOUT_S`` or 1500."""
    timeout_s = timeout_s or float(os.environ.get("B200RL_JOB_TIMEOUT_S", "1500"))
    n = args.gpus
    mode, p, tp, r = job_layout(n)
    total_steps = args.warmup + args.steps
    prompts_per_step = args.prompts_per_gpu * n
    seq_len = args.prompt_len + args.max_response
    tokens_per_step = prompts_per_step * args.group * seq_len
    work = tempfile.mkdtemp(prefix="b200rl_bench_job_")
    out_dir = os.path.join(work, "out")
    os.makedirs(out_dir)
    cfg_path = os.path.join(work, "job.toml")
    with open(cfg_path, "w") as f:
        f.write(dump_toml(job_config(args, n, out_dir)))
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""),
               B200RL_BENCH_PROMPTS=str(prompts_per_step * total_steps), B200RL_BENCH_PROMPT_LEN=str(args.prompt_len),
               B200RL_BENCH_VOCAB=str(named_architectures()[args.model].vocab_size))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "GROUP_RANK"):
        env.pop(k, None)                      # the job builds its own rendezvous
    for k in [k for k in env if k.startswith("TORCHELASTIC_")]:
        env.pop(k)
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", cfg_path, "--policy", "1",
           "--rollout", str(r), "--log-dir", os.path.join(work, "logs"),
           "--rdzv-port", str(getattr(args, "rdzv_port", 29391))]
    if cpu:
        cmd.append("--cpu")
    cmd.append(os.path.join(ROOT, "cosmos_rl_b200", "launcher", "bench_entry.py"))
    clocks = None
    if not cpu:
        from bench import ClockSampler
        clocks = ClockSampler(0)
    import signal
    import threading
    if threading.current_thread() is threading.main_thread():
        def _stop(signum, _frame):            # a terminated benchmark takes its job down with it
            raise KeyboardInterrupt(f"signal {signum}")
        signal.signal(signal.SIGTERM, _stop)
    t0 = time.time()
    proc = subprocess.Popen(cmd, env=env, start_new_session=True)
    metrics = os.path.join(out_dir, "metrics.jsonl")
    started = False
    try:
        while proc.poll() is None:
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"the job did not finish within {timeout_s:.0f} s (logs under {work})")
            if clocks is not None and not started and len(read_steps(metrics)) >= args.warmup:
                clocks.start()                # the timed steps begin at the stamp of step W
                started = True
            time.sleep(0.5)
    except BaseException:
        try:
            os.killpg(proc.pid, signal.SIGTERM)
        except ProcessLookupError:
            pass
        raise
    clk = clocks.stop() if (clocks is not None and started) else None
    rows = read_steps(metrics)
    if proc.returncode != 0:
        raise RuntimeError(f"the job exited with code {proc.returncode} after {len(rows)} steps (logs under {work})")
    tp_ = throughput(rows, args.warmup, args.steps, tokens_per_step)
    timed = [x for x in rows if args.warmup < int(x["step"]) <= total_steps]
    mean = lambda k: sum(float(x.get(k, 0.0)) for x in timed) / max(1, len(timed))   # noqa: E731
    return {
        "metric": "GRPO step tokens/s (prompt+response tokens generated and trained per second)",
        "value": tp_["value"], "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": tp_["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if not cpu else "fp32",
        "data": "synthetic prompts (uniform random token ids), random-init weights, even-token-fraction reward",
        "timing": "host wall clock between the controller's step reports (the job is several processes; no CUDA "
                  "event spans them)",
        "config": {"model": f"{args.model}-arch", "global_batch": prompts_per_step * args.group, "seq_len": seq_len,
                   "prompts": prompts_per_step, "group": args.group, "prompt_len": args.prompt_len,
                   "max_response": args.max_response, "layout": "launcher",
                   "parallelism": ("colocated worker (controller logic in the worker's process), dp1 tp1" if n == 1 else
                                   f"launcher job: controller + policy FSDP{p} + rollout TP{tp} x {r} replicas"),
                   "l2": "inputs larger than L2 (the weights are streamed every decode step and every layer)"},
        "clocks": clk,
        "breakdown": {"train_iteration_s": mean("train/iteration_time"), "step_wall_s": mean("train/step_wall_time"),
                      "tokens_trained_per_step": mean("train/n_tokens"), "job_wall_s": time.time() - t0,
                      "steps_reported": len(rows)},
        "job_dir": work,
    }
