#!/usr/bin/env python
"""Headline benchmark: GRPO step tokens/s on the Qwen2.5-7B architecture (random-init weights, synthetic
prompts, synthetic even-token reward), weak scaling over the GPUs of one node.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

One step = generate `group` responses for each prompt with the built-in rollout engine, score them, run the
GRPO policy update (forward, fused log-prob/loss, backward, clip, AdamW) and make the new weights visible
to the rollout engine. Per-GPU work is fixed (16 prompts x 8 responses x (512 + 1024) tokens per GPU), so
the 8-GPU run is the named configuration: 128 prompts, policy FSDP4 on GPUs 0-3, rollout TP2 x 2 on 4-7.
Rank 0 prints ONE JSON line. `--impl reference` runs the reference arm instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts-per-gpu", type=int, default=16)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--max-response", type=int, default=1024)
    ap.add_argument("--mb-tokens", type=int, default=8192, help="token budget of one training micro-batch")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 5],
                    help="benchmark configuration: 1 = the tiny Qwen2-arch plumbing job on CPU / gloo (controller + 1 "
                         "policy rank + 1 rollout rank through the launcher; fp32, no GPU); 2 = Qwen2.5-7B-arch GRPO "
                         "step (the headline); 5 = weight-sync sweep "
                         "on a separated layout (policy on the first half of the GPUs, rollout TP 1/2/4 on the "
                         "second half; bf16 pull, fused fp8 pull, and the reference-style fp32 send/recv route). The "
                         "MoE and long-context configurations are not wired into this script")
    ap.add_argument("--layout", default="auto", choices=["auto", "colocated", "disaggregated", "launcher"],
                    help="launcher: start the same job through launcher.launch_all (controller, broker and workers as "
                         "a user's job runs) and read tokens/s from the controller's step reports; auto: 8 GPUs use the named disaggregated layout (policy FSDP4 + rollout TP2 x 2); 1, 2 and 4 "
                         "GPUs run colocated data-parallel replicas (each GPU generates and trains its own prompts)")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
def run_reference(args):
    """The reference arm: the unmodified reference tree under baseline/_ref, driven by baseline/run_reference.py
    (its vLLM rollout backend, then its GRPO trainer, on this benchmark's shapes; see that file for what is and is not
    the reference's stock path). Under torchrun every rank runs its own generation engine, the trainer spans all
    ranks with the reference's FSDP plan. Rank 0 prints ONE JSON line."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    out = {"impl": "reference"}

    def finish(obj):
        if rank == 0:
            sys.stdout.write(json.dumps(obj) + "\n")
            sys.stdout.flush()
        return 0

    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29512"),
                   os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        out["unavailable"] = f"WORLD_SIZE={world} does not match --gpus {args.gpus}"
        return finish(out)
    ref = os.path.join(ROOT, "baseline", "_ref")
    driver = os.path.join(ROOT, "baseline", "run_reference.py")
    if not os.path.isdir(os.path.join(ref, "cosmos_rl")):
        out["unavailable"] = ("baseline/_ref is absent (pip install --no-index --no-deps --target baseline/_ref of the "
                              "reference source tree was not done on this box)")
        return finish(out)
    tag = f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid() if world > 1 else os.getpid()}"
    res_dir = os.path.join("/tmp", f"b200rl_ref_res_{tag}")
    os.makedirs(res_dir, exist_ok=True)
    log_dir = os.environ.get("B200RL_REF_LOG_DIR") or res_dir        # where the two halves write their logs
    os.makedirs(log_dir, exist_ok=True)
    common = ["--steps", str(args.steps), "--warmup", str(args.warmup), "--prompts-per-gpu", str(args.prompts_per_gpu),
              "--group", str(args.group), "--prompt-len", str(args.prompt_len), "--max-response", str(args.max_response)]
    limit = float(os.environ.get("B200RL_REF_TIMEOUT_S", "1500"))

    def run_half(half, env, result_path, log_name):
        log = os.path.join(log_dir, log_name)
        with open(log, "w") as lf:
            try:
                rc = subprocess.call([sys.executable, driver, "--half", half, "--result", result_path] + common,
                                     env=env, stdout=lf, stderr=subprocess.STDOUT, timeout=limit)
            except subprocess.TimeoutExpired:
                return None, f"{half} half did not finish within {limit:.0f} s"
        if rc != 0 or not os.path.exists(result_path):
            tail = ""
            try:
                lines = [ln.strip() for ln in open(log, errors="replace").read().splitlines() if ln.strip()]
                errs = [ln for ln in lines if "Error" in ln or "error" in ln]
                tail = (errs[-1] if errs else lines[-1])[:300] if lines else ""
            except Exception:
                pass
            return None, f"{half} half of the reference exited with code {rc}: {tail}"
        return json.load(open(result_path)), None

    # ---- generation half: one engine per GPU, each in its own single-rank world
    env = dict(os.environ)
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    dev = visible.split(",")[local_rank] if visible else str(local_rank)
    env.update({"RANK": "0", "WORLD_SIZE": "1", "LOCAL_RANK": "0", "LOCAL_WORLD_SIZE": "1", "GROUP_RANK": "0",
                "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(29700 + local_rank), "CUDA_VISIBLE_DEVICES": dev})
    # the engine's process is a world of its own: nothing of the launcher's rendezvous may leak into it (with
    # TORCHELASTIC_USE_AGENT_STORE set, env:// would look for the launcher's store on the new port and wait forever)
    for k in list(env):
        if k.startswith("TORCHELASTIC_") or k in ("ROLE_RANK", "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE", "ROLE_NAME"):
            env.pop(k, None)
    r_res, r_err = run_half("rollout", env, os.path.join(res_dir, f"rollout_{rank}.json"), f"ref_rollout_rank{rank}.log")
    with open(os.path.join(res_dir, f"rollout_{rank}.done"), "w") as f:
        f.write(r_err or "ok")
    # every rank finishes its engine (and frees the GPU) before the trainer, which spans all ranks, starts
    deadline = time.time() + limit
    while time.time() < deadline and not all(os.path.exists(os.path.join(res_dir, f"rollout_{r}.done"))
                                             for r in range(world)):
        time.sleep(1.0)
    errs = [open(os.path.join(res_dir, f"rollout_{r}.done")).read() for r in range(world)
            if os.path.exists(os.path.join(res_dir, f"rollout_{r}.done"))]
    bad = [e for e in errs if e != "ok"]
    # ---- training half: the launch environment's ranks
    t_res, t_err = run_half("train", dict(os.environ), os.path.join(res_dir, "train.json"), f"ref_train_rank{rank}.log")
    if rank != 0:
        return 0
    if bad or len(errs) < world or t_err or t_res is None:
        out["unavailable"] = ("; ".join(bad[:1] + ([t_err] if t_err else [])) or "a rank did not report")[:500]
        return finish(out)
    rollout_s = max(json.load(open(os.path.join(res_dir, f"rollout_{r}.json")))["seconds_per_step"] for r in range(world))
    train_s = t_res["seconds_per_step"]
    n_seq = args.prompts_per_gpu * args.group * world
    seq_len = args.prompt_len + args.max_response
    step_s = rollout_s + train_s
    value = n_seq * seq_len / step_s
    out.update({
        "metric": "GRPO step tokens/s (prompt+response tokens generated and trained per second)", "value": value,
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic prompts (uniform random token ids), random-init weights, even-token-fraction reward",
        "config": {"model": "qwen2.5-7b-arch", "global_batch": n_seq, "seq_len": seq_len, "prompts": args.prompts_per_gpu * world,
                   "group": args.group, "prompt_len": args.prompt_len, "max_response": args.max_response,
                   "parallelism": f"colocated sequence rollout -> train on {world} GPU(s): vLLM tp1 per GPU, policy FSDP dp_shard{world}",
                   "settings": "the reference's shipped qwen2-5-7b GRPO job file: compile, gradient checkpointing, mini_batch 8"},
        "path": ("reference vLLMRollout.rollout_generation_single_turn + GRPOTrainer.step_training driven directly, one "
                 "process per half; its controller / worker glue needs redis-server, which this machine lacks; no weight "
                 "hand-over between the halves (upper bound of the reference's throughput)"),
        "breakdown": {"rollout_s": rollout_s, "train_s": train_s},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": n_seq * seq_len * 9,
                "d2h_bytes_per_step": n_seq * args.max_response * 8,
                "api": "tokenisation, host-to-device copies and detokenisation happen inside both timed calls"},
    })
    return finish(out)


# ---------------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.config == 1:
        # 8 prompts of 64 tokens, group 4, 64 response tokens, tiny Qwen2 architecture, two ranks on CPU
        if int(os.environ.get("RANK", "0")) == 0:
            from cosmos_rl_b200.bench_launcher import run
            a = argparse.Namespace(**vars(args))
            a.gpus, a.model, a.prompts_per_gpu, a.group, a.prompt_len, a.max_response = 2, "tiny-qwen2", 4, 4, 64, 64
            a.mb_tokens = 2048
            out = run(a, cpu=True)
            out["n_gpus"], out["config"]["parallelism"] = 0, "CPU / gloo: controller + 1 policy rank + 1 rollout rank"
            print(json.dumps(out))
        return 0
    if args.layout == "launcher":
        # the job starts its own processes: under a multi-rank launch only rank 0 acts, and it holds no GPU itself
        if int(os.environ.get("RANK", "0")) == 0:
            from cosmos_rl_b200.bench_launcher import run
            print(json.dumps(run(args)))
        return 0
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # convenience: re-launch under torchrun
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29511"),
                   os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    torch.cuda.set_device(local_rank)
    if args.config == 5:
        if world < 2:
            raise SystemExit("--config 5 needs at least 2 GPUs (one policy rank, one rollout rank)")
        from cosmos_rl_b200.rollout.weight_sync_bench import main as sweep
        return sweep(["--model", args.model, "--iters", str(max(args.steps, 3)), "--warmup", str(args.warmup)])
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from cosmos_rl_b200.bench_grpo import GRPOBench
    bench = GRPOBench(args, rank, world, local_rank)
    result = bench.run()
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        from cosmos_rl_b200.utils.dist_util import safe_destroy
        dist.barrier()
        safe_destroy(20.0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
