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
    ap.add_argument("--layout", default="auto", choices=["auto", "colocated", "disaggregated"],
                    help="auto: 8 GPUs use the named disaggregated layout (policy FSDP4 + rollout TP2 x 2); 1, 2 and 4 "
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
    """The reference arm: the unmodified reference from baseline/_ref through its own launcher API."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    out = {"impl": "reference"}
    if not os.path.isdir(os.path.join(ref, "cosmos_rl")):
        out["unavailable"] = "baseline/_ref is absent (the offline pip install --no-deps of the reference source tree was not done on this box)"
        print(json.dumps(out))
        return 0
    sys.path.insert(0, ref)
    reasons = []
    try:
        import cosmos_rl  # noqa: F401
    except Exception as e:
        reasons.append(f"import cosmos_rl fails: {type(e).__name__}: {e}")
    for mod in ("redis", "torchao"):
        try:
            __import__(mod)
        except Exception:
            reasons.append(f"python module {mod!r} missing")
    import shutil
    if shutil.which("redis-server") is None:
        reasons.append("redis-server binary missing (the controller hard-requires it)")
    if reasons:
        out["unavailable"] = ("reference installs with --no-deps but cannot run offline: " + "; ".join(reasons))[:400]
        print(json.dumps(out))
        return 0
    out["unavailable"] = "reference imports, but its launcher path was not wired in this build"
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
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
