"""Submit a job to SLURM from a login node: works out how many nodes the policy and rollout replicas need, writes
an sbatch script (code sandbox copy, auto-requeue on time-out, SIGUSR1 ahead of the limit so the trainer can
checkpoint, bounded retries) and calls ``sbatch`` (cosmos_rl/tools/slurm/dispatch_job.py,
cosmos_rl_job_multi_node.sh). ``--dry-run`` prints the script instead.

Every node runs ``node_launch.py``, which derives its index and the node address list from the SLURM environment
and starts the per-node launcher; node 0 also hosts the controller."""
from __future__ import annotations

import argparse
import math
import os
import shlex
import shutil
import subprocess
import sys
from typing import Dict, List, Optional

from cosmos_rl_b200.config import Config, load_toml
from cosmos_rl_b200.launcher.launch_all import gpus_per_replica


def plan_nodes(config: Config, n_policy: int, n_rollout: int, ngpu_per_node: int) -> Dict[str, int]:
    """Nodes per role. A replica larger than a node takes whole nodes; smaller replicas are packed per node."""
    def nodes_for(n_rep: int, gpus_each: int) -> int:
        if n_rep == 0:
            return 0
        if gpus_each >= ngpu_per_node:
            return n_rep * math.ceil(gpus_each / ngpu_per_node)
        return math.ceil(n_rep / (ngpu_per_node // gpus_each))
    gp, gr = gpus_per_replica(config.policy.parallelism), gpus_per_replica(config.rollout.parallelism)
    is_sft = config.train.train_policy.type == "sft"
    if config.mode == "colocated":
        return {"policy": nodes_for(n_policy, gp), "rollout": 0, "policy_gpus": gp, "rollout_gpus": gr}
    return {"policy": nodes_for(n_policy, gp), "rollout": 0 if is_sft else nodes_for(n_rollout, gr),
            "policy_gpus": gp, "rollout_gpus": gr}


def render_sbatch(args, plan: Dict[str, int], sandbox: str) -> str:
    n_nodes = plan["policy"] + plan["rollout"]
    extra = "".join(f"#SBATCH {x}\n" for x in (args.extra_sbatch_args or []))
    launch = (f"{shlex.quote(sys.executable if not args.container else 'python')} -m cosmos_rl_b200.tools.slurm.node_launch "
              f"--config {shlex.quote(args.config_path)} --policy-nodes {plan['policy']} --rollout-nodes {plan['rollout']} "
              f"--n-policy-replicas {args.n_policy_replicas} --n-rollout-replicas {args.n_rollout_replicas} "
              f"--log-dir {shlex.quote(os.path.join(args.output_root_path, args.job_name, 'logs'))}"
              + (f" {shlex.quote(args.launcher_script)}" if args.launcher_script else ""))
    srun = "srun --kill-on-bad-exit=1 " + (f"--container-image={shlex.quote(args.container)} "
                                           f"--container-mounts={shlex.quote(args.container_mounts)} " if args.container else "")
    return f"""#!/bin/bash
#SBATCH --job-name={args.job_name}
#SBATCH --nodes={n_nodes}
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node={args.ngpu_per_node}
#SBATCH --exclusive
#SBATCH --time={args.time}
#SBATCH --signal=B:USR1@{args.signal_lead_s}
#SBATCH --requeue
#SBATCH --output={os.path.join(args.output_root_path, args.job_name, 'slurm-%j.out')}
{f'#SBATCH --partition={args.slurm_partition}' if args.slurm_partition else ''}
{f'#SBATCH --account={args.slurm_account}' if args.slurm_account else ''}
{extra}
set -u
export PYTHONPATH={shlex.quote(sandbox)}:${{PYTHONPATH:-}}
export COSMOS_MAX_RETRIES={args.max_retries}
cd {shlex.quote(sandbox)}

requeue() {{
  echo "[slurm] time limit near: forwarding SIGUSR1 so the trainer checkpoints, then requeueing"
  kill -USR1 "$SRUN_PID" 2>/dev/null
  wait "$SRUN_PID"
  scontrol requeue "$SLURM_JOB_ID"
}}
trap requeue USR1

attempt=0
while :; do
  {srun}{launch} &
  SRUN_PID=$!
  wait "$SRUN_PID"
  rc=$?
  [ "$rc" -eq 0 ] && break
  attempt=$((attempt + 1))
  [ "$attempt" -gt "$COSMOS_MAX_RETRIES" ] && exit "$rc"
  echo "[slurm] attempt $attempt failed with $rc: resuming from the last checkpoint"
done
"""


def make_sandbox(output_root: str, job_name: str, repo_root: str) -> str:
    """Copy of the source tree the job runs from, so edits after submission do not change a queued job."""
    dst = os.path.join(output_root, job_name, "code")
    if not os.path.exists(dst):
        shutil.copytree(repo_root, dst, ignore=shutil.ignore_patterns(".git", "__pycache__", "*.ncu-rep", "outputs"))
    return dst


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="submit a cosmos-rl job to SLURM")
    ap.add_argument("--job-name", required=True)
    ap.add_argument("--config-path", required=True)
    ap.add_argument("--output-root-path", required=True)
    ap.add_argument("--ngpu-per-node", type=int, default=8)
    ap.add_argument("--n-policy-replicas", type=int, default=1)
    ap.add_argument("--n-rollout-replicas", type=int, default=1)
    ap.add_argument("--slurm-partition", default=None)
    ap.add_argument("--slurm-account", default=None)
    ap.add_argument("--time", default="04:00:00")
    ap.add_argument("--signal-lead-s", type=int, default=300, help="seconds before the limit at which SIGUSR1 is sent")
    ap.add_argument("--max-retries", type=int, default=3)
    ap.add_argument("--container", default=None)
    ap.add_argument("--container-mounts", default="")
    ap.add_argument("--extra-sbatch-args", nargs="*", default=None)
    ap.add_argument("--no-sandbox", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("launcher_script", nargs="?", default=None, help="user entry script (dataset / reward definitions)")
    args = ap.parse_args(argv)
    config = Config.from_dict(load_toml(args.config_path))
    plan = plan_nodes(config, args.n_policy_replicas, args.n_rollout_replicas, args.ngpu_per_node)
    repo_root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    sandbox = repo_root if (args.no_sandbox or args.dry_run) else make_sandbox(args.output_root_path, args.job_name, repo_root)
    script = render_sbatch(args, plan, sandbox)
    if args.dry_run:
        print(script)
        return 0
    job_dir = os.path.join(args.output_root_path, args.job_name)
    os.makedirs(job_dir, exist_ok=True)
    path = os.path.join(job_dir, "job.sbatch")
    with open(path, "w") as f:
        f.write(script)
    return subprocess.call(["sbatch", path])


if __name__ == "__main__":
    sys.exit(main())
