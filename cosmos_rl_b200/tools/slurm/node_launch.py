"""Per-node step of a SLURM job: reads this node's index and the node list from the SLURM environment and starts
the launcher with the job-wide replica counts (the launcher's plan decides which replicas, or which part of a
replica that spans nodes, live here); node 0 hosts the controller, the others attach to it (cosmos_rl/tools/slurm/cosmos_rl_slurm_launch.py)."""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
from typing import Dict, List


def expand_nodelist(spec: str) -> List[str]:
    """``node[01-03,07],gpu5`` -> node01 node02 node03 node07 gpu5 (the compact form SLURM_JOB_NODELIST uses)."""
    out: List[str] = []
    for m in re.finditer(r"([^,\[]+)(?:\[([^\]]+)\])?", spec):
        prefix, body = m.group(1), m.group(2)
        if not body:
            out.append(prefix)
            continue
        for part in body.split(","):
            if "-" in part:
                a, b = part.split("-")
                out.extend(f"{prefix}{i:0{len(a)}d}" for i in range(int(a), int(b) + 1))
            else:
                out.append(prefix + part)
    return out


def build_command(args, env: Dict[str, str]) -> List[str]:
    """The launcher call of this node. Every node passes the replica counts of the WHOLE job: the launcher derives the
    same node-by-node plan everywhere (policies first, a replica larger than a node spans whole nodes and meets at
    its first node's rendezvous port) and starts its own row; a node the plan leaves empty exits at once."""
    nodes = expand_nodelist(env.get("SLURM_JOB_NODELIST", "localhost"))
    idx = int(env.get("SLURM_NODEID", "0"))
    port = int(env.get("COSMOS_CONTROLLER_PORT", "8000"))
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", args.config,
           "--policy", str(args.n_policy_replicas), "--rollout", str(args.n_rollout_replicas),
           "--num-workers", str(len(nodes)), "--worker-idx", str(idx), "--node-ip-list", ";".join(nodes),
           "--port", str(port)]
    gpn = getattr(args, "gpus_per_node", None) or env.get("SLURM_GPUS_ON_NODE")
    if gpn:
        cmd += ["--gpus-per-node", str(int(str(gpn).split(":")[-1]))]
    if idx != 0:
        cmd += ["--url", f"{nodes[0]}:{port}", "--no-controller"]
    if args.log_dir:
        cmd += ["--log-dir", os.path.join(args.log_dir, f"node_{idx}")]
    if args.script:
        cmd += [args.script]
    return cmd


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--policy-nodes", type=int, default=0, help="informational: nodes the policies take")
    ap.add_argument("--rollout-nodes", type=int, default=0, help="informational: nodes the rollouts take")
    ap.add_argument("--gpus-per-node", type=int, default=None)
    ap.add_argument("--n-policy-replicas", type=int, default=1)
    ap.add_argument("--n-rollout-replicas", type=int, default=1)
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("script", nargs="?", default=None)
    args = ap.parse_args(argv)
    return subprocess.call(build_command(args, dict(os.environ)))


if __name__ == "__main__":
    sys.exit(main())
