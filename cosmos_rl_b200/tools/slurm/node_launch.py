"""Per-node step of a SLURM job: reads this node's index and the node list from the SLURM environment, decides
which replicas live here (policy nodes first, then rollout nodes) and starts the launcher for them; node 0 hosts the
controller, the others attach to it (cosmos_rl/tools/slurm/cosmos_rl_slurm_launch.py)."""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
from typing import Dict, List, Optional


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


def node_assignment(node_idx: int, policy_nodes: int, rollout_nodes: int, n_policy: int, n_rollout: int) -> Dict[str, int]:
    """How many replicas of each role this node starts. Replicas spanning several nodes are started by the first node
    of their span with the launcher's multi-node rendezvous; packed replicas are split evenly over the role's nodes."""
    def share(n_rep: int, nodes: int, i: int) -> int:
        if nodes == 0 or i < 0 or i >= nodes:
            return 0
        if n_rep <= nodes:                       # each replica spans nodes // n_rep nodes
            return 1 if i % max(1, nodes // n_rep) == 0 and i // max(1, nodes // n_rep) < n_rep else 0
        return n_rep // nodes + (1 if i < n_rep % nodes else 0)
    return {"policy": share(n_policy, policy_nodes, node_idx),
            "rollout": share(n_rollout, rollout_nodes, node_idx - policy_nodes)}


def build_command(args, env: Dict[str, str]) -> Optional[List[str]]:
    nodes = expand_nodelist(env.get("SLURM_JOB_NODELIST", "localhost"))
    idx = int(env.get("SLURM_NODEID", "0"))
    a = node_assignment(idx, args.policy_nodes, args.rollout_nodes, args.n_policy_replicas, args.n_rollout_replicas)
    if a["policy"] == 0 and a["rollout"] == 0 and idx != 0:
        return None
    port = int(env.get("COSMOS_CONTROLLER_PORT", "8000"))
    cmd = [sys.executable, "-m", "cosmos_rl_b200.launcher.launch_all", "--config", args.config,
           "--policy", str(a["policy"]), "--rollout", str(a["rollout"]), "--num-workers", str(len(nodes)),
           "--worker-idx", str(idx), "--node-ip-list", ";".join(nodes), "--port", str(port)]
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
    ap.add_argument("--policy-nodes", type=int, required=True)
    ap.add_argument("--rollout-nodes", type=int, required=True)
    ap.add_argument("--n-policy-replicas", type=int, default=1)
    ap.add_argument("--n-rollout-replicas", type=int, default=1)
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("script", nargs="?", default=None)
    args = ap.parse_args(argv)
    cmd = build_command(args, dict(os.environ))
    if cmd is None:
        return 0
    return subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
