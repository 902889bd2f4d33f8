"""``cosmos-cli``: inspect and steer a running job through the controller's HTTP API
(cosmos_rl/cli/cli.py:26-36, cli/replica.py:38-95, cli/profiler.py:36-127, cli/nccl.py:33-67).

    cosmos-cli --url host:port replica ls            list replicas
    cosmos-cli --url host:port replica lsr NAME      show the ranks of one replica
    cosmos-cli --url host:port profile set NAME [--active-steps N --rank-filter 0 1 ...]
    cosmos-cli --url host:port nccl ls               list the handshake store (communicator rendezvous keys)
    cosmos-cli --url host:port status                step counters and buffers
"""
from __future__ import annotations

import argparse
import json
import sys

from ..dispatcher.api.client import APIClient
from ..utils import api_suffix as S


def _client(url: str) -> APIClient:
    return APIClient("CLI", remote_hosts=[url], max_retries=1)


def cmd_replica(args, api: APIClient):
    st = api.status()
    reps = st["policy_replicas"] + st["rollout_replicas"]
    if args.action == "ls":
        print(f"{'role':10s} {'replica':40s} {'status':14s} {'atoms':>7s} {'weight step':>12s}")
        for r in reps:
            print(f"{r['role']:10s} {r['name']:40s} {r['status']:14s} {r['n_atoms']:3d}/{r['expected_atoms']:<3d} "
                  f"{r['weight_step']:12d}")
    else:
        for r in reps:
            if r["name"] == args.name:
                print(json.dumps(r, indent=2))
                return 0
        print(f"no replica named {args.name}", file=sys.stderr)
        return 1
    return 0


def cmd_profile(args, api: APIClient):
    r = api.set_profile(args.name, active_steps=args.active_steps, rank_filter=args.rank_filter,
                        record_shape=args.record_shape, profile_memory=args.profile_memory,
                        with_stack=args.with_stack, with_modules=args.with_modules)
    print(r.get("message", r))
    return 0


def cmd_nccl(args, api: APIClient):
    info = api.get(S.COSMOS_API_NCCL_COMM_GET_ALL_SUFFIX).get("comm_info", {})
    for k in sorted(info):
        print(k)
    return 0


def cmd_status(args, api: APIClient):
    st = api.status()
    st.pop("policy_replicas", None)
    st.pop("rollout_replicas", None)
    print(json.dumps(st, indent=2))
    return 0


def cmd_algo(args, api: APIClient):
    """``cosmos-cli algo config``: the job configuration the controller serves to every worker
    (cosmos_rl/cli/algo.py)."""
    meta = api.get_controller_metadata()
    print(json.dumps(meta.get("config", meta), indent=2, sort_keys=True))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="cosmos-cli")
    ap.add_argument("--url", default="127.0.0.1:8000", help="controller address host:port")
    sub = ap.add_subparsers(dest="cmd", required=True)
    rp = sub.add_parser("replica")
    rp.add_argument("action", choices=["ls", "lsr"])
    rp.add_argument("name", nargs="?")
    pp = sub.add_parser("profile")
    pp.add_argument("action", choices=["set"])
    pp.add_argument("name")
    pp.add_argument("--active-steps", type=int, default=1)
    pp.add_argument("--rank-filter", type=int, nargs="*", default=[0])
    for flag in ("record-shape", "profile-memory", "with-stack", "with-modules"):
        pp.add_argument("--" + flag, action="store_true")
    np_ = sub.add_parser("nccl")
    np_.add_argument("action", choices=["ls"])
    sub.add_parser("status")
    al = sub.add_parser("algo")
    al.add_argument("action", choices=["config"])
    args = ap.parse_args(argv)
    api = _client(args.url)
    return {"replica": cmd_replica, "profile": cmd_profile, "nccl": cmd_nccl, "status": cmd_status,
            "algo": cmd_algo}[args.cmd](args, api)


if __name__ == "__main__":
    sys.exit(main())
